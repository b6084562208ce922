#!/usr/bin/env python
"""Benchmark of the KDA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference] [--weak]

Default workload `train_bf16`: bf16 chunk_kda forward+backward, B=8 T=8192 H=32 d_k=d_v=128, chunk 64,
seeded synthetic inputs (kda_b200/inputs.py).  One step = one forward+backward over that batch.

With N > 1 (launched by torchrun, one rank per GPU) the stated batch is SHARDED: the (batch, head) recurrences
are independent, so rank r takes the batch rows `kda_b200.shard.batch_slice(B, r, N)` (B/N rows each), there is
no collective on the data path, and value = the whole batch's tokens / max-over-ranks time ("scaling":
"strong").  `--weak` runs N full replicas instead (every rank its own batch of the full shape).

Prints ONE JSON line:
  metric / value      tokens/s with the inputs resident in HBM (CUDA events, max over ranks);
  e2e                 the same step through the public host-resident API with pinned HOST buffers: host->device
                      copies of every input and device->host copies of every output inside the timed region;
  roofline            the kernel with the largest share of the step: ALGORITHMIC bytes (the operator-boundary
                      tensors that kernel must read and write: q, k, v, g, beta, o, dO and the gradients) per
                      launch / its average launch time (CUDA events recorded by the library around each kernel
                      during the timed steps) / the measured HBM copy bandwidth.  Beside it `design_bytes_per_launch`
                      (boundary tensors + the tiles this design exchanges between its kernels), `dram_efficiency`
                      (that figure / time / peak: how well the kernel streams what it does move), `traffic` (ncu DRAM
                      bytes of a smaller case scaled by units) and `wasted_traffic_ratio` = traffic / algorithmic;
  step_roofline       the whole step against both roofs (4,364 B and 559,787 FLOP per (token, head));
  workloads           (N = 1, default run) the other stated workloads, each timed on its own after the headline:
                      prefill forward, packed varlen forward+backward, decode (256 consecutive steps, GB/s against the
                      measured copy bandwidth and against the nominal 8 TB/s), and `gpu_bar`: flash-linear-attention's
                      own Triton kernels on the same GPU and shapes (a comparison; nothing of it is on the product path);
  cpu_baseline        the float32 token-recurrent PyTorch restatement on the host cores, bounded sample;
  clocks, gpu_launches, checks (outputs finite, device status words 0).

`--impl reference` times the CPU restatement alone, on all host threads (the NVlabs/kda repository has no
implementation of this operator to run).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from kda_b200.inputs import (WORKLOADS, decode_bytes_per_seq_head, flops_per_token_head, make_inputs,  # noqa: E402
                             make_workload, min_hbm_bytes_per_token_head)
from kda_b200.shard import balance_sequences, batch_head_block, batch_slice, take_sequences  # noqa: E402

METRIC = "KDA fwd+bwd tokens/s (H=32,d=128,bf16)"
NOMINAL_HBM_GBS = 8000.0

K_, V_, C_ = 128, 128, 64
_IN = 2 * K_ + 2 * K_ + 2 * V_ + 4 * K_ + 4                      # q,k,v bf16 + g fp32 + beta = 1,284 B
_GRADS = 2 * K_ + 2 * K_ + 2 * V_ + 4 * K_ + 4                   # dq,dk,dv bf16 + dg fp32 + dbeta = 1,284 B
_TK, _TT, _VK = 2 * K_, 2 * C_, 2 * K_ * V_ / C_                 # bytes per token of a [64x128], [64x64], [128x128] bf16 tile
# Per kernel and per (token, head): (FLOPs, ALGORITHMIC bytes, DESIGN bytes).
#   algorithmic = the operator-boundary tensors the kernel must touch.  Forward 1,540 B = prepare 1,284 (q,k,v,g,beta)
#                 + scan 256 (o).  Backward 2,824 B = q,k,v,g,beta,dO read + dq,dk,dv,dg,dbeta written, all of it by
#                 bwd_main; the reverse scan reads dO (256 B) a second time, which is its only boundary tensor.
#   design      = algorithmic + the per-chunk tiles this design moves between its kernels through HBM.
# GEMM = 2mnk, triangular products counted full, the 64x64 inverse as (2/3) C^2 per token.
KERNEL_WORK = {
    "prepare": (2 * C_ * (3 * K_ + V_) + (2.0 / 3.0) * C_ * C_, _IN, _IN + 4 * _TK + _TT + 2 * _TT + 8),
    "scan": (6 * K_ * V_ + 2 * C_ * V_, 2 * V_, 4 * _TK + _TT + 8 + 2 * V_ + _VK + _TK),
    "bwd_scan": (6 * K_ * V_ + 2 * C_ * V_, 2 * V_, 3 * _TK + _TT + 8 + 2 * V_ + _VK + _TK),
    "bwd_main": (6 * K_ * V_ + 12 * C_ * K_ + 6 * C_ * V_ + 4 * C_ * C_, _IN + 2 * V_ + _GRADS,
                 _IN + 2 * V_ + 2 * _TT + 2 * _VK + 2 * _TK + _GRADS),
    "gate_fwd": (12 * K_, 2 * K_ + 4 * K_ + 2 + 4, 2 * K_ + 4 * K_ + 2 + 4),
    "gate_bwd": (20 * K_, 4 * K_ + 2 * K_ + 2 * K_ + 4 + 2 + 2, 4 * K_ + 2 * K_ + 2 * K_ + 4 + 2 + 2),
}
# DRAM bytes per (token, head) that ncu measured (dram__bytes_read.sum + dram__bytes_write.sum of one launch) on a
# small case of each kernel (B=1 T=8192, 262,144 (token, head) units; the one-CTA-per-unit scans at B=2; summaries under
# profiles/).  Traffic grows in proportion to the units, so a launch's traffic is this figure times its units.
KERNEL_TRAFFIC = {"prepare": 2524.0, "scan": 2112.0, "bwd_scan": 1870.0, "bwd_main": 4572.0, "decode": 125600.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sust=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sust=1400.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, interval_ms: int = 20):
        self.index, self.proc, self.lines, self.interval_ms = index, None, [], interval_ms

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", str(self.interval_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
            return
        # nvidia-smi needs up to a second to initialise, and while it does the driver delays other processes'
        # launches (measured: +4 % on a 150 ms timed region that overlapped it, nothing once it is sampling):
        # wait for its first line before any step runs
        t0 = time.time()
        while not self.lines and self.proc.poll() is None and time.time() - t0 < 10.0:
            time.sleep(0.05)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()          # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        load = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
        return dict(sm_mhz=(statistics.median(load) if load else None), sm_max_mhz=(max(mx) if mx else None),
                    reasons=sorted(reasons), samples=len(sm))


def cpu_baseline(threads: int, T: int = 1024, backward: bool = True):
    """The oracle's recurrence in float32 on the host cores (fla/ops/kda/naive.py:12-66 restated in
    oracle/kda_oracle.py), forward+backward by autograd, B=1 H=32 d=128.  Returns tokens/s."""
    from oracle.kda_oracle import recurrent_kda
    torch.set_num_threads(threads)
    d = make_inputs(1, T, 32, 128, 128, torch.float32, seed=0, h0_std=0.02, backward=True)
    leaves = [d[n].clone().requires_grad_(backward) for n in ("q", "k", "v", "g", "beta")]
    h0 = d["h0"].clone().requires_grad_(backward)
    t0 = time.perf_counter()
    o, ht = recurrent_kda(*leaves, initial_state=h0, output_final_state=True, dtype=torch.float32)
    if backward:
        torch.autograd.grad([o, ht], leaves + [h0], [d["do"], d["dht"]])
    dt = time.perf_counter() - t0
    return T / dt, dt


def run_reference(args, rank):
    """Reference arm: the CPU restatement, all host threads, bounded sample per step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    T = 512
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline(threads, T=128)
    times = []
    for _ in range(args.steps):
        tps, dt = cpu_baseline(threads, T=T)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = T / (ms / 1e3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak" if args.weak else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "train_bf16 (B=8 T=8192 H=32 K=V=128 fwd+bwd)",
                   "sample": f"B=1 T={T} H=32 K=V=128 per step"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"token-recurrent float32 PyTorch forward+backward, B=1 T={T} H=32 K=V=128 per step"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# =====================================================================================================================
# steps of the workloads on device-resident inputs
# =====================================================================================================================

def make_step(workload: str, x: dict, cu, gate: bool = False, l2: bool = False, safe: bool = False):
    """Returns (step function over a dict of device tensors, kernel launches per step, names that get gradients)."""
    from kda_b200 import chunk_kda, fused_recurrent_kda_fwd
    w = WORKLOADS[workload]
    if workload == "decode":
        state = x["h0"].clone()
        dec_kw = dict(use_qk_l2norm_in_kernel=l2)
        if gate:       # the layer's decode call: raw gate input, beta logits; activated inside the one kernel
            dec_kw.update(use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, A_log=x["A_log"], dt_bias=x["dt_bias"])

        def step(x=x):
            return fused_recurrent_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=128 ** -0.5, initial_state=state,
                                           inplace_final_state=True, **dec_kw)
        return step, 1, []
    if w.backward:
        grad_names = ["q", "k", "v", "g", "beta"] + (["h0"] if x.get("h0") is not None else []) + (["A_log", "dt_bias"] if gate else [])
        gate_kw = dict(use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True) if gate else {}

        def step(x=x):
            leaves = [x[n].requires_grad_(True) for n in grad_names]
            kw = dict(gate_kw, A_log=x["A_log"], dt_bias=x["dt_bias"]) if gate else {}
            o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"),
                              output_final_state=True, cu_seqlens=cu, use_qk_l2norm_in_kernel=l2, safe_gate=safe, **kw)
            grads = torch.autograd.grad([o, ht], leaves, [x["do"], x["dht"]])
            return (o, ht) + tuple(grads)
        if x["q"].dtype == torch.float32:
            return step, 3, grad_names                    # token-recurrent forward, backward, its finishing kernel
        return step, (10 if gate else 5), grad_names      # gate: + activation, beta sigmoid; + their backward and the reduction

    def step(x=x):
        with torch.no_grad():
            return chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"),
                             output_final_state=True, cu_seqlens=cu, use_qk_l2norm_in_kernel=l2, safe_gate=safe)
    return step, (1 if x["q"].dtype == torch.float32 else 3), []


def time_steps(step, steps: int, warmup: int) -> float:
    """Milliseconds per step: CUDA events on the current stream, after `warmup` untimed steps, synchronised both sides."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def other_workloads(peaks, dev) -> dict:
    """The stated workloads beside the headline one, each timed on its own on device-resident inputs that are
    drawn on the device (seeded).  Inputs exceed L2 by far in every case, so no flush between steps."""
    from kda_b200 import _lib
    out = {}
    for name, steps in (("prefill_bf16", 20), ("varlen_bf16", 5), ("decode", 256)):
        w = WORKLOADS[name]
        try:
            x = make_workload(name, seed=0, device=dev, generate_on_device=True)
            cu = x.pop("cu_seqlens")
            step, launches, _ = make_step(name, x, cu)
            ms = time_steps(step, steps, 3)
            B, T, H = x["q"].shape[:3]
            tokens, th = B * T, B * T * H
            rec = {"config": f"B={B} T={T} H={H} K=V=128" + (f", {cu.numel() - 1} packed sequences" if cu is not None else ""),
                   "ms_per_step": ms, "steps": steps, "value": tokens / (ms / 1e3), "unit": "tokens/s",
                   "gpu_launches": launches * steps}
            if name == "decode":
                byt = B * H * decode_bytes_per_seq_head()
                gbs = byt / (ms * 1e-3) / 1e9
                rec.update({"hbm_gbs": gbs, "hbm_frac_of_measured": gbs / peaks["hbm"], "hbm_frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS,
                            "algorithmic_bytes_per_step": byt, "status": _lib.recurrent_status()})
            else:
                by = min_hbm_bytes_per_token_head(backward=w.backward) * th
                fl = flops_per_token_head(backward=w.backward) * th
                rec.update({"hbm_frac_min_traffic": by / (ms * 1e-3) / 1e9 / peaks["hbm"],
                            "tensor_frac_sustained": fl / (ms * 1e-3) / 1e12 / peaks["tf_sust"]})
            out[name] = rec
            del x, step
        except Exception as e:          # noqa: BLE001   (a workload that does not fit must not lose the headline line)
            out[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
    return out


# =====================================================================================================================
# the on-box GPU comparison: flash-linear-attention's Triton kernels, in a child process with a deadline
# =====================================================================================================================

def gpu_bar_child():
    """Runs in a child process: times fla.ops.kda on train / prefill / decode shapes and prints one JSON line per
    workload as soon as it is measured (so that a deadline in the parent keeps what finished)."""
    try:
        import fla
        import triton
        from fla.ops.kda import chunk_kda as fla_chunk_kda
        from fla.ops.kda import fused_recurrent_kda as fla_recurrent_kda
    except Exception as e:          # noqa: BLE001
        print(json.dumps({"workload": "*", "unavailable": f"unavailable on this box: {type(e).__name__}: {e}"[:300]}), flush=True)
        return
    impl = f"flash-linear-attention {getattr(fla, '__version__', '?')}, Triton {triton.__version__}"
    dev = torch.device("cuda", 0)
    for name, steps in (("train_bf16", 5), ("prefill_bf16", 10), ("decode", 64)):
        w = WORKLOADS[name]
        try:
            x = make_workload(name, seed=0, device=dev, generate_on_device=True)
            x.pop("cu_seqlens")
            grad_names = ["q", "k", "v", "g", "beta", "h0"]

            def step():
                if name == "decode":      # fla's public entry point returns the new state in a second buffer (same bytes moved)
                    with torch.no_grad():
                        return fla_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=128 ** -0.5,
                                                 initial_state=x["h0"], output_final_state=True)
                if w.backward:
                    leaves = [x[n].detach().requires_grad_(True) for n in grad_names]
                    t = dict(zip(grad_names, leaves))
                    o, ht = fla_chunk_kda(t["q"], t["k"], t["v"], t["g"], t["beta"], initial_state=t["h0"], output_final_state=True)
                    return torch.autograd.grad([o, ht], leaves, [x["do"], x["dht"]])
                with torch.no_grad():
                    return fla_chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True)
            ms = time_steps(step, steps, 3)
            B, T = x["q"].shape[:2]
            print(json.dumps({"workload": name, "impl": f"fla.ops.kda ({impl})", "ms_per_step": ms, "steps": steps,
                              "value": B * T / (ms / 1e3), "unit": "tokens/s"}), flush=True)
            del x
            torch.cuda.empty_cache()
        except Exception as e:          # noqa: BLE001
            print(json.dumps({"workload": name, "unavailable": f"unavailable on this box: {type(e).__name__}: {e}"[:300]}), flush=True)


def gpu_bar(deadline_s: float) -> dict:
    """Runs gpu_bar_child() in a child process (Triton compiles for a minute or more) and keeps what it measured
    before the deadline."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0])
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    out = {}
    try:
        p = subprocess.Popen([sys.executable, os.path.abspath(__file__), "--gpu-bar-child"], stdout=subprocess.PIPE,
                             stderr=subprocess.DEVNULL, text=True, env=env)
    except OSError as e:
        return {"unavailable": f"unavailable on this box: {e}"}
    try:
        stdout, _ = p.communicate(timeout=deadline_s)
    except subprocess.TimeoutExpired:
        p.kill()                         # the exact child started above
        stdout, _ = p.communicate()
        out["note"] = f"stopped at the {deadline_s:.0f} s deadline; workloads not listed were not reached"
    for ln in (stdout or "").splitlines():
        try:
            rec = json.loads(ln)
        except ValueError:
            continue
        out[rec.pop("workload", "?")] = rec
    if not out:
        out["unavailable"] = "unavailable on this box: the comparison process printed nothing"
    return out


# =====================================================================================================================

def shard_inputs(args, w, rank, world, dev):
    """This rank's share of the workload as host tensors (headline workload: CPU generator, one seed per batch row,
    so that the union over ranks is the same batch for every N) or device tensors (the others)."""
    B = max(1, w.B // args.scale_down)
    if args.workload == "train_bf16" and not w.n_seqs:
        rows = range(B) if (args.weak or world == 1) else range(B)[batch_slice(B, rank, world)]
        seed0 = rank * 1000 if args.weak else 0
        parts = [make_inputs(1, w.T, w.H, w.K, w.V, w.dtype, seed=seed0 + r, h0_std=w.h0_std, backward=True) for r in rows]
        host = {n: torch.cat([p[n] for p in parts], 0) for n in parts[0] if parts[0][n] is not None}
        return host, None, B * w.T * (world if args.weak else 1)
    # other workloads: drawn on the device, then this rank's share is cut out
    x = make_workload(args.workload, seed=(rank if args.weak else 0), device=dev, scale_down=args.scale_down, generate_on_device=True)
    cu = x.pop("cu_seqlens")
    x = {n: t for n, t in x.items() if t is not None}
    total = x["q"].shape[0] * x["q"].shape[1]
    if args.weak or world == 1:
        return x, cu, total * world
    if cu is not None:                                   # whole sequences, balanced by token count
        lens = (cu[1:] - cu[:-1]).tolist()
        mine = balance_sequences(lens, world)[rank]
        cul = cu.tolist()
        y = {}
        for n, t in x.items():
            if n in ("h0", "dht"):
                y[n] = t[mine].contiguous()
            else:
                y[n], new_cu = take_sequences(t, cul, mine)
        return y, new_cu.to(dev), total
    if args.workload == "decode":
        sl = batch_slice(x["q"].shape[0], rank, world)
        return {n: t[sl].contiguous() for n, t in x.items()}, None, total
    b0, b1, h0, h1 = batch_head_block(x["q"].shape[0], w.H, rank, world)      # (batch x head) units, contiguous block
    return {n: (t[b0:b1, h0:h1] if n in ("h0", "dht") else t[b0:b1, :, h0:h1]).contiguous() for n, t in x.items()}, None, total


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_bf16", choices=sorted(WORKLOADS))
    ap.add_argument("--weak", action="store_true", help="N > 1: every rank runs its own full batch (replicas) instead of a shard")
    ap.add_argument("--scale-down", type=int, default=1, help="divide the batch (smaller case for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the other workloads and the Triton comparison")
    ap.add_argument("--gate", action="store_true",
                    help="call the operator as the layer does: raw bf16 gate input + A_log + dt_bias and beta logits "
                         "(use_gate_in_kernel, use_beta_sigmoid_in_kernel); training workloads and decode")
    ap.add_argument("--l2norm", action="store_true", help="use_qk_l2norm_in_kernel=True (chunked workloads)")
    ap.add_argument("--safe-gate", action="store_true",
                    help="bounded gates g = -5 sigmoid(x) and safe_gate=True: the forward's tensor-core diagonal blocks (chunked workloads)")
    ap.add_argument("--gpu-bar-deadline", type=float, default=240.0, help="seconds the Triton comparison may take (0: skip it)")
    ap.add_argument("--clock-interval-ms", type=int, default=20, help="nvidia-smi sampling interval during the timed region")
    ap.add_argument("--gpu-bar-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()

    if args.gpu_bar_child:
        gpu_bar_child()
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; kda_b200 has no CPU path")
    args.warmup = max(args.warmup, 3)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from kda_b200 import _lib
    w = WORKLOADS[args.workload]
    peaks = load_peaks()
    mine, cu, job_tokens = shard_inputs(args, w, rank, world, dev)
    if args.gate:
        if not w.backward and args.workload != "decode":
            raise SystemExit("--gate needs a forward+backward workload or the decode workload")
        gen = torch.Generator().manual_seed(1000 + rank)
        mine["g"] = torch.randn(mine["g"].shape, generator=gen).bfloat16().to(mine["g"].device)            # raw gate input
        mine["beta"] = torch.randn(mine["beta"].shape, generator=gen).bfloat16().to(mine["beta"].device)   # beta logits
        mine["A_log"] = torch.log(torch.empty(w.H).uniform_(1, 16, generator=gen))
        mine["dt_bias"] = torch.randn(w.H * w.K, generator=gen)
    if args.safe_gate:
        if args.gate or args.workload == "decode" or w.dtype != torch.bfloat16:
            raise SystemExit("--safe-gate goes with the bf16 chunked workloads, without --gate")
        gen = torch.Generator().manual_seed(2000 + rank)
        mine["g"] = (-5.0 * torch.sigmoid(2.0 * torch.randn(mine["g"].shape, generator=gen))).to(mine["g"].device)      # g >= -5
    names = list(mine)
    host_resident = not mine["q"].is_cuda
    pinned = {n: mine[n].pin_memory() for n in names} if host_resident else None
    devt = {n: (pinned[n].to(dev, non_blocking=True) if host_resident else mine[n].to(dev)) for n in names}
    B, T, H = devt["q"].shape[:3]
    tokens = B * T                                       # this rank's tokens per step
    torch.cuda.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def maxms(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    step, launches_per_step, grad_names = make_step(args.workload, devt, cu, args.gate, args.l2norm, args.safe_gate)

    # ---------------- kernel-resident timing ----------------
    sampler = ClockSampler(local_rank if os.environ.get("CUDA_VISIBLE_DEVICES") is None else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]), args.clock_interval_ms)
    if rank == 0:
        sampler.start()          # returns once nvidia-smi delivers samples
    # the warm-up keeps each step's results alive until the next step has produced its own, exactly as the timed loop
    # does: otherwise the caching allocator meets the second set of output and workspace blocks only inside the timed
    # region, and its cudaMalloc calls (milliseconds, longer when several ranks of a box allocate at once) stall the host
    # while the GPU runs dry
    outs = None
    for _ in range(args.warmup):
        outs = step()
    barrier()
    _lib.profile_enable(True)      # the library's event pair around every kernel: per-kernel times over the timed region itself
    _lib.profile_read(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_host = time.perf_counter()
    e0.record()
    host_marks = []
    for _ in range(args.steps):
        outs = step()
        host_marks.append(time.perf_counter())
    e1.record()
    host_issue_ms = (time.perf_counter() - t_host) * 1e3 / args.steps      # what the host needs to queue one step
    if os.environ.get("KDA_BENCH_HOST_MARKS"):
        print("host ms per step:", [round((b - a) * 1e3, 3) for a, b in zip([t_host] + host_marks[:-1], host_marks)], file=sys.stderr, flush=True)
    barrier()
    ms_rank = e0.elapsed_time(e1)
    ms_total = maxms(ms_rank)
    if world > 1:
        per_rank = torch.zeros(world, 2, device=dev, dtype=torch.float64)
        per_rank[rank, 0], per_rank[rank, 1] = ms_rank / args.steps, host_issue_ms
        dist.all_reduce(per_rank)
        ranks_ms, ranks_host = [round(x, 4) for x in per_rank[:, 0].tolist()], [round(x, 4) for x in per_rank[:, 1].tolist()]
    else:
        ranks_ms, ranks_host = [round(ms_rank / args.steps, 4)], [round(host_issue_ms, 4)]
    stages = _lib.profile_read(reset=True)
    _lib.profile_enable(False)
    # what was timed is checked: every output finite, no bounded wait gave up, cu_seqlens accepted
    checks = {"outputs_finite": all(bool(torch.isfinite(t.float()).all()) for t in outs if isinstance(t, torch.Tensor)),
              "decode_status": _lib.recurrent_status()}
    del outs
    clocks = None
    if rank == 0:
        # a timed region of a few milliseconds (decode) ends before nvidia-smi delivers: keep the same step running,
        # untimed, until a few samples under load exist
        extended = False
        t_ext = time.time()
        while len(sampler.lines) < 5 and sampler.proc is not None and time.time() - t_ext < 4.0:
            extended = True
            for _ in range(8):
                step()
            torch.cuda.synchronize()
        clocks = sampler.stop()
        if extended:
            clocks["note"] = "timed region shorter than the sampling interval: sampled over untimed repeats of the same step right after it"
    ms_step = ms_total / args.steps
    value = job_tokens / (ms_step / 1e3)

    # ---------------- end to end: pinned host buffers in, every output back out ----------------
    e2e = None
    if not args.no_e2e and host_resident:
        out_host = None
        pipelined = w.backward and cu is None and args.workload != "decode" and not args.gate and not args.l2norm and not args.safe_gate
        head_groups = 4 if (pipelined and B < 4) else None      # few batch rows: cut the pieces along the heads as well

        def e2e_step():
            nonlocal out_host
            if pipelined:
                # public host-resident API: batch slices pipelined over copy-in / compute / copy-out streams; consecutive
                # steps are queued without waiting (two alternating sets of pinned output buffers), so step i+1's
                # copy-in runs under step i's copy-out; the timed region ends after the last result has landed
                from kda_b200.host import chunk_kda_fwd_bwd_host
                out_sets[e2e_count[0] & 1] = out_host = chunk_kda_fwd_bwd_host(pinned, out_sets[e2e_count[0] & 1], wait=False,
                                                                              head_groups=head_groups)
                e2e_count[0] += 1
                return
            x = {n: pinned[n].to(dev, non_blocking=True) for n in names}
            res = [t for t in step(x) if t is not None]
            if out_host is None:
                out_host = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res]
            for hbuf, t in zip(out_host, res):
                hbuf.copy_(t, non_blocking=True)

        def e2e_drain():
            if pipelined:
                from kda_b200.host import host_synchronize
                host_synchronize()
        out_sets, e2e_count = [None, None], [0]
        e2e_step()
        e2e_step()              # both output sets exist (pinned allocations stay outside the timed region)
        e2e_drain()
        barrier()
        n_e2e = max(1, min(args.steps, 10))
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e2e_drain()             # every step's results are in host memory
        e1.record()
        barrier()
        ms_e2e = maxms(e0.elapsed_time(e1)) / n_e2e
        h2d = sum(pinned[n].numel() * pinned[n].element_size() for n in names)
        d2h = sum(t.numel() * t.element_size() for t in (out_host.values() if isinstance(out_host, dict) else out_host))
        e2e = {"value": job_tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "bytes": "per rank", "steps": n_e2e,
               "api": "kda_b200.host.chunk_kda_fwd_bwd_host(wait=False) + host_synchronize (batch slices pipelined over 3 streams, "
                      "consecutive steps overlapped, results of all steps in host memory before the clock stops)" if pipelined else "kda_b200.chunk_kda"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- roofline of the dominant kernel ----------------
    th = tokens * H                                      # (token, head) units one launch of this rank processes
    roof = None
    if args.workload == "decode":
        byt = B * H * decode_bytes_per_seq_head()
        ach = byt / (ms_step * 1e-3) / 1e9
        roof = {"kernel": "kda_decode_bulk_kernel", "bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": ach / peaks["hbm"], "frac_of_nominal_8tbs": ach / NOMINAL_HBM_GBS, "traffic": KERNEL_TRAFFIC["decode"] * B * H,
                "traffic_source": "ncu capture of a smaller case, scaled by units", "peak_source": peaks["src"]}
        kernels = {}
    else:
        kernels = {s: {"ms_per_launch": (ms / n), "launches": n} for s, (ms, n) in stages.items() if n > 0}
        for s_, kv in kernels.items():
            if s_ in KERNEL_WORK:
                sec_ = kv["ms_per_launch"] * 1e-3
                kv["hbm_frac"] = KERNEL_WORK[s_][1] * th / sec_ / 1e9 / peaks["hbm"]          # algorithmic bytes, "of measured"
                kv["dram_efficiency"] = KERNEL_WORK[s_][2] * th / sec_ / 1e9 / peaks["hbm"]   # design bytes (boundary + tiles)
                kv["tensor_frac_sustained"] = KERNEL_WORK[s_][0] * th / sec_ / 1e12 / peaks["tf_sust"]
        staged = [s for s in kernels if s in KERNEL_WORK]
        dom = max(staged, key=lambda s: kernels[s]["ms_per_launch"] * kernels[s]["launches"]) if staged else None
        if dom is None:
            # float32 tensors: the token-recurrent pair of kernels, which the library does not time one by one; the whole
            # step against the operator-boundary bytes (all tensors float32)
            io = 4 * (3 * 128 + 2 * 128 + 1) + (4 * (4 * 128 + 2 * 128 + 1) if w.backward else 0)
            ach = io * th / (ms_step * 1e-3) / 1e9
            roof = {"kernel": "kda_recurrent_kernel" + (" + kda_recurrent_bwd_kernel" if w.backward else ""), "bound": "hbm",
                    "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s", "frac": ach / peaks["hbm"], "traffic": None,
                    "peak_source": peaks["src"], "algorithmic_bytes_per_launch": io * th,
                    "note": "exact fp32 path: one warp (forward) or CTA (backward) per (sequence, head), token-serial; not HBM-bound"}
    if roof is None:
        fl, by, design = KERNEL_WORK[dom]
        sec = kernels[dom]["ms_per_launch"] * 1e-3
        ridge = peaks["tf_sust"] * 1e12 / (peaks["hbm"] * 1e9)
        if fl / by >= ridge:
            ach = fl * th / sec / 1e12
            roof = {"kernel": dom, "bound": "tensor", "achieved": ach, "peak": peaks["tf_sust"], "unit": "TFLOP/s",
                    "frac": ach / peaks["tf_sust"]}
        else:
            ach = by * th / sec / 1e9
            roof = {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                    "frac": ach / peaks["hbm"]}
        traffic = KERNEL_TRAFFIC[dom] * th if dom in KERNEL_TRAFFIC else None
        roof.update({"traffic": traffic, "traffic_source": "ncu capture of a smaller case, scaled by units",
                     "wasted_traffic_ratio": (traffic / (by * th)) if traffic else None,
                     "peak_source": peaks["src"], "ms_per_launch": kernels[dom]["ms_per_launch"],
                     "algorithmic_flops_per_launch": fl * th, "algorithmic_bytes_per_launch": by * th,
                     "design_bytes_per_launch": design * th, "dram_efficiency": design * th / sec / 1e9 / peaks["hbm"],
                     "tensor_frac_sustained": fl * th / sec / 1e12 / peaks["tf_sust"]})
    # whole-step roofline fractions (both bounds) of this rank's share
    fl_step = flops_per_token_head(backward=w.backward) * th
    by_step = min_hbm_bytes_per_token_head(backward=w.backward) * th
    whole = {"tensor_frac_sustained": fl_step / (ms_step * 1e-3) / 1e12 / peaks["tf_sust"],
             "hbm_frac_min_traffic": by_step / (ms_step * 1e-3) / 1e9 / peaks["hbm"]}

    cpu = None
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        cpu_baseline(threads, T=64, backward=w.backward)          # warm-up of the thread pool and the allocator
        reps, spent = 0, 0.0
        while spent < 10.0 and reps < 64:                          # a bounded sample: about ten seconds of CPU work
            _, dt = cpu_baseline(threads, T=512, backward=w.backward)
            reps += 1
            spent += dt
        cpu = {"value": reps * 512 / spent, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": f"token-recurrent float32 PyTorch {'forward+backward' if w.backward else 'forward'}, "
                         f"{reps} x (B=1 T=512 H=32 K=V=128), {spent:.1f} s"}

    workloads = None
    default_run = args.workload == "train_bf16" and not args.gate and not args.l2norm and not args.safe_gate and args.scale_down == 1
    if default_run and world == 1 and not args.no_workloads:
        del devt, step
        torch.cuda.empty_cache()
        workloads = other_workloads(peaks, dev)
        workloads["gpu_bar"] = gpu_bar(args.gpu_bar_deadline) if args.gpu_bar_deadline > 0 else {"unavailable": "skipped (--gpu-bar-deadline 0)"}
        ours = {"train_bf16": ms_step, "prefill_bf16": workloads.get("prefill_bf16", {}).get("ms_per_step"),
                "decode": workloads.get("decode", {}).get("ms_per_step")}
        for n, rec in workloads["gpu_bar"].items():
            if isinstance(rec, dict) and rec.get("ms_per_step") and ours.get(n):
                rec["kda_b200_ms_per_step"] = ours[n]
                rec["speedup_over_it"] = rec["ms_per_step"] / ours[n]

    strong = world > 1 and not args.weak
    line = {
        "metric": METRIC if (args.workload == "train_bf16" and not args.gate and not args.l2norm and not args.safe_gate) else
                  f"KDA {args.workload}{' +gate' if args.gate else ''}{' +l2norm' if args.l2norm else ''} tokens/s",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if (args.weak and world > 1) else "strong",
        "vs_baseline": None, "dtype": "f32" if w.dtype == torch.float32 else "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} (B={B * (world if strong else 1)} T={T} H={H} K=V=128, chunk 64"
                               f"{', fwd+bwd' if w.backward else ''}{', packed varlen' if cu is not None else ''}"
                               f"{', gate + beta sigmoid in kernel' if args.gate else ''}{', q/k l2norm in kernel' if args.l2norm else ''}"
                               f"{', bounded gates + safe_gate' if args.safe_gate else ''})",
                   "per_gpu_batch": B, "sharding": ("batch rows over ranks, no collective on the data path" if strong else
                                                    ("replicas" if world > 1 else "one GPU")),
                   "l2": "inputs of a step far exceed the 126 MB L2; no flush needed",
                   "seed": "one per batch row" if host_resident else "0 (drawn on the device)"},
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks, "checks": checks,
        "ms_per_step_by_rank": ranks_ms, "host_issue_ms_per_step_by_rank": ranks_host,
        "roofline": roof, "step_roofline": whole, "kernels": kernels, "cpu_baseline": cpu,
    }
    if workloads is not None:
        line["workloads"] = workloads
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
