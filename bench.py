#!/usr/bin/env python
"""Benchmark of the KDA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Default workload `train_bf16`: bf16 chunk_kda forward+backward, B=8 T=8192 H=32 d_k=d_v=128, chunk 64,
seeded synthetic inputs (kda_b200/inputs.py).  One step = one forward+backward over that batch.
With N > 1 (launched by torchrun, one rank per GPU) every rank runs its own batch of the same shape
(independent (batch, head) shards, no collective on the data path): weak scaling, value = all ranks'
tokens / max-over-ranks time.

Prints ONE JSON line: metric/value (inputs resident in HBM), `e2e` (same step through the public
operator with pinned HOST buffers: host->device copies of every input and device->host copies of
every output inside the timed region), `roofline` of the dominant kernel (per-kernel times from CUDA
events recorded by the library around each kernel during the timed steps), `cpu_baseline` (the
float32 token-recurrent PyTorch restatement on the host cores, bounded sample), clocks, launches.

`--impl reference` times that CPU restatement alone, on all host threads (the NVlabs/kda repository
has no implementation of this operator to run).  `--gpu-bar` adds a `gpu_bar` object: flash-linear-attention's
own Triton chunk_kda timed on the same GPU and inputs, when that package imports (a comparison, off by default).
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

METRIC = "KDA fwd+bwd tokens/s (H=32,d=128,bf16)"

# Algorithmic work of each kernel per (token, head): C=64, K=V=128; GEMM = 2mnk, triangular products
# counted full, the 64x64 inverse as (2/3) C^2 per token; bytes = the tensors the kernel must read and
# write at the operator boundary plus the tiles it exchanges with the neighbouring kernels.
K_, V_, C_ = 128, 128, 64
_IN = 2 * K_ + 2 * K_ + 2 * V_ + 4 * K_ + 4                      # q,k,v bf16 + g fp32 + beta
_TK, _TT, _VK = 2 * K_, 2 * C_, 2 * K_ * V_ / C_                 # bytes per token of a [64x128], [64x64], [128x128] bf16 tile
KERNEL_WORK = {
    # name: (flops, bytes) per (token, head)
    "prepare": (2 * C_ * (3 * K_ + V_) + (2.0 / 3.0) * C_ * C_, _IN + 4 * _TK + _TT + 2 * _TT + 8),
    "scan": (6 * K_ * V_ + 2 * C_ * V_, 4 * _TK + _TT + 8 + 2 * V_ + _VK + _TK),
    "bwd_scan": (6 * K_ * V_ + 2 * C_ * V_, 3 * _TK + _TT + 8 + 2 * V_ + _VK + _TK),
    "bwd_main": (6 * K_ * V_ + 12 * C_ * K_ + 6 * C_ * V_ + 4 * C_ * C_,
                 _IN + 2 * V_ + 2 * _TT + 2 * _VK + 2 * _TK + (2 * K_ + 2 * K_ + 2 * V_ + 4 * K_ + 4)),   # = 4,616 B
    # gate front end with bf16 raw inputs: fwd reads g_raw, beta logits, writes g, beta (fp32);
    # bwd reads dg, dbeta (fp32), g_raw, beta logits, writes dg_raw, dbeta_raw (bf16)
    "gate_fwd": (12 * K_, 2 * K_ + 4 * K_ + 2 + 4),                # = 774 B
    "gate_bwd": (20 * K_, 4 * K_ + 2 * K_ + 2 * K_ + 4 + 2 + 2),   # = 1,032 B
}
# DRAM bytes per (token, head) that ncu measured (dram__bytes_read.sum + dram__bytes_write.sum of one launch) on a
# small case of each kernel (B=1 T=8192, 262,144 (token, head) units; summaries under profiles/).  Traffic grows in
# proportion to the units, so a launch's traffic is this figure times its units.
KERNEL_TRAFFIC = {"prepare": 2533.0, "scan": 2043.0, "bwd_scan": 1814.0, "bwd_main": 4577.0, "decode": 125600.0}


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

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

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
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "train_bf16 (B=8 T=8192 H=32 K=V=128 fwd+bwd)",
                   "sample": f"B=1 T={T} H=32 K=V=128 per step"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"token-recurrent float32 PyTorch forward+backward, B=1 T={T} H=32 K=V=128 per step"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_fla_triton(args, w, devt, cu, grad_names, tokens):
    """The on-box GPU comparison: flash-linear-attention's own chunk_kda (Triton) on the same inputs, same step
    definition (forward, or forward + backward with the same output gradients), CUDA events, same warm-up rule.
    A comparison line only: nothing of it is on the product path."""
    if args.gate:
        return {"unavailable": "timed without the gate front end"}
    try:
        from fla.ops.kda import chunk_kda as fla_chunk_kda
        from fla.ops.kda import fused_recurrent_kda as fla_recurrent_kda
    except Exception as e:          # noqa: BLE001
        return {"unavailable": f"fla does not import on this box: {type(e).__name__}: {e}"[:200]}
    x = devt
    name = "fused_recurrent_kda" if args.workload == "decode" else "chunk_kda"

    def step():
        if args.workload == "decode":
            # fla's public entry point returns the new state in a second buffer (same bytes moved as in place)
            with torch.no_grad():
                return fla_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=128 ** -0.5,
                                         initial_state=x["h0"], output_final_state=True)
        if w.backward:
            leaves = [x[n].detach().requires_grad_(True) for n in grad_names]
            t = dict(zip(grad_names, leaves))
            o, ht = fla_chunk_kda(t["q"], t["k"], t["v"], t["g"], t["beta"], initial_state=t.get("h0"),
                                  output_final_state=True, cu_seqlens=cu)
            return torch.autograd.grad([o, ht], leaves, [x["do"], x["dht"]])
        with torch.no_grad():
            return fla_chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"),
                                 output_final_state=True, cu_seqlens=cu)
    try:
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(1, min(args.steps, 10))
        e0.record()
        for _ in range(n):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
    except Exception as e:          # noqa: BLE001
        return {"unavailable": f"fla.ops.kda.{name} failed on this box: {type(e).__name__}: {e}"[:300]}
    import fla
    import triton
    return {"impl": f"fla.ops.kda.{name} (flash-linear-attention {getattr(fla, '__version__', '?')}, Triton {triton.__version__})",
            "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "steps": n}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_bf16", choices=sorted(WORKLOADS))
    ap.add_argument("--scale-down", type=int, default=1, help="divide the batch (smaller case for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gate", action="store_true",
                    help="call the operator as the layer does: raw bf16 gate input + A_log + dt_bias and beta logits "
                         "(use_gate_in_kernel, use_beta_sigmoid_in_kernel); training workloads and decode")
    ap.add_argument("--l2norm", action="store_true", help="use_qk_l2norm_in_kernel=True (chunked workloads)")
    ap.add_argument("--gpu-bar", action="store_true",
                    help="also time fla.ops.kda.chunk_kda (the Triton kernels of flash-linear-attention, if it imports on "
                         "this box) on the same device-resident inputs: the on-box GPU comparison; 1 GPU only")
    args = ap.parse_args()

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

    from kda_b200 import _lib, chunk_kda, fused_recurrent_kda_fwd
    w = WORKLOADS[args.workload]
    peaks = load_peaks()
    host = make_workload(args.workload, seed=rank, scale_down=args.scale_down)
    cu_host = host.pop("cu_seqlens")
    if args.gate:
        if not w.backward and args.workload != "decode":
            raise SystemExit("--gate needs a forward+backward workload or the decode workload")
        gen = torch.Generator().manual_seed(1000 + rank)
        host["g"] = torch.randn(host["g"].shape, generator=gen).bfloat16()                      # raw gate input
        host["beta"] = torch.randn(host["beta"].shape, generator=gen).bfloat16()                # beta logits
        host["A_log"] = torch.log(torch.empty(w.H).uniform_(1, 16, generator=gen))
        host["dt_bias"] = torch.randn(w.H * w.K, generator=gen)
    names = [n for n, t in host.items() if t is not None]
    pinned = {n: host[n].pin_memory() for n in names}
    devt = {n: pinned[n].to(dev, non_blocking=True) for n in names}
    cu = cu_host.to(dev) if cu_host is not None else None
    B, T, H = devt["q"].shape[:3]
    tokens = B * T
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

    launches_per_step = 0
    if args.workload == "decode":
        state = devt["h0"].clone()
        scale = 128 ** -0.5

        dec_kw = dict(use_qk_l2norm_in_kernel=args.l2norm)
        if args.gate:       # the layer's decode call: raw gate input, beta logits; activated inside the one kernel
            dec_kw.update(use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True, A_log=devt["A_log"], dt_bias=devt["dt_bias"])

        def step(x=devt):
            return fused_recurrent_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=scale, initial_state=state,
                                           inplace_final_state=True, **dec_kw)
        launches_per_step = 1
        grad_names = []
    elif w.backward:
        grad_names = ["q", "k", "v", "g", "beta"] + (["h0"] if "h0" in devt else []) + (["A_log", "dt_bias"] if args.gate else [])
        gate_kw = dict(use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True) if args.gate else {}

        def step(x=devt):
            leaves = [x[n].requires_grad_(True) for n in grad_names]
            kw = dict(gate_kw, A_log=x["A_log"], dt_bias=x["dt_bias"]) if args.gate else {}
            o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"),
                              output_final_state=True, cu_seqlens=cu, use_qk_l2norm_in_kernel=args.l2norm, **kw)
            grads = torch.autograd.grad([o, ht], leaves, [x["do"], x["dht"]])
            return (o, ht) + tuple(grads)
        launches_per_step = 10 if args.gate else 5      # gate: + activation, beta sigmoid; + their backward and the reduction
    else:
        grad_names = []

        def step(x=devt):
            with torch.no_grad():
                return chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x.get("h0"),
                                 output_final_state=True, cu_seqlens=cu, use_qk_l2norm_in_kernel=args.l2norm)
        launches_per_step = 3

    # ---------------- kernel-resident timing ----------------
    sampler = ClockSampler(local_rank if os.environ.get("CUDA_VISIBLE_DEVICES") is None else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()          # started before the warm-up: nvidia-smi needs a moment to deliver samples
    for _ in range(args.warmup):
        step()
    barrier()
    _lib.profile_enable(True)
    _lib.profile_read(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = maxms(e0.elapsed_time(e1))
    stages = _lib.profile_read(reset=True)
    _lib.profile_enable(False)
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
    value = world * tokens / (ms_step / 1e3)

    # ---------------- end to end: pinned host buffers in, every output back out ----------------
    e2e = None
    if not args.no_e2e:
        out_host = None
        pipelined = w.backward and cu is None and args.workload != "decode" and not args.gate and not args.l2norm

        def e2e_step():
            nonlocal out_host
            if pipelined:
                # public host-resident API: batch slices pipelined over copy-in / compute / copy-out streams; consecutive
                # steps are queued without waiting (two alternating sets of pinned output buffers), so step i+1's
                # copy-in runs under step i's copy-out; the timed region ends after the last result has landed
                from kda_b200.host import chunk_kda_fwd_bwd_host
                out_sets[e2e_count[0] & 1] = out_host = chunk_kda_fwd_bwd_host(pinned, out_sets[e2e_count[0] & 1], wait=False)
                e2e_count[0] += 1
                return
            x = {n: pinned[n].to(dev, non_blocking=True) for n in names}
            outs = step(x)
            outs = [t for t in outs if t is not None]
            if out_host is None:
                out_host = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
            for hbuf, t in zip(out_host, outs):
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
        e2e = {"value": world * tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "api": "kda_b200.host.chunk_kda_fwd_bwd_host(wait=False) + host_synchronize (batch slices pipelined over 3 streams, "
                      "consecutive steps overlapped, results of all steps in host memory before the clock stops)" if pipelined else "kda_b200.chunk_kda"}

    gpu_bar = None
    if args.gpu_bar:
        gpu_bar = time_fla_triton(args, w, devt, cu, grad_names, tokens) if world == 1 else {"unavailable": "timed on 1 GPU only"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- roofline of the dominant kernel ----------------
    th = tokens * H
    if args.workload == "decode":
        byt = B * H * decode_bytes_per_seq_head()
        ach = byt / (ms_step * 1e-3) / 1e9
        roof = {"kernel": "kda_decode_bulk_kernel", "bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": ach / peaks["hbm"], "traffic": KERNEL_TRAFFIC["decode"] * B * H,
                "traffic_source": "ncu capture of a smaller case, scaled by units", "peak_source": peaks["src"]}
        kernels = {}
    else:
        kernels = {s: {"ms_per_launch": (ms / n), "launches": n} for s, (ms, n) in stages.items() if n > 0}
        for s_, kv in kernels.items():          # every kernel against the HBM roof at its algorithmic bytes ("of measured")
            if s_ in KERNEL_WORK:
                kv["hbm_frac"] = KERNEL_WORK[s_][1] * th / (kv["ms_per_launch"] * 1e-3) / 1e9 / peaks["hbm"]
        dom = max((s for s in kernels if s in KERNEL_WORK), key=lambda s: kernels[s]["ms_per_launch"] * kernels[s]["launches"])
        fl, by = KERNEL_WORK[dom]
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
        roof.update({"traffic": KERNEL_TRAFFIC[dom] * th if dom in KERNEL_TRAFFIC else None, "traffic_source": "ncu capture of a smaller case, scaled by units",
                     "peak_source": peaks["src"], "ms_per_launch": kernels[dom]["ms_per_launch"],
                     "algorithmic_flops_per_launch": fl * th, "algorithmic_bytes_per_launch": by * th})
    # whole-step roofline fractions (both bounds), for context
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

    line = {
        "metric": METRIC if (args.workload == "train_bf16" and not args.gate and not args.l2norm) else
                  f"KDA {args.workload}{' +gate' if args.gate else ''}{' +l2norm' if args.l2norm else ''} tokens/s",
        "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} (B={B} T={T} H={H} K=V=128, chunk 64"
                               f"{', fwd+bwd' if w.backward else ''}{', packed varlen' if cu is not None else ''}"
                               f"{', gate + beta sigmoid in kernel' if args.gate else ''}{', q/k l2norm in kernel' if args.l2norm else ''})",
                   "per_gpu_batch": B, "l2": "inputs (>= 3 GB per step) far exceed the 126 MB L2; no flush needed",
                   "seed": "rank"},
        "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "roofline": roof, "step_roofline": whole, "kernels": kernels, "cpu_baseline": cpu,
    }
    if gpu_bar is not None:
        line["gpu_bar"] = gpu_bar
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
