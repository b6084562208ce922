// Token-recurrent KDA backward in fp32: the exact counterpart of kda_recurrent_kernel for training with float32
// tensors (any K, V in {32, 64, 128}).  Reverse-mode through the recurrence of fla/ops/kda/naive.py:12-66,
//
//   S' = Diag(exp g_t) S_{t-1};   r = v_t - S'^T k_t;   w = beta_t r;   S_t = S' + k_t w^T;   o_t = scale S_t^T q_t,
//
// needs S' of every token in reverse order.  One CTA owns one (sequence, head) and walks it three times:
//   pass 1  forward over the whole sequence, leaving the state at the start of every 64-token chunk in the workspace;
//   pass 2  per chunk, last chunk first: forward again from the chunk's start state, leaving S', r, w of each of its
//           tokens in a per-CTA scratch area (the same thread writes and later reads a value: L2-resident), then
//           backward over the chunk's tokens with dL/dS in registers:
//             dS += scale q do^T;  dq^ = scale S_t do;  dw = dS^T k;  dk^ = dS w - S' (beta dw);  dbeta = <dw, r>;
//             dv = beta dw;  dS' = dS - k (beta dw)^T;  dg = rowsum(dS' . S');  dS <- Diag(exp g) dS'.
// A warp holds eight value columns of S and dS (lane = 16 row groups x 2 column quads, rows rg + 16 i); reductions over
// K are register sums and four shuffles, reductions over V (dq^, dk^, dg, dbeta) go through per-warp partial rows in
// shared memory that 3K + 1 threads add up in a fixed order: results do not depend on scheduling.
// dq^, dk^ (gradients w.r.t. the possibly L2-normalised rows, per VALUE head) go to the workspace; a second kernel
// sums grouped value heads, applies the normalisation's backward (fla/modules/l2norm.py:190-240) and writes dq, dk.
#include <algorithm>

#include "kda_common.cuh"
#include "kda_device.cuh"

namespace kda {

namespace {

constexpr int RB_CHUNK = 64;      // tokens between two kept states

struct RecBwdParams {
  const float *q, *k, *v, *g, *beta, *h0, *d_o, *d_ht;
  const int32_t* cu;
  float *dqh, *dkh;      // [tokens, H, K] per value head, w.r.t. the normalised rows
  float *dv, *dg, *dbeta, *dh0;
  float *ckpt;           // [tokens / 64 + N + 1][H][K][V] chunk-start states
  float *stash;          // [grid][64][K][V] S' of the chunk in flight
  float *rw;             // [grid][64][2][V]  r and w of the chunk in flight
  long long T;
  int N, H, HQ;
  int use_l2;
  float scale;
};

__device__ __forceinline__ float dot4(const float4 a, const float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float4 fma4(const float s, const float4 a, const float4 c) {
  return make_float4(fmaf(s, a.x, c.x), fmaf(s, a.y, c.y), fmaf(s, a.z, c.z), fmaf(s, a.w, c.w));
}
__device__ __forceinline__ float4 mul4(const float s, const float4 a) { return make_float4(s * a.x, s * a.y, s * a.z, s * a.w); }
// sum over the 16 row groups of a warp (lane bits 1..4); every lane ends with the total
__device__ __forceinline__ float4 sum_rows(float4 x) {
#pragma unroll
  for (int off = 2; off < 32; off <<= 1) {
    x.x += __shfl_xor_sync(0xffffffffu, x.x, off);
    x.y += __shfl_xor_sync(0xffffffffu, x.y, off);
    x.z += __shfl_xor_sync(0xffffffffu, x.z, off);
    x.w += __shfl_xor_sync(0xffffffffu, x.w, off);
  }
  return x;
}

template <int K, int V>
struct RecBwdSmem {
  static constexpr int NW = V / 8;
  float q[RB_CHUNK][K];          // scale * q^ of the chunk's tokens
  float k[RB_CHUNK][K];          // k^
  float a[RB_CHUNK][K];          // exp g
  float beta[RB_CHUNK];
  float part[2][NW][3][K];       // per-warp partial sums over its eight value columns: dq^, dk^, dg (two tokens in flight)
  float partb[2][NW];            // dbeta
};

template <int K, int V>
__global__ void __launch_bounds__(V * 4, 1) kda_recurrent_bwd_kernel(const RecBwdParams p) {
  constexpr int NW = V / 8, NT = NW * 32, R = K / 16, E = K / 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  RecBwdSmem<K, V>& s = *reinterpret_cast<RecBwdSmem<K, V>*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cg = lane & 1, rg = lane >> 1;
  const int col = warp * 8 + cg * 4;
  const int grp = p.H / p.HQ;
  float* const stash = p.stash + static_cast<size_t>(blockIdx.x) * RB_CHUNK * K * V;
  float* const rw = p.rw + static_cast<size_t>(blockIdx.x) * RB_CHUNK * 2 * V;

  for (long long item = blockIdx.x; item < static_cast<long long>(p.N) * p.H; item += gridDim.x) {
    const int n = static_cast<int>(item / p.H), h = static_cast<int>(item % p.H);
    const long long bos = p.cu ? p.cu[n] : n * p.T, eos = p.cu ? p.cu[n + 1] : bos + p.T;
    const long long len = eos - bos;
    const int nchunks = static_cast<int>((len + RB_CHUNK - 1) / RB_CHUNK);
    float* const ckpt = p.ckpt + ((bos / RB_CHUNK + n) * p.H + h) * static_cast<size_t>(K) * V;
    const size_t sbase = (static_cast<size_t>(n) * p.H + h) * K * V + col;

    // q^, k^, exp g, beta of chunk c into shared memory: one warp per token
    auto setup = [&](int c) {
      const int lenc = static_cast<int>(min(static_cast<long long>(RB_CHUNK), len - static_cast<long long>(c) * RB_CHUNK));
      for (int j = warp; j < lenc; j += NW) {
        const size_t tok = static_cast<size_t>(bos + static_cast<long long>(c) * RB_CHUNK + j);
        const size_t rowq = (tok * p.HQ + h / grp) * K + lane * E, rowg = (tok * p.H + h) * K + lane * E;
        float qf[E], kf[E];
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
          qf[e] = __ldg(p.q + rowq + e);
          kf[e] = __ldg(p.k + rowq + e);
          sq += qf[e] * qf[e];
          sk += kf[e] * kf[e];
        }
        float qs = p.scale, ks = 1.f;
        if (p.use_l2) {
          qs *= rsqrtf(warp_sum(sq) + L2NORM_EPS);
          ks = rsqrtf(warp_sum(sk) + L2NORM_EPS);
        }
#pragma unroll
        for (int e = 0; e < E; ++e) {
          s.q[j][lane * E + e] = qf[e] * qs;
          s.k[j][lane * E + e] = kf[e] * ks;
          s.a[j][lane * E + e] = expf(__ldg(p.g + rowg + e));
        }
        if (lane == 0) s.beta[j] = __ldg(p.beta + tok * p.H + h);
      }
      return lenc;
    };
    // one forward step on token j of the chunk in shared memory; STASH: leave S', r, w for the backward step
    auto forward_step = [&](float4 (&S)[R], int j, long long tok, bool keep) {
      const float4 vt = __ldg(reinterpret_cast<const float4*>(p.v + (static_cast<size_t>(tok) * p.H + h) * V + col));
      float4 hk = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int r = rg + 16 * i;
        S[i] = mul4(s.a[j][r], S[i]);
        hk = fma4(s.k[j][r], S[i], hk);
        if (keep) *reinterpret_cast<float4*>(stash + (static_cast<size_t>(j) * K + r) * V + col) = S[i];
      }
      hk = sum_rows(hk);
      const float b = s.beta[j];
      const float4 r4 = make_float4(vt.x - hk.x, vt.y - hk.y, vt.z - hk.z, vt.w - hk.w);
      const float4 w4 = mul4(b, r4);
      if (keep && rg == 0) {
        *reinterpret_cast<float4*>(rw + (static_cast<size_t>(j) * 2 + 0) * V + col) = r4;
        *reinterpret_cast<float4*>(rw + (static_cast<size_t>(j) * 2 + 1) * V + col) = w4;
      }
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] = fma4(s.k[j][rg + 16 * i], w4, S[i]);
    };

    // ---------------- pass 1: chunk-start states ----------------
    float4 S[R];
#pragma unroll
    for (int i = 0; i < R; ++i)
      S[i] = p.h0 ? __ldg(reinterpret_cast<const float4*>(p.h0 + sbase + static_cast<size_t>(rg + 16 * i) * V)) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 0; c < nchunks; ++c) {
#pragma unroll
      for (int i = 0; i < R; ++i)
        *reinterpret_cast<float4*>(ckpt + (static_cast<size_t>(c) * p.H * K + rg + 16 * i) * V + col) = S[i];
      if (c == nchunks - 1) break;      // the state after the last chunk is not needed
      __syncthreads();                  // the previous chunk's rows in shared memory are no longer read
      setup(c);
      __syncthreads();
      for (int j = 0; j < RB_CHUNK; ++j) forward_step(S, j, bos + static_cast<long long>(c) * RB_CHUNK + j, false);
    }

    // ---------------- pass 2: chunks in reverse ----------------
    float4 dS[R];
#pragma unroll
    for (int i = 0; i < R; ++i)
      dS[i] = p.d_ht ? __ldg(reinterpret_cast<const float4*>(p.d_ht + sbase + static_cast<size_t>(rg + 16 * i) * V)) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = nchunks - 1; c >= 0; --c) {
      __syncthreads();
      const int lenc = setup(c);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < R; ++i)      // written by this very thread in pass 1
        S[i] = *reinterpret_cast<const float4*>(ckpt + (static_cast<size_t>(c) * p.H * K + rg + 16 * i) * V + col);
      const long long tok0 = bos + static_cast<long long>(c) * RB_CHUNK;
      for (int j = 0; j < lenc; ++j) forward_step(S, j, tok0 + j, true);
      __syncwarp();      // r, w were written by the lanes of row group 0 and are read by the whole warp
      for (int j = lenc - 1; j >= 0; --j) {
        const size_t tok = static_cast<size_t>(tok0 + j);
        const int buf = j & 1;
        const float4 do4 = __ldg(reinterpret_cast<const float4*>(p.d_o + (tok * p.H + h) * V + col));
        const float4 r4 = *reinterpret_cast<const float4*>(rw + (static_cast<size_t>(j) * 2 + 0) * V + col);
        const float4 w4 = *reinterpret_cast<const float4*>(rw + (static_cast<size_t>(j) * 2 + 1) * V + col);
        const float b = s.beta[j];
        float4 Sp[R];
        float pq[R], pk[R], pg[R];
        float4 dw = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int r = rg + 16 * i;
          const float kk = s.k[j][r];
          Sp[i] = *reinterpret_cast<const float4*>(stash + (static_cast<size_t>(j) * K + r) * V + col);
          dS[i] = fma4(s.q[j][r], do4, dS[i]);                       // o_t = scale S_t^T q_t
          pq[i] = dot4(fma4(kk, w4, Sp[i]), do4);                    // S_t do  (the scale is applied by the second kernel)
          dw = fma4(kk, dS[i], dw);
          pk[i] = dot4(dS[i], w4);
        }
        dw = sum_rows(dw);
        const float4 dr = mul4(b, dw);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const int r = rg + 16 * i;
          const float4 dSp = fma4(-s.k[j][r], dr, dS[i]);
          pk[i] -= dot4(Sp[i], dr);
          pg[i] = dot4(dSp, Sp[i]);
          dS[i] = mul4(s.a[j][r], dSp);
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {      // the warp's two column quads
          pq[i] += __shfl_xor_sync(0xffffffffu, pq[i], 1);
          pk[i] += __shfl_xor_sync(0xffffffffu, pk[i], 1);
          pg[i] += __shfl_xor_sync(0xffffffffu, pg[i], 1);
        }
        if (cg == 0) {
#pragma unroll
          for (int i = 0; i < R; ++i) {
            s.part[buf][warp][0][rg + 16 * i] = pq[i];
            s.part[buf][warp][1][rg + 16 * i] = pk[i];
            s.part[buf][warp][2][rg + 16 * i] = pg[i];
          }
        }
        float pb = dot4(dw, r4);
        pb += __shfl_xor_sync(0xffffffffu, pb, 1);
        if (lane == 0) s.partb[buf][warp] = pb;
        if (rg == 0) *reinterpret_cast<float4*>(p.dv + (tok * p.H + h) * V + col) = dr;
        __syncthreads();
        for (int idx = tid; idx < 3 * K + 1; idx += NT) {
          if (idx == 3 * K) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) acc += s.partb[buf][w];
            p.dbeta[tok * p.H + h] = acc;
          } else {
            const int which = idx / K, kk = idx % K;
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) acc += s.part[buf][w][which][kk];
            float* const out = which == 0 ? p.dqh : (which == 1 ? p.dkh : p.dg);
            out[(tok * p.H + h) * K + kk] = acc;
          }
        }
      }
    }
    if (p.dh0) {
#pragma unroll
      for (int i = 0; i < R; ++i) *reinterpret_cast<float4*>(p.dh0 + sbase + static_cast<size_t>(rg + 16 * i) * V) = dS[i];
    }
    __syncthreads();      // shared memory and the scratch areas go to the next (sequence, head)
  }
}

// dq, dk from the per-value-head gradients w.r.t. the rows the recurrence saw: sum over the value heads of a group,
// scale (q only), then the backward of x^ = x rsqrt(sum x^2 + eps) when the rows were normalised.  One warp per row.
template <int K>
__global__ void __launch_bounds__(256) kda_recurrent_bwd_finish_kernel(const RecBwdParams p, float* __restrict__ dq, float* __restrict__ dk,
                                                                       long long rows) {
  constexpr int E = K / 32;
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);      // token * HQ + q head
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int grp = p.H / p.HQ;
  const long long tok = row / p.HQ;
  const int hq = static_cast<int>(row % p.HQ);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const float* x = (which ? p.k : p.q) + row * K + lane * E;
    const float* src = (which ? p.dkh : p.dqh) + (tok * p.H + static_cast<long long>(hq) * grp) * K + lane * E;
    float d[E], xf[E];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      float acc = 0.f;
      for (int j = 0; j < grp; ++j) acc += src[static_cast<size_t>(j) * K + e];
      d[e] = which ? acc : acc * p.scale;
      xf[e] = __ldg(x + e);
      ss += xf[e] * xf[e];
    }
    if (p.use_l2) {
      const float rs = rsqrtf(warp_sum(ss) + L2NORM_EPS);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) dot += xf[e] * rs * d[e];
      dot = warp_sum(dot);
#pragma unroll
      for (int e = 0; e < E; ++e) d[e] = rs * (d[e] - xf[e] * rs * dot);
    }
    float* out = (which ? dk : dq) + row * K + lane * E;
#pragma unroll
    for (int e = 0; e < E; ++e) out[e] = d[e];
  }
}

int rec_bwd_grid(int N, int H) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long items = static_cast<long long>(N) * H;
  return static_cast<int>(std::max(1LL, std::min<long long>(items, sms)));
}

struct RecBwdLayout {
  size_t dqh, dkh, ckpt, stash, rw, total;
};
RecBwdLayout rec_bwd_layout(long long tokens, int N, int H, int K, int V) {
  auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
  RecBwdLayout l{};
  size_t off = 0;
  const size_t grid = 148 * 2;      // an upper bound of rec_bwd_grid on any device this library runs on
  l.dqh = off; off = up(off + static_cast<size_t>(tokens) * H * K * 4);
  l.dkh = off; off = up(off + static_cast<size_t>(tokens) * H * K * 4);
  l.ckpt = off; off = up(off + (static_cast<size_t>(tokens) / RB_CHUNK + N + 1) * H * K * V * 4);
  l.stash = off; off = up(off + grid * RB_CHUNK * K * V * 4);
  l.rw = off; off = up(off + grid * RB_CHUNK * 2 * V * 4);
  l.total = off;
  return l;
}

template <int K, int V>
int launch_rec_bwd(const RecBwdParams& p, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(RecBwdSmem<K, V>));
  const int rc = once.run([&] { return cudaFuncSetAttribute(kda_recurrent_bwd_kernel<K, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != KDA_OK) return rc;
  const int grid = std::min(rec_bwd_grid(p.N, p.H), 148 * 2);
  kda_recurrent_bwd_kernel<K, V><<<grid, V * 4, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <int K>
int launch_rec_bwd_v(const RecBwdParams& p, int V, cudaStream_t st) {
  switch (V) {
    case 32: return launch_rec_bwd<K, 32>(p, st);
    case 64: return launch_rec_bwd<K, 64>(p, st);
    case 128: return launch_rec_bwd<K, 128>(p, st);
    default: return KDA_E_SHAPE;
  }
}

}  // namespace

}  // namespace kda

using namespace kda;

extern "C" size_t kda_recurrent_bwd_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V) {
  if (tokens < 0 || N < 0 || H <= 0 || K <= 0 || V <= 0) return 0;
  return rec_bwd_layout(tokens, N, H, K, V).total;
}

extern "C" int kda_recurrent_bwd(const kda_recurrent_bwd_args* a, void* stream) {
  if (!a) return KDA_E_NULL;
  if (!a->q || !a->k || !a->v || !a->g || !a->beta || !a->d_o || !a->dq || !a->dk || !a->dv || !a->dg || !a->dbeta || !a->workspace)
    return KDA_E_NULL;
  if (a->io_dtype != KDA_FP32) return KDA_E_DTYPE;
  if (a->N < 0 || a->H <= 0 || a->tokens < 0 || (!a->cu_seqlens && a->T < 0)) return KDA_E_SHAPE;
  if ((a->K != 32 && a->K != 64 && a->K != 128) || (a->V != 32 && a->V != 64 && a->V != 128)) return KDA_E_SHAPE;
  const int HQ = a->HQ > 0 ? a->HQ : a->H;
  if (a->H % HQ) return KDA_E_SHAPE;
  const RecBwdLayout l = rec_bwd_layout(a->tokens, a->N, a->H, a->K, a->V);
  if (a->workspace_bytes < l.total) return KDA_E_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(a->workspace) & 255) return KDA_E_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->N == 0) return KDA_OK;
  if (a->tokens == 0) {      // empty sequences: the initial state is the final state
    if (!a->dh0) return KDA_OK;
    const size_t bytes = static_cast<size_t>(a->N) * a->H * a->K * a->V * sizeof(float);
    return static_cast<int>(a->d_ht ? cudaMemcpyAsync(a->dh0, a->d_ht, bytes, cudaMemcpyDeviceToDevice, st) : cudaMemsetAsync(a->dh0, 0, bytes, st));
  }
  if (!a->cu_seqlens && static_cast<int64_t>(a->N) * a->T != a->tokens) return KDA_E_SHAPE;
  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  RecBwdParams p{};
  p.q = static_cast<const float*>(a->q); p.k = static_cast<const float*>(a->k); p.v = static_cast<const float*>(a->v);
  p.g = a->g; p.beta = a->beta; p.h0 = a->h0; p.d_o = static_cast<const float*>(a->d_o); p.d_ht = a->d_ht;
  p.cu = a->cu_seqlens;
  p.dqh = reinterpret_cast<float*>(ws + l.dqh); p.dkh = reinterpret_cast<float*>(ws + l.dkh);
  p.dv = static_cast<float*>(a->dv); p.dg = a->dg; p.dbeta = a->dbeta; p.dh0 = a->dh0;
  p.ckpt = reinterpret_cast<float*>(ws + l.ckpt); p.stash = reinterpret_cast<float*>(ws + l.stash); p.rw = reinterpret_cast<float*>(ws + l.rw);
  p.T = a->T; p.N = a->N; p.H = a->H; p.HQ = HQ; p.use_l2 = a->use_qk_l2norm; p.scale = a->scale;
  int rc;
  switch (a->K) {
    case 32: rc = launch_rec_bwd_v<32>(p, a->V, st); break;
    case 64: rc = launch_rec_bwd_v<64>(p, a->V, st); break;
    default: rc = launch_rec_bwd_v<128>(p, a->V, st); break;
  }
  if (rc != KDA_OK) return rc;
  const long long rows = a->tokens * HQ;
  const int blocks = static_cast<int>((rows + 7) / 8);
  switch (a->K) {
    case 32: kda_recurrent_bwd_finish_kernel<32><<<blocks, 256, 0, st>>>(p, static_cast<float*>(a->dq), static_cast<float*>(a->dk), rows); break;
    case 64: kda_recurrent_bwd_finish_kernel<64><<<blocks, 256, 0, st>>>(p, static_cast<float*>(a->dq), static_cast<float*>(a->dk), rows); break;
    default: kda_recurrent_bwd_finish_kernel<128><<<blocks, 256, 0, st>>>(p, static_cast<float*>(a->dq), static_cast<float*>(a->dk), rows); break;
  }
  return static_cast<int>(cudaGetLastError());
}
