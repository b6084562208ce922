// Token-recurrent KDA forward: decode (one token per sequence, HBM-bound) and exact fp32 scans.
//
// One warp owns one (sequence, head, V-slice) and keeps its [K x VS] slice of the fp32 state in
// registers for the whole call.  Lanes are arranged as RG row groups x CL column lanes; a lane holds
// rows rg, rg+RG, ... and four consecutive V columns, so every state load/store is a 128-bit access
// and a warp-wide access covers RG rows x (VS*4) contiguous bytes.  Both reductions over K (S^T k for the
// delta rule, S^T q for the read-out) are register sums followed by log2(RG) shuffles: no shared-memory
// reduction, no block barrier, warps are independent.
// Per token (order as in fla/ops/kda/fused_recurrent.py:146-192): S *= exp(g); v' = beta (v - S^T k);
// S += k v'^T; o = scale S^T q.
#include "kda_common.cuh"

namespace kda {

template <typename IO> struct IoTraits;
template <> struct IoTraits<float> {
  static __device__ __forceinline__ float ld(const float* p) { return __ldg(p); }
  static __device__ __forceinline__ void st4(float* p, float4 x) { *reinterpret_cast<float4*>(p) = x; }
  static __device__ __forceinline__ float4 ld4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
};
template <> struct IoTraits<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st4(__nv_bfloat16* p, float4 x) {
    uint2 u = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
    *reinterpret_cast<uint2*>(p) = u;
  }
  static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    return make_float4(a.x, a.y, b.x, b.y);
  }
};

constexpr int REC_WARPS = 4;

// Sum over the 32 lanes of 32 per-lane values at once: lane L returns the total of v[L] (31 shuffles).
__device__ __forceinline__ float butterfly_sum32(float (&v)[32], int lane) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {
      const float mine = up ? v[i + o] : v[i];
      const float other = up ? v[i] : v[i + o];
      v[i] = mine + __shfl_xor_sync(0xffffffffu, other, o);
    }
  }
  return v[0];
}

template <typename IO, int K, int VS>
__global__ void __launch_bounds__(REC_WARPS * 32) kda_recurrent_kernel(const kda_recurrent_args a) {
  constexpr int CL = VS / 4;      // lanes across the V slice (4 columns each)
  constexpr int RG = 32 / CL;     // row groups
  constexpr int R = K / RG;       // state rows per lane
  constexpr int E = K / 32;       // q/k/g elements staged per lane
  static_assert(K % RG == 0 && K % 32 == 0, "unsupported K");

  __shared__ float s_k[REC_WARPS][K], s_q[REC_WARPS][K], s_eg[REC_WARPS][K];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvs = a.V / VS;
  const long long wid = static_cast<long long>(blockIdx.x) * REC_WARPS + warp;
  const long long total = static_cast<long long>(a.N) * a.H * nvs;
  if (wid >= total) return;   // whole warps leave; only __syncwarp is used below
  const int vs = static_cast<int>(wid % nvs);
  const int h = static_cast<int>((wid / nvs) % a.H);
  const int n = static_cast<int>(wid / (static_cast<long long>(nvs) * a.H));
  const int HQ = a.HQ > 0 ? a.HQ : a.H, grp = a.H / HQ;      // grouped value heads
  const int cg = lane % CL, rg = lane / CL;
  const int col = vs * VS + cg * 4;

  long long bos, eos;
  if (a.cu_seqlens) {
    bos = a.cu_seqlens[n];
    eos = a.cu_seqlens[n + 1];
  } else {
    bos = static_cast<long long>(n) * a.T;
    eos = bos + a.T;
  }
  // continuous batching: the sequence's row of slot numbers; it starts from the slot of the last accepted token
  const int32_t* slots = a.state_indices ? a.state_indices + static_cast<size_t>(n) * a.state_indices_stride : nullptr;
  const long long slot = slots ? slots[a.num_accepted_tokens ? a.num_accepted_tokens[n] - 1 : 0] : n;
  const size_t sbase = (static_cast<size_t>(slot) * a.H + h) * K * a.V + col;

  float4 S[R];
  if (a.h0) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      S[i] = __ldcs(reinterpret_cast<const float4*>(a.h0 + sbase + static_cast<size_t>(rg + RG * i) * a.V));
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  const IO* qp = static_cast<const IO*>(a.q);
  const IO* kp = static_cast<const IO*>(a.k);
  const IO* vp = static_cast<const IO*>(a.v);
  IO* op = static_cast<IO*>(a.o);

  for (long long t = bos; t < eos; ++t) {
    const size_t rowq = (static_cast<size_t>(t) * HQ + h / grp) * K + lane * E;   // q, k row (their own head count)
    float qf[E], kf[E], gf[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      qf[e] = IoTraits<IO>::ld(qp + rowq + e);
      kf[e] = IoTraits<IO>::ld(kp + rowq + e);
      gf[e] = recurrent_log_decay(a, static_cast<size_t>(t) * a.H + h, h, lane * E + e, K);
    }
    float qs = a.scale;
    if (a.use_qk_l2norm) {
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        sq += qf[e] * qf[e];
        sk += kf[e] * kf[e];
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      qs *= rsqrtf(sq + L2NORM_EPS);
      const float ks = rsqrtf(sk + L2NORM_EPS);
#pragma unroll
      for (int e = 0; e < E; ++e) kf[e] *= ks;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      s_k[warp][lane * E + e] = kf[e];
      s_q[warp][lane * E + e] = qf[e] * qs;
      s_eg[warp][lane * E + e] = expf(gf[e]);
    }
    const float beta = recurrent_beta(a, static_cast<size_t>(t) * a.H + h);
    const float4 vt = IoTraits<IO>::ld4(vp + (static_cast<size_t>(t) * a.H + h) * a.V + col);
    __syncwarp();

    float4 hk = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = rg + RG * i;
      const float eg = s_eg[warp][r], kk = s_k[warp][r];
      S[i].x *= eg; S[i].y *= eg; S[i].z *= eg; S[i].w *= eg;
      hk.x += kk * S[i].x; hk.y += kk * S[i].y; hk.z += kk * S[i].z; hk.w += kk * S[i].w;
    }
#pragma unroll
    for (int off = CL; off < 32; off <<= 1) {
      hk.x += __shfl_xor_sync(0xffffffffu, hk.x, off);
      hk.y += __shfl_xor_sync(0xffffffffu, hk.y, off);
      hk.z += __shfl_xor_sync(0xffffffffu, hk.z, off);
      hk.w += __shfl_xor_sync(0xffffffffu, hk.w, off);
    }
    const float4 dv = make_float4(beta * (vt.x - hk.x), beta * (vt.y - hk.y), beta * (vt.z - hk.z), beta * (vt.w - hk.w));
    float4 oa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int r = rg + RG * i;
      const float kk = s_k[warp][r], qq = s_q[warp][r];
      S[i].x += kk * dv.x; S[i].y += kk * dv.y; S[i].z += kk * dv.z; S[i].w += kk * dv.w;
      oa.x += qq * S[i].x; oa.y += qq * S[i].y; oa.z += qq * S[i].z; oa.w += qq * S[i].w;
    }
#pragma unroll
    for (int off = CL; off < 32; off <<= 1) {
      oa.x += __shfl_xor_sync(0xffffffffu, oa.x, off);
      oa.y += __shfl_xor_sync(0xffffffffu, oa.y, off);
      oa.z += __shfl_xor_sync(0xffffffffu, oa.z, off);
      oa.w += __shfl_xor_sync(0xffffffffu, oa.w, off);
    }
    if (rg == 0) IoTraits<IO>::st4(op + (static_cast<size_t>(t) * a.H + h) * a.V + col, oa);
    if (slots && a.ht) {      // the state after every token goes to that token's slot
      const size_t tb = (static_cast<size_t>(slots[t - bos]) * a.H + h) * K * a.V + col;
#pragma unroll
      for (int i = 0; i < R; ++i) __stcs(reinterpret_cast<float4*>(a.ht + tb + static_cast<size_t>(rg + RG * i) * a.V), S[i]);
    }
    __syncwarp();
  }

  if (a.ht && !slots) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      __stcs(reinterpret_cast<float4*>(a.ht + sbase + static_cast<size_t>(rg + RG * i) * a.V), S[i]);
  }
}

// E (2 or 4) consecutive floats of a state row, streaming loads / stores of 8 or 16 bytes
template <int E>
__device__ __forceinline__ void ld_row(float (&d)[E], const float* p) {
  if constexpr (E == 4) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(p));
    d[0] = x.x; d[1] = x.y; d[2] = x.z; d[3] = x.w;
  } else {
    const float2 x = __ldcs(reinterpret_cast<const float2*>(p));
    d[0] = x.x; d[1] = x.y;
  }
}
template <int E>
__device__ __forceinline__ void st_row(float* p, const float (&d)[E]) {
  if constexpr (E == 4) __stcs(reinterpret_cast<float4*>(p), make_float4(d[0], d[1], d[2], d[3]));
  else __stcs(reinterpret_cast<float2*>(p), make_float2(d[0], d[1]));
}

// ---- transposed state layout [slots, H, V, K] (K contiguous) ------------------------------------------------------
// One warp owns (sequence, head, 32 value rows); a lane holds the 32 x (K / 32) slice of key columns
// lane*(K/32) .. of those rows, so every state access is again contiguous over the warp.  The two reductions over K
// are per-lane partial dot products summed over the lanes 32 values at a time by a butterfly (lane L ends up with
// the total of value row L); the delta-rule update needs every row's dv in every lane: one shuffle per row.
template <typename IO, int K>
__global__ void __launch_bounds__(REC_WARPS * 32) kda_recurrent_t_kernel(const kda_recurrent_args a) {
  constexpr int E = K / 32;       // key columns per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvs = a.V / 32;
  const long long wid = static_cast<long long>(blockIdx.x) * REC_WARPS + warp;
  const long long total = static_cast<long long>(a.N) * a.H * nvs;
  if (wid >= total) return;
  const int vs = static_cast<int>(wid % nvs);
  const int h = static_cast<int>((wid / nvs) % a.H);
  const int n = static_cast<int>(wid / (static_cast<long long>(nvs) * a.H));
  const int HQ = a.HQ > 0 ? a.HQ : a.H, grp = a.H / HQ;      // grouped value heads
  long long bos, eos;
  if (a.cu_seqlens) {
    bos = a.cu_seqlens[n];
    eos = a.cu_seqlens[n + 1];
  } else {
    bos = static_cast<long long>(n) * a.T;
    eos = bos + a.T;
  }
  const int32_t* slots = a.state_indices ? a.state_indices + static_cast<size_t>(n) * a.state_indices_stride : nullptr;
  const long long slot = slots ? slots[a.num_accepted_tokens ? a.num_accepted_tokens[n] - 1 : 0] : n;
  auto state_ptr = [&](const float* base, long long sl) {
    return base + ((static_cast<size_t>(sl) * a.H + h) * a.V + vs * 32) * K + lane * E;
  };
  float S[32][E];
  if (a.h0) {
    const float* p0 = state_ptr(a.h0, slot);
#pragma unroll
    for (int r = 0; r < 32; ++r) ld_row<E>(S[r], p0 + static_cast<size_t>(r) * K);
  } else {
#pragma unroll
    for (int r = 0; r < 32; ++r)
#pragma unroll
      for (int e = 0; e < E; ++e) S[r][e] = 0.f;
  }
  const IO* qp = static_cast<const IO*>(a.q);
  const IO* kp = static_cast<const IO*>(a.k);
  const IO* vp = static_cast<const IO*>(a.v);
  IO* op = static_cast<IO*>(a.o);
  for (long long t = bos; t < eos; ++t) {
    const size_t rowq = (static_cast<size_t>(t) * HQ + h / grp) * K + lane * E;   // q, k row (their own head count)
    float qf[E], kf[E], eg[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
      qf[e] = IoTraits<IO>::ld(qp + rowq + e);
      kf[e] = IoTraits<IO>::ld(kp + rowq + e);
      eg[e] = expf(recurrent_log_decay(a, static_cast<size_t>(t) * a.H + h, h, lane * E + e, K));
    }
    float qs = a.scale;
    if (a.use_qk_l2norm) {
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        sq += qf[e] * qf[e];
        sk += kf[e] * kf[e];
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      qs *= rsqrtf(sq + L2NORM_EPS);
      const float ks = rsqrtf(sk + L2NORM_EPS);
#pragma unroll
      for (int e = 0; e < E; ++e) kf[e] *= ks;
    }
#pragma unroll
    for (int e = 0; e < E; ++e) qf[e] *= qs;
    const float beta = recurrent_beta(a, static_cast<size_t>(t) * a.H + h);
    const float vt = IoTraits<IO>::ld(vp + (static_cast<size_t>(t) * a.H + h) * a.V + vs * 32 + lane);      // value row `lane`
    float part[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        S[r][e] *= eg[e];
        acc = fmaf(kf[e], S[r][e], acc);
      }
      part[r] = acc;
    }
    const float hk = butterfly_sum32(part, lane);            // S^T k for value row `lane`
    const float dv = beta * (vt - hk);
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const float dvr = __shfl_sync(0xffffffffu, dv, r);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        S[r][e] = fmaf(kf[e], dvr, S[r][e]);
        acc = fmaf(qf[e], S[r][e], acc);
      }
      part[r] = acc;
    }
    const float o = butterfly_sum32(part, lane);
    if (sizeof(IO) == 2) reinterpret_cast<__nv_bfloat16*>(op)[(static_cast<size_t>(t) * a.H + h) * a.V + vs * 32 + lane] = __float2bfloat16_rn(o);
    else reinterpret_cast<float*>(op)[(static_cast<size_t>(t) * a.H + h) * a.V + vs * 32 + lane] = o;
    if (slots && a.ht) {
      float* pt = const_cast<float*>(state_ptr(a.ht, slots[t - bos]));
#pragma unroll
      for (int r = 0; r < 32; ++r) st_row<E>(pt + static_cast<size_t>(r) * K, S[r]);
    }
  }
  if (a.ht && !slots) {
    float* pt = const_cast<float*>(state_ptr(a.ht, slot));
#pragma unroll
    for (int r = 0; r < 32; ++r) st_row<E>(pt + static_cast<size_t>(r) * K, S[r]);
  }
}

template <typename IO, int K>
static int launch_rec_t(const kda_recurrent_args& a, cudaStream_t st) {
  const long long total = static_cast<long long>(a.N) * a.H * (a.V / 32);
  const long long blocks = (total + REC_WARPS - 1) / REC_WARPS;
  if (blocks <= 0) return KDA_OK;
  if (blocks > 0x7fffffffLL) return KDA_E_SHAPE;
  kda_recurrent_t_kernel<IO, K><<<static_cast<unsigned>(blocks), REC_WARPS * 32, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

template <typename IO, int K, int VS>
static int launch_rec(const kda_recurrent_args& a, cudaStream_t st) {
  const long long total = static_cast<long long>(a.N) * a.H * (a.V / VS);
  const long long blocks = (total + REC_WARPS - 1) / REC_WARPS;
  if (blocks <= 0) return KDA_OK;
  if (blocks > 0x7fffffffLL) return KDA_E_SHAPE;
  kda_recurrent_kernel<IO, K, VS><<<static_cast<unsigned>(blocks), REC_WARPS * 32, 0, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

template <typename IO>
static int dispatch_rec(const kda_recurrent_args& a, cudaStream_t st) {
  if (a.transpose_state) {
    switch (a.K) {
      case 64: return launch_rec_t<IO, 64>(a, st);
      case 128: return launch_rec_t<IO, 128>(a, st);
      default: return KDA_E_SHAPE;
    }
  }
  switch (a.K) {
    case 32: return launch_rec<IO, 32, 32>(a, st);
    case 64: return launch_rec<IO, 64, 32>(a, st);
    case 128: return launch_rec<IO, 128, 32>(a, st);
    case 256: return (a.V % 32 == 0) ? launch_rec<IO, 256, 16>(a, st) : KDA_E_SHAPE;
    default: return KDA_E_SHAPE;
  }
}

bool decode_bulk_covers(const kda_recurrent_args& a);                    // kda_decode_bulk.cu
int decode_bulk_launch(const kda_recurrent_args& a, cudaStream_t st);

}  // namespace kda

extern "C" int kda_recurrent_fwd(const kda_recurrent_args* args, void* stream) {
  if (!args) return KDA_E_NULL;
  kda_recurrent_args a = *args;
  if (a.state_indices) {
    if (a.state_indices_stride <= 0) a.state_indices_stride = 1;
    if (a.ht && a.ht != a.h0) return KDA_E_SHAPE;      // slot-addressed states are updated in place
  } else if (a.num_accepted_tokens) {
    return KDA_E_NULL;                                 // accepted-token counts only mean something with slots
  }
  if (a.N < 0 || a.H <= 0 || a.V <= 0 || a.V % 32 != 0 || a.tokens < 0) return KDA_E_SHAPE;
  if (a.HQ < 0 || (a.HQ > 0 && (a.HQ > a.H || a.H % a.HQ != 0))) return KDA_E_SHAPE;
  if (a.N == 0 || a.tokens == 0) {
    // nothing to scan; with distinct h0/ht buffers the final state is the initial one
    if (a.N > 0 && a.ht && a.ht != a.h0) {
      const size_t bytes = static_cast<size_t>(a.N) * a.H * a.K * a.V * sizeof(float);
      cudaError_t e = a.h0 ? cudaMemcpyAsync(a.ht, a.h0, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream))
                           : cudaMemsetAsync(a.ht, 0, bytes, static_cast<cudaStream_t>(stream));
      return static_cast<int>(e);
    }
    return KDA_OK;
  }
  if (!a.q || !a.k || !a.v || !a.g || !a.beta || !a.o) return KDA_E_NULL;
  if (!a.cu_seqlens && static_cast<int64_t>(a.N) * a.T != a.tokens) return KDA_E_SHAPE;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) |
                         reinterpret_cast<uintptr_t>(a.v) | reinterpret_cast<uintptr_t>(a.g) |
                         reinterpret_cast<uintptr_t>(a.o) | reinterpret_cast<uintptr_t>(a.h0) |
                         reinterpret_cast<uintptr_t>(a.ht);
  if (bits & 15u) return KDA_E_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kda::decode_bulk_covers(a)) return kda::decode_bulk_launch(a, st);
  if (a.io_dtype == KDA_BF16) return kda::dispatch_rec<__nv_bfloat16>(a, st);
  if (a.io_dtype == KDA_FP32) return kda::dispatch_rec<float>(a, st);
  return KDA_E_DTYPE;
}
