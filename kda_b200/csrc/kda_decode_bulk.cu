// Decode step of KDA (one token per sequence) for large batches: the [K x V] fp32 state of one (sequence, head)
// is 64 KiB of contiguous memory that has to be read and written once per step -- nothing else matters for speed.
// One persistent CTA per SM moves whole state tiles with the bulk-copy engine through a ring of three
// shared-memory stages: while the threads update tile i in place, the loads of tiles i+1 and i+2 and the store of
// tile i-1 are in flight, so the memory system always has work queued from every SM (the register-resident
// kernel in kda_recurrent.cu alternates between loading, computing and storing).
// Per token (order as in fla/ops/kda/fused_recurrent.py:146-192): S *= exp(g); v' = beta (v - S^T k);
// S += k v'^T; o = scale S^T q.
#include <mutex>

#include "kda_common.cuh"
#include "kda_device.cuh"

namespace kda {

namespace {

constexpr int DK = 128, DV = 128;
constexpr int DEC_STAGES = 3;
#ifndef KDA_DECODE_BULK_MIN_UNITS_PER_SM
#define KDA_DECODE_BULK_MIN_UNITS_PER_SM 4      // fewer (sequence, head) units per SM: the per-warp kernel is used
#endif
constexpr int DEC_THREADS = 256;                 // 8 warps: warp w owns the 16 state rows 16 w .., a lane 4 value columns
constexpr unsigned DEC_TILE = DK * DV * 4;       // bytes of one state tile

struct DecSmem {
  float S[DEC_STAGES][DK * DV];
  float red[8][DV];          // per-warp partial sums of S^T k
  float red2[8][DV];         // per-warp partial sums of S^T q
  float kv[2][DK], qv[2][DK], eg[2][DK], vv[2][DV];   // the token's vectors, double-buffered over units
  float nrm[2][8];           // partial sums of squares: q (warps 0..3), k (warps 0..3)
  float beta[2];
  uint64_t full[DEC_STAGES];
};
static_assert(sizeof(DecSmem) + 128 <= 227 * 1024, "DecSmem too large");

// Bit 0: a bounded wait on a state tile gave up (the step's results are incomplete).
__device__ unsigned g_decode_status = 0;

template <typename IO> __device__ __forceinline__ float ld1(const IO* p);
template <> __device__ __forceinline__ float ld1<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st4o(float* p, float4 x) { *reinterpret_cast<float4*>(p) = x; }
__device__ __forceinline__ void st4o(__nv_bfloat16* p, float4 x) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w));
}
__device__ __forceinline__ void st1o(float* p, float x) { *p = x; }
__device__ __forceinline__ void st1o(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// Sum over the 32 lanes of 16 per-lane values at once: afterwards lane L holds the total of v[L & 15] (31 shuffles).
__device__ __forceinline__ float butterfly_sum16(float (&v)[16], int lane) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], 16);
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) {
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

// TR: the states are [slots, H, V, K] (fla's transpose_state_layout): a warp owns 16 value rows of the tile and a lane
// four key columns, so both sums over K stay inside the warp (two butterflies) and no block-wide reduction is needed.
// GATE: g and / or beta are the raw layer outputs and are activated here (see kda_recurrent_args::A_log, beta_sigmoid).
template <typename IO, bool TR, bool GATE>
__global__ void __launch_bounds__(DEC_THREADS, 1) kda_decode_bulk_kernel(const kda_recurrent_args a) {
  extern __shared__ unsigned char smem_raw[];
  DecSmem& s = *reinterpret_cast<DecSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long total = static_cast<long long>(a.N) * a.H;
  const int HQ = a.HQ > 0 ? a.HQ : a.H, grp = a.H / HQ;
  const IO* qp = static_cast<const IO*>(a.q);
  const IO* kp = static_cast<const IO*>(a.k);
  const IO* vp = static_cast<const IO*>(a.v);
  IO* op = static_cast<IO*>(a.o);

  // unit u = (sequence n, value head h); one token per sequence: token index = n
  auto slot_of = [&](long long u) -> size_t {
    const long long n = u / a.H;
    const int h = static_cast<int>(u % a.H);
    const long long slot = a.state_indices ? a.state_indices[static_cast<size_t>(n) * a.state_indices_stride] : n;
    return (static_cast<size_t>(slot) * a.H + h) * (DK * DV);
  };
  // A thread fetches two elements of the unit's vectors: q, k (threads 0..127) or g, v (threads 128..255).  The loaded
  // bits stay untouched in registers until stash_vec: an instruction that depends on a load makes the thread wait for it
  // right there, and a small load takes longer than a unit's update when the memory system is saturated.
  struct Raw { uint32_t x0, x1, b, al, bias; };
  auto ld_bits = [&](const void* p, size_t i, bool bf16) -> uint32_t {
    if (bf16) return static_cast<const unsigned short*>(p)[i];
    return __float_as_uint(__ldg(static_cast<const float*>(p) + i));
  };
  auto to_float = [&](uint32_t bits, bool bf16) -> float { return __uint_as_float(bf16 ? bits << 16 : bits); };
  constexpr bool IO16 = sizeof(IO) == 2;
  auto load_vec = [&](long long u, Raw& r) {
    const long long n = u / a.H;
    const int h = static_cast<int>(u % a.H);
    const size_t rowv = static_cast<size_t>(n) * a.H + h;
    if (tid < DK) {
      const size_t row = (static_cast<size_t>(n) * HQ + h / grp) * DK + tid;
      r.x0 = ld_bits(qp, row, IO16);
      r.x1 = ld_bits(kp, row, IO16);
    } else {
      const int kk = tid - DK;
      if constexpr (GATE) {
        if (a.A_log) {
          r.x0 = ld_bits(a.g, rowv * DK + kk, a.g_raw_dtype == KDA_BF16);
          r.al = __float_as_uint(__ldg(a.A_log + h));
          r.bias = a.dt_bias ? __float_as_uint(__ldg(a.dt_bias + static_cast<size_t>(h) * DK + kk)) : 0u;
        } else {
          r.x0 = __float_as_uint(__ldg(a.g + rowv * DK + kk));
        }
      } else {
        r.x0 = __float_as_uint(__ldg(a.g + rowv * DK + kk));
      }
      r.x1 = ld_bits(vp, rowv * DV + kk, IO16);
    }
    if (tid == 0) {
      if constexpr (GATE) r.b = a.beta_sigmoid ? ld_bits(a.beta, rowv, a.beta_raw_dtype == KDA_BF16) : __float_as_uint(__ldg(a.beta + rowv));
      else r.b = __float_as_uint(__ldg(a.beta + rowv));
    }
  };
  auto stash_vec = [&](int buf, const Raw& r) {
    const float x1 = to_float(r.x1, IO16);
    float b = __uint_as_float(r.b);
    if (tid < DK) {
      const float x0 = to_float(r.x0, IO16);
      s.qv[buf][tid] = x0;
      s.kv[buf][tid] = x1;
      if (a.use_qk_l2norm) {
        const float sq = warp_sum(x0 * x0), sk = warp_sum(x1 * x1);
        if (lane == 0) {
          s.nrm[buf][warp] = sq;
          s.nrm[buf][4 + warp] = sk;
        }
      }
    } else {
      float g = __uint_as_float(r.x0);
      if constexpr (GATE) {
        if (a.A_log) {
          const float x = to_float(r.x0, a.g_raw_dtype == KDA_BF16) + __uint_as_float(r.bias);
          const float al = __expf(__uint_as_float(r.al));
          g = a.use_lower_bound ? a.lower_bound * sigmoid_fast(al * x) : -al * softplus_fast(x);
        }
      }
      s.eg[buf][tid - DK] = __expf(g);
      s.vv[buf][tid - DK] = x1;
    }
    if constexpr (GATE) {
      if (a.beta_sigmoid) b = sigmoid_fast(to_float(r.b, a.beta_raw_dtype == KDA_BF16));
    }
    if (tid == 0) s.beta[buf] = b;
  };

  if (tid == 0) {
    for (int i = 0; i < DEC_STAGES; ++i) mbar_init(&s.full[i], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const long long u0 = blockIdx.x, step = gridDim.x;
  if (u0 >= total) return;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      const long long u = u0 + i * step;
      if (u < total) {
        mbar_expect_tx(&s.full[i], DEC_TILE);
        bulk_g2s(s.S[i], a.h0 + slot_of(u), DEC_TILE, &s.full[i]);
      }
    }
  }
  // The vectors travel two units ahead of their use, in registers: under a saturated memory system a small load takes
  // longer than one unit's update, and a thread that waits for it holds up the whole ring.
  Raw rx = {0u, 0u, 0u, 0u, 0u};                    // unit it + 1
  {
    Raw rf = {0u, 0u, 0u, 0u, 0u};
    load_vec(u0, rf);
    if (u0 + step < total) load_vec(u0 + step, rx);
    stash_vec(0, rf);
  }
  __syncthreads();

  bool alive = true;
  int it = 0;
  for (long long u = u0; u < total; u += step, ++it) {
    const int st = it % DEC_STAGES, buf = it & 1;
    const bool has_next = u + step < total;
    Raw ry = {0u, 0u, 0u, 0u, 0u};                  // unit it + 2
    if (u + 2 * step < total) load_vec(u + 2 * step, ry);

    if (!mbar_wait(&s.full[st], static_cast<unsigned>(it / DEC_STAGES) & 1u)) alive = false;
    float rq = a.scale, rk = 1.f;
    if (a.use_qk_l2norm) {
      rq *= rsqrtf(s.nrm[buf][0] + s.nrm[buf][1] + s.nrm[buf][2] + s.nrm[buf][3] + L2NORM_EPS);
      rk = rsqrtf(s.nrm[buf][4] + s.nrm[buf][5] + s.nrm[buf][6] + s.nrm[buf][7] + L2NORM_EPS);
    }
    float* const tile = s.S[st];
    float4 Sr[16];
    float o_tr = 0.f;
    if constexpr (TR) {
      // tile[v][k]: rows 16 warp .. of the value axis, key columns 4 lane ..
      const float4 e4 = *reinterpret_cast<const float4*>(&s.eg[buf][4 * lane]);
      float4 k4 = *reinterpret_cast<const float4*>(&s.kv[buf][4 * lane]);
      float4 q4 = *reinterpret_cast<const float4*>(&s.qv[buf][4 * lane]);
      k4.x *= rk; k4.y *= rk; k4.z *= rk; k4.w *= rk;
      q4.x *= rq; q4.y *= rq; q4.z *= rq; q4.w *= rq;
      float part[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        Sr[i] = *reinterpret_cast<const float4*>(&tile[(16 * warp + i) * DK + 4 * lane]);
        Sr[i].x *= e4.x; Sr[i].y *= e4.y; Sr[i].z *= e4.z; Sr[i].w *= e4.w;
        part[i] = fmaf(k4.x, Sr[i].x, fmaf(k4.y, Sr[i].y, fmaf(k4.z, Sr[i].z, k4.w * Sr[i].w)));
      }
      const float hk = butterfly_sum16(part, lane);                     // value row 16 warp + (lane & 15)
      const float dvl = s.beta[buf] * (s.vv[buf][16 * warp + (lane & 15)] - hk);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float dvi = __shfl_sync(0xffffffffu, dvl, i);
        Sr[i].x = fmaf(k4.x, dvi, Sr[i].x); Sr[i].y = fmaf(k4.y, dvi, Sr[i].y); Sr[i].z = fmaf(k4.z, dvi, Sr[i].z); Sr[i].w = fmaf(k4.w, dvi, Sr[i].w);
        part[i] = fmaf(q4.x, Sr[i].x, fmaf(q4.y, Sr[i].y, fmaf(q4.z, Sr[i].z, q4.w * Sr[i].w)));
        *reinterpret_cast<float4*>(&tile[(16 * warp + i) * DK + 4 * lane]) = Sr[i];
      }
      o_tr = butterfly_sum16(part, lane);
    } else {
    float4 hk = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = 16 * warp + i;
      Sr[i] = *reinterpret_cast<const float4*>(&tile[r * DV + 4 * lane]);
      const float e = s.eg[buf][r], kk = s.kv[buf][r] * rk;
      Sr[i].x *= e; Sr[i].y *= e; Sr[i].z *= e; Sr[i].w *= e;
      hk.x = fmaf(kk, Sr[i].x, hk.x); hk.y = fmaf(kk, Sr[i].y, hk.y); hk.z = fmaf(kk, Sr[i].z, hk.z); hk.w = fmaf(kk, Sr[i].w, hk.w);
    }
    *reinterpret_cast<float4*>(&s.red[warp][4 * lane]) = hk;
    __syncthreads();
    hk = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(&s.red[w][4 * lane]);
      hk.x += x.x; hk.y += x.y; hk.z += x.z; hk.w += x.w;
    }
    const float4 vt = *reinterpret_cast<const float4*>(&s.vv[buf][4 * lane]);
    const float beta = s.beta[buf];
    const float4 dv = make_float4(beta * (vt.x - hk.x), beta * (vt.y - hk.y), beta * (vt.z - hk.z), beta * (vt.w - hk.w));
    float4 oa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = 16 * warp + i;
      const float kk = s.kv[buf][r] * rk, qq = s.qv[buf][r] * rq;
      Sr[i].x = fmaf(kk, dv.x, Sr[i].x); Sr[i].y = fmaf(kk, dv.y, Sr[i].y); Sr[i].z = fmaf(kk, dv.z, Sr[i].z); Sr[i].w = fmaf(kk, dv.w, Sr[i].w);
      oa.x = fmaf(qq, Sr[i].x, oa.x); oa.y = fmaf(qq, Sr[i].y, oa.y); oa.z = fmaf(qq, Sr[i].z, oa.z); oa.w = fmaf(qq, Sr[i].w, oa.w);
      *reinterpret_cast<float4*>(&tile[r * DV + 4 * lane]) = Sr[i];
    }
    *reinterpret_cast<float4*>(&s.red2[warp][4 * lane]) = oa;
    }
    if (has_next) stash_vec(buf ^ 1, rx);
    rx = ry;
    fence_proxy_async();          // the updated tile becomes visible to the bulk-copy engine
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) {
        atomicOr(&g_decode_status, 1u);
        // loads of the next two tiles may still be in flight into this CTA's shared memory: give them a bounded wait too
        for (int j = 1; j <= 2; ++j)
          if (u + j * step < total) mbar_wait(&s.full[(it + j) % DEC_STAGES], static_cast<unsigned>((it + j) / DEC_STAGES) & 1u);
      }
      break;
    }
    if (tid == 0) {
      bulk_s2g(a.ht + slot_of(u), tile, DEC_TILE);
      bulk_commit();
      const long long u2 = u + 2 * step;
      if (u2 < total) {
        const int s2 = (it + 2) % DEC_STAGES;       // last used by the previous unit, whose store was committed one group ago
        bulk_wait_read<1>();
        mbar_expect_tx(&s.full[s2], DEC_TILE);
        bulk_g2s(s.S[s2], a.h0 + slot_of(u2), DEC_TILE, &s.full[s2]);
      }
    }
    if constexpr (TR) {
      if (lane < 16) st1o(op + static_cast<size_t>(u) * DV + 16 * warp + lane, o_tr);
    } else if (warp == 0) {
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(&s.red2[w][4 * lane]);
        o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
      }
      st4o(op + static_cast<size_t>(u) * DV + 4 * lane, o);     // token n, head h: row u of [N, H, V]
    }
  }
  // the stores read shared memory and write the states: both must be complete before the CTA leaves
  if (tid == 0) bulk_wait<0>();
  __syncthreads();
}

template <typename IO, bool TR, bool GATE>
int launch(const kda_recurrent_args& a, cudaStream_t st) {
  const int smem = static_cast<int>(sizeof(DecSmem)) + 128;
  static DeviceOnce once;      // per template variant, per device
  const int rc = once.run([&] {
    return cudaFuncSetAttribute(kda_decode_bulk_kernel<IO, TR, GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (rc != KDA_OK) return rc;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long total = static_cast<long long>(a.N) * a.H;
  const unsigned grid = static_cast<unsigned>(total < sms ? total : sms);
  kda_decode_bulk_kernel<IO, TR, GATE><<<grid, DEC_THREADS, smem, st>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Whether the bulk-copy decode kernel covers this call: one token per sequence, K = V = 128, states carried from h0 to
// ht (either layout), and enough (sequence, head) units to keep every SM's ring busy (with few units per SM the
// per-warp kernel spreads the work more finely).
bool decode_bulk_covers(const kda_recurrent_args& a) {
  if (a.K != DK || a.V != DV || !a.h0 || !a.ht || a.cu_seqlens || a.T != 1 || a.num_accepted_tokens) return false;
  if (a.io_dtype != KDA_BF16 && a.io_dtype != KDA_FP32) return false;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
  return static_cast<long long>(a.N) * a.H >= static_cast<long long>(KDA_DECODE_BULK_MIN_UNITS_PER_SM) * sms;
}

int decode_bulk_launch(const kda_recurrent_args& a, cudaStream_t st) {
  const bool gate = a.A_log != nullptr || a.beta_sigmoid != 0;
  const int which = (a.io_dtype == KDA_BF16 ? 0 : 4) + (a.transpose_state ? 2 : 0) + (gate ? 1 : 0);
  switch (which) {
    case 0: return launch<__nv_bfloat16, false, false>(a, st);
    case 1: return launch<__nv_bfloat16, false, true>(a, st);
    case 2: return launch<__nv_bfloat16, true, false>(a, st);
    case 3: return launch<__nv_bfloat16, true, true>(a, st);
    case 4: return launch<float, false, false>(a, st);
    case 5: return launch<float, false, true>(a, st);
    case 6: return launch<float, true, false>(a, st);
    default: return launch<float, true, true>(a, st);
  }
}

}  // namespace kda

extern "C" int kda_recurrent_status(uint32_t* host_out) {
  if (!host_out) return KDA_E_NULL;
  unsigned v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, kda::g_decode_status, sizeof(v));
  if (e == cudaSuccess && v) e = cudaMemcpyToSymbol(kda::g_decode_status, &zero, sizeof(zero));
  *host_out = v;
  return static_cast<int>(e);
}
