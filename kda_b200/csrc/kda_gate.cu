// Gate front end of KDA: the decay activation and the beta sigmoid that the layer applies before the chunked
// or recurrent operator, and their backward.  Plain HBM-bound elementwise kernels with 16-byte accesses; the
// backward's reductions over tokens (d dt_bias, d A_log) go through per-CTA partial sums in a caller-provided
// workspace and a second small kernel, so the result does not depend on scheduling.
//
//   x = g_raw + dt_bias[h, k]
//   g = -exp(A_log[h]) * softplus(x)                       (softplus(x) = x for x > 20)
//   g = lower_bound * sigmoid(exp(A_log[h]) * x)           (when a lower bound is given)
//   beta = sigmoid(beta_raw)
#include "kda_chunk.cuh"

namespace kda {

constexpr int GATE_THREADS = 256;
constexpr int GATE_BWD_THREADS = 256;

__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// softplus and its derivative (the sigmoid) from one exponential: log(1 + e^x), e^x / (1 + e^x); identity / 1 above 20.
// Below -15 the sum 1 + e^x would round the small term away: log(1 + e) = e there to fp32 accuracy.
__device__ __forceinline__ float softplusf_(float x, float& sig) {
  const float e = __expf(fminf(x, 20.f));
  const float t = 1.f + e;
  sig = x > 20.f ? 1.f : __fdividef(e, t);
  return x > 20.f ? x : (x < -15.f ? e : __logf(t));
}
__device__ __forceinline__ float softplusf_(float x) {
  const float e = __expf(fminf(x, 20.f));
  return x > 20.f ? x : (x < -15.f ? e : __logf(1.f + e));
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y), c = unpack_bf16(r.z), d = unpack_bf16(r.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
template <typename T>
__device__ __forceinline__ float load1(const T* p);
template <>
__device__ __forceinline__ float load1<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void store1(T* p, float v);
template <>
__device__ __forceinline__ void store1<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// ---- forward: one thread per group of eight key columns -------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GATE_THREADS) kda_gate_fwd_kernel(const T* __restrict__ g_raw, const float* __restrict__ A_log,
                                                                    const float* __restrict__ dt_bias, float* __restrict__ g,
                                                                    long long groups, int HK, int K, int use_lb, float lb) {
  const int gpr = HK >> 3;                                   // groups per token row
  const long long stride = static_cast<long long>(gridDim.x) * GATE_THREADS;
  // two independent groups per iteration keep two 16-byte loads in flight per thread
  for (long long i0 = static_cast<long long>(blockIdx.x) * GATE_THREADS + threadIdx.x; i0 < groups; i0 += 2 * stride) {
    const long long i1 = i0 + stride;
    const bool two = i1 < groups;
    float x[2][8];
    load8(g_raw + i0 * 8, x[0]);
    if (two) load8(g_raw + i1 * 8, x[1]);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
      const long long i = u ? i1 : i0;
      const int col = static_cast<int>(i % gpr) << 3;
      const float a = __expf(A_log[col / K]);
      if (dt_bias) {
        float b[8];
        load8(dt_bias + col, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[u][e] += b[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) x[u][e] = use_lb ? lb * sigmoidf_(a * x[u][e]) : -a * softplusf_(x[u][e]);
      store8(g + i * 8, x[u]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(GATE_THREADS) kda_beta_sigmoid_fwd_kernel(const T* __restrict__ beta_raw, float* __restrict__ beta,
                                                                            long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * GATE_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * GATE_THREADS)
    beta[i] = sigmoidf_(load1(beta_raw + i));
}

template <typename T>
__global__ void __launch_bounds__(GATE_THREADS) kda_beta_sigmoid_bwd_kernel(const T* __restrict__ beta_raw, const float* __restrict__ dbeta,
                                                                            T* __restrict__ dbeta_raw, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * GATE_THREADS + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * GATE_THREADS) {
    const float b = sigmoidf_(load1(beta_raw + i));
    store1(dbeta_raw + i, dbeta[i] * b * (1.f - b));
  }
}

// ---- backward: CTA (cb, rb) owns 256 groups of eight columns and the token rows rb, rb + nblk, ...; two rows per
// iteration keep 96 bytes of loads in flight per thread.
//   dx = dg * dg/dx;   part_dx[rb][col] = sum over the CTA's rows of dx;   part_dA[rb][group] = sum of dg * dg/dA_log
template <typename T>
__global__ void __launch_bounds__(GATE_BWD_THREADS, 3) kda_gate_bwd_kernel(const T* __restrict__ g_raw, const float* __restrict__ A_log,
                                                                           const float* __restrict__ dt_bias, const float* __restrict__ dg,
                                                                           T* __restrict__ dg_raw, float* __restrict__ part_dx,
                                                                           float* __restrict__ part_dA, long long tokens, int HK, int K,
                                                                           int use_lb, float lb) {
  const int gpr = HK >> 3;
  const int cg = blockIdx.x * GATE_BWD_THREADS + threadIdx.x;
  if (cg >= gpr) return;
  const int col = cg << 3, nblk = gridDim.y, rb = blockIdx.y;
  const float a = __expf(A_log[col / K]);
  float b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) b[e] = 0.f;
  if (dt_bias) load8(dt_bias + col, b);
  float sdx[8], sA = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) sdx[e] = 0.f;
  for (long long r0 = rb; r0 < tokens; r0 += 2LL * nblk) {
    const long long r1 = r0 + nblk;
    const bool two = r1 < tokens;
    float x[2][8], d[2][8];
    load8(g_raw + r0 * HK + col, x[0]);
    load8(dg + r0 * HK + col, d[0]);
    if (two) {
      load8(g_raw + r1 * HK + col, x[1]);
      load8(dg + r1 * HK + col, d[1]);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && !two) break;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xe = x[u][e] + b[e];
        float dx;
        if (use_lb) {
          const float sg = sigmoidf_(a * xe);
          dx = d[u][e] * lb * sg * (1.f - sg) * a;    // d/dx of lb sigmoid(a x);  d/dA_log = dx * x
          sA = fmaf(dx, xe, sA);
        } else {
          float sg;
          const float sp = softplusf_(xe, sg);
          dx = -a * d[u][e] * sg;                     // d/dx of -a softplus(x);   d/dA_log = g itself
          sA = fmaf(d[u][e], -a * sp, sA);
        }
        sdx[e] += dx;
        d[u][e] = dx;
      }
      store8(dg_raw + (u ? r1 : r0) * HK + col, d[u]);
    }
  }
  store8(part_dx + static_cast<size_t>(rb) * HK + col, sdx);
  part_dA[static_cast<size_t>(rb) * gpr + cg] = sA;
}

// Sums the partials in a fixed order (bit-reproducible).  Blocks [0, ceil(HK / 256)): one thread per column of
// d dt_bias.  Then one block per head for d A_log: thread i adds elements i, i + 256, ... of that head's
// nblk x K/8 partials, and a shared-memory tree adds the 256 thread sums.
__global__ void __launch_bounds__(GATE_THREADS) kda_gate_bwd_finish_kernel(const float* __restrict__ part_dx, const float* __restrict__ part_dA,
                                                                           float* __restrict__ ddt_bias, float* __restrict__ dA_log, int nblk,
                                                                           int HK, int K) {
  __shared__ float red[GATE_THREADS];
  const int col_blocks = (HK + GATE_THREADS - 1) / GATE_THREADS;
  const int gpr = HK >> 3, gph = K >> 3;
  if (static_cast<int>(blockIdx.x) < col_blocks) {
    const int i = blockIdx.x * GATE_THREADS + threadIdx.x;
    if (i < HK && ddt_bias) {
      float s = 0.f;
#pragma unroll 8
      for (int b = 0; b < nblk; ++b) s += part_dx[static_cast<size_t>(b) * HK + i];
      ddt_bias[i] = s;
    }
    return;
  }
  const int h = blockIdx.x - col_blocks;
  float s = 0.f;
  for (int i = threadIdx.x; i < nblk * gph; i += GATE_THREADS) s += part_dA[static_cast<size_t>(i / gph) * gpr + h * gph + (i % gph)];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = GATE_THREADS / 2; o > 0; o >>= 1) {
    if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) dA_log[h] = red[0];
}

constexpr int GATE_BWD_MAX_ROW_BLOCKS = 148 * 2;       // the workspace is sized for this many partial sums per column
static int gate_bwd_blocks(long long tokens, int col_blocks) {     // row blocks: about three CTAs per SM in total
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long want = (3LL * sms + col_blocks - 1) / col_blocks;
  if (want > GATE_BWD_MAX_ROW_BLOCKS) want = GATE_BWD_MAX_ROW_BLOCKS;
  if (want > tokens) want = tokens;
  return static_cast<int>(want < 1 ? 1 : want);
}

static int validate_gate(const kda_gate_args* a, bool bwd) {
  if (!a || (!a->g_raw && !a->beta_raw)) return KDA_E_NULL;        // g_raw == NULL: beta sigmoid only
  if (a->g_raw && !a->A_log) return KDA_E_NULL;
  if (a->tokens < 0 || a->H <= 0 || a->K <= 0 || (a->K & 7)) return KDA_E_SHAPE;
  if ((a->g_dtype != KDA_BF16 && a->g_dtype != KDA_FP32) || (a->beta_dtype != KDA_BF16 && a->beta_dtype != KDA_FP32)) return KDA_E_DTYPE;
  if (!bwd) {
    if (a->g_raw && !a->g) return KDA_E_NULL;
    if (a->beta_raw && !a->beta) return KDA_E_NULL;
  } else {
    if (a->g_raw && (!a->dg || !a->dg_raw || !a->dA_log || !a->workspace)) return KDA_E_NULL;
    if (a->beta_raw && (!a->dbeta || !a->dbeta_raw)) return KDA_E_NULL;
    if (a->g_raw && a->workspace_bytes < kda_gate_bwd_workspace_bytes(a->tokens, a->H, a->K)) return KDA_E_WORKSPACE;
  }
  const void* ptrs[] = {a->g_raw, a->dt_bias, a->g, a->dg, a->dg_raw, a->workspace};
  for (const void* p : ptrs)
    if (p && (reinterpret_cast<uintptr_t>(p) & 15)) return KDA_E_ALIGN;
  return KDA_OK;
}

static int ew_blocks(long long n) {
  const long long b = (n + GATE_THREADS - 1) / GATE_THREADS;
  return static_cast<int>(b < 1 ? 1 : (b > 148LL * 64 ? 148LL * 64 : b));
}

}  // namespace kda

extern "C" size_t kda_gate_bwd_workspace_bytes(int64_t tokens, int32_t H, int32_t K) {
  if (tokens < 0 || H <= 0 || K <= 0) return 0;
  const size_t HK = static_cast<size_t>(H) * K;
  return static_cast<size_t>(kda::GATE_BWD_MAX_ROW_BLOCKS) * (HK + HK / 8) * sizeof(float);
}

extern "C" int kda_gate_fwd(const kda_gate_args* a, void* stream) {
  using namespace kda;
  const int rc = validate_gate(a, false);
  if (rc != KDA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ProfCall* pc = prof_begin(st);
  const int HK = a->H * a->K;
  const long long groups = a->g_raw ? a->tokens * (HK >> 3) : 0;
  if (groups > 0) {
    if (a->g_dtype == KDA_BF16)
      kda_gate_fwd_kernel<__nv_bfloat16><<<ew_blocks(groups), GATE_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(a->g_raw), a->A_log, a->dt_bias,
                                                                                      a->g, groups, HK, a->K, a->use_lower_bound, a->lower_bound);
    else
      kda_gate_fwd_kernel<float><<<ew_blocks(groups), GATE_THREADS, 0, st>>>(static_cast<const float*>(a->g_raw), a->A_log, a->dt_bias, a->g, groups,
                                                                              HK, a->K, a->use_lower_bound, a->lower_bound);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long long nb = a->tokens * a->H;
  if (a->beta_raw && nb > 0) {
    if (a->beta_dtype == KDA_BF16)
      kda_beta_sigmoid_fwd_kernel<__nv_bfloat16><<<ew_blocks(nb), GATE_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(a->beta_raw), a->beta, nb);
    else
      kda_beta_sigmoid_fwd_kernel<float><<<ew_blocks(nb), GATE_THREADS, 0, st>>>(static_cast<const float*>(a->beta_raw), a->beta, nb);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  prof_mark(pc, KDA_STAGE_GATE_FWD, st);
  return KDA_OK;
}

extern "C" int kda_gate_bwd(const kda_gate_args* a, void* stream) {
  using namespace kda;
  const int rc = validate_gate(a, true);
  if (rc != KDA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ProfCall* pc = prof_begin(st);
  const int HK = a->H * a->K;
  const int col_blocks = ((HK >> 3) + GATE_BWD_THREADS - 1) / GATE_BWD_THREADS;
  const int nblk = gate_bwd_blocks(a->tokens, col_blocks);
  const dim3 grid(col_blocks, nblk);
  float* part_dx = static_cast<float*>(a->workspace);
  float* part_dA = part_dx + static_cast<size_t>(GATE_BWD_MAX_ROW_BLOCKS) * HK;
  if (!a->g_raw) {
    // beta sigmoid only
  } else if (a->g_dtype == KDA_BF16)
    kda_gate_bwd_kernel<__nv_bfloat16><<<grid, GATE_BWD_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(a->g_raw), a->A_log, a->dt_bias, a->dg,
                                                                            static_cast<__nv_bfloat16*>(a->dg_raw), part_dx, part_dA, a->tokens, HK, a->K,
                                                                            a->use_lower_bound, a->lower_bound);
  else
    kda_gate_bwd_kernel<float><<<grid, GATE_BWD_THREADS, 0, st>>>(static_cast<const float*>(a->g_raw), a->A_log, a->dt_bias, a->dg,
                                                                    static_cast<float*>(a->dg_raw), part_dx, part_dA, a->tokens, HK, a->K, a->use_lower_bound,
                                                                    a->lower_bound);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (a->g_raw)
    kda_gate_bwd_finish_kernel<<<(HK + GATE_THREADS - 1) / GATE_THREADS + a->H, GATE_THREADS, 0, st>>>(part_dx, part_dA, a->ddt_bias, a->dA_log, nblk,
                                                                                                         HK, a->K);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long nb = a->tokens * a->H;
  if (a->beta_raw && nb > 0) {
    if (a->beta_dtype == KDA_BF16)
      kda_beta_sigmoid_bwd_kernel<__nv_bfloat16><<<ew_blocks(nb), GATE_THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(a->beta_raw), a->dbeta,
                                                                                          static_cast<__nv_bfloat16*>(a->dbeta_raw), nb);
    else
      kda_beta_sigmoid_bwd_kernel<float><<<ew_blocks(nb), GATE_THREADS, 0, st>>>(static_cast<const float*>(a->beta_raw), a->dbeta,
                                                                                  static_cast<float*>(a->dbeta_raw), nb);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  prof_mark(pc, KDA_STAGE_GATE_BWD, st);
  return KDA_OK;
}
