// Device-side helpers shared by the KDA kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kda_b200.h"

namespace kda {

constexpr int C = KDA_CHUNK;              // tokens per chunk
constexpr float LOG2E = 1.4426950408889634f;
constexpr float L2NORM_EPS = 1e-6f;

// ---- small numeric helpers ---------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {  // 2^x, ex2.approx (flushes tiny results to 0, never overflows for x<=0)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);   // .x = lo (low 16 bits), .y = hi
  return *reinterpret_cast<uint32_t*>(&p);
}

__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 p = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(p);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// ---- gate front end of the recurrent kernels: activated log-decay and beta from the raw layer outputs -------------
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// softplus(x) = log(1 + e^x); identity above 20; below -15 the sum would round e^x away and log(1 + e) = e to fp32 accuracy
__device__ __forceinline__ float softplus_fast(float x) {
  const float e = __expf(fminf(x, 20.f));
  return x > 20.f ? x : (x < -15.f ? e : __logf(1.f + e));
}
__device__ __forceinline__ float load_raw(const void* p, size_t i, int dtype) {      // dtype: KDA_BF16 or KDA_FP32
  return dtype == KDA_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]) : __ldg(static_cast<const float*>(p) + i);
}
// log-decay of (token row `row` = token * H + h, key column k) as the kernels use it
__device__ __forceinline__ float recurrent_log_decay(const kda_recurrent_args& a, size_t row, int h, int k, int K) {
  if (!a.A_log) return __ldg(a.g + row * K + k);
  float x = load_raw(a.g, row * K + k, a.g_raw_dtype);
  if (a.dt_bias) x += __ldg(a.dt_bias + static_cast<size_t>(h) * K + k);
  const float al = __expf(__ldg(a.A_log + h));
  return a.use_lower_bound ? a.lower_bound * sigmoid_fast(al * x) : -al * softplus_fast(x);
}
__device__ __forceinline__ float recurrent_beta(const kda_recurrent_args& a, size_t row) {
  return a.beta_sigmoid ? sigmoid_fast(load_raw(a.beta, row, a.beta_raw_dtype)) : __ldg(a.beta + row);
}

// ---- tensor-core primitives (warp-level, bf16 in / fp32 accumulate) ------------------------------
// D(16x8) += A(16x16, row) * B(16x8, col).  Fragment ownership (gid = lane/4, tig = lane%4):
//   a0:(gid, 2tig..+1) a1:(gid+8, 2tig..) a2:(gid, 2tig+8..) a3:(gid+8, 2tig+8..)
//   b0:(k=2tig..+1, n=gid) b1:(k=2tig+8..+9, n=gid)
//   c0,c1:(gid, 2tig, 2tig+1) c2,c3:(gid+8, 2tig, 2tig+1)
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// ---- shared-memory tile addressing --------------------------------------------------------------
// A bf16 tile with ROWB bytes per row (128 or 256) is stored with its 16-byte pieces XOR-swizzled by the
// row index, so that the eight row addresses of one ldmatrix 8x8 load, and the eight rows touched by
// one warp-wide fragment access, fall in distinct bank groups.  `col` is a bf16 element index.
template <int ROWB>
__device__ __forceinline__ uint32_t swz(int row, int col) {
  const int piece = (col >> 3) ^ (row & 7);
  return static_cast<uint32_t>(row * ROWB + (piece << 4) + ((col & 7) << 1));
}

// ---- TMA 1-D bulk copy + mbarrier, with bounded waits ------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Waits for the phase with the given parity.  Gives up after a bounded number of polls and returns false; the
// caller then records an error and leaves its loop instead of spinning forever.  One poll (a try_wait that the
// hardware suspends for a short while, plus the sleep) takes about 4 microseconds on B200, so 2^18 polls are
// about one second -- four orders of magnitude above the longest wait of a healthy run.
constexpr unsigned MBAR_WAIT_POLLS = 1u << 18;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  for (unsigned i = 0; i < MBAR_WAIT_POLLS; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}
// global -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned; completion on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// shared -> global bulk store (commit + wait by the issuing thread)
__device__ __forceinline__ void bulk_s2g(void* dst_gmem, const void* src_smem, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- Ampere-style 16-byte async copies for strided rows ------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem, bool valid) {
  const unsigned sz = valid ? 16u : 0u;   // src-size 0 -> destination is zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src_gmem, bool valid) {
  const unsigned sz = valid ? 4u : 0u;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

}  // namespace kda
