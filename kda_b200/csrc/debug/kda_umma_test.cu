// Development check of the tcgen05 primitives in kda_umma.cuh (built into libkda_b200_debug.so, not into the product library): one CTA computes D[128 x N] = A[128 x 128] * B[N x 128]^T
// with the operands placed in shared memory K-major or MN-major.  Reached through an exported debug entry
// (not part of the public header, not in libkda_b200.so); tests/test_umma_gpu.py compares it with a plain matrix product.
#include "kda_umma.cuh"

namespace kda {

__global__ void __launch_bounds__(128, 1) umma_test_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                                                          float* __restrict__ D, int N, int a_mn, int b_mn, uint32_t idesc,
                                                          unsigned* __restrict__ status, int M, int NB, int n_off) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = base;
  unsigned char* sB = base + 32768;
  uint64_t* bar = reinterpret_cast<uint64_t*>(base + 65536);
  uint32_t* slot = reinterpret_cast<uint32_t*>(base + 65536 + 16);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  for (int i = tid; i < 128 * 128; i += 128) {
    const int m = i >> 7, k = i & 127;
    const uint32_t off = a_mn ? (m >> 6) * 16384u + umma::sw128(k, m & 63) : (k >> 6) * 16384u + umma::sw128(m, k & 63);
    *reinterpret_cast<__nv_bfloat16*>(sA + off) = A[i];
  }
  for (int i = tid; i < NB * 128; i += 128) {
    const int n = i >> 7, k = i & 127;
    const uint32_t off = b_mn ? (n >> 6) * 16384u + umma::sw128(k, n & 63) : (k >> 6) * (NB * 128u) + umma::sw128(n, k & 63);
    *reinterpret_cast<__nv_bfloat16*>(sB + off) = B[i];
  }
  fence_proxy_async();
  const uint32_t ncols = (N <= 64) ? 64u : (N <= 128 ? 128u : 256u);
  if (warp == 0) umma::tmem_alloc(slot, ncols);
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t taddr = *slot;

  if (tid == 0) {
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
    for (int s = 0; s < 8; ++s) {
      const uint64_t ad = a_mn ? umma::desc_mnmajor(a0, s, 16384u) : umma::desc_kmajor(a0 + (s >> 2) * 16384u, s & 3);
      const uint64_t bd = b_mn ? umma::desc_mnmajor(b0 + n_off * 2u, s, 16384u)
                               : umma::desc_kmajor(b0 + (s >> 2) * (NB * 128u) + n_off * 128u, s & 3);
      umma::mma_ss(taddr, ad, bd, idesc, s > 0 ? 1u : 0u);
    }
    umma::commit(bar);
  }
  const bool ok = mbar_wait(bar, 0);
  umma::fence_after_sync();
  if (ok) {
    for (int c0 = 0; c0 < N; c0 += 16) {
      float v[16];
      umma::tmem_ld16(umma::tmem_addr(taddr, 32 * warp, c0), v);
      umma::tmem_ld_wait();
      // M = 128: row = TMEM lane.  M = 64: rows 16q..16q+15 sit in lanes 32q..32q+15 (q = warp).
      const int row = (M == 128) ? 32 * warp + lane : 16 * warp + lane;
      if (M == 128 || lane < 16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) D[static_cast<size_t>(row) * N + c0 + i] = v[i];
      }
    }
  } else if (tid == 0) {
    atomicOr(status, 1u);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(taddr, ncols);
}

}  // namespace kda

// D[M x N] (fp32) = A[M x 128] * B[n_off : n_off+N, 128]^T (optionally with B negated); M in {64, 128}, N in {16, 32, 64, 128};
// B has NB rows in shared memory and the instruction reads N of them starting at row n_off.
// a_mn / b_mn select the shared-memory placement (0 = K-major, 1 = MN-major).  status: device word, nonzero if a
// bounded wait gave up.
extern "C" __attribute__((visibility("default"))) int kda_b200_debug_umma_gemm(const void* A, const void* B, float* D, int N, int a_mn,
                                                                               int b_mn, int neg_b, unsigned* status, void* stream, int M, int NB, int n_off) {
  if (!A || !B || !D || !status) return KDA_E_NULL;
  if ((N != 16 && N != 32 && N != 64 && N != 128) || (M != 64 && M != 128) || NB < N + n_off || NB > 128) return KDA_E_SHAPE;
  const int smem = 65536 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kda::umma_test_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const uint32_t idesc = kda::umma::instr_desc(M, N, a_mn != 0, b_mn != 0, false, neg_b != 0);
  kda::umma_test_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), D, N, a_mn, b_mn, idesc, status, M, NB, n_off);
  return static_cast<int>(cudaGetLastError());
}
