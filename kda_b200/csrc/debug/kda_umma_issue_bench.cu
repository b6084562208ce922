// Development measurement (libkda_b200_debug.so only): what a sequence of small tcgen05.mma instructions costs the issuing
// thread and the tensor pipe, depending on how many accumulators the sequence is spread over and on whether it is issued
// from a single-thread branch or by the lead lane of a converged warp.  One CTA, operands are zero-filled shared memory.
// out[0] = cycles the issuing thread spent in the issue loop (including the commit), out[1] = cycles until the commit's
// barrier completed.
#include "kda_umma.cuh"

namespace kda {

__global__ void __launch_bounds__(128, 1) umma_issue_bench_kernel(long long* __restrict__ out, int M, int N, int count, int naccum,
                                                                  int converged, unsigned* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = base;              // [128][64] SW128 tiles x 2
  unsigned char* sB = base + 32768;
  uint64_t* bar = reinterpret_cast<uint64_t*>(base + 65536);
  uint32_t* slot = reinterpret_cast<uint32_t*>(base + 65536 + 16);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 65536 / 16; i += 128) reinterpret_cast<uint4*>(base)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  if (warp == 0) umma::tmem_alloc(slot, 512);
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t taddr = *slot;
  const uint32_t idesc = umma::instr_desc(M, N, false, true);
  const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
  long long t0 = 0, t1 = 0, t2 = 0;
  if (warp == 0) {
    if (converged == 1) {
      const uint32_t leadf = lane == 0;
      t0 = clock64();
#pragma unroll 1
      for (int r = 0; r < count; r += 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma::mma_ss_lead(taddr + static_cast<uint32_t>(((r + s) % naccum) * N), umma::desc_kmajor(a0 + (s >> 2) * 16384u, s & 3),
                            umma::desc_mnmajor(b0, s, 16384u), idesc, (r + s) >= naccum, leadf);
      }
      if (leadf) umma::commit(bar);
      t1 = clock64();
    } else if (converged == 2) {
      // converged warp, everything provably warp-uniform (tensor-memory address through a shuffle), descriptors as
      // base + constant, the lead lane issues
      const uint32_t leadf = lane == 0;
      const uint32_t tu = __shfl_sync(0xffffffffu, taddr, 0);
      const uint64_t dA0 = umma::desc_kmajor(a0, 0), dA1 = umma::desc_kmajor(a0 + 16384u, 0), dB = umma::desc_mnmajor(b0, 0, 16384u);
      t0 = clock64();
#pragma unroll 1
      for (int r = 0; r < count; r += 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma::mma_ss_lead(tu + static_cast<uint32_t>(((r + s) % naccum) * N), ((s >> 2) ? dA1 : dA0) + static_cast<uint64_t>(s & 3) * 2u,
                            dB + static_cast<uint64_t>(s) * 128u, idesc, (r + s) >= naccum, leadf);
      }
      if (leadf) umma::commit(bar);
      t1 = clock64();
    } else if (converged == 3) {
      // one asm block with eight products: descriptor arithmetic and the predicate live inside it
      const uint64_t dA0 = umma::desc_kmajor(a0, 0), dA1 = umma::desc_kmajor(a0 + 16384u, 0), dB = umma::desc_mnmajor(b0, 0, 16384u);
      if (lane == 0) {
        t0 = clock64();
#pragma unroll 1
        for (int r = 0; r < count; r += 8) {
          asm volatile(
              "{\n\t"
              ".reg .pred p;\n\t"
              ".reg .b64 a, b;\n\t"
              "setp.ne.b32 p, %5, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %3, %4, p;\n\t"
              "add.u64 a, %1, 2;\n\t add.u64 b, %3, 128;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "add.u64 a, %1, 4;\n\t add.u64 b, %3, 256;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "add.u64 a, %1, 6;\n\t add.u64 b, %3, 384;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "add.u64 b, %3, 512;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, b, %4, p;\n\t"
              "add.u64 a, %2, 2;\n\t add.u64 b, %3, 640;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "add.u64 a, %2, 4;\n\t add.u64 b, %3, 768;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "add.u64 a, %2, 6;\n\t add.u64 b, %3, 896;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %4, p;\n\t"
              "}\n" ::"r"(taddr),
              "l"(dA0), "l"(dA1), "l"(dB), "r"(idesc), "r"(1)
              : "memory");
        }
        umma::commit(bar);
        t1 = clock64();
      }
    } else if (converged == 4) {
      // like 0, but the second and later groups of eight go to their own accumulators and nothing else differs: shows
      // whether the constant cost is the issue or a dependence between consecutive products
      if (lane == 0) {
        t0 = clock64();
#pragma unroll 1
        for (int r = 0; r < count; r += 8) {
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma::mma_ss(taddr + static_cast<uint32_t>(s * N), umma::desc_kmajor(a0 + (s >> 2) * 16384u, s & 3),
                         umma::desc_mnmajor(b0, s, 16384u), idesc, 0);
        }
        umma::commit(bar);
        t1 = clock64();
      }
    } else if (lane == 0) {
      t0 = clock64();
#pragma unroll 1
      for (int r = 0; r < count; r += 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma::mma_ss(taddr + static_cast<uint32_t>(((r + s) % naccum) * N), umma::desc_kmajor(a0 + (s >> 2) * 16384u, s & 3),
                       umma::desc_mnmajor(b0, s, 16384u), idesc, (r + s) >= naccum);
      }
      umma::commit(bar);
      t1 = clock64();
    }
    __syncwarp();
    const bool ok = mbar_wait(bar, 0);
    t2 = clock64();
    if (lane == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
      if (!ok) atomicOr(status, 1u);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(taddr, 512);
}

}  // namespace kda

// count: multiple of 8, naccum * N <= 512 (variant 4 uses eight accumulators: 8 N <= 512); N <= 128 (the B operand region holds two 64-column spans)
extern "C" __attribute__((visibility("default"))) int kda_b200_debug_umma_issue_bench(long long* out, int M, int N, int count, int naccum,
                                                                                       int converged, unsigned* status, void* stream) {
  if (!out || !status) return KDA_E_NULL;
  if ((M != 64 && M != 128) || N < 16 || N > 128 || N % 16 || count < 8 || count % 8 || naccum < 1 || naccum * N > 512 || (converged == 4 && 8 * N > 512)) return KDA_E_SHAPE;
  const int smem = 65536 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kda::umma_issue_bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  kda::umma_issue_bench_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(out, M, N, count, naccum, converged, status);
  return static_cast<int>(cudaGetLastError());
}

// Round trip of one hand-over: a "compute" warp arrives on an mbarrier, the issuing thread (lane 0 of another warp) wakes,
// issues `nmma` products (0, 4 or 8; M=64 N=32) and commits, the compute warp waits for the commit.  out[0] = average
// cycles per round trip over `rounds` rounds, measured by the compute warp.
namespace kda {

__global__ void __launch_bounds__(64, 1) umma_roundtrip_kernel(long long* __restrict__ out, int nmma, int rounds, unsigned* __restrict__ status,
                                                               int variant, int extra) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* barX = reinterpret_cast<uint64_t*>(base + 65536);
  uint64_t* barY = barX + 1;
  uint32_t* slot = reinterpret_cast<uint32_t*>(base + 65536 + 32);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 65536 / 16; i += 64) reinterpret_cast<uint4*>(base)[i] = make_uint4(0u, 0u, 0u, 0u);
  fence_proxy_async();
  if (warp == 0) umma::tmem_alloc(slot, 64);
  if (tid == 0) {
    mbar_init(barX, 1);
    mbar_init(barY, 1);
    fence_mbar_init();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t taddr = *slot;
  // variant 0: M=64, A K-major (the shape of the sliced scans' products 1); variant 1: M=128, A MN-major in two spans of 64
  // (their products 2: kg^T read from a [64 t][128 k] tile)
  const uint32_t idesc = variant ? umma::instr_desc(128, 32, true, true) : umma::instr_desc(64, 32, false, true);
  const uint64_t dA = variant ? umma::desc_mnmajor(smem_u32(base), 0, 8192u) : umma::desc_kmajor(smem_u32(base), 0);
  const uint64_t dB = umma::desc_mnmajor(smem_u32(base + 32768), 0, 16384u);
  const uint64_t dB0k = umma::desc_kmajor(smem_u32(base + 16384), 0);
  bool ok = true;
  if (warp == 0) {
    const long long t0 = clock64();
    for (int r = 0; r < rounds && ok; ++r) {
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(barX);
      ok = __all_sync(0xffffffffu, mbar_wait(barY, r & 1));
      umma::fence_after_sync();
    }
    const long long t1 = clock64();
    if (lane == 0) {
      out[0] = (t1 - t0) / (rounds > 0 ? rounds : 1);
      if (!ok) atomicOr(status, 1u);
    }
  } else if (lane == 0) {
    for (int r = 0; r < rounds && ok; ++r) {
      ok = mbar_wait(barX, r & 1);
      umma::fence_after_sync();
      if (variant) {
        if (nmma >= 4) umma::mma4<umma::KSTEP_MNMAJOR, umma::KSTEP_MNMAJOR>(taddr, dA, dB, idesc, 0);
      } else {
        if (nmma >= 4) umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(taddr, dA, dB, idesc, 0);
        if (nmma >= 8) umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(taddr, dA + 8u, dB + 4u * umma::KSTEP_MNMAJOR, idesc, 1);
      }
      umma::commit(barY);
      // `extra` products into another accumulator behind the commit (the way the scans issue their o products behind the
      // chain's): does the next round's hand-over find the issuing thread late?
      if (extra >= 4) umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(taddr + 32, dB0k, dB, umma::instr_desc(64, 32, false, true), 0);
      if (extra >= 8) umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(taddr + 32, dB0k + 8u, dB + 4u * umma::KSTEP_MNMAJOR, umma::instr_desc(64, 32, false, true), 1);
    }
    if (!ok) atomicOr(status, 2u);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(taddr, 64);
}

}  // namespace kda

extern "C" __attribute__((visibility("default"))) int kda_b200_debug_umma_roundtrip(long long* out, int nmma, int rounds, unsigned* status,
                                                                                    void* stream, int variant, int extra) {
  if (!out || !status) return KDA_E_NULL;
  if ((nmma != 0 && nmma != 4 && nmma != 8) || rounds < 1 || rounds > 4096 || (variant != 0 && variant != 1) || (variant == 1 && nmma == 8) ||
      (extra != 0 && extra != 4 && extra != 8))
    return KDA_E_SHAPE;
  const int smem = 65536 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kda::umma_roundtrip_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  kda::umma_roundtrip_kernel<<<1, 64, smem, static_cast<cudaStream_t>(stream)>>>(out, nmma, rounds, status, variant, extra);
  return static_cast<int>(cudaGetLastError());
}
