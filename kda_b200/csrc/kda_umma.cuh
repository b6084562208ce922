// tcgen05 (5th-generation tensor core) primitives for sm_100a: shared-memory matrix descriptors for
// 128-byte-swizzled bf16 tiles, the instruction descriptor of kind::f16, TMEM allocation, MMA issue,
// commit-to-mbarrier and TMEM loads.  Everything is inline PTX; no CUTLASS dependency.
//
// Operand tiles ("SW128 tiles"): [R rows][64 bf16], 128-byte rows, the 16-byte pieces of a row XOR-ed with
// (row & 7), eight rows = one 1024-byte swizzle atom, atoms stacked contiguously; the tile base is
// 1024-byte aligned.  The same memory image serves two roles:
//   K-major  : rows = M (or N) index, the 64 columns = K.   One MMA (K = 16) reads 32 bytes of each row.
//   MN-major : rows = K index, the 64 columns = M (or N).   One MMA (K = 16) reads 16 rows = two atoms.
// A 128-wide dimension is two such tiles ("spans"); for MN-major the distance between the two spans is
// the descriptor's leading byte offset.
#pragma once

#include "kda_common.cuh"

namespace kda {
namespace umma {

constexpr uint32_t ATOM_BYTES = 1024;   // 8 rows x 128 bytes

// byte offset of element (row, col) inside one SW128 tile, col in [0, 64)
__device__ __forceinline__ uint32_t sw128(int row, int col) {
  return static_cast<uint32_t>(row * 128 + ((((col >> 3) ^ row) & 7) << 4) + ((col & 7) << 1));
}

// Shared-memory matrix descriptor (64-bit), SWIZZLE_128B:
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version = 1 (Blackwell)   [61,64) layout type = 2 (128-byte swizzle)
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_byte_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_byte_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// K-major operand, k-step s (16 columns) of a tile: +32 bytes per step inside the 128-byte rows
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kstep_in_tile) {
  return smem_desc(tile_addr + static_cast<uint32_t>(kstep_in_tile) * 32u, 16u, ATOM_BYTES);
}
// MN-major operand, k-step s (16 rows = two atoms); span_stride = bytes between the two 64-wide spans
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int kstep, uint32_t span_stride_bytes) {
  return smem_desc(tile_addr + static_cast<uint32_t>(kstep) * 2u * ATOM_BYTES, span_stride_bytes, ATOM_BYTES);
}

// Instruction descriptor, kind::f16 with bf16 inputs and fp32 accumulation:
//   [4,6) D format (1 = f32)  [7,10) A format (1 = bf16)  [10,13) B format (1 = bf16)
//   [13] negate A  [14] negate B  [15] A major (0 = K, 1 = MN)  [16] B major  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool a_mn_major, bool b_mn_major, bool neg_a = false,
                                                  bool neg_b = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(neg_a) << 13) | (static_cast<uint32_t>(neg_b) << 14) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ---- TMEM allocation (one full warp executes these) -----------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // ncols: power of two >= 32
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate = 0 overwrites D.
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same, issued inside a converged warp whose lanes all hold the same operands: only the lane with
// leader != 0 issues.  Keeping the whole warp on one instruction stream lets the compiler hold the descriptors
// in uniform registers instead of moving them there before every MMA.
__device__ __forceinline__ void mma_ss_lead(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                            uint32_t leader) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
// Four products of one accumulation chain in ONE asm block: D (+)= A_s B_s for k-steps s = 0..3, the descriptors of step s
// being a + s * A_INC and b + s * B_INC (in descriptor units of 16 bytes: 2 per k-step of a K-major tile, 128 per k-step
// of an MN-major tile).  The first product accumulates iff acc_first != 0, the others always.  Keeping the descriptor
// arithmetic and the predicates inside the block lets consecutive products issue about 56 cycles apart; issued as four
// separate asm statements with their operands prepared in between, the same thread needs about 90 cycles per product.
template <int A_INC, int B_INC>
__device__ __forceinline__ void mma4(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 a1, b1;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\t"
      "setp.eq.b32 p1, %4, %4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "add.u64 a1, %1, %5;\n\t"
      "add.u64 b1, %2, %8;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "add.u64 a1, %1, %6;\n\t"
      "add.u64 b1, %2, %9;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "add.u64 a1, %1, %7;\n\t"
      "add.u64 b1, %2, %10;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, p1;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc_first), "n"(A_INC), "n"(2 * A_INC), "n"(3 * A_INC), "n"(B_INC), "n"(2 * B_INC), "n"(3 * B_INC)
      : "memory");
}
constexpr int KSTEP_KMAJOR = 2;      // descriptor units per k-step (16 columns = 32 bytes) inside a K-major SW128 tile
constexpr int KSTEP_MNMAJOR = 128;   // descriptor units per k-step (16 rows = two atoms = 2048 bytes) of an MN-major SW128 tile

// Makes the mbarrier receive one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// TMEM -> registers: this warp's 32 lanes (quadrant warp%4), 16 consecutive 32-bit columns per thread.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// registers -> TMEM, same shape
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMEM address of (lane, column) relative to an allocation base
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
  return base + (static_cast<uint32_t>(lane) << 16) + static_cast<uint32_t>(col);
}

}  // namespace umma
}  // namespace kda
