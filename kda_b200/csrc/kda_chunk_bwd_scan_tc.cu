// Reverse state scan of chunked KDA on tcgen05 with the fp32 state gradient resident in tensor memory (sm_100a).
//
// One CTA per (sequence, head) walks the sequence's chunks from the last to the first.  TMEM lane = value column v;
// dhT[v][k] (128 lanes x 128 fp32 columns) is the gradient w.r.t. the state at the END of the current chunk.
// Per chunk:
//   state pass   bf16 copy of dhT (A operand of the next product; also stored as the chunk's DH tile), dhT *= Gam_last;
//   products 1   dv_new^T = dO^T Aqk + dhT_bf16 kg^T                                    (M=128 v, N=64 j)
//   epilogue 1   dv_new^T -> bf16 tile (A operand of products 2; stored as the chunk's DVNEWT tile)
//   products 2   dhT += dO^T qg - dv_new^T w                                            (M=128 v, N=128 k, K=64 tokens)
// dO arrives by TMA tiled loads (two boxes of 64 value columns, 128-byte swizzled) together with the W, QG, KG, AQK,
// GL tiles of the chunk through a 2-stage mbarrier ring.
#include "kda_chunk_bwd.cuh"
#include "kda_device.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

constexpr int RNT = 256;     // 8 warps: TMEM lane quadrant = warp & 3, column half = warp >> 2

struct TcRScanStage {
  unsigned char W[TILE_TK], QG[TILE_TK], KG[TILE_TK], AQK[TILE_TT], dO[TILE_TK];
  float GL[KD];
  unsigned char pad[512];
};
static_assert(sizeof(TcRScanStage) % 1024 == 0, "stage must keep 1024-byte alignment");
constexpr unsigned TC_RSTAGE_TX = 4 * TILE_TK + TILE_TT + TILE_GL;

struct TcRScanSmem {
  TcRScanStage st[2];
  unsigned char DHb[TILE_VK];    // bf16 copy of dhT: two [128 v][64 k] spans (= the DH tile image)
  unsigned char DVNT[TILE_VT];   // bf16 dv_new^T [128 v][64 j] (= the DVNEWT tile image)
  uint64_t full[2], barM;
  uint32_t tmem_slot;
};
static_assert(sizeof(TcRScanSmem) + 1024 <= 227 * 1024, "TcRScanSmem too large");

constexpr int C_H = 0, C_VN = 128;      // TMEM columns

__device__ __forceinline__ uint4 pack8g(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ unsigned char* swq(unsigned char* tile, int row, int chunk) {
  return tile + row * 128 + (((chunk ^ row) & 7) << 4);
}

}  // namespace

__global__ void __launch_bounds__(RNT, 1) kda_chunk_bwd_scan_tc_kernel(const __grid_constant__ RScanParams p) {
  extern __shared__ unsigned char smem_raw[];
  TcRScanSmem& s = *reinterpret_cast<TcRScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, half = warp >> 2;
  const int seq = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int c_begin = p.seq_chunk_off[seq], c_end = p.seq_chunk_off[seq + 1];
  const int nchunks = c_end - c_begin;
  const long long seq_tok0 = p.cu[seq];
  const int v = 32 * q4 + lane;

  if (tid == 0) {
    mbar_init(&s.full[0], 1);
    mbar_init(&s.full[1], 1);
    mbar_init(&s.barM, 1);
    fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, 256);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = s.tmem_slot;
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);

  auto issue_load = [&](int i) {                      // thread 0: step i handles chunk c_end - 1 - i
    TcRScanStage& d = s.st[i & 1];
    const int c = c_end - 1 - i;
    const size_t tile = static_cast<size_t>(c) * p.H + h;
    const long long tok0 = seq_tok0 + static_cast<long long>(c - c_begin) * C;      // the CTA's one sequence: no table look-up
    mbar_expect_tx(&s.full[i & 1], TC_RSTAGE_TX);
    bulk_g2s(d.W, p.W + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.QG, p.QG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.KG, p.KG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.AQK, p.AQK + tile * TILE_TT, TILE_TT, &s.full[i & 1]);
    bulk_g2s(d.GL, p.GL + tile * TILE_GL, TILE_GL, &s.full[i & 1]);
    tma_load_rows(d.dO, &p.tm_do, 0, h, static_cast<int>(tok0), &s.full[i & 1]);
    tma_load_rows(d.dO + 8192, &p.tm_do, 64, h, static_cast<int>(tok0), &s.full[i & 1]);
  };
  if (tid == 0) {
    if (nchunks > 0) issue_load(0);
    if (nchunks > 1) issue_load(1);
  }

  {
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kk = 64 * half + 16 * g + i;
        x[i] = p.d_ht ? __ldg(p.d_ht + sb + static_cast<size_t>(kk) * VD + v) : 0.f;
      }
      umma::tmem_st16(tq + C_H + 64 * half + 16 * g, x);
    }
    umma::tmem_st_wait();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();

  uint32_t mph = 0;
  bool alive = true;
  for (int i = 0; i < nchunks; ++i) {       // a failed wait leaves through the uniform vote at the top of the next iteration
    TcRScanStage& d = s.st[i & 1];
    const int c = c_end - 1 - i;
    const size_t tile = static_cast<size_t>(c) * p.H + h;
    long long* const dbg = (i == 8) ? p.dbg : nullptr;      // development aid: clocks of a steady-state chunk
    KDA_DBG_CLOCK(dbg, 40);

    if (!mbar_wait(&s.full[i & 1], (i >> 1) & 1)) alive = false;
    if (tid == 0) bulk_wait_read<0>();      // the previous chunk's tile stores have read DHb / DVNT
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 4u);
      break;
    }
    KDA_DBG_CLOCK(dbg, 41);

    // ---- state pass ------------------------------------------------------------------------------------------------------
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[16];
      umma::tmem_ld16(tq + C_H + 64 * half + 16 * g, x);
      umma::tmem_ld_wait();
      *reinterpret_cast<uint4*>(swq(s.DHb + half * 16384, v, 2 * g)) = pack8g(&x[0]);
      *reinterpret_cast<uint4*>(swq(s.DHb + half * 16384, v, 2 * g + 1)) = pack8g(&x[8]);
#pragma unroll
      for (int e = 0; e < 16; ++e) x[e] *= d.GL[64 * half + 16 * g + e];
      umma::tmem_st16(tq + C_H + 64 * half + 16 * g, x);
    }
    umma::tmem_st_wait();
    fence_proxy_async();
    KDA_DBG_CLOCK(dbg, 42);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 43);

    // ---- products 1: dv_new^T = dO^T Aqk + dhT kg^T ---------------------------------------------------------------------
    if (tid == 0) {
      const uint32_t aDO = smem_u32(d.dO), aAQ = smem_u32(d.AQK), aDH = smem_u32(s.DHb), aKG = smem_u32(d.KG);
      constexpr uint32_t idA = umma::instr_desc(128, 64, true, true);      // A = dO (rows t, two spans of 64 v), B = Aqk (rows t)
      constexpr uint32_t idB = umma::instr_desc(128, 64, false, false);    // A = dhT (K-major), B = kg (rows j, K-major)
      const uint64_t dDO = umma::smem_desc(aDO, 8192, umma::ATOM_BYTES), dAQ = umma::smem_desc(aAQ, 8192, umma::ATOM_BYTES);
      const uint64_t dH0 = umma::desc_kmajor(aDH, 0), dH1 = umma::desc_kmajor(aDH + 16384, 0);
      const uint64_t dK0 = umma::desc_kmajor(aKG, 0), dK1 = umma::desc_kmajor(aKG + 8192, 0);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK)
        umma::mma_ss(tb + C_VN, dDO + static_cast<uint64_t>(sK) * 128u, dAQ + static_cast<uint64_t>(sK) * 128u, idA, sK > 0);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t o2 = static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss(tb + C_VN, ((sK >> 2) ? dH1 : dH0) + o2, ((sK >> 2) ? dK1 : dK0) + o2, idB, 1);
      }
      umma::commit(&s.barM);
      bulk_s2g(p.DH + tile * TILE_VK, s.DHb, TILE_VK);       // the bf16 image of dh' is the chunk's DH tile
      bulk_commit();
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 44);

    // ---- epilogue 1: dv_new^T -> bf16 tile -----------------------------------------------------------------------------------
    if (alive) {
      float x[16], y[16];
      umma::tmem_ld16(tq + C_VN + 32 * half, x);
      umma::tmem_ld16(tq + C_VN + 32 * half + 16, y);
      umma::tmem_ld_wait();
      *reinterpret_cast<uint4*>(swq(s.DVNT, v, 4 * half)) = pack8g(&x[0]);
      *reinterpret_cast<uint4*>(swq(s.DVNT, v, 4 * half + 1)) = pack8g(&x[8]);
      *reinterpret_cast<uint4*>(swq(s.DVNT, v, 4 * half + 2)) = pack8g(&y[0]);
      *reinterpret_cast<uint4*>(swq(s.DVNT, v, 4 * half + 3)) = pack8g(&y[8]);
    }
    fence_proxy_async();
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 8u);
      break;
    }
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 45);

    // ---- products 2: dhT += dO^T qg - dv_new^T w ------------------------------------------------------------------------------
    if (tid == 0) {
      const uint32_t aDO = smem_u32(d.dO), aQG = smem_u32(d.QG), aDV = smem_u32(s.DVNT), aW = smem_u32(d.W);
      constexpr uint32_t idQ = umma::instr_desc(128, 128, true, true);                   // A = dO rows t, B = qg rows t (two spans of 64 k)
      constexpr uint32_t idW = umma::instr_desc(128, 128, false, true, false, true);     // A = dv_new^T (K-major), B = -w rows j
      const uint64_t dDO = umma::smem_desc(aDO, 8192, umma::ATOM_BYTES), dQ = umma::smem_desc(aQG, 8192, umma::ATOM_BYTES);
      const uint64_t dDV = umma::desc_kmajor(aDV, 0), dW = umma::smem_desc(aW, 8192, umma::ATOM_BYTES);
      // first every dO^T qg term, then every dv_new^T w term: the order in which the sliced kernel (kda_chunk_bwd_scan_vs.cu)
      // has to add them, so that both layouts give the same bits
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) umma::mma_ss(tb + C_H, dDO + static_cast<uint64_t>(sK) * 128u, dQ + static_cast<uint64_t>(sK) * 128u, idQ, 1);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) umma::mma_ss(tb + C_H, dDV + static_cast<uint64_t>(sK) * 2u, dW + static_cast<uint64_t>(sK) * 128u, idW, 1);
      umma::commit(&s.barM);
      bulk_s2g(p.DVNEWT + tile * TILE_VT, s.DVNT, TILE_VT);
      bulk_commit();
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 46);
    if (tid == 0 && alive && i + 2 < nchunks) issue_load(i + 2);      // this stage's tiles are free again
  }

  alive = __syncthreads_and(alive);      // uniform: either every thread writes dh0 or none does
  if (alive && p.dh0) {
    umma::fence_after_sync();
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[16];
      umma::tmem_ld16(tq + C_H + 64 * half + 16 * g, x);
      umma::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 16; ++e) p.dh0[sb + static_cast<size_t>(64 * half + 16 * g + e) * VD + v] = x[e];
    }
  }
  if (tid == 0) bulk_wait<0>();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tb, 256);
}

int launch_bwd_scan_tc(const RScanParams& p, int blocks, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(TcRScanSmem)) + 1024;
  const int rc = once.run([&] { return cudaFuncSetAttribute(kda_chunk_bwd_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != KDA_OK) return rc;
  kda_chunk_bwd_scan_tc_kernel<<<blocks, RNT, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace kda
