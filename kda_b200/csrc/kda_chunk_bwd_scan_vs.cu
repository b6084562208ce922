// Reverse state scan of chunked KDA for FEW (sequence, head) units: several CTAs per unit, one per slice of the value
// columns (sm_100a, tcgen05 + TMEM).  The counterpart of kda_chunk_scan_vs.cu for the backward.
//
// A unit is cut into 128 / VS slices of VS value columns (VS = 32: four slices); each CTA walks the unit's chunks from the last
// to the first with its slice of the state gradient in tensor memory, TMEM lane = KEY row k: dh[k][v].  Per chunk:
//   state pass   thread k writes its VS/2 columns of dh as bf16 into row k of DHb ([128 k][VS v], MN-major B operand;
//                transposed into the chunk's DH tile rows beside the products) and scales the fp32 copy by Gam_last[k];
//   products 1   dv_new[t][v] = Aqk[:][t] dO[:][v] + kg[t][:] dh[:][v]                   (M=64 t, N=VS, K=64 + 128)
//   epilogue 1   dv_new -> bf16 rows of DVN ([64 t][VS v], MN-major B operand; transposed into the DVNEWT tile rows)
//   products 2   dh[k][v] += qg[:][k] dO[:][v] - w[:][k] dv_new[:][v]                    (M=128 k, N=VS, K=64 t)
// The halves of the products that do not depend on the step's own results (Aqk^T dO; qg^T dO) are issued early, so that
// the chain carries only kg dh (eight products) and w^T dv_new (four).
// dO arrives by a tiled TMA load of the 64-column box that holds the slice (128-byte swizzled rows t: an MN-major B
// operand as it lands); W, QG, KG, AQK, GL are the tiles the forward left.  DH and DVNEWT keep the [v][k] / [v][t]
// formats of the one-CTA kernel, so the per-chunk backward reads them unchanged.
#include "kda_chunk_bwd.cuh"
#include "kda_device.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

// warps: 0..7 compute (TMEM lane quadrant = warp & 3, column half = warp >> 2), 8 issues the products, 9 refills the
// operand stages, 10 stores the DH / DVNEWT rows.  As in the forward kernel the loops hold no CTA-wide barrier: every
// hand-over is an mbarrier with a bounded wait, so the issuing thread carries nothing but the chain's products.
constexpr int RVS_WARPS = 11;
constexpr int RVS_THREADS = RVS_WARPS * 32;
constexpr int RW_ISSUE = 8, RW_LOAD = 9, RW_STORE = 10;

struct RvsStage {
  unsigned char W[TILE_TK], QG[TILE_TK], KG[TILE_TK], AQK[TILE_TT];
  unsigned char dO[TILE_TT];             // [64 t][64 v]: the 64-column box of dO that holds the slice
  float GL[KD];
  unsigned char pad[1024 - TILE_GL];
};
static_assert(sizeof(RvsStage) % 1024 == 0, "stage must keep 1024-byte alignment");
constexpr unsigned RVS_STAGE_TX = 3 * TILE_TK + 2 * TILE_TT + TILE_GL;

template <int VS>
struct RvsSmem {
  RvsStage st[2];
  unsigned char DHb[KD * 128];           // bf16 dh: [128 k] rows of 128 bytes, the first VS columns in use
  unsigned char DVN[C * 128];            // bf16 dv_new: [64 t] rows of 128 bytes, the first VS columns in use
  unsigned char DHst[2 * VS * 128];      // rows v of the slice of the DH tile, two spans of [VS v][64 k]
  unsigned char DVNTst[VS * 128];        // rows v of the slice of the DVNEWT tile, [VS v][64 t]
  uint64_t full[2], stageFree[2];        // operand stage loaded / every product that reads it complete
  uint64_t stReady, vnReady;             // compute warps -> issuing thread: DHb resp. DVN written (8 arrivals)
  uint64_t barM;                         // products 1 / products 2 complete (alternating phases)
  uint64_t sgReady, sgFree;              // staging tiles written (8 arrivals) / stored (1 arrival)
  uint32_t tmem_slot;
  volatile int dead;
};

__device__ __forceinline__ uint4 pack8r(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ unsigned char* rpiece(unsigned char* tile, int row, int pc) {
  return tile + row * 128 + (((pc ^ row) & 7) << 4);
}
__device__ __forceinline__ void rstore_bf16_at(unsigned char* tile, int row, int col, uint32_t packed_pair, int which) {
  *reinterpret_cast<uint16_t*>(tile + umma::sw128(row, col)) = static_cast<uint16_t>(which ? (packed_pair >> 16) : (packed_pair & 0xffffu));
}
__device__ __forceinline__ bool rwarp_wait(uint64_t* bar, unsigned parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); }
__device__ __forceinline__ void rwarp_arrive(uint64_t* bar, int lane) {
  umma::fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

}  // namespace

template <int VS>
__global__ void __launch_bounds__(RVS_THREADS, 1) kda_chunk_bwd_scan_vs_kernel(const __grid_constant__ RScanParams p) {
  constexpr int NS = VD / VS;
  constexpr int HC = VS / 2;
  constexpr int C_H = 0, C_VN = VS;      // TMEM columns
  constexpr uint32_t TM_COLS = 2 * VS < 32 ? 32 : 2 * VS;
  extern __shared__ unsigned char smem_raw[];
  RvsSmem<VS>& s = *reinterpret_cast<RvsSmem<VS>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, half = (warp >> 2) & 1;
  const int unit = blockIdx.x / NS, slice = blockIdx.x % NS;
  const int seq = unit / p.H, h = unit % p.H;
  const int c_begin = p.seq_chunk_off[seq], c_end = p.seq_chunk_off[seq + 1];
  const int nchunks = c_end - c_begin;
  const long long seq_tok0 = p.cu[seq];
  const int k = 32 * q4 + lane;          // compute thread: its key row = TMEM lane of the state gradient
  const int t = 16 * q4 + lane;          // lanes 0..15 of a quadrant hold rows 16 q4 .. of an M = 64 accumulator
  const int v0 = VS * slice;             // first value column of the slice
  const int box0 = (v0 / 64) * 64;       // first column of the 64-column dO box that holds the slice
  const uint32_t n_off = static_cast<uint32_t>(v0 - box0) * 2u;      // byte offset of the slice inside the box's 128-byte rows

  if (tid == 0) {
    mbar_init(&s.full[0], 1);
    mbar_init(&s.full[1], 1);
    mbar_init(&s.stageFree[0], 1);
    mbar_init(&s.stageFree[1], 1);
    mbar_init(&s.stReady, 8);
    mbar_init(&s.vnReady, 8);
    mbar_init(&s.barM, 1);
    mbar_init(&s.sgReady, 8);
    mbar_init(&s.sgFree, 1);
    s.dead = 0;
    fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, TM_COLS);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = s.tmem_slot;
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);

  auto issue_load = [&](int i) {                      // one thread: step i handles chunk c_end - 1 - i
    RvsStage& d = s.st[i & 1];
    const int c = c_end - 1 - i;
    const size_t tile = static_cast<size_t>(c) * p.H + h;
    const long long tok0 = seq_tok0 + static_cast<long long>(c - c_begin) * C;
    mbar_expect_tx(&s.full[i & 1], RVS_STAGE_TX);
    bulk_g2s(d.AQK, p.AQK + tile * TILE_TT, TILE_TT, &s.full[i & 1]);
    tma_load_rows(d.dO, &p.tm_do, box0, h, static_cast<int>(tok0), &s.full[i & 1]);
    bulk_g2s(d.GL, p.GL + tile * TILE_GL, TILE_GL, &s.full[i & 1]);
    bulk_g2s(d.KG, p.KG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.QG, p.QG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.W, p.W + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
  };
  if (warp == RW_LOAD && lane == 0) {
    if (nchunks > 0) issue_load(0);
    if (nchunks > 1) issue_load(1);
  }

  if (warp < 8) {                                     // gradient w.r.t. the final state -> TMEM: lane k, the slice's columns
    const size_t sb = ((static_cast<size_t>(seq) * p.H + h) * KD + k) * VD + v0 + HC * half;
#pragma unroll
    for (int g = 0; g < HC / 16; ++g) {
      float x[16];
#pragma unroll
      for (int e = 0; e < 16; e += 4) {
        const float4 f = p.d_ht ? __ldg(reinterpret_cast<const float4*>(p.d_ht + sb + 16 * g + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[e] = f.x; x[e + 1] = f.y; x[e + 2] = f.z; x[e + 3] = f.w;
      }
      umma::tmem_st16(tq + C_H + HC * half + 16 * g, x);
    }
    umma::tmem_st_wait();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();

  if (warp < 8) {
    // ================= compute warps: the chain =================
    bool ok = true;
    for (int i = 0; i < nchunks && ok; ++i) {
      RvsStage& d = s.st[i & 1];
      if (__any_sync(0xffffffffu, s.dead != 0)) break;
      if (!rwarp_wait(&s.full[i & 1], (i >> 1) & 1)) { ok = false; break; }      // GL is there

      // ---- state pass ---------------------------------------------------------------------------------------------------
      uint4 hp[HC / 8];                                  // this thread's bf16 values of dh (kept for the DH tile)
      {
        const float gl = d.GL[k];
#pragma unroll
        for (int g = 0; g < HC / 16; ++g) {
          float x[16];
          umma::tmem_ld16(tq + C_H + HC * half + 16 * g, x);
          umma::tmem_ld_wait();
          hp[2 * g] = pack8r(&x[0]);
          hp[2 * g + 1] = pack8r(&x[8]);
          *reinterpret_cast<uint4*>(rpiece(s.DHb, k, (HC * half) / 8 + 2 * g)) = hp[2 * g];
          *reinterpret_cast<uint4*>(rpiece(s.DHb, k, (HC * half) / 8 + 2 * g + 1)) = hp[2 * g + 1];
#pragma unroll
          for (int e = 0; e < 16; ++e) x[e] *= gl;
          umma::tmem_st16(tq + C_H + HC * half + 16 * g, x);
        }
        umma::tmem_st_wait();
        fence_proxy_async();
      }
      rwarp_arrive(&s.stReady, lane);

      // ---- beside products 1: dh transposed into the DH staging tile ------------------------------------------------------
      if (i > 0 && !rwarp_wait(&s.sgFree, (i - 1) & 1)) { ok = false; break; }      // the previous step's rows have been stored
#pragma unroll
      for (int e = 0; e < HC / 8; ++e) {
        const uint32_t wds[4] = {hp[e].x, hp[e].y, hp[e].z, hp[e].w};
#pragma unroll
        for (int j = 0; j < 8; ++j)                      // element (v, k) of the slice's rows of span k / 64
          rstore_bf16_at(s.DHst + (k >> 6) * (VS * 128), HC * half + 8 * e + j, k & 63, wds[j >> 1], j & 1);
      }

      // ---- epilogue 1: dv_new -> bf16 rows of DVN (the loads are warp-wide; lanes 16..31 hold no row) --------------------
      if (!rwarp_wait(&s.barM, 0)) { ok = false; break; }
      umma::fence_after_sync();
      uint4 vp[HC / 8];                                  // this thread's bf16 dv_new values (kept for the DVNEWT tile)
#pragma unroll
      for (int g = 0; g < HC / 16; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_VN + HC * half + 16 * g, x);
        umma::tmem_ld_wait();
        vp[2 * g] = pack8r(&x[0]);
        vp[2 * g + 1] = pack8r(&x[8]);
        if (lane < 16) {
          *reinterpret_cast<uint4*>(rpiece(s.DVN, t, (HC * half) / 8 + 2 * g)) = vp[2 * g];
          *reinterpret_cast<uint4*>(rpiece(s.DVN, t, (HC * half) / 8 + 2 * g + 1)) = vp[2 * g + 1];
        }
      }
      fence_proxy_async();
      rwarp_arrive(&s.vnReady, lane);

      // ---- beside products 2: dv_new transposed into the DVNEWT staging tile ---------------------------------------------
      if (lane < 16) {
#pragma unroll
        for (int e = 0; e < HC / 8; ++e) {
          const uint32_t wds[4] = {vp[e].x, vp[e].y, vp[e].z, vp[e].w};
#pragma unroll
          for (int j = 0; j < 8; ++j) rstore_bf16_at(s.DVNTst, HC * half + 8 * e + j, t, wds[j >> 1], j & 1);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.sgReady);
      if (!rwarp_wait(&s.barM, 1)) { ok = false; break; }      // products 2 complete
      umma::fence_after_sync();
    }
    if (!ok) s.dead = 1;
    if (__any_sync(0xffffffffu, s.dead != 0)) {
      if (lane == 0) atomicOr(p.status, KDA_STATUS_BWD_SCAN_MMA_WAIT);
    } else if (p.dh0) {
      const size_t sb = ((static_cast<size_t>(seq) * p.H + h) * KD + k) * VD + v0 + HC * half;
#pragma unroll
      for (int g = 0; g < HC / 16; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_H + HC * half + 16 * g, x);
        umma::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 4)
          *reinterpret_cast<float4*>(p.dh0 + sb + 16 * g + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
      }
    }
  } else if (warp == RW_ISSUE) {
    // ================= the issuing thread: nothing but products =================
    if (lane == 0) {
      constexpr uint32_t idA = umma::instr_desc(64, VS, true, true);      // A = Aqk rows j (columns t: MN-major), B = dO rows j
      constexpr uint32_t idB = umma::instr_desc(64, VS, false, true);     // A = kg rows t (K-major), B = dh rows k
      constexpr uint32_t idQ = umma::instr_desc(128, VS, true, true);     // A = qg rows t, two spans of 64 k; B = dO rows t
      constexpr uint32_t idW = umma::instr_desc(128, VS, true, true, false, true);      // A = w rows t; B = -dv_new rows t
      const uint64_t dDH = umma::desc_mnmajor(smem_u32(s.DHb), 0, 16384u), dDV = umma::desc_mnmajor(smem_u32(s.DVN), 0, 16384u);
      bool ok = true;
      for (int i = 0; i < nchunks; ++i) {
        RvsStage& d = s.st[i & 1];
        const uint64_t dDO = umma::desc_mnmajor(smem_u32(d.dO) + n_off, 0, 8192u), dAQ = umma::desc_mnmajor(smem_u32(d.AQK), 0, 8192u);
        const uint64_t dKG = umma::desc_kmajor(smem_u32(d.KG), 0);
        const uint64_t dQG = umma::desc_mnmajor(smem_u32(d.QG), 0, 8192u), dW = umma::desc_mnmajor(smem_u32(d.W), 0, 8192u);
        if (s.dead) break;
        if (!mbar_wait(&s.full[i & 1], (i >> 1) & 1)) { ok = false; break; }
        // products 1, the part that does not need the state: dv_new = Aqk^T dO (the accumulator was read by the previous
        // step's epilogue, whose hand-over this thread has waited for)
        umma::mma4<umma::KSTEP_MNMAJOR, umma::KSTEP_MNMAJOR>(tb + C_VN, dAQ, dDO, idA, 0);
        if (!mbar_wait(&s.stReady, i & 1)) { ok = false; break; }
        umma::fence_after_sync();
        // products 1: dv_new += kg dh
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(tb + C_VN, dKG, dDH, idB, 1);
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(tb + C_VN, dKG + 512u, dDH + 4u * umma::KSTEP_MNMAJOR, idB, 1);
        umma::commit(&s.barM);
        // products 2, the part that does not need dv_new: dh += qg^T dO (the state has been scaled: stReady)
        umma::mma4<umma::KSTEP_MNMAJOR, umma::KSTEP_MNMAJOR>(tb + C_H, dQG, dDO, idQ, 1);
        if (!mbar_wait(&s.vnReady, i & 1)) { ok = false; break; }
        umma::fence_after_sync();
        // products 2: dh -= w^T dv_new
        umma::mma4<umma::KSTEP_MNMAJOR, umma::KSTEP_MNMAJOR>(tb + C_H, dW, dDV, idW, 1);
        umma::commit(&s.barM);
        umma::commit(&s.stageFree[i & 1]);
      }
      if (!ok) {
        s.dead = 1;
        atomicOr(p.status, KDA_STATUS_BWD_SCAN_MMA_WAIT);
      }
    }
    __syncwarp();
  } else if (warp == RW_LOAD) {
    if (lane == 0) {
      for (int i = 0; i + 2 < nchunks; ++i) {
        if (s.dead) break;
        if (!mbar_wait(&s.stageFree[i & 1], (i >> 1) & 1)) {
          s.dead = 1;
          atomicOr(p.status, KDA_STATUS_BWD_SCAN_LOAD_WAIT);
          break;
        }
        issue_load(i + 2);
      }
    }
    __syncwarp();
  } else if (warp == RW_STORE) {
    if (lane == 0) {
      for (int i = 0; i < nchunks; ++i) {
        const size_t tile = static_cast<size_t>(c_end - 1 - i) * p.H + h;
        if (s.dead) break;
        if (!mbar_wait(&s.sgReady, i & 1)) {
          s.dead = 1;
          break;
        }
        bulk_s2g(p.DH + tile * TILE_VK + static_cast<size_t>(v0) * 128, s.DHst, VS * 128);
        bulk_s2g(p.DH + tile * TILE_VK + 16384 + static_cast<size_t>(v0) * 128, s.DHst + VS * 128, VS * 128);
        bulk_s2g(p.DVNEWT + tile * TILE_VT + static_cast<size_t>(v0) * 128, s.DVNTst, VS * 128);
        bulk_commit();
        bulk_wait_read<0>();                             // the staging tiles may be rewritten
        mbar_arrive(&s.sgFree);
      }
      bulk_wait<0>();                                    // the stores read shared memory that dies with the CTA
    }
    __syncwarp();
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tb, TM_COLS);
}

template <int VS>
static int launch_rvs(const RScanParams& p, int units, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(RvsSmem<VS>)) + 1024;
  const int rc = once.run([&] { return cudaFuncSetAttribute(kda_chunk_bwd_scan_vs_kernel<VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != KDA_OK) return rc;
  kda_chunk_bwd_scan_vs_kernel<VS><<<units * (VD / VS), RVS_THREADS, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int launch_bwd_scan_vs(const RScanParams& p, int units, cudaStream_t st) { return launch_rvs<32>(p, units, st); }

}  // namespace kda
