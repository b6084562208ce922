// Forward state scan of chunked KDA on tcgen05 with the fp32 state resident in tensor memory (sm_100a).
//
// One CTA per (sequence, head) walks the sequence's chunks in order.  TMEM lane = value column v, so the state
// is held transposed, hT[v][k] (128 lanes x 128 fp32 columns), for the whole sequence.  Per chunk:
//   state pass   every thread reads its slice of hT, writes the bf16 copy that the next products use as their A
//                operand (shared memory, K-major; in training the same image is stored as the chunk's HS tile),
//                and writes hT * Gam_last back to TMEM;
//   products 1   v_part^T = hT_bf16 w^T,   o^T = hT_bf16 qg^T                          (M=128 v, N=64 t, K=128 k)
//   epilogue 1   v_new^T = u^T - v_part^T  -> bf16 tile (A operand of products 2; the chunk's VNEWT tile in training)
//   products 2   hT += v_new^T kg,   o^T += v_new^T Aqk^T                              (K = 64 tokens)
//   epilogue 2   o^T -> bf16 -> staged in shared memory -> coalesced stores of o[t][v].
// Operand tiles (W, QG, KG, AQK, UT, GL of the chunk) arrive through a 2-stage TMA bulk-copy / mbarrier ring.
#include "kda_chunk.cuh"
#include "kda_device.cuh"
#include "kda_scan.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

constexpr int SCT = 256;     // 8 compute warps: TMEM lane quadrant = warp & 3, column half = warp >> 2
constexpr int SNT = SCT + 32;  // + one warp whose first lane issues every MMA, bulk copy and bulk store: the time it spends issuing
                             // (about 75 cycles per product, 760 cycles for a stage refill) stays off the compute warps' path

struct TcScanStage {
  unsigned char W[TILE_TK], QG[TILE_TK], KG[TILE_TK], AQK[TILE_TT], UT[TILE_VT];
  float GL[KD];
  unsigned char pad[512];
};
static_assert(sizeof(TcScanStage) % 1024 == 0, "stage must keep 1024-byte alignment");
constexpr unsigned TC_STAGE_TX = 3 * TILE_TK + TILE_TT + TILE_VT + TILE_GL;

struct TcScanSmem {
  TcScanStage st[2];
  unsigned char Hb[TILE_VK];     // bf16 copy of hT: two [128 v][64 k] spans (K-major A operand; = the HS tile image)
  unsigned char VNT[TILE_VT];    // bf16 v_new^T [128 v][64 t] (K-major A operand; = the VNEWT tile image)
  __nv_bfloat16 oS[C * VD];      // o staged as [64 t][128 v]
  uint64_t full[2], barM;
  uint32_t tmem_slot;
};
static_assert(sizeof(TcScanSmem) + 1024 <= 227 * 1024, "TcScanSmem too large");

constexpr int C_H = 0, C_VN = 128, C_O = 192;      // TMEM columns; o is double buffered: C_O + 64 * (chunk & 1)

__device__ __forceinline__ uint4 pack8f(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ unsigned char* swp(unsigned char* tile, int row, int chunk) {
  return tile + row * 128 + (((chunk ^ row) & 7) << 4);
}

}  // namespace

__global__ void __launch_bounds__(SNT, 1) kda_chunk_scan_tc_kernel(const ScanParams p) {
  extern __shared__ unsigned char smem_raw[];
  TcScanSmem& s = *reinterpret_cast<TcScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, half = warp >> 2;
  const int seq = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int c_begin = p.seq_chunk_off[seq], c_end = p.seq_chunk_off[seq + 1];
  const int nchunks = c_end - c_begin;
  const long long seq_tok0 = p.cu[seq], seq_tok1 = p.cu[seq + 1];
  const int v = 32 * q4 + lane;                       // this thread's value column = TMEM lane

  if (tid == 0) {
    mbar_init(&s.full[0], 1);
    mbar_init(&s.full[1], 1);
    mbar_init(&s.barM, 1);
    fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = s.tmem_slot;
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);

  auto issue_load = [&](int i) {                      // issuing thread: operand tiles of the sequence's chunk i
    TcScanStage& d = s.st[i & 1];
    const size_t tile = static_cast<size_t>(c_begin + i) * p.H + h;
    mbar_expect_tx(&s.full[i & 1], TC_STAGE_TX);
    bulk_g2s(d.W, p.W + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.QG, p.QG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.KG, p.KG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.AQK, p.AQK + tile * TILE_TT, TILE_TT, &s.full[i & 1]);
    bulk_g2s(d.UT, p.UT + tile * TILE_VT, TILE_VT, &s.full[i & 1]);
    bulk_g2s(d.GL, p.GL + tile * TILE_GL, TILE_GL, &s.full[i & 1]);
  };
  const bool issuer = warp == 8, lead = issuer && lane == 0;
  if (lead) {
    if (nchunks > 0) issue_load(0);
    if (nchunks > 1) issue_load(1);
  }

  // initial state -> TMEM: lane v, columns k = 64 half .. +63
  if (!issuer) {
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kk = 64 * half + 16 * g + i;
        x[i] = p.h0 ? __ldg(p.h0 + sb + static_cast<size_t>(kk) * VD + v) : 0.f;
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
    TcScanStage& d = s.st[i & 1];
    const int c = c_begin + i;
    // every chunk of this CTA belongs to its one sequence: first token and length by arithmetic (a table look-up would
    // be three dependent loads on the chunk-to-chunk chain)
    struct { long long tok0; int len; } ci;
    ci.tok0 = seq_tok0 + static_cast<long long>(i) * C;
    ci.len = static_cast<int>(seq_tok1 - ci.tok0 < C ? seq_tok1 - ci.tok0 : C);
    const size_t tile = static_cast<size_t>(c) * p.H + h;
    const uint32_t to = C_O + 64 * (i & 1);
    long long* const dbg = (i == 8) ? p.dbg : nullptr;      // development aid: clocks of a steady-state chunk
    KDA_DBG_CLOCK(dbg, 32);

    if (!mbar_wait(&s.full[i & 1], (i >> 1) & 1)) alive = false;
    // the previous chunk's bulk stores must have read Hb / VNT before they are rewritten
    if (lead) bulk_wait_read<0>();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 1u);
      break;
    }
    KDA_DBG_CLOCK(dbg, 33);

    // ---- state pass: bf16 copy of hT for the products, hT *= Gam_last in TMEM ----------------------------------
    if (!issuer) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_H + 64 * half + 16 * g, x);
        umma::tmem_ld_wait();
        *reinterpret_cast<uint4*>(swp(s.Hb + half * 16384, v, 2 * g)) = pack8f(&x[0]);
        *reinterpret_cast<uint4*>(swp(s.Hb + half * 16384, v, 2 * g + 1)) = pack8f(&x[8]);
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] *= d.GL[64 * half + 16 * g + e];
        umma::tmem_st16(tq + C_H + 64 * half + 16 * g, x);
      }
      umma::tmem_st_wait();
      fence_proxy_async();
    }
    KDA_DBG_CLOCK(dbg, 34);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 35);

    // ---- products 1: the chain from chunk to chunk runs through v_part only; it goes first with its own commit, the
    // products for o execute behind it while the compute warps already turn v_part into v_new
    if (lead) {
      const uint32_t aHb = smem_u32(s.Hb), aW = smem_u32(d.W), aQG = smem_u32(d.QG);
      constexpr uint32_t id1 = umma::instr_desc(128, 64, false, false);
      const uint64_t dH0 = umma::desc_kmajor(aHb, 0), dH1 = umma::desc_kmajor(aHb + 16384, 0);
      const uint64_t dW0 = umma::desc_kmajor(aW, 0), dW1 = umma::desc_kmajor(aW + 8192, 0);
      const uint64_t dQ0 = umma::desc_kmajor(aQG, 0), dQ1 = umma::desc_kmajor(aQG + 8192, 0);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t o2 = static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss(tb + C_VN, ((sK >> 2) ? dH1 : dH0) + o2, ((sK >> 2) ? dW1 : dW0) + o2, id1, sK > 0);      // v_part^T = hT w^T
      }
      umma::commit(&s.barM);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t o2 = static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss(tb + to, ((sK >> 2) ? dH1 : dH0) + o2, ((sK >> 2) ? dQ1 : dQ0) + o2, id1, sK > 0);        // o^T = hT qg^T
      }
      if (p.HS) {                                       // training: the bf16 state image is the chunk's HS tile
        bulk_s2g(p.HS + tile * TILE_VK, s.Hb, TILE_VK);
        bulk_commit();
      }
    }
    __syncwarp();

    // ---- epilogue 1: v_new^T = u^T - v_part^T -> bf16 tile --------------------------------------------------------------
    if (!issuer) {
      if (!mbar_wait(&s.barM, mph & 1)) alive = false;
      umma::fence_after_sync();
      KDA_DBG_CLOCK(dbg, 36);
      if (alive) {
        float x[16], y[16];
        umma::tmem_ld16(tq + C_VN + 32 * half, x);
        umma::tmem_ld16(tq + C_VN + 32 * half + 16, y);
        umma::tmem_ld_wait();
#pragma unroll
        for (int cix = 0; cix < 4; ++cix) {
          const uint4 u4 = *reinterpret_cast<const uint4*>(swp(d.UT, v, 4 * half + cix));
          const uint32_t uw[4] = {u4.x, u4.y, u4.z, u4.w};
          float* src = (cix < 2) ? &x[8 * cix] : &y[8 * (cix - 2)];
          float r[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 uu = unpack_bf16(uw[e]);
            r[2 * e] = uu.x - src[2 * e];
            r[2 * e + 1] = uu.y - src[2 * e + 1];
          }
          *reinterpret_cast<uint4*>(swp(s.VNT, v, 4 * half + cix)) = pack8f(r);
        }
      }
      fence_proxy_async();
    }
    ++mph;
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 2u);
      break;
    }
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 37);

    // ---- products 2 ---------------------------------------------------------------------------------------------------
    if (lead) {
      const uint32_t aVN = smem_u32(s.VNT), aKG = smem_u32(d.KG), aAQ = smem_u32(d.AQK);
      constexpr uint32_t idH = umma::instr_desc(128, 128, false, true);      // B = kg as MN-major: rows t, two spans of 64 k
      constexpr uint32_t idO = umma::instr_desc(128, 64, false, false);
      const uint64_t dV = umma::desc_kmajor(aVN, 0), dK = umma::smem_desc(aKG, 8192, umma::ATOM_BYTES), dA = umma::desc_kmajor(aAQ, 0);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) {
        umma::mma_ss(tb + C_H, dV + static_cast<uint64_t>(sK) * 2u, dK + static_cast<uint64_t>(sK) * 128u, idH, 1);      // hT += v_new^T kg
        umma::mma_ss(tb + to, dV + static_cast<uint64_t>(sK) * 2u, dA + static_cast<uint64_t>(sK) * 2u, idO, 1);         // o^T += v_new^T Aqk^T
      }
      umma::commit(&s.barM);
      if (p.VNEWT) {
        bulk_s2g(p.VNEWT + tile * TILE_VT, s.VNT, TILE_VT);
        bulk_commit();
      }
    }
    __syncwarp();
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 38);
    if (issuer) {
      // this stage's operand tiles are free: fetch chunk i + 2 into it (the compute warps do not wait for this)
      if (lead && alive && i + 2 < nchunks) issue_load(i + 2);
      __syncwarp();
      continue;
    }

    // ---- epilogue 2 (compute warps): o^T -> bf16 -> staged [t][v] -> coalesced rows --------------------------------------
    if (alive) {
      float x[16], y[16];
      umma::tmem_ld16(tq + to + 32 * half, x);
      umma::tmem_ld16(tq + to + 32 * half + 16, y);
      umma::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        s.oS[(32 * half + e) * VD + v] = __float2bfloat16_rn(x[e]);
        s.oS[(32 * half + 16 + e) * VD + v] = __float2bfloat16_rn(y[e]);
      }
    }
    umma::fence_before_sync();
    asm volatile("bar.sync 1, 256;" ::: "memory");      // the eight compute warps only
    for (int e = tid; e < C * 16; e += SCT) {
      const int r = e >> 4, pc = e & 15;
      if (r < ci.len)
        *reinterpret_cast<uint4*>(p.o + (static_cast<size_t>(ci.tok0 + r) * p.H + h) * VD + pc * 8) =
            *reinterpret_cast<const uint4*>(&s.oS[r * VD + pc * 8]);
    }
    // (the next iteration's first barrier orders these reads of oS before it is rewritten)
    KDA_DBG_CLOCK(dbg, 39);
  }
  alive = __syncthreads_and(alive);

  // final state
  if (alive && p.ht && !issuer) {
    umma::fence_after_sync();
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float x[16];
      umma::tmem_ld16(tq + C_H + 64 * half + 16 * g, x);
      umma::tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 16; ++e) p.ht[sb + static_cast<size_t>(64 * half + 16 * g + e) * VD + v] = x[e];
    }
  }
  if (lead) bulk_wait<0>();              // outstanding bulk stores read shared memory that dies with the CTA
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tb, 512);
}

int launch_scan_tc(const ScanParams& p, int blocks, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(TcScanSmem)) + 1024;
  const int rc = once.run([&] { return cudaFuncSetAttribute(kda_chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != KDA_OK) return rc;
  kda_chunk_scan_tc_kernel<<<blocks, SNT, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace kda
