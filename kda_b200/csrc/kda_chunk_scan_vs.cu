// Forward state scan of chunked KDA for FEW (sequence, head) units: several CTAs per unit, one per slice of the value
// columns (sm_100a, tcgen05 + TMEM).
//
// The recurrence is independent per value column, and the time of a scan with fewer units than SMs is set by the
// chunk-to-chunk chain of one CTA.  Here a unit is cut into 128 / VS slices of VS value columns (VS = 32: four slices), each
// walked by its own CTA, and the state is held the other way round than in the one-CTA-per-unit kernel: TMEM lane =
// KEY row k, columns = the slice's value columns, h[k][v].  That makes every product's N dimension the slice width, so
// the state pass and the epilogue of a chunk shrink with the slice.  Per chunk:
//   state pass   thread k reads its VS/2 columns of h, writes them as bf16 into row k of Hb (a [128 k][VS v] tile, the
//                MN-major B operand of products 1) and scales the fp32 copy by Gam_last[k] (one scalar per thread);
//   products 1   v_part[t][v] = w[t][:] h[:][v]                                               (M=64 t, N=VS, K=128 k)
//   epilogue 1   v_new[t][v] = u[t][v] - v_part[t][v] -> bf16 rows of VN ([64 t][VS v], MN-major B of products 2)
//   products 2   h[k][v] += kg[:][k] v_new[:][v]                                              (M=128 k, N=VS, K=64 t)
//   beside them  o[t][v] = qg[t][:] h[:][v] + Aqk[t][:] v_new[:][v]  (issued behind products 1 resp. 2, so that they
//                execute while the compute warps are busy), read out of a double-buffered accumulator by four extra warps.
// What the chain costs is mostly fixed latency: a small tcgen05.mma issues every ~56 cycles whatever its shape, and every
// hand-over between the compute warps and the issuing thread costs a barrier round trip.  So the chain carries nothing
// but its own twelve products: the issuing thread does nothing else (the compute warps signal it through mbarriers and
// never wait for it at a CTA barrier), operand tiles are refilled by a read-out warp, tile stores by a warp of their own.
// The operand tiles (W, QG, KG, AQK, GL and the slice's rows of UT) are the ones the prepare kernel writes for the
// one-CTA kernel; the second and later slices of a unit find them in L2.  In training the chunk's HS and VNEWT tiles
// are written in the same [v][k] / [v][t] formats as by the one-CTA kernel (the per-chunk backward reads them): the
// threads transpose their bf16 values into staging tiles with 2-byte stores while the products execute.
// Every sum is formed in the same order as in the one-CTA kernel, so both give the same bits.
#include "kda_chunk.cuh"
#include "kda_device.cuh"
#include "kda_scan.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

// warps: 0..7 compute (TMEM lane quadrant = warp & 3, column half = warp >> 2), 8 issues the products, 9..12 read o out
// (quadrant = warp & 3; warp 12 also refills the operand stages), 13 stores the HS / VNEWT rows
constexpr int VS_WARPS = 14;
constexpr int VS_THREADS = VS_WARPS * 32;
constexpr int W_ISSUE = 8, W_READ0 = 9, W_LOAD = 12, W_STORE = 13;

template <int VS>
struct VsStage {
  unsigned char W[TILE_TK], QG[TILE_TK], KG[TILE_TK], AQK[TILE_TT];
  unsigned char UT[VS * 128];            // rows v of the slice of the chunk's UT tile ([128 v][64 t])
  float GL[KD];
  unsigned char pad[1024 - TILE_GL];
};

template <int VS>
struct VsSmem {
  VsStage<VS> st[2];
  unsigned char Hb[KD * 128];            // bf16 h: [128 k] rows of 128 bytes, the first VS columns in use
  unsigned char VN[C * 128];             // bf16 v_new: [64 t] rows of 128 bytes, the first VS columns in use
  unsigned char HSst[2 * VS * 128];      // training: rows v of the slice of the HS tile, two spans of [VS v][64 k]
  unsigned char VNTst[VS * 128];         // training: rows v of the slice of the VNEWT tile, [VS v][64 t]
  uint64_t full[2];                      // operand stage loaded (bulk copies)
  uint64_t stReady, vnReady;             // compute warps -> issuing thread: Hb resp. VN written (8 arrivals, one per warp)
  uint64_t barM;                         // products 1 / products 2 complete (alternating phases)
  uint64_t barO[2], oFree[2];            // o accumulator complete (this also frees the operand stage) / read out (4 arrivals)
  uint64_t sgReady, sgFree;              // staging tiles written (8 arrivals) / stored (1 arrival)
  uint32_t tmem_slot;
  volatile int dead;                     // a bounded wait gave up somewhere: everybody leaves at the next look
};

template <int VS>
constexpr unsigned VS_STAGE_TX = 3 * TILE_TK + TILE_TT + VS * 128 + TILE_GL;

__device__ __forceinline__ uint4 pack8v(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ unsigned char* piece(unsigned char* tile, int row, int pc) {      // 16-byte piece pc of a 128-byte row
  return tile + row * 128 + (((pc ^ row) & 7) << 4);
}
__device__ __forceinline__ void store_bf16_at(unsigned char* tile, int row, int col, uint32_t packed_pair, int which) {
  *reinterpret_cast<uint16_t*>(tile + umma::sw128(row, col)) = static_cast<uint16_t>(which ? (packed_pair >> 16) : (packed_pair & 0xffffu));
}
// A wait whose answer is the same for every lane of the warp (the tensor-memory loads and stores behind it need all 32).
__device__ __forceinline__ bool warp_wait(uint64_t* bar, unsigned parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity)); }
// one arrival per warp, after every lane's shared-memory and tensor-memory writes
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  umma::fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

}  // namespace

template <int VS>
__global__ void __launch_bounds__(VS_THREADS, 1) kda_chunk_scan_vs_kernel(const ScanParams p) {
  constexpr int NS = VD / VS;            // slices (CTAs) per unit
  constexpr int HC = VS / 2;             // columns per compute thread (two column halves)
  constexpr int C_H = 0, C_VN = VS, C_O = 2 * VS;      // TMEM columns; o double buffered: C_O + VS * (chunk & 1)
  extern __shared__ unsigned char smem_raw[];
  VsSmem<VS>& s = *reinterpret_cast<VsSmem<VS>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, half = (warp >> 2) & 1;
  const int unit = blockIdx.x / NS, slice = blockIdx.x % NS;
  const int seq = unit / p.H, h = unit % p.H;
  const int c_begin = p.seq_chunk_off[seq], c_end = p.seq_chunk_off[seq + 1];
  const int nchunks = c_end - c_begin;
  const long long seq_tok0 = p.cu[seq], seq_tok1 = p.cu[seq + 1];
  const int k = 32 * q4 + lane;          // compute thread: its key row = TMEM lane of the state
  const int t = 16 * q4 + lane;          // lanes 0..15 of a quadrant hold rows 16 q4 .. of an M = 64 accumulator
  const int v0 = VS * slice;             // first value column of the slice
  const bool save = p.HS != nullptr;

  if (tid == 0) {
    mbar_init(&s.full[0], 1);
    mbar_init(&s.full[1], 1);
    mbar_init(&s.stReady, 8);
    mbar_init(&s.vnReady, 8);
    mbar_init(&s.barM, 1);
    mbar_init(&s.barO[0], 1);
    mbar_init(&s.barO[1], 1);
    mbar_init(&s.oFree[0], 4);
    mbar_init(&s.oFree[1], 4);
    mbar_init(&s.sgReady, 8);
    mbar_init(&s.sgFree, 1);
    s.dead = 0;
    fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, 4 * VS);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = s.tmem_slot;
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);

  auto issue_load = [&](int i) {                      // one thread: operand tiles of the sequence's chunk i
    VsStage<VS>& d = s.st[i & 1];
    const size_t tile = static_cast<size_t>(c_begin + i) * p.H + h;
    mbar_expect_tx(&s.full[i & 1], VS_STAGE_TX<VS>);
    bulk_g2s(d.W, p.W + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.KG, p.KG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.UT, p.UT + tile * TILE_VT + static_cast<size_t>(v0) * 128, VS * 128, &s.full[i & 1]);
    bulk_g2s(d.GL, p.GL + tile * TILE_GL, TILE_GL, &s.full[i & 1]);
    bulk_g2s(d.QG, p.QG + tile * TILE_TK, TILE_TK, &s.full[i & 1]);
    bulk_g2s(d.AQK, p.AQK + tile * TILE_TT, TILE_TT, &s.full[i & 1]);
  };
  if (warp == W_LOAD && lane == 0) {
    if (nchunks > 0) issue_load(0);
    if (nchunks > 1) issue_load(1);
  }

  // initial state -> TMEM: lane k, the slice's columns
  if (warp < 8) {
    const size_t sb = ((static_cast<size_t>(seq) * p.H + h) * KD + k) * VD + v0 + HC * half;
#pragma unroll
    for (int g = 0; g < HC / 16; ++g) {
      float x[16];
#pragma unroll
      for (int e = 0; e < 16; e += 4) {
        const float4 f = p.h0 ? __ldg(reinterpret_cast<const float4*>(p.h0 + sb + 16 * g + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
        x[e] = f.x; x[e + 1] = f.y; x[e + 2] = f.z; x[e + 3] = f.w;
      }
      umma::tmem_st16(tq + C_H + HC * half + 16 * g, x);
    }
    umma::tmem_st_wait();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();

  // No CTA-wide barrier inside the loops below: every hand-over is an mbarrier with a bounded wait, a thread whose wait
  // gave up raises s.dead and leaves, and the others follow at their next look (or when their own wait runs out).
  if (warp < 8) {
    // ================= compute warps: the chain =================
    bool ok = nchunks == 0 || warp_wait(&s.full[0], 0);      // the first chunk's GL and UT rows are there
    float gl = (ok && nchunks > 0) ? s.st[0].GL[k] : 0.f;    // Gam_last[k] of the current chunk (read one chunk ahead, see below)
    for (int i = 0; i < nchunks && ok; ++i) {
      VsStage<VS>& d = s.st[i & 1];
      long long* const dbg = (i == 8) ? p.dbg : nullptr;      // development aid: clocks of a steady-state chunk
      KDA_DBG_CLOCK(dbg, 48);
      KDA_DBG_CLOCK(dbg, 49);

      // ---- state pass ---------------------------------------------------------------------------------------------------
      uint4 hp[HC / 8];                                  // this thread's bf16 state values (kept for the HS tile)
      {
#pragma unroll
        for (int g = 0; g < HC / 16; ++g) {
          float x[16];
          umma::tmem_ld16(tq + C_H + HC * half + 16 * g, x);
          umma::tmem_ld_wait();
          hp[2 * g] = pack8v(&x[0]);
          hp[2 * g + 1] = pack8v(&x[8]);
          *reinterpret_cast<uint4*>(piece(s.Hb, k, (HC * half) / 8 + 2 * g)) = hp[2 * g];
          *reinterpret_cast<uint4*>(piece(s.Hb, k, (HC * half) / 8 + 2 * g + 1)) = hp[2 * g + 1];
#pragma unroll
          for (int e = 0; e < 16; ++e) x[e] *= gl;
          umma::tmem_st16(tq + C_H + HC * half + 16 * g, x);
        }
        umma::tmem_st_wait();
        fence_proxy_async();
      }
      warp_arrive(&s.stReady, lane);
      KDA_DBG_CLOCK(dbg, 50);

      // ---- beside products 1: u of this thread's row; the state values transposed into the HS staging tile -----------------
      uint32_t up[HC / 2];                               // u[t][HC half ..] as bf16 pairs (rows t exist in lanes 0..15)
#pragma unroll
      for (int e = 0; e < HC / 2; ++e) {
        uint32_t lo = 0, hi = 0;
        if (lane < 16) {
          lo = *reinterpret_cast<const uint16_t*>(d.UT + umma::sw128(HC * half + 2 * e, t));
          hi = *reinterpret_cast<const uint16_t*>(d.UT + umma::sw128(HC * half + 2 * e + 1, t));
        }
        up[e] = lo | (hi << 16);
      }
      if (save) {
        if (i > 0 && !warp_wait(&s.sgFree, (i - 1) & 1)) { ok = false; break; }      // the previous chunk's rows have been stored
#pragma unroll
        for (int e = 0; e < HC / 8; ++e) {
          const uint32_t wds[4] = {hp[e].x, hp[e].y, hp[e].z, hp[e].w};
#pragma unroll
          for (int j = 0; j < 8; ++j)                    // element (v, k) of the slice's rows of span k / 64
            store_bf16_at(s.HSst + (k >> 6) * (VS * 128), HC * half + 8 * e + j, k & 63, wds[j >> 1], j & 1);
        }
      }
      KDA_DBG_CLOCK(dbg, 51);

      // ---- epilogue 1: v_new = u - v_part -> bf16 rows of VN (the loads are warp-wide; lanes 16..31 hold no row) ----------
      if (!warp_wait(&s.barM, 0)) { ok = false; break; }
      umma::fence_after_sync();
      KDA_DBG_CLOCK(dbg, 52);
      uint4 vp[HC / 8];                                  // this thread's bf16 v_new values (kept for the VNEWT tile)
#pragma unroll
      for (int g = 0; g < HC / 16; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_VN + HC * half + 16 * g, x);
        umma::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 uu = unpack_bf16(up[8 * g + e]);
          x[2 * e] = uu.x - x[2 * e];
          x[2 * e + 1] = uu.y - x[2 * e + 1];
        }
        vp[2 * g] = pack8v(&x[0]);
        vp[2 * g + 1] = pack8v(&x[8]);
        if (lane < 16) {
          *reinterpret_cast<uint4*>(piece(s.VN, t, (HC * half) / 8 + 2 * g)) = vp[2 * g];
          *reinterpret_cast<uint4*>(piece(s.VN, t, (HC * half) / 8 + 2 * g + 1)) = vp[2 * g + 1];
        }
      }
      fence_proxy_async();
      warp_arrive(&s.vnReady, lane);
      KDA_DBG_CLOCK(dbg, 53);

      // ---- beside products 2: v_new transposed into the VNEWT staging tile ------------------------------------------------
      if (save) {
        if (lane < 16) {
#pragma unroll
          for (int e = 0; e < HC / 8; ++e) {
            const uint32_t wds[4] = {vp[e].x, vp[e].y, vp[e].z, vp[e].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) store_bf16_at(s.VNTst, HC * half + 8 * e + j, t, wds[j >> 1], j & 1);
          }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s.sgReady);
      }
      KDA_DBG_CLOCK(dbg, 54);
      // beside products 2 (nothing else to do until they complete): make sure the next chunk's operand stage has landed
      // and fetch its Gam_last, so that the next state pass starts without a look at a barrier or a shared-memory read;
      // a raised s.dead is noticed here as well
      if (i + 1 < nchunks) {
        if (__any_sync(0xffffffffu, s.dead != 0) || !warp_wait(&s.full[(i + 1) & 1], ((i + 1) >> 1) & 1)) { ok = false; break; }
        gl = s.st[(i + 1) & 1].GL[k];
      }
      if (!warp_wait(&s.barM, 1)) { ok = false; break; }      // products 2 complete: the state is that of the next chunk's start
      umma::fence_after_sync();
      KDA_DBG_CLOCK(dbg, 55);
    }
    if (!ok) s.dead = 1;
    if (__any_sync(0xffffffffu, s.dead != 0)) {
      if (lane == 0) atomicOr(p.status, KDA_STATUS_SCAN_MMA_WAIT);
    } else if (p.ht) {
      const size_t sb = ((static_cast<size_t>(seq) * p.H + h) * KD + k) * VD + v0 + HC * half;
#pragma unroll
      for (int g = 0; g < HC / 16; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_H + HC * half + 16 * g, x);
        umma::tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; e += 4)
          *reinterpret_cast<float4*>(p.ht + sb + 16 * g + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
      }
    }
  } else if (warp == W_ISSUE) {
    // ================= the issuing thread: nothing but products =================
    if (lane == 0) {
      constexpr uint32_t id1 = umma::instr_desc(64, VS, false, true);      // A = w / qg / Aqk rows t (K-major), B = h rows k / v_new rows j (MN-major)
      constexpr uint32_t idH = umma::instr_desc(128, VS, true, true);      // A = kg rows t, two spans of 64 k (MN-major); B = v_new rows t
      const uint64_t dHb = umma::desc_mnmajor(smem_u32(s.Hb), 0, 16384u), dVN = umma::desc_mnmajor(smem_u32(s.VN), 0, 16384u);
      bool ok = nchunks == 0 || mbar_wait(&s.full[0], 0);
      for (int i = 0; i < nchunks && ok; ++i) {
        VsStage<VS>& d = s.st[i & 1];
        const uint32_t to = tb + C_O + VS * (i & 1);
        const uint64_t dW = umma::desc_kmajor(smem_u32(d.W), 0), dQ = umma::desc_kmajor(smem_u32(d.QG), 0);
        const uint64_t dKG = umma::desc_mnmajor(smem_u32(d.KG), 0, 8192u), dAQ = umma::desc_kmajor(smem_u32(d.AQK), 0);
        if (!mbar_wait(&s.stReady, i & 1)) { ok = false; break; }      // (the stage itself was waited for one chunk ahead)
        umma::fence_after_sync();
        // products 1: v_part = w h (k-steps 0..3 in the first sub-tile of W, 4..7 in the second)
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(tb + C_VN, dW, dHb, id1, 0);
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(tb + C_VN, dW + 512u, dHb + 4u * umma::KSTEP_MNMAJOR, id1, 1);
        umma::commit(&s.barM);
        // beside epilogue 1: o = qg h (the accumulator of chunk i - 2 must have been read out)
        if (i >= 2 && !mbar_wait(&s.oFree[i & 1], ((i >> 1) + 1) & 1)) { ok = false; break; }
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(to, dQ, dHb, id1, 0);
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(to, dQ + 512u, dHb + 4u * umma::KSTEP_MNMAJOR, id1, 1);
        if (!mbar_wait(&s.vnReady, i & 1)) { ok = false; break; }
        umma::fence_after_sync();
        // products 2: h += kg^T v_new;  behind them o += Aqk v_new
        umma::mma4<umma::KSTEP_MNMAJOR, umma::KSTEP_MNMAJOR>(tb + C_H, dKG, dVN, idH, 1);
        umma::commit(&s.barM);
        umma::mma4<umma::KSTEP_KMAJOR, umma::KSTEP_MNMAJOR>(to, dAQ, dVN, id1, 1);
        umma::commit(&s.barO[i & 1]);      // every product of this chunk is complete when this fires: o is final, the stage is free
        // off the chain: the next chunk's operand stage has landed; somebody gave up?
        if (s.dead || (i + 1 < nchunks && !mbar_wait(&s.full[(i + 1) & 1], ((i + 1) >> 1) & 1))) { ok = s.dead == 0 ? false : ok; break; }
      }
      if (!ok) {
        s.dead = 1;
        atomicOr(p.status, KDA_STATUS_SCAN_MMA_WAIT);
      }
    }
    __syncwarp();
  } else if (warp >= W_READ0 && warp <= W_LOAD) {
    // ================= read-out warps: o of chunk i as soon as its products are complete =================
    for (int i = 0; i < nchunks; ++i) {
      const int b = i & 1;
      if (__any_sync(0xffffffffu, s.dead != 0)) break;
      if (!warp_wait(&s.barO[b], (i >> 1) & 1)) {        // bounded; also ends a wait for a chain that stopped
        s.dead = 1;
        break;
      }
      umma::fence_after_sync();
      if (warp == W_LOAD && lane == 0 && i + 2 < nchunks) issue_load(i + 2);      // this stage's operand tiles are free again
      const long long tok0 = seq_tok0 + static_cast<long long>(i) * C;
      const int len = static_cast<int>(seq_tok1 - tok0 < C ? seq_tok1 - tok0 : C);
      uint4 out[VS / 8];
#pragma unroll
      for (int g = 0; g < VS / 16; ++g) {
        float x[16];
        umma::tmem_ld16(tq + C_O + VS * b + 16 * g, x);
        umma::tmem_ld_wait();
        out[2 * g] = pack8v(&x[0]);
        out[2 * g + 1] = pack8v(&x[8]);
      }
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.oFree[b]);          // the accumulator may be overwritten (chunk i + 2)
      if (lane < 16 && t < len) {
        uint4* dst = reinterpret_cast<uint4*>(p.o + (static_cast<size_t>(tok0 + t) * p.H + h) * VD + v0);
#pragma unroll
        for (int e = 0; e < VS / 8; ++e) dst[e] = out[e];
      }
    }
  } else if (warp == W_STORE) {
    // ================= tile stores (training): the slice's rows of the HS and VNEWT tiles of every chunk =================
    if (lane == 0 && save) {
      for (int i = 0; i < nchunks; ++i) {
        const size_t tile = static_cast<size_t>(c_begin + i) * p.H + h;
        if (s.dead) break;
        if (!mbar_wait(&s.sgReady, i & 1)) {
          s.dead = 1;
          break;
        }
        bulk_s2g(p.HS + tile * TILE_VK + static_cast<size_t>(v0) * 128, s.HSst, VS * 128);
        bulk_s2g(p.HS + tile * TILE_VK + 16384 + static_cast<size_t>(v0) * 128, s.HSst + VS * 128, VS * 128);
        bulk_s2g(p.VNEWT + tile * TILE_VT + static_cast<size_t>(v0) * 128, s.VNTst, VS * 128);
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
  if (warp == 0) umma::tmem_dealloc(tb, 4 * VS);
}

template <int VS>
static int launch_vs(const ScanParams& p, int units, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(VsSmem<VS>)) + 1024;
  const int rc = once.run([&] { return cudaFuncSetAttribute(kda_chunk_scan_vs_kernel<VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != KDA_OK) return rc;
  kda_chunk_scan_vs_kernel<VS><<<units * (VD / VS), VS_THREADS, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int launch_scan_vs(const ScanParams& p, int units, cudaStream_t st) { return launch_vs<32>(p, units, st); }

}  // namespace kda
