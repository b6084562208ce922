// Per-chunk KDA backward on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// One persistent CTA per SM walks (chunk, head) tiles.  Every matrix product of the chunk's backward is a
// tcgen05.mma issued by one thread, with bf16 operands in 128-byte-swizzled shared-memory tiles and fp32
// accumulators in tensor memory.  The products are arranged so that the accumulators that end up in dq / dk
// have the KEY COLUMN as their TMEM lane ("transposed": D^T[kk][t]); a thread then owns one key column, which
// is exactly what the last phase needs (pairwise decay inside the diagonal 16x16 blocks, reverse cumsum for
// dg) -- no shared-memory transposition of fp32 matrices is needed.  The 64 x 64 products of the backward
// through Tm = (I + Akk)^-1 use M = 64 (token row = TMEM lane).
//
// Phases per tile (G = in-chunk cumsum of g in the log2 domain, Gam = 2^G, D[t,j] = 2^(G_t - G_j)):
//   A   dqg^T = h dO^T,  dw^T = -h dv_new^T,  dkg^T = dh' v_new^T      (M=128 kk, N=64 t, K=128 v)
//       dAqk  = dO v_new^T                                             (M=64 t,  N=64 j)
//   B1  dTm = du (beta v)^T + dw (beta k Gam)^T, and its transpose     (M=64)
//       dbv^T = du^T Tm,  dbk^T = dw^T Tm                              (M=128, N=64 t, K=64 t')
//   B2  X = dTm Tm^T      B3  Y = Tm^T X,  dAkk = -tril(Y, -1)
//   C   off-diagonal 16x16 blocks of the intra-chunk terms, decay factored around a row that lies between
//       j and t (both factors <= 1):  Cq^T, Cp^T (reference = first row of t's block),
//       Cn^T (reference = last row of j's block)                       (M=128 kk, N=16, K=16..48)
//   D   per key column: diagonal blocks pairwise with running products of 2^(g), dG = q dq + k (dk+ - dk-),
//       dg = reverse cumsum, final dq, dk, dg;  dbeta from  <Tm, dTm_raw> + <dAkk, raw kk>.
#include <mutex>

#include "kda_chunk_bwd.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

constexpr uint32_t SPAN = 16384;    // bytes of one [128 rows][64] tile

struct TcSmem {
  // ---- SW128 operand tiles; every offset is a multiple of 1024 -------------------------------------------------
  unsigned char HS[TILE_VK];    // A.  later: KG = k Gam [64 j][128 kk] (16K) | DWT = dw^T [128 kk][64 t] (16K);  C: kL span 0 (12K)
  unsigned char DH[TILE_VK];    // A.  later: DT (8K) | X (8K) | DAQ (8K) | DAK (8K)
  unsigned char VN[TILE_VT];    // A.  C: kR span 0 (12K)
  unsigned char DVN[TILE_VT];   // A, B1.  C: qL span 0 (12K)
  unsigned char dO[TILE_TK];    // A (two [64 t][64 v] sub-tiles).  C: kR span 1
  unsigned char V[TILE_TK];     // B1 (two [64 j][64 v] sub-tiles).  C: qL span 1
  unsigned char TI[TILE_TT];    // B1..B3.  C (with RKK): kL span 1 (12K)
  unsigned char RKK[TILE_TT];   // post-B3
  // ---- plain arrays -----------------------------------------------------------------------------------------------
  __nv_bfloat16 q[C * KD];      // [64][128]; at the end dq
  __nv_bfloat16 k[C * KD];      // at the end dk
  float G[C * KD];              // log2-domain cumsum of g; at the end dg
  float4 Ad[2][16][16];         // diagonal blocks: (a1[b], a1[b+2], a2[b], a2[b+2]), a1 = scale dAqk, a2 = beta dAkk
  float beta[C];
  float hdh[4][KD];             // partial sums over v of h dh'
  float dbp[4][C];              // dbeta partial sums
  float dglp[2][KD];            // partial sums over rows of k dk_end
  float carry[4][KD];           // block totals of the reverse cumsum
  uint64_t barS, barB, barM;
  uint32_t tmem_slot;
};
static_assert(sizeof(TcSmem) + 1024 <= 227 * 1024, "TcSmem too large");

// TMEM columns (512 allocated): 64 each
constexpr int C_DQG = 0, C_DKG = 64, C_DW = 128 /* later dbk^T */, C_DAQ = 192 /* later dTm, later Cn */, C_DTT = 256,
              C_XY = 320, C_DBV = 384 /* later Cq */, C_CP = 448;
constexpr int C_CQ = C_DBV, C_CN = C_DAQ, C_DBK = C_DW;

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  float a[16], b[16];
  umma::tmem_ld16(taddr, a);
  umma::tmem_ld16(taddr + 16, b);
  umma::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[i] = a[i];
    v[16 + i] = b[i];
  }
}
// eight floats -> one 16-byte piece of bf16
__device__ __forceinline__ uint4 pack8(const float* v) {
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
// address of the 16-byte piece `chunk` (0..7) of row `row` in an SW128 tile
__device__ __forceinline__ unsigned char* sw_piece(unsigned char* tile, int row, int chunk) {
  return tile + row * 128 + (((chunk ^ row) & 7) << 4);
}

}  // namespace

__global__ void __launch_bounds__(256, 1) kda_chunk_bwd_main_tc_kernel(const MainParams p) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& s = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, half = warp >> 2;          // TMEM lane quadrant of this warp; which half of the columns
  const long long total_tiles = static_cast<long long>(p.seq_chunk_off[p.N]) * p.H;

  // aliases inside the tile regions
  unsigned char* const sKG = s.HS;
  unsigned char* const sDWT = s.HS + SPAN;
  unsigned char* const sDT = s.DH;
  unsigned char* const sX = s.DH + 8192;
  unsigned char* const sDAQ = s.DH + 16384;
  unsigned char* const sDAK = s.DH + 24576;
  unsigned char* const sKR0 = s.VN;
  unsigned char* const sKR1 = s.dO;
  unsigned char* const sQL0 = s.DVN;
  unsigned char* const sQL1 = s.V;
  unsigned char* const sKL0 = s.HS;
  unsigned char* const sKL1 = s.TI;

  if (tid == 0) {
    mbar_init(&s.barS, 1);
    mbar_init(&s.barB, 1);
    mbar_init(&s.barM, 1);
    fence_mbar_init();
  }
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = s.tmem_slot;
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);     // this warp's lanes

  auto fetch_state = [&](long long idx) {      // thread 0: HS, DH, v_new^T, dv_new^T of tile idx
    const size_t tl = static_cast<size_t>(idx);
    mbar_expect_tx(&s.barS, 2 * TILE_VK + 2 * TILE_VT);
    bulk_g2s(s.HS, p.HS + tl * TILE_VK, TILE_VK, &s.barS);
    bulk_g2s(s.DH, p.DH + tl * TILE_VK, TILE_VK, &s.barS);
    bulk_g2s(s.VN, p.VNEWT + tl * TILE_VT, TILE_VT, &s.barS);
    bulk_g2s(s.DVN, p.DVNEWT + tl * TILE_VT, TILE_VT, &s.barS);
  };
  auto fetch_do = [&](long long idx) {          // all threads: dO rows of tile idx as two K-major sub-tiles
    const int cc = static_cast<int>(idx / p.H), hh = static_cast<int>(idx % p.H);
    const ChunkInfo cn = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, cc);
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const bool ok = r < cn.len;
      const size_t row = (static_cast<size_t>(cn.tok0 + (ok ? r : 0)) * p.H + hh) * KD + pc * 8;
      cp_async16(sw_piece(s.dO + (pc >> 3) * 8192, r, pc & 7), p.d_o + row, ok);
    }
    cp_async_commit();
  };
  if (static_cast<long long>(blockIdx.x) < total_tiles) {
    if (tid == 0) fetch_state(blockIdx.x);
    fetch_do(blockIdx.x);
  }

  uint32_t mph = 0;      // phase counter of barM
  bool alive = true;
  int it = 0;
  for (long long idx = blockIdx.x; idx < total_tiles && alive; idx += gridDim.x, ++it) {
    const int c = static_cast<int>(idx / p.H), h = static_cast<int>(idx % p.H);
    const ChunkInfo ci = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, c);
    const int len = ci.len;
    const size_t tile = static_cast<size_t>(idx);
    const long long next_idx = idx + gridDim.x;

    // ---- second load group: Tm, raw kk (bulk); q, k, g, v, beta (async copies); lands behind phase A ------------
    if (tid == 0) {
      mbar_expect_tx(&s.barB, 2 * TILE_TT);
      bulk_g2s(s.TI, p.TI + tile * TILE_TT, TILE_TT, &s.barB);
      bulk_g2s(s.RKK, p.RKK + tile * TILE_TT, TILE_TT, &s.barB);
    }
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const bool ok = r < len;
      const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 8;
      cp_async16(&s.q[r * KD + pc * 8], p.q + row, ok);
      cp_async16(&s.k[r * KD + pc * 8], p.k + row, ok);
      cp_async16(sw_piece(s.V + (pc >> 3) * 8192, r, pc & 7), p.v + row, ok);
    }
    for (int i = tid; i < C * 32; i += 256) {
      const int r = i >> 5, pc = i & 31;
      const bool ok = r < len;
      const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 4;
      cp_async16(&s.G[r * KD + pc * 4], p.g + row, ok);
    }
    if (tid < C) cp_async4(&s.beta[tid], p.beta + static_cast<size_t>(ci.tok0 + (tid < len ? tid : 0)) * p.H + h, tid < len);
    cp_async_commit();
    cp_async_wait<1>();          // this tile's dO (issued one tile ago, or in the prologue)
    fence_proxy_async();         // async-copy writes -> tensor-core (async proxy) reads
    __syncthreads();
    if (!mbar_wait(&s.barS, it & 1)) {
      if (tid == 0) atomicOr(p.status, 32u);
      alive = false;
    }
    umma::fence_after_sync();

    // =========================== phase A: state-dependent products ==================================================
    if (tid == 0 && alive) {
      const uint32_t aHS = smem_u32(s.HS), aDH = smem_u32(s.DH), aVN = smem_u32(s.VN), aDVN = smem_u32(s.DVN), aDO = smem_u32(s.dO);
      constexpr uint32_t i1 = umma::instr_desc(128, 64, true, false);
      constexpr uint32_t i2 = umma::instr_desc(128, 64, true, true, false, true);
      constexpr uint32_t i3 = umma::instr_desc(128, 64, true, true);
      constexpr uint32_t i4 = umma::instr_desc(64, 64, false, true);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t dHS = umma::desc_mnmajor(aHS, sK, SPAN);
        const uint64_t dDOk = umma::desc_kmajor(aDO + (sK >> 2) * 8192, sK & 3);
        umma::mma_ss(tb + C_DQG, dHS, dDOk, i1, sK > 0);                                          // dqg^T = h dO^T
        umma::mma_ss(tb + C_DW, dHS, umma::desc_mnmajor(aDVN, sK, SPAN), i2, sK > 0);              // dw^T = -h dv_new^T
        umma::mma_ss(tb + C_DKG, umma::desc_mnmajor(aDH, sK, SPAN), umma::desc_mnmajor(aVN, sK, SPAN), i3, sK > 0);   // dkg^T
        umma::mma_ss(tb + C_DAQ, dDOk, umma::desc_mnmajor(aVN, sK, SPAN), i4, sK > 0);             // dAqk = dO v_new^T
      }
      umma::commit(&s.barM);
    }
    // ---- meanwhile: the second load group, G = cumsum(g) log2(e), sum_v h dh' ------------------------------------
    cp_async_wait<0>();
    __syncthreads();
    {
      const int col = tid & 127, hf = tid >> 7;
      float gv[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) gv[i] = s.G[(hf * 32 + i) * KD + col];
      float run = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        run += gv[i];
        gv[i] = run;
      }
      if (hf == 0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) s.G[i * KD + col] = gv[i] * LOG2E;
      }
      __syncthreads();
      if (hf == 1) {
        const float carry = s.G[31 * KD + col];
#pragma unroll
        for (int i = 0; i < 32; ++i) s.G[(32 + i) * KD + col] = carry + gv[i] * LOG2E;
      }
    }
    {
      const int kp = tid & 63, vq = tid >> 6;
      float ax = 0.f, ay = 0.f;
#pragma unroll 4
      for (int vv = vq * 32; vv < vq * 32 + 32; ++vv) {
        const float2 hh = unpack_bf16(*reinterpret_cast<const uint32_t*>(s.HS + vk_off(vv, 2 * kp)));
        const float2 dd = unpack_bf16(*reinterpret_cast<const uint32_t*>(s.DH + vk_off(vv, 2 * kp)));
        ax += hh.x * dd.x;
        ay += hh.y * dd.y;
      }
      s.hdh[vq][2 * kp] = ax;
      s.hdh[vq][2 * kp + 1] = ay;
    }
    if (alive && !mbar_wait(&s.barB, it & 1)) {
      if (tid == 0) atomicOr(p.status, 32u);
      alive = false;
    }
    if (alive && !mbar_wait(&s.barM, mph & 1)) {
      if (tid == 0) atomicOr(p.status, 64u);
      alive = false;
    }
    ++mph;
    alive = __syncthreads_and(alive);      // also: G complete, hdh complete, phase A products complete for everybody
    if (!alive) break;
    umma::fence_after_sync();

    // ---- post-A: dw^T -> bf16 tile; dAqk -> masked bf16 tile + diagonal blocks; k Gam tile -------------------------
    {
      float v[32];
      tmem_ld32(tq + C_DW + 32 * half, v);
      const int kk = 32 * q4 + lane;
#pragma unroll
      for (int cix = 0; cix < 4; ++cix) *reinterpret_cast<uint4*>(sw_piece(sDWT, kk, 4 * half + cix)) = pack8(&v[8 * cix]);
      tmem_ld32(tq + C_DAQ + 32 * half, v);            // M = 64: rows 16 q4 .. +15 live in lanes 0..15 of this quadrant
      if (lane < 16) {
        const int t = 16 * q4 + lane;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = (32 * half + i <= t) ? v[i] : 0.f;
#pragma unroll
        for (int cix = 0; cix < 4; ++cix) *reinterpret_cast<uint4*>(sw_piece(sDAQ, t, 4 * half + cix)) = pack8(&v[8 * cix]);
        if ((q4 >> 1) == half) {                       // the diagonal block of row block q4 lies in this half of the columns
          float* ad = reinterpret_cast<float*>(&s.Ad[q4 & 1][lane][0]);
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) ad[cc * 4 + (q4 >> 1)] = p.scale * v[16 * (q4 & 1) + cc];
        }
      }
    }
    for (int i = tid; i < C * 16; i += 256) {          // k Gam as two K-major sub-tiles [64 j][64 kk]
      const int j = i >> 4, pc = i & 15;
      const uint4 kr = *reinterpret_cast<const uint4*>(&s.k[j * KD + pc * 8]);
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[j * KD + pc * 8]);
      const float4 Gb = *reinterpret_cast<const float4*>(&s.G[j * KD + pc * 8 + 4]);
      const float2 k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y), k2 = unpack_bf16(kr.z), k3 = unpack_bf16(kr.w);
      *reinterpret_cast<uint4*>(sw_piece(sKG + (pc >> 3) * 8192, j, pc & 7)) =
          make_uint4(pack_bf16(k0.x * ex2(Ga.x), k0.y * ex2(Ga.y)), pack_bf16(k1.x * ex2(Ga.z), k1.y * ex2(Ga.w)),
                     pack_bf16(k2.x * ex2(Gb.x), k2.y * ex2(Gb.y)), pack_bf16(k3.x * ex2(Gb.z), k3.y * ex2(Gb.w)));
    }
    fence_proxy_async();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();

    // =========================== phase B1 ===========================================================================
    if (tid == 0) {
      const uint32_t aDVN = smem_u32(s.DVN), aV = smem_u32(s.V), aDWT = smem_u32(sDWT), aKG = smem_u32(sKG), aTI = smem_u32(s.TI);
      constexpr uint32_t iT = umma::instr_desc(64, 64, true, false);
      constexpr uint32_t iTt = umma::instr_desc(64, 64, false, true);
      constexpr uint32_t iB = umma::instr_desc(128, 64, false, true);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t dDu = umma::desc_mnmajor(aDVN, sK, SPAN), dVk = umma::desc_kmajor(aV + (sK >> 2) * 8192, sK & 3);
        umma::mma_ss(tb + C_DAQ, dDu, dVk, iT, sK > 0);       // dTm[t][j]   += sum_v du[t][v] v[j][v]
        umma::mma_ss(tb + C_DTT, dVk, dDu, iTt, sK > 0);      // dTm^T[j][t] += the same
      }
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t dDw = umma::desc_mnmajor(aDWT, sK, SPAN), dKg = umma::desc_kmajor(aKG + (sK >> 2) * 8192, sK & 3);
        umma::mma_ss(tb + C_DAQ, dDw, dKg, iT, 1);            // += sum_kk dw[t][kk] kGam[j][kk]
        umma::mma_ss(tb + C_DTT, dKg, dDw, iTt, 1);
      }
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) {
        const uint64_t dTi = umma::desc_mnmajor(aTI, sK, SPAN);
        umma::mma_ss(tb + C_DBV, umma::desc_kmajor(aDVN, sK), dTi, iB, sK > 0);     // dbv^T[v][t] = sum_t' du[t'][v] Tm[t'][t]
        umma::mma_ss(tb + C_DBK, umma::desc_kmajor(aDWT, sK), dTi, iB, sK > 0);     // dbk^T[kk][t] = sum_t' dw[t'][kk] Tm[t'][t]
      }
      umma::commit(&s.barM);
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    if (alive) {
      float v[32];
      tmem_ld32(tq + C_DAQ + 32 * half, v);            // dTm rows (M = 64 layout): scale the columns by beta_j
      if (lane < 16) {
        const int t = 16 * q4 + lane;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= s.beta[32 * half + i];
#pragma unroll
        for (int cix = 0; cix < 4; ++cix) *reinterpret_cast<uint4*>(sw_piece(sDT, t, 4 * half + cix)) = pack8(&v[8 * cix]);
      }
      tmem_ld32(tq + C_DTT + 32 * half, v);            // dTm_raw^T rows j: dbeta_j += sum_t' Tm[t'][j] dTm_raw[t'][j]
      if (lane < 16) {
        const int j = 16 * q4 + lane;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t2 = 32 * half + i;
          acc += v[i] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(s.TI + umma::sw128(t2, j)));
        }
        s.dbp[half][j] = acc;
      }
      tmem_ld32(tq + C_DBV + 32 * half, v);            // dbv^T rows v: dv[t][v] = beta_t dbv[t][v]
      {
        const int vcol = 32 * q4 + lane;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = 32 * half + i;
          if (t < len) p.dv[(static_cast<size_t>(ci.tok0 + t) * p.H + h) * VD + vcol] = __float2bfloat16_rn(s.beta[t] * v[i]);
        }
      }
    }
    fence_proxy_async();
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 64u);
      break;
    }
    umma::fence_after_sync();

    // =========================== phase B2: X = dTm Tm^T ============================================================
    if (tid == 0) {
      const uint32_t aDT = smem_u32(sDT), aTI = smem_u32(s.TI);
      constexpr uint32_t iX = umma::instr_desc(64, 64, false, false);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) umma::mma_ss(tb + C_XY, umma::desc_kmajor(aDT, sK), umma::desc_kmajor(aTI, sK), iX, sK > 0);
      umma::commit(&s.barM);
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    if (alive) {
      float v[32];
      tmem_ld32(tq + C_XY + 32 * half, v);
      if (lane < 16) {
        const int m = 16 * q4 + lane;
#pragma unroll
        for (int cix = 0; cix < 4; ++cix) *reinterpret_cast<uint4*>(sw_piece(sX, m, 4 * half + cix)) = pack8(&v[8 * cix]);
      }
    }
    fence_proxy_async();
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 64u);
      break;
    }
    umma::fence_after_sync();

    // =========================== phase B3: Y = Tm^T X,  dAkk = -tril(Y, -1) ==========================================
    if (tid == 0) {
      const uint32_t aX = smem_u32(sX), aTI = smem_u32(s.TI);
      constexpr uint32_t iY = umma::instr_desc(64, 64, true, true);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK)
        umma::mma_ss(tb + C_XY, umma::desc_mnmajor(aTI, sK, SPAN), umma::desc_mnmajor(aX, sK, SPAN), iY, sK > 0);
      umma::commit(&s.barM);
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    if (alive) {
      float v[32];
      tmem_ld32(tq + C_XY + 32 * half, v);
      if (lane < 16) {
        const int i0 = 16 * q4 + lane;                 // row i of dAkk
        const float br = s.beta[i0];
        float pb = 0.f;
#pragma unroll
        for (int cix = 0; cix < 4; ++cix) {
          const uint4 rw = *reinterpret_cast<const uint4*>(sw_piece(s.RKK, i0, 4 * half + cix));
          const uint32_t rws[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 raw = unpack_bf16(rws[e]);
            const int j = 32 * half + 8 * cix + 2 * e;
            const float x0 = (j < i0) ? -v[8 * cix + 2 * e] : 0.f;
            const float x1 = (j + 1 < i0) ? -v[8 * cix + 2 * e + 1] : 0.f;
            pb += x0 * raw.x + x1 * raw.y;
            v[8 * cix + 2 * e] = br * x0;
            v[8 * cix + 2 * e + 1] = br * x1;
          }
          *reinterpret_cast<uint4*>(sw_piece(sDAK, i0, 4 * half + cix)) = pack8(&v[8 * cix]);
        }
        s.dbp[2 + half][i0] = pb;
        if ((q4 >> 1) == half) {
          float* ad = reinterpret_cast<float*>(&s.Ad[q4 & 1][lane][0]);
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) ad[cc * 4 + 2 + (q4 >> 1)] = v[16 * (q4 & 1) + cc];
        }
      }
    }
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);      // TI / RKK are dead: their memory now takes phase-C operands
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 64u);
      break;
    }

    // ---- operands of phase C -------------------------------------------------------------------------------------------
    // kR_I[j][kk] = k_j 2^(G_r - G_j),  r = 16 I,  j < 16 I            rows stacked: I=1 -> 0..15, I=2 -> 16..47, I=3 -> 48..95
    // qL_J[t][kk] = scale q_t 2^(G_t - G_e), kL_J = k_t 2^(G_t - G_e), e = 16 J + 15, t >= 16 (J+1)
    //                                                                   rows stacked: J=0 -> 0..47, J=1 -> 48..79, J=2 -> 80..95
    for (int i = tid; i < 96 * 16; i += 256) {
      const int R = i >> 4, pc = i & 15;
      {
        const int I = (R < 16) ? 1 : (R < 48 ? 2 : 3);
        const int j = R - (I == 1 ? 0 : (I == 2 ? 16 : 48));
        const int r = 16 * I;
        const uint4 kr = *reinterpret_cast<const uint4*>(&s.k[j * KD + pc * 8]);
        const float4 Ga = *reinterpret_cast<const float4*>(&s.G[j * KD + pc * 8]);
        const float4 Gb = *reinterpret_cast<const float4*>(&s.G[j * KD + pc * 8 + 4]);
        const float4 Ra = *reinterpret_cast<const float4*>(&s.G[r * KD + pc * 8]);
        const float4 Rb = *reinterpret_cast<const float4*>(&s.G[r * KD + pc * 8 + 4]);
        const float2 k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y), k2 = unpack_bf16(kr.z), k3 = unpack_bf16(kr.w);
        *reinterpret_cast<uint4*>(sw_piece((pc >> 3) ? sKR1 : sKR0, R, pc & 7)) =
            make_uint4(pack_bf16(k0.x * ex2(Ra.x - Ga.x), k0.y * ex2(Ra.y - Ga.y)), pack_bf16(k1.x * ex2(Ra.z - Ga.z), k1.y * ex2(Ra.w - Ga.w)),
                       pack_bf16(k2.x * ex2(Rb.x - Gb.x), k2.y * ex2(Rb.y - Gb.y)), pack_bf16(k3.x * ex2(Rb.z - Gb.z), k3.y * ex2(Rb.w - Gb.w)));
      }
      {
        const int J = (R < 48) ? 0 : (R < 80 ? 1 : 2);
        const int t = 16 * (J + 1) + R - (J == 0 ? 0 : (J == 1 ? 48 : 80));
        const int e = 16 * J + 15;
        const uint4 qr = *reinterpret_cast<const uint4*>(&s.q[t * KD + pc * 8]);
        const uint4 kr = *reinterpret_cast<const uint4*>(&s.k[t * KD + pc * 8]);
        const float4 Ga = *reinterpret_cast<const float4*>(&s.G[t * KD + pc * 8]);
        const float4 Gb = *reinterpret_cast<const float4*>(&s.G[t * KD + pc * 8 + 4]);
        const float4 Ea = *reinterpret_cast<const float4*>(&s.G[e * KD + pc * 8]);
        const float4 Eb = *reinterpret_cast<const float4*>(&s.G[e * KD + pc * 8 + 4]);
        const float f[8] = {ex2(Ga.x - Ea.x), ex2(Ga.y - Ea.y), ex2(Ga.z - Ea.z), ex2(Ga.w - Ea.w),
                            ex2(Gb.x - Eb.x), ex2(Gb.y - Eb.y), ex2(Gb.z - Eb.z), ex2(Gb.w - Eb.w)};
        const uint32_t qw[4] = {qr.x, qr.y, qr.z, qr.w}, kw[4] = {kr.x, kr.y, kr.z, kr.w};
        uint32_t oq[4], ok[4];
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
          const float2 qq = unpack_bf16(qw[e2]), kk2 = unpack_bf16(kw[e2]);
          oq[e2] = pack_bf16(p.scale * qq.x * f[2 * e2], p.scale * qq.y * f[2 * e2 + 1]);
          ok[e2] = pack_bf16(kk2.x * f[2 * e2], kk2.y * f[2 * e2 + 1]);
        }
        *reinterpret_cast<uint4*>(sw_piece((pc >> 3) ? sQL1 : sQL0, R, pc & 7)) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
        *reinterpret_cast<uint4*>(sw_piece((pc >> 3) ? sKL1 : sKL0, R, pc & 7)) = make_uint4(ok[0], ok[1], ok[2], ok[3]);
      }
    }
    fence_proxy_async();
    __syncthreads();
    umma::fence_after_sync();

    // =========================== phase C: off-diagonal blocks of the intra-chunk terms ==============================
    if (tid == 0) {
      const uint32_t aKR = smem_u32(sKR0), aQL = smem_u32(sQL0), aKL = smem_u32(sKL0), aDAQ = smem_u32(sDAQ), aDAK = smem_u32(sDAK);
      const uint32_t lKR = smem_u32(sKR1) - aKR, lQL = smem_u32(sQL1) - aQL, lKL = smem_u32(sKL1) - aKL;
      constexpr uint32_t iC1 = umma::instr_desc(128, 16, true, false);
      constexpr uint32_t iC2 = umma::instr_desc(128, 16, true, true);
#pragma unroll
      for (int I = 1; I < 4; ++I) {
        const int rb = (I == 1) ? 0 : (I == 2 ? 16 : 48);
        for (int sK = 0; sK < I; ++sK) {
          const uint64_t dA = umma::smem_desc(aKR + (rb + 16 * sK) * 128, lKR, umma::ATOM_BYTES);     // A[kk][j] = kR_I[j][kk]
          umma::mma_ss(tb + C_CQ + 16 * I, dA, umma::smem_desc(aDAQ + 16 * I * 128 + sK * 32, 16, umma::ATOM_BYTES), iC1, sK > 0);
          umma::mma_ss(tb + C_CP + 16 * I, dA, umma::smem_desc(aDAK + 16 * I * 128 + sK * 32, 16, umma::ATOM_BYTES), iC1, sK > 0);
        }
      }
#pragma unroll
      for (int J = 0; J < 3; ++J) {
        const int rb = (J == 0) ? 0 : (J == 1 ? 48 : 80);
        for (int sK = 0; sK < 3 - J; ++sK) {
          const uint32_t boff = (16 * (J + 1) + 16 * sK) * 128 + 32 * J;                               // B[j][t] = dA[t][j]
          umma::mma_ss(tb + C_CN + 16 * J, umma::smem_desc(aQL + (rb + 16 * sK) * 128, lQL, umma::ATOM_BYTES),
                       umma::smem_desc(aDAQ + boff, 16, umma::ATOM_BYTES), iC2, sK > 0);
          umma::mma_ss(tb + C_CN + 16 * J, umma::smem_desc(aKL + (rb + 16 * sK) * 128, lKL, umma::ATOM_BYTES),
                       umma::smem_desc(aDAK + boff, 16, umma::ATOM_BYTES), iC2, 1);
        }
      }
      umma::commit(&s.barM);
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 64u);
      break;
    }
    umma::fence_after_sync();
    // every shared-memory operand tile is dead now: fetch the next tile's phase-A operands behind phase D
    if (next_idx < total_tiles) {
      if (tid == 0) fetch_state(next_idx);
      fetch_do(next_idx);
    }
    if (tid < len) p.dbeta[static_cast<size_t>(ci.tok0 + tid) * p.H + h] = s.dbp[0][tid] + s.dbp[1][tid] + s.dbp[2][tid] + s.dbp[3][tid];

    // =========================== phase D: one thread per key column and pair of 16-row blocks (half, half+2) =======
    {
      const int kk = 32 * q4 + lane;
      float2 cq[16], cp[16], cn[16], lam[16], qv[16], kv[16];
      float dglp = 0.f;
#pragma unroll
      for (int hb = 0; hb < 2; ++hb) {                 // component .x: block `half`, component .y: block `half + 2`
        const int blk = half + 2 * hb, t0 = 16 * blk;
        float Gc[16], a[16], b[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) Gc[i] = s.G[(t0 + i) * KD + kk];
        const float Glast = s.G[(C - 1) * KD + kk];
        // dq: scale (Gam dqg + L Cq)
        umma::tmem_ld16(tq + C_DQG + t0, a);
        umma::tmem_ld16(tq + C_CQ + t0, b);
        umma::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = ex2(Gc[i]) * a[i];
          if (blk > 0) x = fmaf(ex2(Gc[i] - Gc[0]), b[i], x);
          (hb ? cq[i].y : cq[i].x) = p.scale * x;
        }
        // dk+: Gam beta dbk + L Cp
        umma::tmem_ld16(tq + C_DBK + t0, a);
        umma::tmem_ld16(tq + C_CP + t0, b);
        umma::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = ex2(Gc[i]) * s.beta[t0 + i] * a[i];
          if (blk > 0) x = fmaf(ex2(Gc[i] - Gc[0]), b[i], x);
          (hb ? cp[i].y : cp[i].x) = x;
        }
        // dk-: dkg 2^(G_last - G) + 2^(G_e - G) Cn ;  sum of k dk_end feeds dG at the chunk's last row
        umma::tmem_ld16(tq + C_DKG + t0, a);
        umma::tmem_ld16(tq + C_CN + t0, b);
        umma::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 kq = make_float2(__bfloat162float(s.q[(t0 + i) * KD + kk]), __bfloat162float(s.k[(t0 + i) * KD + kk]));
          const float dke = a[i] * ex2(Glast - Gc[i]);
          dglp = fmaf(kq.y, dke, dglp);
          float x = dke;
          if (blk < 3) x = fmaf(ex2(Gc[15] - Gc[i]), b[i], x);
          (hb ? cn[i].y : cn[i].x) = x;
          (hb ? qv[i].y : qv[i].x) = kq.x;
          (hb ? kv[i].y : kv[i].x) = kq.y;
          (hb ? lam[i].y : lam[i].x) = (i > 0) ? ex2(Gc[i] - Gc[i - 1]) : 1.f;
        }
      }
      s.dglp[half][kk] = dglp;
      // diagonal blocks, pairwise; D = running product of lam (range-safe)
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        float2 D = make_float2(1.f, 1.f);
#pragma unroll
        for (int j = t; j >= 0; --j) {
          const float4 a = s.Ad[half][t][j];
          const float2 a1 = make_float2(a.x, a.y), a2 = make_float2(a.z, a.w);
          const float2 kd = __fmul2_rn(kv[j], D);
          cq[t] = __ffma2_rn(a1, kd, cq[t]);
          cp[t] = __ffma2_rn(a2, kd, cp[t]);
          const float2 tmp = __ffma2_rn(a2, kv[t], __fmul2_rn(a1, qv[t]));
          cn[j] = __ffma2_rn(D, tmp, cn[j]);
          D = __fmul2_rn(D, lam[j]);
        }
      }
      // dG, dq, dk (in place of q, k)
      float2 dGv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        dGv[i] = make_float2(qv[i].x * cq[i].x + kv[i].x * (cp[i].x - cn[i].x), qv[i].y * cq[i].y + kv[i].y * (cp[i].y - cn[i].y));
        const int ta = 16 * half + i, tb2 = 16 * (half + 2) + i;
        s.q[ta * KD + kk] = __float2bfloat16_rn(cq[i].x);
        s.q[tb2 * KD + kk] = __float2bfloat16_rn(cq[i].y);
        s.k[ta * KD + kk] = __float2bfloat16_rn(cp[i].x + cn[i].x);
        s.k[tb2 * KD + kk] = __float2bfloat16_rn(cp[i].y + cn[i].y);
      }
      __syncthreads();       // dglp complete
      if (half == 1)         // this thread owns block 3 (.y): the chunk's last row carries the chunk-end terms
        dGv[15].y += s.dglp[0][kk] + s.dglp[1][kk] +
                     ex2(s.G[(C - 1) * KD + kk]) * (s.hdh[0][kk] + s.hdh[1][kk] + s.hdh[2][kk] + s.hdh[3][kk]);
      {
        float2 run = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 15; i >= 0; --i) {
          run.x += dGv[i].x;
          run.y += dGv[i].y;
          dGv[i] = run;
        }
        s.carry[half][kk] = run.x;
        s.carry[half + 2][kk] = run.y;
      }
      __syncthreads();
      {
        float addx = 0.f, addy = 0.f;        // totals of the later blocks
#pragma unroll
        for (int bb = 1; bb < 4; ++bb) {
          const float cb = s.carry[bb][kk];
          if (bb > half) addx += cb;
          if (bb > half + 2) addy += cb;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          s.G[(16 * half + i) * KD + kk] = dGv[i].x + addx;
          s.G[(16 * (half + 2) + i) * KD + kk] = dGv[i].y + addy;
        }
      }
      umma::fence_before_sync();
      __syncthreads();
      for (int i = tid; i < C * 16; i += 256) {
        const int r = i >> 4, pc = i & 15;
        if (r < len) {
          const size_t row = (static_cast<size_t>(ci.tok0 + r) * p.H + h) * KD + pc * 8;
          *reinterpret_cast<uint4*>(p.dq + row) = *reinterpret_cast<const uint4*>(&s.q[r * KD + pc * 8]);
          *reinterpret_cast<uint4*>(p.dk + row) = *reinterpret_cast<const uint4*>(&s.k[r * KD + pc * 8]);
        }
      }
      for (int i = tid; i < C * 32; i += 256) {
        const int r = i >> 5, pc = i & 31;
        if (r < len) {
          const size_t row = (static_cast<size_t>(ci.tok0 + r) * p.H + h) * KD + pc * 4;
          *reinterpret_cast<float4*>(p.dg + row) = *reinterpret_cast<const float4*>(&s.G[r * KD + pc * 4]);
        }
      }
    }
    __syncthreads();   // q, k, G, beta, Ad, ... may be overwritten by the next tile
  }

  // drain: a copy that is still in flight must not outlive the CTA's shared memory
  cp_async_wait<0>();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tb, 512);
}

cudaError_t launch_bwd_main_tc(const MainParams& p, int grid, cudaStream_t st) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  const int smem = static_cast<int>(sizeof(TcSmem)) + 1024;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kda_chunk_bwd_main_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  });
  if (attr_err != cudaSuccess) return attr_err;
  kda_chunk_bwd_main_tc_kernel<<<grid, 256, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace kda
