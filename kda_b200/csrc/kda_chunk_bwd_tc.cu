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
#include "kda_chunk_bwd.cuh"
#include "kda_device.cuh"
#include "kda_umma.cuh"

namespace kda {

namespace {

constexpr uint32_t SPAN = 16384;    // bytes of one [128 rows][64] tile
constexpr int NT = 512;             // threads per CTA: 16 warps = 4 TMEM lane quadrants x 4 column parts

struct TcSmem {
  // ---- SW128 operand tiles; every offset is a multiple of 1024 -------------------------------------------------
  unsigned char HS[TILE_VK];    // A.  later: KG = k Gam [64 j][128 kk] (16K) | DWT = dw^T [128 kk][64 t] (16K);  C: kL span 0 | kL span 1 (12K each)
  unsigned char DH[TILE_VK];    // A.  later: DT (8K) | X (8K) | DAQ (8K) | DAK (8K)
  unsigned char VN[TILE_VT];    // A.  C: kR span 0 (12K)
  unsigned char DVN[TILE_VT];   // A, B1.  C: qL span 0 (12K)
  unsigned char dO[TILE_TK];    // A (two [64 t][64 v] sub-tiles).  C: kR span 1
  unsigned char V[TILE_TK];     // B1 (two [64 j][64 v] sub-tiles).  C: qL span 1.  D: dq staging [64][128]
  unsigned char TI[TILE_TT];    // B1..B3.  D (with RKK): dk staging [64][128]
  unsigned char RKK[TILE_TT];   // post-B3
  // ---- plain arrays -----------------------------------------------------------------------------------------------
  __nv_bfloat16 q[C * KD];      // [64][128]   (q, k, g of the NEXT tile arrive here during phase D)
  __nv_bfloat16 k[C * KD];
  float G[C * KD];              // log2-domain cumsum of g
  float2 Ad[4][16][17];         // diagonal blocks: (a1, a2) = (scale dAqk, beta dAkk); rows padded against bank conflicts
  float beta[C];
  float hdh[KD];                // sum over v of h dh'
  union {
    float hdh_part[8][KD];      // its partial sums (phase A only)
    struct {
      float dbp[8][C];          // dbeta partial sums (from phase B1 on)
      float dglp[4][KD];        // partial sums over rows of k dk_end (phase D)
    };
  };
  float carry[4][KD];           // block totals of the reverse cumsum
  uint64_t barS, barQ, barB, barM;
  long long ci_tok0[2];         // first token and length of the chunk of the current / next tile (written by thread 0)
  int ci_len[2];
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

// L2: q, k are L2-normalised rows and dq, dk leave through the normalisation's backward (fla/modules/l2norm.py:190-240).
template <bool L2>
__global__ void __launch_bounds__(512, 1) kda_chunk_bwd_main_tc_kernel(const __grid_constant__ MainParams p) {
  extern __shared__ unsigned char smem_raw[];
  TcSmem& s = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, part = warp >> 2;          // TMEM lane quadrant of this warp; which 16 of the 64 columns
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
  unsigned char* const sKL1 = s.HS + SPAN;
  __nv_bfloat16* const stq = reinterpret_cast<__nv_bfloat16*>(s.V);      // phase D: dq, dk before their coalesced stores
  __nv_bfloat16* const stk = reinterpret_cast<__nv_bfloat16*>(s.TI);

  // thread 0: the phase-A operands of tile idx -- state tiles by bulk copy, dO by two tiled loads (64 value columns each)
  // thread 0: first token and length of tile idx's chunk into slot (two dependent global loads: done early, off the
  // critical path, while phase B2 executes and the other warps build operands)
  auto stash_chunk = [&](long long idx, int slot) {
    const ChunkInfo cn = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, static_cast<int>(idx / p.H));
    s.ci_tok0[slot] = cn.tok0;
    s.ci_len[slot] = cn.len;
  };
  auto fetch_state = [&](long long idx, int slot) {      // after stash_chunk(idx, slot)
    const size_t tl = static_cast<size_t>(idx);
    const int hh = static_cast<int>(idx % p.H);
    struct { long long tok0; } cn;
    cn.tok0 = s.ci_tok0[slot];
    mbar_expect_tx(&s.barS, 2 * TILE_VK + 2 * TILE_VT + TILE_TK);
    bulk_g2s(s.HS, p.HS + tl * TILE_VK, TILE_VK, &s.barS);
    bulk_g2s(s.DH, p.DH + tl * TILE_VK, TILE_VK, &s.barS);
    bulk_g2s(s.VN, p.VNEWT + tl * TILE_VT, TILE_VT, &s.barS);
    bulk_g2s(s.DVN, p.DVNEWT + tl * TILE_VT, TILE_VT, &s.barS);
    tma_load_rows(s.dO, &p.tm_do, 0, hh, static_cast<int>(cn.tok0), &s.barS);
    tma_load_rows(s.dO + 8192, &p.tm_do, 64, hh, static_cast<int>(cn.tok0), &s.barS);
  };
  // thread 0: q, k, g of tile idx
  auto fetch_qkg = [&](long long idx, int slot) {      // after fetch_state(idx, slot)
    const int hh = static_cast<int>(idx % p.H);
    const int tk = static_cast<int>(s.ci_tok0[slot]);
    mbar_expect_tx(&s.barQ, 2 * TILE_TK + C * KD * 4);
    tma_load_rows(s.q, &p.tm_q, 0, hh / p.grp, tk, &s.barQ);
    tma_load_rows(s.k, &p.tm_k, 0, hh / p.grp, tk, &s.barQ);
    tma_load_rows(s.G, &p.tm_g, 0, hh, tk, &s.barQ);
  };
  // rows of a partial chunk beyond its length hold the next sequence's tokens after a tiled load: clear them
  auto zero_rows_sw = [&](unsigned char* tile, int len) {          // [64][64] bf16 sub-tile, 128-byte rows
    for (int i = len * 8 + tid; i < C * 8; i += NT) *reinterpret_cast<uint4*>(tile + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  };
  if (tid == 0) {
    mbar_init(&s.barS, 1);
    mbar_init(&s.barQ, 1);
    mbar_init(&s.barB, 1);
    mbar_init(&s.barM, 1);
    fence_mbar_init();
    if (static_cast<long long>(blockIdx.x) < total_tiles) {
      stash_chunk(blockIdx.x, 0);
      fetch_state(blockIdx.x, 0);
      fetch_qkg(blockIdx.x, 0);
    }
  }
  __syncwarp();
  if (warp == 0) umma::tmem_alloc(&s.tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tb = __shfl_sync(0xffffffffu, s.tmem_slot, 0);          // warp-uniform for the compiler
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);
  const uint32_t lead = lane == 0;                                      // the lane of warp 0 that issues the MMAs
  const uint32_t tq = tb + (static_cast<uint32_t>(32 * q4) << 16);     // this warp's lanes

  // Operands of phase C, built while the phase-B products run (rows R of the stacked tiles, 16-byte pieces pc):
  // kR_I[j][kk] = k_j 2^(G_r - G_j),  r = 16 I,  j < 16 I            rows stacked: I=1 -> 0..15, I=2 -> 16..47, I=3 -> 48..95
  // qL_J[t][kk] = scale q_t 2^(G_t - G_e), kL_J = k_t 2^(G_t - G_e), e = 16 J + 15, t >= 16 (J+1)
  //                                                                   rows stacked: J=0 -> 0..47, J=1 -> 48..79, J=2 -> 80..95
  // One item = four key columns of one row (a warp covers one row: conflict-free 8- and 16-byte accesses).
  auto build_kR = [&](int first, int stride) {
    for (int i = first; i < 96 * 32; i += stride) {
      const int R = i >> 5, g4 = i & 31;
      const int I = (R < 16) ? 1 : (R < 48 ? 2 : 3);
      const int j = R - (I == 1 ? 0 : (I == 2 ? 16 : 48));
      const int r = 16 * I;
      const uint2 kr = *reinterpret_cast<const uint2*>(&s.k[j * KD + g4 * 4]);
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[j * KD + g4 * 4]);
      const float4 Ra = *reinterpret_cast<const float4*>(&s.G[r * KD + g4 * 4]);
      const float2 k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y);
      *reinterpret_cast<uint2*>(sw_piece((g4 >> 4) ? sKR1 : sKR0, R, (g4 >> 1) & 7) + (g4 & 1) * 8) =
          make_uint2(pack_bf16(k0.x * ex2(Ra.x - Ga.x), k0.y * ex2(Ra.y - Ga.y)), pack_bf16(k1.x * ex2(Ra.z - Ga.z), k1.y * ex2(Ra.w - Ga.w)));
    }
  };
  auto build_qkL = [&](int R0, int R1, int first, int stride) {
    for (int i = R0 * 32 + first; i < R1 * 32; i += stride) {
      const int R = i >> 5, g4 = i & 31;
      const int J = (R < 48) ? 0 : (R < 80 ? 1 : 2);
      const int t = 16 * (J + 1) + R - (J == 0 ? 0 : (J == 1 ? 48 : 80));
      const int e = 16 * J + 15;
      const uint2 qr = *reinterpret_cast<const uint2*>(&s.q[t * KD + g4 * 4]);
      const uint2 kr = *reinterpret_cast<const uint2*>(&s.k[t * KD + g4 * 4]);
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[t * KD + g4 * 4]);
      const float4 Ea = *reinterpret_cast<const float4*>(&s.G[e * KD + g4 * 4]);
      const float f0 = ex2(Ga.x - Ea.x), f1 = ex2(Ga.y - Ea.y), f2 = ex2(Ga.z - Ea.z), f3 = ex2(Ga.w - Ea.w);
      const float2 q0 = unpack_bf16(qr.x), q1 = unpack_bf16(qr.y), k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y);
      const int off = (g4 & 1) * 8, pc = (g4 >> 1) & 7;
      *reinterpret_cast<uint2*>(sw_piece((g4 >> 4) ? sQL1 : sQL0, R, pc) + off) =
          make_uint2(pack_bf16(p.scale * q0.x * f0, p.scale * q0.y * f1), pack_bf16(p.scale * q1.x * f2, p.scale * q1.y * f3));
      *reinterpret_cast<uint2*>(sw_piece((g4 >> 4) ? sKL1 : sKL0, R, pc) + off) =
          make_uint2(pack_bf16(k0.x * f0, k0.y * f1), pack_bf16(k1.x * f2, k1.y * f3));
    }
  };

  uint32_t mph = 0;      // phase counter of barM
  bool alive = true;
  int it = 0;
  for (long long idx = blockIdx.x; idx < total_tiles && alive; idx += gridDim.x, ++it) {
    const int h = static_cast<int>(idx % p.H);
    struct { long long tok0; int len; } ci;
    ci.tok0 = s.ci_tok0[it & 1];
    ci.len = s.ci_len[it & 1];
    const int len = ci.len;
    const size_t tile = static_cast<size_t>(idx);
    const long long next_idx = idx + gridDim.x;
    long long* const dbg = (it == 2) ? p.dbg : nullptr;   // development aid: clocks of a steady-state tile

    KDA_DBG_CLOCK(dbg, 0);
    // ---- third load group: Tm, raw kk (bulk), v (tiled), beta (async copies); needed from phase B1 on ---------------
    if (tid == 0) {
      fence_proxy_async();        // the previous tile read its dq / dk staging out of this memory
      mbar_expect_tx(&s.barB, 2 * TILE_TT + TILE_TK);
      bulk_g2s(s.TI, p.TI + tile * TILE_TT, TILE_TT, &s.barB);
      bulk_g2s(s.RKK, p.RKK + tile * TILE_TT, TILE_TT, &s.barB);
      const int tk = static_cast<int>(ci.tok0);
      tma_load_rows(s.V, &p.tm_v, 0, h, tk, &s.barB);
      tma_load_rows(s.V + 8192, &p.tm_v, 64, h, tk, &s.barB);
    }
    if (tid < C) cp_async4(&s.beta[tid], p.beta + static_cast<size_t>(ci.tok0 + (tid < len ? tid : 0)) * p.H + h, tid < len);
    cp_async_commit();
    if (!mbar_wait(&s.barS, it & 1)) {
      if (tid == 0) atomicOr(p.status, 32u);
      alive = false;
    }
    if (len < C) {                 // uniform over the CTA
      zero_rows_sw(s.dO, len);
      zero_rows_sw(s.dO + 8192, len);
      fence_proxy_async();
      __syncthreads();
    }
    umma::fence_after_sync();

    KDA_DBG_CLOCK(dbg, 1);
    // ---- sum_v h dh' (all warps, before warp 0 starts issuing) -------------------------------------------------------
    {
      const int kp = tid & 63, vq = tid >> 6;
      float ax = 0.f, ay = 0.f;
#pragma unroll 4
      for (int vv = vq * 16; vv < vq * 16 + 16; ++vv) {
        const float2 hh = unpack_bf16(*reinterpret_cast<const uint32_t*>(s.HS + vk_off(vv, 2 * kp)));
        const float2 dd = unpack_bf16(*reinterpret_cast<const uint32_t*>(s.DH + vk_off(vv, 2 * kp)));
        ax += hh.x * dd.x;
        ay += hh.y * dd.y;
      }
      s.hdh_part[vq][2 * kp] = ax;
      s.hdh_part[vq][2 * kp + 1] = ay;
    }
    // =========================== phase A: state-dependent products ==================================================
    if (warp_u == 0 && alive) {
      const uint32_t aHS = smem_u32(s.HS), aDH = smem_u32(s.DH), aVN = smem_u32(s.VN), aDVN = smem_u32(s.DVN), aDO = smem_u32(s.dO);
      constexpr uint32_t i1 = umma::instr_desc(128, 64, true, false);
      constexpr uint32_t i2 = umma::instr_desc(128, 64, true, true, false, true);
      constexpr uint32_t i3 = umma::instr_desc(128, 64, true, true);
      constexpr uint32_t i4 = umma::instr_desc(64, 64, false, true);
      // base descriptors once; a k-step advances an MN-major operand by two atoms (2048 B) and a K-major one by 32 B
      const uint64_t dHS = umma::desc_mnmajor(aHS, 0, SPAN), dDHm = umma::desc_mnmajor(aDH, 0, SPAN);
      const uint64_t dVNm = umma::desc_mnmajor(aVN, 0, SPAN), dDVNm = umma::desc_mnmajor(aDVN, 0, SPAN);
      const uint64_t dDO0 = umma::desc_kmajor(aDO, 0), dDO1 = umma::desc_kmajor(aDO + 8192, 0);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t mn = static_cast<uint64_t>(sK) * 128u, dDOk = ((sK >> 2) ? dDO1 : dDO0) + static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss_lead(tb + C_DQG, dHS + mn, dDOk, i1, sK > 0, lead);                 // dqg^T = h dO^T
        umma::mma_ss_lead(tb + C_DW, dHS + mn, dDVNm + mn, i2, sK > 0, lead);            // dw^T = -h dv_new^T
        umma::mma_ss_lead(tb + C_DKG, dDHm + mn, dVNm + mn, i3, sK > 0, lead);           // dkg^T = dh' v_new^T
        umma::mma_ss_lead(tb + C_DAQ, dDOk, dVNm + mn, i4, sK > 0, lead);                // dAqk = dO v_new^T
      }
      if (lead) umma::commit(&s.barM);
    }
    KDA_DBG_CLOCK(dbg, 2);
    // ---- meanwhile, on warps 1..15 (warp 0 is held up by the issue loop; a barrier that includes it would make
    // everybody wait for the loop's end, so these warps meet at named barrier 1 and warp 1 takes warp 0's columns):
    // G = cumsum(g) log2(e)  (q, k, g arrived during the previous tile's phase D) ------------------------------------
    if (warp_u != 0) {
      if (alive && !mbar_wait(&s.barQ, it & 1)) alive = false;
      if (len < C) {
        for (int i = len * 16 + tid - 32; i < C * 16; i += NT - 32) {
          reinterpret_cast<uint4*>(s.q)[i] = make_uint4(0u, 0u, 0u, 0u);
          reinterpret_cast<uint4*>(s.k)[i] = make_uint4(0u, 0u, 0u, 0u);
          reinterpret_cast<uint4*>(s.G)[2 * i] = make_uint4(0u, 0u, 0u, 0u);
          reinterpret_cast<uint4*>(s.G)[2 * i + 1] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      asm volatile("bar.sync 1, 480;" ::: "memory");
      // item = (column, quarter of 16 rows): a thread's own, and for warp 1 also the one warp 0 would have had
      float gv[2][16];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r == 1 && warp_u != 1) break;
        const int item = r ? tid - 32 : tid;
        const int col = item & 127, qr = item >> 7;
#pragma unroll
        for (int i = 0; i < 16; ++i) gv[r][i] = s.G[(qr * 16 + i) * KD + col];
        float run = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          run += gv[r][i];
          gv[r][i] = run;
        }
        s.carry[qr][col] = run;
      }
      asm volatile("bar.sync 1, 480;" ::: "memory");
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (r == 1 && warp_u != 1) break;
        const int item = r ? tid - 32 : tid;
        const int col = item & 127, qr = item >> 7;
        float pre = 0.f;
#pragma unroll
        for (int b = 0; b < 3; ++b) pre += (b < qr) ? s.carry[b][col] : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) s.G[(qr * 16 + i) * KD + col] = (pre + gv[r][i]) * LOG2E;
      }
    }
    if (alive && !mbar_wait(&s.barM, mph & 1)) {
      if (tid == 0) atomicOr(p.status, 64u);
      alive = false;
    }
    ++mph;
    alive = __syncthreads_and(alive);      // also: G complete, hdh partials complete, phase A products complete for everybody
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 32u);
      break;
    }
    umma::fence_after_sync();
    if (tid < KD)
      s.hdh[tid] = s.hdh_part[0][tid] + s.hdh_part[1][tid] + s.hdh_part[2][tid] + s.hdh_part[3][tid] + s.hdh_part[4][tid] +
                   s.hdh_part[5][tid] + s.hdh_part[6][tid] + s.hdh_part[7][tid];      // consumed long before dbp is written

    KDA_DBG_CLOCK(dbg, 3);
    // ---- post-A: dw^T -> bf16 tile; dAqk -> masked bf16 tile + diagonal blocks; k Gam tile -------------------------
    {
      float v[16], w16[16];                            // both loads in flight together
      umma::tmem_ld16(tq + C_DW + 16 * part, w16);
      umma::tmem_ld16(tq + C_DAQ + 16 * part, v);      // M = 64: rows 16 q4 .. +15 live in lanes 0..15 of this quadrant
      umma::tmem_ld_wait();
      const int kk = 32 * q4 + lane;
      *reinterpret_cast<uint4*>(sw_piece(sDWT, kk, 2 * part)) = pack8(&w16[0]);
      *reinterpret_cast<uint4*>(sw_piece(sDWT, kk, 2 * part + 1)) = pack8(&w16[8]);
      if (lane < 16) {
        const int t = 16 * q4 + lane;
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = (16 * part + i <= t) ? v[i] : 0.f;
        *reinterpret_cast<uint4*>(sw_piece(sDAQ, t, 2 * part)) = pack8(&v[0]);
        *reinterpret_cast<uint4*>(sw_piece(sDAQ, t, 2 * part + 1)) = pack8(&v[8]);
        if (part == q4) {                              // these 16 columns are the diagonal block of row block q4
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) s.Ad[q4][lane][cc].x = p.scale * v[cc];
        }
      }
    }
    for (int i = tid; i < C * 32; i += NT) {          // k Gam as two K-major sub-tiles [64 j][64 kk]
      const int j = i >> 5, g4 = i & 31;
      const uint2 kr = *reinterpret_cast<const uint2*>(&s.k[j * KD + g4 * 4]);
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[j * KD + g4 * 4]);
      const float2 k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y);
      *reinterpret_cast<uint2*>(sw_piece(sKG + (g4 >> 4) * 8192, j, (g4 >> 1) & 7) + (g4 & 1) * 8) =
          make_uint2(pack_bf16(k0.x * ex2(Ga.x), k0.y * ex2(Ga.y)), pack_bf16(k1.x * ex2(Ga.z), k1.y * ex2(Ga.w)));
    }
    cp_async_wait<0>();
    if (!mbar_wait(&s.barB, it & 1)) alive = false;       // Tm, raw kk, v
    if (len < C) {
      zero_rows_sw(s.V, len);
      zero_rows_sw(s.V + 8192, len);
    }
    fence_proxy_async();
    umma::fence_before_sync();
    alive = __syncthreads_and(alive);
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 32u);
      break;
    }
    umma::fence_after_sync();

    KDA_DBG_CLOCK(dbg, 4);
    // =========================== phase B1 ===========================================================================
    if (warp_u == 0) {
      const uint32_t aDVN = smem_u32(s.DVN), aV = smem_u32(s.V), aDWT = smem_u32(sDWT), aKG = smem_u32(sKG), aTI = smem_u32(s.TI);
      constexpr uint32_t iT = umma::instr_desc(64, 64, true, false);
      constexpr uint32_t iTt = umma::instr_desc(64, 64, false, true);
      constexpr uint32_t iB = umma::instr_desc(128, 64, false, true);
      const uint64_t dDuM = umma::desc_mnmajor(aDVN, 0, SPAN), dDwM = umma::desc_mnmajor(aDWT, 0, SPAN), dTiM = umma::desc_mnmajor(aTI, 0, SPAN);
      const uint64_t dV0 = umma::desc_kmajor(aV, 0), dV1 = umma::desc_kmajor(aV + 8192, 0);
      const uint64_t dKg0 = umma::desc_kmajor(aKG, 0), dKg1 = umma::desc_kmajor(aKG + 8192, 0);
      const uint64_t dDuK = umma::desc_kmajor(aDVN, 0), dDwK = umma::desc_kmajor(aDWT, 0);
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t mn = static_cast<uint64_t>(sK) * 128u, dVk = ((sK >> 2) ? dV1 : dV0) + static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss_lead(tb + C_DAQ, dDuM + mn, dVk, iT, sK > 0, lead);       // dTm[t][j]   += sum_v du[t][v] v[j][v]
        umma::mma_ss_lead(tb + C_DTT, dVk, dDuM + mn, iTt, sK > 0, lead);      // dTm^T[j][t] += the same
      }
#pragma unroll
      for (int sK = 0; sK < 8; ++sK) {
        const uint64_t mn = static_cast<uint64_t>(sK) * 128u, dKg = ((sK >> 2) ? dKg1 : dKg0) + static_cast<uint64_t>(sK & 3) * 2u;
        umma::mma_ss_lead(tb + C_DAQ, dDwM + mn, dKg, iT, 1, lead);            // += sum_kk dw[t][kk] kGam[j][kk]
        umma::mma_ss_lead(tb + C_DTT, dKg, dDwM + mn, iTt, 1, lead);
      }
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) {
        const uint64_t dTi = dTiM + static_cast<uint64_t>(sK) * 128u;
        umma::mma_ss_lead(tb + C_DBV, dDuK + static_cast<uint64_t>(sK) * 2u, dTi, iB, sK > 0, lead);     // dbv^T[v][t] = sum_t' du[t'][v] Tm[t'][t]
        umma::mma_ss_lead(tb + C_DBK, dDwK + static_cast<uint64_t>(sK) * 2u, dTi, iB, sK > 0, lead);     // dbk^T[kk][t] = sum_t' dw[t'][kk] Tm[t'][t]
      }
      if (lead) umma::commit(&s.barM);
    }
    if (warp_u != 0) build_kR(tid - 32, NT - 32);      // warp 0 is busy issuing; into the v_new and dO tiles, which only phase A read
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 5);
    if (alive) {
      float v[16], v2[16], v3[16];                     // the three loads are in flight together
      umma::tmem_ld16(tq + C_DAQ + 16 * part, v);      // dTm rows (M = 64 layout): scale the columns by beta_j
      umma::tmem_ld16(tq + C_DTT + 16 * part, v2);     // dTm_raw^T rows j: dbeta_j += sum_t' Tm[t'][j] dTm_raw[t'][j]
      umma::tmem_ld16(tq + C_DBV + 16 * part, v3);     // dbv^T rows v: dv[t][v] = beta_t dbv[t][v]
      umma::tmem_ld_wait();
      if (lane < 16) {
        const int t = 16 * q4 + lane;
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] *= s.beta[16 * part + i];
        *reinterpret_cast<uint4*>(sw_piece(sDT, t, 2 * part)) = pack8(&v[0]);
        *reinterpret_cast<uint4*>(sw_piece(sDT, t, 2 * part + 1)) = pack8(&v[8]);
      }
      if (lane < 16) {
        const int j = 16 * q4 + lane;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int t2 = 16 * part + i;
          acc += v2[i] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(s.TI + umma::sw128(t2, j)));
        }
        s.dbp[part][j] = acc;
      }
      {
        const int vcol = 32 * q4 + lane;
        __nv_bfloat16* const dvp = p.dv + (static_cast<size_t>(ci.tok0 + 16 * part) * p.H + h) * VD + vcol;
        const size_t tstride = static_cast<size_t>(p.H) * VD;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (16 * part + i < len) dvp[i * tstride] = __float2bfloat16_rn(s.beta[16 * part + i] * v3[i]);
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

    KDA_DBG_CLOCK(dbg, 6);
    // =========================== phase B2: X = dTm Tm^T ============================================================
    if (warp_u == 0) {
      const uint32_t aDT = smem_u32(sDT), aTI = smem_u32(s.TI);
      constexpr uint32_t iX = umma::instr_desc(64, 64, false, false);
#pragma unroll
      const uint64_t dDt = umma::desc_kmajor(aDT, 0), dTiK = umma::desc_kmajor(aTI, 0);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK) umma::mma_ss_lead(tb + C_XY, dDt + static_cast<uint64_t>(sK) * 2u, dTiK + static_cast<uint64_t>(sK) * 2u, iX, sK > 0, lead);
      if (lead) {
        umma::commit(&s.barM);
        if (next_idx < total_tiles) stash_chunk(next_idx, (it + 1) & 1);      // warp 0 sits this build out: the look-up's latency hides here
      }
    }
    if (warp_u != 0) build_qkL(0, 48, tid - 32, NT - 32);      // into the dv_new, v, k Gam and dw^T tiles, which phase B1 read last
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    if (alive) {
      float v[16];
      umma::tmem_ld16(tq + C_XY + 16 * part, v);
      umma::tmem_ld_wait();
      if (lane < 16) {
        const int m = 16 * q4 + lane;
        *reinterpret_cast<uint4*>(sw_piece(sX, m, 2 * part)) = pack8(&v[0]);
        *reinterpret_cast<uint4*>(sw_piece(sX, m, 2 * part + 1)) = pack8(&v[8]);
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

    KDA_DBG_CLOCK(dbg, 7);
    // =========================== phase B3: Y = Tm^T X,  dAkk = -tril(Y, -1) ==========================================
    if (warp_u == 0) {
      const uint32_t aX = smem_u32(sX), aTI = smem_u32(s.TI);
      constexpr uint32_t iY = umma::instr_desc(64, 64, true, true);
#pragma unroll
      const uint64_t dTiM = umma::desc_mnmajor(aTI, 0, SPAN), dXm = umma::desc_mnmajor(aX, 0, SPAN);
#pragma unroll
      for (int sK = 0; sK < 4; ++sK)
        umma::mma_ss_lead(tb + C_XY, dTiM + static_cast<uint64_t>(sK) * 128u, dXm + static_cast<uint64_t>(sK) * 128u, iY, sK > 0, lead);
      if (lead) umma::commit(&s.barM);
    }
    build_qkL(48, 96, tid, NT);
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    umma::fence_after_sync();
    if (alive) {
      float v[16];
      umma::tmem_ld16(tq + C_XY + 16 * part, v);
      umma::tmem_ld_wait();
      if (lane < 16) {
        const int i0 = 16 * q4 + lane;                 // row i of dAkk
        const float br = s.beta[i0];
        float pb = 0.f;
#pragma unroll
        for (int cix = 0; cix < 2; ++cix) {
          const uint4 rw = *reinterpret_cast<const uint4*>(sw_piece(s.RKK, i0, 2 * part + cix));
          const uint32_t rws[4] = {rw.x, rw.y, rw.z, rw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 raw = unpack_bf16(rws[e]);
            const int j = 16 * part + 8 * cix + 2 * e;
            const float x0 = (j < i0) ? -v[8 * cix + 2 * e] : 0.f;
            const float x1 = (j + 1 < i0) ? -v[8 * cix + 2 * e + 1] : 0.f;
            pb += x0 * raw.x + x1 * raw.y;
            v[8 * cix + 2 * e] = br * x0;
            v[8 * cix + 2 * e + 1] = br * x1;
          }
        }
        *reinterpret_cast<uint4*>(sw_piece(sDAK, i0, 2 * part)) = pack8(&v[0]);
        *reinterpret_cast<uint4*>(sw_piece(sDAK, i0, 2 * part + 1)) = pack8(&v[8]);
        s.dbp[4 + part][i0] = pb;
        if (part == q4) {
#pragma unroll
          for (int cc = 0; cc < 16; ++cc) s.Ad[q4][lane][cc].y = v[cc];
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
    KDA_DBG_CLOCK(dbg, 8);

    KDA_DBG_CLOCK(dbg, 9);
    // =========================== phase C: off-diagonal blocks of the intra-chunk terms ==============================
    if (warp_u == 0) {
      const uint32_t aKR = smem_u32(sKR0), aQL = smem_u32(sQL0), aKL = smem_u32(sKL0), aDAQ = smem_u32(sDAQ), aDAK = smem_u32(sDAK);
      const uint32_t lKR = smem_u32(sKR1) - aKR, lQL = smem_u32(sQL1) - aQL, lKL = smem_u32(sKL1) - aKL;
      constexpr uint32_t iC1 = umma::instr_desc(128, 16, true, false);
      constexpr uint32_t iC2 = umma::instr_desc(128, 16, true, true);
      const uint64_t dKr = umma::smem_desc(aKR, lKR, umma::ATOM_BYTES), dQl = umma::smem_desc(aQL, lQL, umma::ATOM_BYTES);
      const uint64_t dKl = umma::smem_desc(aKL, lKL, umma::ATOM_BYTES);
      const uint64_t dAq = umma::smem_desc(aDAQ, 16, umma::ATOM_BYTES), dAk = umma::smem_desc(aDAK, 16, umma::ATOM_BYTES);
#pragma unroll
      for (int I = 1; I < 4; ++I) {
        const int rb = (I == 1) ? 0 : (I == 2 ? 16 : 48);
#pragma unroll
        for (int sK = 0; sK < I; ++sK) {
          const uint64_t dA = dKr + static_cast<uint64_t>((rb + 16 * sK) * 8);                 // A[kk][j] = kR_I[j][kk]: row offset in 16-byte units
          const uint64_t bo = static_cast<uint64_t>(16 * I * 8 + sK * 2);                      // B[t][j]: rows 16 I.., k-step sK
          umma::mma_ss_lead(tb + C_CQ + 16 * I, dA, dAq + bo, iC1, sK > 0, lead);
          umma::mma_ss_lead(tb + C_CP + 16 * I, dA, dAk + bo, iC1, sK > 0, lead);
        }
      }
#pragma unroll
      for (int J = 0; J < 3; ++J) {
        const int rb = (J == 0) ? 0 : (J == 1 ? 48 : 80);
#pragma unroll
        for (int sK = 0; sK < 3 - J; ++sK) {
          const uint64_t ao = static_cast<uint64_t>((rb + 16 * sK) * 8);
          const uint64_t bo = static_cast<uint64_t>((16 * (J + 1) + 16 * sK) * 8 + 2 * J);     // B[j][t] = dA[t][j]: rows t, columns 16 J..
          umma::mma_ss_lead(tb + C_CN + 16 * J, dQl + ao, dAq + bo, iC2, sK > 0, lead);
          umma::mma_ss_lead(tb + C_CN + 16 * J, dKl + ao, dAk + bo, iC2, 1, lead);
        }
      }
      if (lead) umma::commit(&s.barM);
    }
    // =========================== phase D: one thread per key column and 16-row block ================================
    // Part 1 needs only accumulators of phases A and B1 and runs while phase C executes.
    const int kk = 32 * q4 + lane, blk = part, t0 = 16 * blk;
    float cq[16], cp[16], cn[16], lam[16], qv[16], kv[16];
    float gam_last;
    {
      // Decay inside the block as running products of lam_i = 2^(G_i - G_{i-1}) (every factor <= 1):
      //   2^(G_i - G_first) = fl_i,  2^(G_i) = 2^(G_first) fl_i,  2^(G_e - G_i) = fr_i,  2^(G_last - G_i) = 2^(G_last - G_e) fr_i
      float a[16], a2[16];
      float g_first, e_last;
      {
        float prev = s.G[t0 * KD + kk];
        g_first = ex2(prev);
        lam[0] = 1.f;
#pragma unroll
        for (int i = 1; i < 16; ++i) {
          const float cur = s.G[(t0 + i) * KD + kk];
          lam[i] = ex2(cur - prev);
          prev = cur;
        }
        const float Glast = s.G[(C - 1) * KD + kk];
        gam_last = ex2(Glast);
        e_last = ex2(Glast - prev);
      }
      // dk-: dkg 2^(G_last - G);  sum of k dk_end feeds dG at the chunk's last row
      umma::tmem_ld16(tq + C_DKG + t0, a);
      umma::tmem_ld16(tq + C_DQG + t0, a2);
      umma::tmem_ld_wait();
      {
        float dglp = 0.f, fr = 1.f;
#pragma unroll
        for (int i = 15; i >= 0; --i) {
          const float dke = a[i] * (e_last * fr);
          dglp = fmaf(__bfloat162float(s.k[(t0 + i) * KD + kk]), dke, dglp);
          cn[i] = dke;
          fr *= lam[i];
        }
        s.dglp[blk][kk] = dglp;
      }
      // dq: scale Gam dqg
      {
        float fl = p.scale * g_first;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          fl *= lam[i];
          cq[i] = fl * a2[i];
        }
      }
      // dk+: Gam beta dbk
      umma::tmem_ld16(tq + C_DBK + t0, a);
      umma::tmem_ld_wait();
      {
        float fl = g_first;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          fl *= lam[i];
          cp[i] = fl * s.beta[t0 + i] * a[i];
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        qv[i] = __bfloat162float(s.q[(t0 + i) * KD + kk]);
        kv[i] = __bfloat162float(s.k[(t0 + i) * KD + kk]);
      }
    }
    if (!mbar_wait(&s.barM, mph & 1)) alive = false;
    ++mph;
    alive = __syncthreads_and(alive);      // phase C complete; q, k, G have been read by everybody; dglp is complete
    if (!alive) {
      if (tid == 0) atomicOr(p.status, 64u);
      break;
    }
    umma::fence_after_sync();
    KDA_DBG_CLOCK(dbg, 10);
    // every shared-memory operand tile is dead now and q, k, g are in registers: fetch the next tile behind the rest
    if (next_idx < total_tiles && tid == 0) {
      fetch_state(next_idx, (it + 1) & 1);
      fetch_qkg(next_idx, (it + 1) & 1);
    }
    if (tid < len)
      p.dbeta[static_cast<size_t>(ci.tok0 + tid) * p.H + h] = s.dbp[0][tid] + s.dbp[1][tid] + s.dbp[2][tid] + s.dbp[3][tid] +
                                                             s.dbp[4][tid] + s.dbp[5][tid] + s.dbp[6][tid] + s.dbp[7][tid];

    KDA_DBG_CLOCK(dbg, 11);
    {
      {
        // part 2: the off-diagonal blocks of phase C, scaled back from their reference rows
        float b[16];
        if (blk < 3) {                          // dk-: + 2^(G_e - G) Cn
          umma::tmem_ld16(tq + C_CN + t0, b);
          umma::tmem_ld_wait();
          float fr = 1.f;
#pragma unroll
          for (int i = 15; i >= 0; --i) {
            cn[i] = fmaf(fr, b[i], cn[i]);
            fr *= lam[i];
          }
        }
        if (blk > 0) {                          // dq: + scale L Cq;  dk+: + L Cp
          umma::tmem_ld16(tq + C_CQ + t0, b);
          umma::tmem_ld_wait();
          float fl = 1.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            fl *= lam[i];
            cq[i] = fmaf(p.scale * fl, b[i], cq[i]);
          }
          umma::tmem_ld16(tq + C_CP + t0, b);
          umma::tmem_ld_wait();
          fl = 1.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            fl *= lam[i];
            cp[i] = fmaf(fl, b[i], cp[i]);
          }
        }
      }
      KDA_DBG_CLOCK(dbg, 12);
      // diagonal block, pairwise; D = running product of lam (range-safe)
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        float D = 1.f;
#pragma unroll
        for (int j = t; j >= 0; --j) {
          const float2 a = s.Ad[blk][t][j];
          const float kd = kv[j] * D;
          cq[t] = fmaf(a.x, kd, cq[t]);
          cp[t] = fmaf(a.y, kd, cp[t]);
          cn[j] = fmaf(D, fmaf(a.y, kv[t], a.x * qv[t]), cn[j]);
          D *= lam[j];
        }
      }
      KDA_DBG_CLOCK(dbg, 13);
      // dG; dq, dk into their staging tiles
      float dGv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        dGv[i] = qv[i] * cq[i] + kv[i] * (cp[i] - cn[i]);
        stq[(t0 + i) * KD + kk] = __float2bfloat16_rn(cq[i]);
        stk[(t0 + i) * KD + kk] = __float2bfloat16_rn(cp[i] + cn[i]);
      }
      if (blk == 3)          // the chunk's last row carries the chunk-end terms
        dGv[15] += s.dglp[0][kk] + s.dglp[1][kk] + s.dglp[2][kk] + s.dglp[3][kk] + gam_last * s.hdh[kk];
      {
        float run = 0.f;
#pragma unroll
        for (int i = 15; i >= 0; --i) {
          run += dGv[i];
          dGv[i] = run;
        }
        s.carry[blk][kk] = run;
      }
      // L2: the normalised q, k pieces and the reciprocal norms this thread needs for its two copy-out pieces, asked
      // for before the barrier so that they arrive behind it
      uint4 yq2[2], yk2[2];
      float rq2[2], rk2[2];
      if constexpr (L2) {
        static_assert(C * 16 == 2 * NT, "two copy-out pieces per thread");
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int i = tid + u * NT, r = i >> 4, pc = i & 15;
          const size_t grow = static_cast<size_t>(ci.tok0 + (r < len ? r : 0)) * p.H + h;
          yq2[u] = __ldg(reinterpret_cast<const uint4*>(p.q + grow * KD + pc * 8));
          yk2[u] = __ldg(reinterpret_cast<const uint4*>(p.k + grow * KD + pc * 8));
          rq2[u] = __ldg(p.rstd + grow);
          rk2[u] = __ldg(p.rstd + p.qrows + grow);
        }
      }
      __syncthreads();       // block totals and the staged dq, dk are complete
      {
        float add = 0.f;             // totals of the later blocks
#pragma unroll
        for (int bb = 1; bb < 4; ++bb) add += (bb > blk) ? s.carry[bb][kk] : 0.f;
        float* const dgp = p.dg + (static_cast<size_t>(ci.tok0 + t0) * p.H + h) * KD + kk;      // a warp stores 128 contiguous bytes
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (t0 + i < len) dgp[static_cast<size_t>(i) * p.H * KD] = dGv[i] + add;
      }
#pragma unroll
      for (int u = 0; u < C * 16 / NT; ++u) {
        const int i = tid + u * NT, r = i >> 4, pc = i & 15;
        const size_t row = (static_cast<size_t>(ci.tok0 + (r < len ? r : 0)) * p.H + h) * KD + pc * 8;
        uint4 oq = *reinterpret_cast<const uint4*>(&stq[r * KD + pc * 8]);
        uint4 ok = *reinterpret_cast<const uint4*>(&stk[r * KD + pc * 8]);
        if constexpr (L2) {
          // dx = rstd (dy - y <y, dy>) per row; sixteen consecutive lanes hold one row (y: the normalised q, k, re-read
          // from global memory -- the tile loaded them a few microseconds ago; dy: the staged bf16 values, as the
          // separate pass would read them)
          const uint4 yq = yq2[u], yk = yk2[u];
          const uint32_t dqw[4] = {oq.x, oq.y, oq.z, oq.w}, dkw[4] = {ok.x, ok.y, ok.z, ok.w};
          const uint32_t yqw[4] = {yq.x, yq.y, yq.z, yq.w}, ykw[4] = {yk.x, yk.y, yk.z, yk.w};
          float2 dqf[4], dkf[4], yqf[4], ykf[4];
          float sq = 0.f, sk = 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            dqf[e] = unpack_bf16(dqw[e]); dkf[e] = unpack_bf16(dkw[e]);
            yqf[e] = unpack_bf16(yqw[e]); ykf[e] = unpack_bf16(ykw[e]);
            sq = fmaf(yqf[e].x, dqf[e].x, fmaf(yqf[e].y, dqf[e].y, sq));
            sk = fmaf(ykf[e].x, dkf[e].x, fmaf(ykf[e].y, dkf[e].y, sk));
          }
#pragma unroll
          for (int o = 8; o >= 1; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
          }
          const float rq = rq2[u], rk = rk2[u];
          uint32_t wq[4], wk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            wq[e] = pack_bf16(rq * (dqf[e].x - yqf[e].x * sq), rq * (dqf[e].y - yqf[e].y * sq));
            wk[e] = pack_bf16(rk * (dkf[e].x - ykf[e].x * sk), rk * (dkf[e].y - ykf[e].y * sk));
          }
          oq = make_uint4(wq[0], wq[1], wq[2], wq[3]);
          ok = make_uint4(wk[0], wk[1], wk[2], wk[3]);
        }
        if (r < len) {
          *reinterpret_cast<uint4*>(p.dq + row) = oq;
          *reinterpret_cast<uint4*>(p.dk + row) = ok;
        }
      }
    }
    KDA_DBG_CLOCK(dbg, 14);
    umma::fence_before_sync();
    __syncthreads();   // beta, Ad, the staging tiles, TMEM ... may be overwritten by the next tile
  }

  // drain: a copy that is still in flight must not outlive the CTA's shared memory
  cp_async_wait<0>();
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tb, 512);
}

int launch_bwd_main_tc(const MainParams& p, int grid, cudaStream_t st) {
  static DeviceOnce once;
  const int smem = static_cast<int>(sizeof(TcSmem)) + 1024;
  const int rc = once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(kda_chunk_bwd_main_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kda_chunk_bwd_main_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    return e;
  });
  if (rc != KDA_OK) return rc;
  if (p.rstd != nullptr && p.grp == 1) kda_chunk_bwd_main_tc_kernel<true><<<grid, NT, smem, st>>>(p);
  else kda_chunk_bwd_main_tc_kernel<false><<<grid, NT, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace kda
