// Chunked KDA backward for sm_100a.  Two kernels, both reading the tiles the forward left behind:
//
//  kda_chunk_bwd_scan_kernel   one CTA per (sequence, head): chunks in REVERSE order with the fp32 state
//                              gradient in registers (transposed, one warp per 16 value columns):
//                                 dv_new = Aqk^T dO + kg dh';   dh = Diag(Gam_last) dh' + qg^T dO - w^T dv_new
//                              stores dh' (gradient w.r.t. the state at the chunk's end) and dv_new per chunk.
//  kda_chunk_bwd_main_kernel   one CTA per (chunk, head): every tensor-core product of the chunk's backward
//                              (state-dependent terms, the backward through Tm = (I+Akk)^-1, the
//                              off-diagonal 16x16 blocks of the intra-chunk terms), then, one thread per key
//                              column, the diagonal 16x16 blocks pairwise (range-safe), dg = reverse cumsum,
//                              and the final dq, dk, dv, dg, dbeta.
//
// Gradient identities (G = in-chunk cumsum of g, Gam = exp G, D[t,j] = exp(G_t - G_j)):
//   dqg = dO h^T,  dAqk = tril(dO v_new^T),  dkg = v_new dh'^T,  dw = -dv_new h^T,  du = dv_new
//   dv = beta (Tm^T du),  dkGam = beta (Tm^T dw),  dTm = du (beta v)^T + dw (beta k Gam)^T
//   dAkk = -Tm^T dTm Tm^T (strictly lower),  dbeta = <Tm^T du, v> + <Tm^T dw, k Gam> + <dAkk, Akk/beta>
//   dq = scale Gam dqg + scale sum_j dAqk[t,j] D[t,j] k_j
//   dk+ = Gam dkGam + sum_j beta_t dAkk[t,j] D[t,j] k_j        (terms in which k_t enters as k_t Gam_t)
//   dk- = dkg exp(G_last - G) + sum_t D[t,j] (scale dAqk[t,j] q_t + beta_t dAkk[t,j] k_t)   (k_j / Gam_j)
//   dk = dk+ + dk-;   dG = q dq + k (dk+ - dk-);   dG_last += sum_j k_j dk_end_j + Gam_last sum_v h dh'
//   dg = reverse cumsum of dG inside the chunk.
#include <mutex>

#include "kda_chunk.cuh"
#include "kda_chunk_bwd.cuh"

namespace kda {

int validate_chunk_args(const kda_chunk_args& a, bool backward);

// =================================================================================================
// reverse state scan
// =================================================================================================
constexpr int RS_STAGES = 3;
constexpr int RS_WARPS = 8;
constexpr int RS_THREADS = RS_WARPS * 32;

struct RScanStage {
  unsigned char W[TILE_TK], QG[TILE_TK], KG[TILE_TK], AQK[TILE_TT];
  float GL[KD];
};
constexpr unsigned RS_STAGE_TX = 3 * TILE_TK + TILE_TT + TILE_GL;

struct RScanSmem {
  RScanStage st[RS_STAGES];
  unsigned char dO[RS_WARPS][2][C * 32];   // per warp, double buffered: [64 t][16 v] bf16, 32-byte rows
  uint64_t full[RS_STAGES], empty[RS_STAGES];
};

struct RScanParams {
  const int* cu;
  const int *seq_chunk_off, *chunk_seq;
  const unsigned char *W, *KG, *QG, *AQK, *GL;
  unsigned char *DH, *DVNEWT;
  const __nv_bfloat16* d_o;
  const float* d_ht;
  float* dh0;
  unsigned* status;
  int N, H;
};

// 16-byte piece p (0/1) of row t in a warp's dO slab; the XOR keeps ldmatrix rows on distinct banks
__device__ __forceinline__ uint32_t do_slab_off(int t, int p) { return static_cast<uint32_t>(t * 32 + ((p ^ ((t >> 2) & 1)) << 4)); }

__global__ void __launch_bounds__(RS_THREADS, 1) kda_chunk_bwd_scan_kernel(const RScanParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  RScanSmem& s = *reinterpret_cast<RScanSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int seq = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int c_begin = p.seq_chunk_off[seq], c_end = p.seq_chunk_off[seq + 1];
  const int nchunks = c_end - c_begin;
  const int v0 = warp * 16;

  if (tid == 0) {
    for (int i = 0; i < RS_STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], RS_WARPS);
    }
    fence_mbar_init();
  }
  __syncthreads();

  // step i handles chunk c_end-1-i
  auto issue = [&](int i) -> bool {
    const int stg = i % RS_STAGES;
    if (i >= RS_STAGES) {
      if (!mbar_wait(&s.empty[stg], ((i / RS_STAGES) & 1) ^ 1)) return false;
    }
    const size_t tile = static_cast<size_t>(c_end - 1 - i) * p.H + h;
    RScanStage& d = s.st[stg];
    mbar_expect_tx(&s.full[stg], RS_STAGE_TX);
    bulk_g2s(d.W, p.W + tile * TILE_TK, TILE_TK, &s.full[stg]);
    bulk_g2s(d.QG, p.QG + tile * TILE_TK, TILE_TK, &s.full[stg]);
    bulk_g2s(d.KG, p.KG + tile * TILE_TK, TILE_TK, &s.full[stg]);
    bulk_g2s(d.AQK, p.AQK + tile * TILE_TT, TILE_TT, &s.full[stg]);
    bulk_g2s(d.GL, p.GL + tile * TILE_GL, TILE_GL, &s.full[stg]);
    return true;
  };
  // each warp fetches its own 16 value columns of dO for step i (rows beyond the chunk are zero-filled)
  auto fetch_do = [&](int i) {
    const ChunkInfo ci = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, c_end - 1 - i);
    unsigned char* slab = s.dO[warp][i & 1];
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int pc = lane + 32 * it, t = pc >> 1, half = pc & 1;
      const bool ok = t < ci.len;
      const __nv_bfloat16* src = p.d_o + (static_cast<size_t>(ci.tok0 + (ok ? t : 0)) * p.H + h) * VD + v0 + half * 8;
      cp_async16(slab + do_slab_off(t, half), src, ok);
    }
    cp_async_commit();
  };

  if (tid == 0) {
    for (int i = 0; i < RS_STAGES - 1 && i < nchunks; ++i) issue(i);
  }
  if (nchunks > 0) fetch_do(0);

  float dhT[16][4];   // transposed state gradient: rows v0+gid (+8), columns nt*8 + 2 tig (+1)
  {
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int kk = nt * 8 + tig * 2;
      if (p.d_ht) {
        dhT[nt][0] = __ldg(p.d_ht + sb + static_cast<size_t>(kk) * VD + v0 + gid);
        dhT[nt][1] = __ldg(p.d_ht + sb + static_cast<size_t>(kk + 1) * VD + v0 + gid);
        dhT[nt][2] = __ldg(p.d_ht + sb + static_cast<size_t>(kk) * VD + v0 + gid + 8);
        dhT[nt][3] = __ldg(p.d_ht + sb + static_cast<size_t>(kk + 1) * VD + v0 + gid + 8);
      } else {
        dhT[nt][0] = dhT[nt][1] = dhT[nt][2] = dhT[nt][3] = 0.f;
      }
    }
  }

  bool failed = false;
  for (int i = 0; i < nchunks; ++i) {
    const int stg = i % RS_STAGES;
    const int c = c_end - 1 - i;
    if (tid == 0 && i + RS_STAGES - 1 < nchunks) {
      if (!issue(i + RS_STAGES - 1)) atomicOr(p.status, 4u);
    }
    __syncwarp();
    if (i + 1 < nchunks) {
      fetch_do(i + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    if (!mbar_wait(&s.full[stg], (i / RS_STAGES) & 1)) {
      failed = true;
      break;
    }
    const RScanStage& d = s.st[stg];
    const size_t tile = static_cast<size_t>(c) * p.H + h;
    const uint32_t slab = smem_u32(s.dO[warp][i & 1]);

    // dh' as bf16 A fragments; this is also what the per-chunk kernel reads back
    uint32_t dhA[8][4];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      dhA[ks][0] = pack_bf16(dhT[2 * ks][0], dhT[2 * ks][1]);
      dhA[ks][1] = pack_bf16(dhT[2 * ks][2], dhT[2 * ks][3]);
      dhA[ks][2] = pack_bf16(dhT[2 * ks + 1][0], dhT[2 * ks + 1][1]);
      dhA[ks][3] = pack_bf16(dhT[2 * ks + 1][2], dhT[2 * ks + 1][3]);
    }
    {
      unsigned char* g = p.DH + tile * TILE_VK;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int kk = ks * 16 + tig * 2;
        *reinterpret_cast<uint32_t*>(g + vk_off(v0 + gid, kk)) = dhA[ks][0];
        *reinterpret_cast<uint32_t*>(g + vk_off(v0 + gid + 8, kk)) = dhA[ks][1];
        *reinterpret_cast<uint32_t*>(g + vk_off(v0 + gid, kk + 8)) = dhA[ks][2];
        *reinterpret_cast<uint32_t*>(g + vk_off(v0 + gid + 8, kk + 8)) = dhA[ks][3];
      }
    }
    // dO^T as A fragments: A[m = v][k = t] from the slab stored [t][v]  (transposed ldmatrix)
    uint32_t doA[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int t = ks * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldsm_x4_t(doA[ks], slab + do_slab_off(t, (lane >> 3) & 1));
    }
    // dv_new^T = dO^T Aqk + dh'^T kg^T      (rows: value columns; columns: tokens j)
    float dvn[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) dvn[nt][0] = dvn[nt][1] = dvn[nt][2] = dvn[nt][3] = 0.f;
    const uint32_t abase = smem_u32(d.AQK), kbase = smem_u32(d.KG), qbase = smem_u32(d.QG), wbase = smem_u32(d.W);
    const int brow = (lane & 7) + ((lane >> 4) << 3), bcol = ((lane >> 3) & 1) << 3;            // B stored [n][k]
    const int trow = (lane & 7) + (((lane >> 3) & 1) << 3), tcol = (lane >> 4) << 3;            // B stored [k][n]
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm_x4_t(b, abase + swz<128>(ks * 16 + trow, np * 16 + tcol));     // B[k=t][n=j] = Aqk[t][j]
        mma16816(dvn[2 * np], doA[ks], b[0], b[1]);
        mma16816(dvn[2 * np + 1], doA[ks], b[2], b[3]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm_x4(b, kbase + swz<256>(np * 16 + brow, ks * 16 + bcol));       // B[k=kk][n=j] = kg[j][kk]
        mma16816(dvn[2 * np], dhA[ks], b[0], b[1]);
        mma16816(dvn[2 * np + 1], dhA[ks], b[2], b[3]);
      }
    }
    uint32_t dvA[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      dvA[ks][0] = pack_bf16(dvn[2 * ks][0], dvn[2 * ks][1]);
      dvA[ks][1] = pack_bf16(dvn[2 * ks][2], dvn[2 * ks][3]);
      dvA[ks][2] = pack_bf16(dvn[2 * ks + 1][0], dvn[2 * ks + 1][1]);
      dvA[ks][3] = pack_bf16(dvn[2 * ks + 1][2], dvn[2 * ks + 1][3]);
    }
    {
      unsigned char* g = p.DVNEWT + tile * TILE_VT;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const int t = ks * 16 + tig * 2;
        *reinterpret_cast<uint32_t*>(g + swz<128>(v0 + gid, t)) = dvA[ks][0];
        *reinterpret_cast<uint32_t*>(g + swz<128>(v0 + gid + 8, t)) = dvA[ks][1];
        *reinterpret_cast<uint32_t*>(g + swz<128>(v0 + gid, t + 8)) = dvA[ks][2];
        *reinterpret_cast<uint32_t*>(g + swz<128>(v0 + gid + 8, t + 8)) = dvA[ks][3];
      }
    }
    // dh^T = dh'^T Diag(Gam_last) + dO^T qg - dv_new^T w
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const float2 gl = *reinterpret_cast<const float2*>(&d.GL[nt * 8 + tig * 2]);
      dhT[nt][0] *= gl.x; dhT[nt][1] *= gl.y; dhT[nt][2] *= gl.x; dhT[nt][3] *= gl.y;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t dneg[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) dneg[e] = dvA[ks][e] ^ 0x80008000u;
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b[4];
        ldsm_x4_t(b, qbase + swz<256>(ks * 16 + trow, np * 16 + tcol));     // B[k=t][n=kk] = qg[t][kk]
        mma16816(dhT[2 * np], doA[ks], b[0], b[1]);
        mma16816(dhT[2 * np + 1], doA[ks], b[2], b[3]);
        ldsm_x4_t(b, wbase + swz<256>(ks * 16 + trow, np * 16 + tcol));     // B[k=j][n=kk] = w[j][kk]
        mma16816(dhT[2 * np], dneg, b[0], b[1]);
        mma16816(dhT[2 * np + 1], dneg, b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&s.empty[stg]);
  }
  if (failed && lane == 0) atomicOr(p.status, 8u);

  if (p.dh0 && !failed) {
    const size_t sb = (static_cast<size_t>(seq) * p.H + h) * KD * VD;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int kk = nt * 8 + tig * 2;
      p.dh0[sb + static_cast<size_t>(kk) * VD + v0 + gid] = dhT[nt][0];
      p.dh0[sb + static_cast<size_t>(kk + 1) * VD + v0 + gid] = dhT[nt][1];
      p.dh0[sb + static_cast<size_t>(kk) * VD + v0 + gid + 8] = dhT[nt][2];
      p.dh0[sb + static_cast<size_t>(kk + 1) * VD + v0 + gid + 8] = dhT[nt][3];
    }
  }
}


// =================================================================================================
// per-chunk backward: tensor-core part
// =================================================================================================
constexpr int QS = 136;   // bf16 elements per padded 128-wide row (272 B)
constexpr int GS = 136;   // floats per padded row of G
constexpr int TS = 72;    // bf16 elements per padded 64-wide row (144 B)

struct MainSmem {
  __nv_bfloat16 q[C * QS];
  __nv_bfloat16 k[C * QS];
  __nv_bfloat16 v[C * QS];
  float G[C * GS];
  float beta[C];
  union {
    float red[8][C];        // per-warp partial row sums of dbeta (end of the kernel)
    float hdh[4][KD];       // partial sums over v of h * dh' (phase A)
  };
  float dgl[KD];            // extra gradient of G at the chunk's last row
  float2 Ad[4][16][16];     // diagonal 16x16 blocks of (dAqk, beta dAkk), fp32
  unsigned char TI[TILE_TT];
  unsigned char RKK[TILE_TT];
  __nv_bfloat16 dO[C * QS];            // phase A;  later X  [64][TS]
  unsigned char HS[TILE_VK];           // phase A;  later kG [64][QS] + dT [64][TS]
  unsigned char DH[TILE_VK];           // phase A;  later dw [64][QS] + dAk [64][TS]
  unsigned char VN[TILE_VT];           // phase A;  later dAq [64][TS]
  unsigned char DVN[TILE_VT];          // phases A and B
  uint64_t bar, bar2;
};
constexpr int FS = 136;   // floats per padded row of the staged fp32 [64][128] matrices
static_assert(3 * C * FS * 4 <= C * QS * 2 + 2 * TILE_VK + 2 * TILE_VT, "staged dq/dk+/dk- must fit the dead regions");
static_assert(sizeof(MainSmem) <= 227 * 1024, "MainSmem too large");
static_assert(C * QS * 2 + C * TS * 2 <= TILE_VK, "aliasing of HS/DH regions");
static_assert(C * TS * 2 <= TILE_VT && C * TS * 2 <= C * QS * 2, "aliasing of VN/dO regions");

__global__ void __launch_bounds__(256, 1) kda_chunk_bwd_main_kernel(const MainParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  MainSmem& s = *reinterpret_cast<MainSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  // Persistent CTAs: tile = (chunk, head), walked with stride gridDim.x.  The state tiles and dO of the NEXT
  // tile are fetched while this tile's last phase runs, so only the first tile waits for its loads.
  const long long total_tiles = static_cast<long long>(p.seq_chunk_off[p.N]) * p.H;
  if (tid == 0) {
    mbar_init(&s.bar, 1);
    mbar_init(&s.bar2, 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto fetch_state = [&](long long idx) {      // thread 0: HS, DH, v_new^T, dv_new^T of tile idx
    const size_t tl = static_cast<size_t>(idx);
    mbar_expect_tx(&s.bar, 2 * TILE_VK + 2 * TILE_VT);
    bulk_g2s(s.HS, p.HS + tl * TILE_VK, TILE_VK, &s.bar);
    bulk_g2s(s.DH, p.DH + tl * TILE_VK, TILE_VK, &s.bar);
    bulk_g2s(s.VN, p.VNEWT + tl * TILE_VT, TILE_VT, &s.bar);
    bulk_g2s(s.DVN, p.DVNEWT + tl * TILE_VT, TILE_VT, &s.bar);
  };
  auto fetch_do = [&](long long idx) {          // all threads: dO rows of tile idx (one cp.async group)
    const int cc = static_cast<int>(idx / p.H), hh = static_cast<int>(idx % p.H);
    const ChunkInfo cn = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, cc);
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const bool ok = r < cn.len;
      const size_t row = (static_cast<size_t>(cn.tok0 + (ok ? r : 0)) * p.H + hh) * KD + pc * 8;
      cp_async16(&s.dO[r * QS + pc * 8], p.d_o + row, ok);
    }
    cp_async_commit();
  };
  if (static_cast<long long>(blockIdx.x) < total_tiles) {
    if (tid == 0) fetch_state(blockIdx.x);
    fetch_do(blockIdx.x);
  }

  int it = 0;
  for (long long idx = blockIdx.x; idx < total_tiles; idx += gridDim.x, ++it) {
  const int c = static_cast<int>(idx / p.H), h = static_cast<int>(idx % p.H);
  const ChunkInfo ci = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, c);
  const int len = ci.len;
  const size_t tile = static_cast<size_t>(idx);
  const long long next_idx = idx + gridDim.x;
  long long* const dbg = (it == 2) ? p.dbg : nullptr;   // development aid: clocks of a steady-state tile
  KDA_DBG_CLOCK(dbg, 0);

  // ---- second load group (q, k, v, g, Tm, raw kk): lands behind phase A ------------------------------
  if (tid == 0) {
    mbar_expect_tx(&s.bar2, 2 * TILE_TT);
    bulk_g2s(s.TI, p.TI + tile * TILE_TT, TILE_TT, &s.bar2);
    bulk_g2s(s.RKK, p.RKK + tile * TILE_TT, TILE_TT, &s.bar2);
  }
  for (int i = tid; i < C * 16; i += 256) {
    const int r = i >> 4, pc = i & 15;
    const bool ok = r < len;
    const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 8;
    cp_async16(&s.q[r * QS + pc * 8], p.q + row, ok);
    cp_async16(&s.k[r * QS + pc * 8], p.k + row, ok);
    cp_async16(&s.v[r * QS + pc * 8], p.v + row, ok);
  }
  for (int i = tid; i < C * 32; i += 256) {
    const int r = i >> 5, pc = i & 31;
    const bool ok = r < len;
    const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 4;
    cp_async16(&s.G[r * GS + pc * 4], p.g + row, ok);
  }
  cp_async_commit();
  if (tid < C) s.beta[tid] = (tid < len) ? __ldg(p.beta + static_cast<size_t>(ci.tok0 + tid) * p.H + h) : 0.f;
  cp_async_wait<1>();   // this tile's dO (issued one tile ago, or in the prologue) has landed
  __syncthreads();
  const bool tiles_ok = mbar_wait(&s.bar, it & 1);
  if (!tiles_ok && tid == 0) atomicOr(p.status, 16u);

  KDA_DBG_CLOCK(dbg, 1);
  const int n0 = warp * 16;                                    // this warp's 16 output columns (kk or v)
  const int j0 = warp * 8;                                     // this warp's 8 columns of the 64x64 products
  const int trow = (lane & 7) + (((lane >> 3) & 1) << 3), tcol = (lane >> 4) << 3;   // B stored [k][n]
  const int arow = lane & 15, acol = (lane >> 4) << 3;                                // A stored [m][k]
  const int atrow = (lane & 7) + ((lane >> 4) << 3), atcol = ((lane >> 3) & 1) << 3;  // A stored [k][m]
  const uint32_t uHS = smem_u32(s.HS), uDH = smem_u32(s.DH), uVN = smem_u32(s.VN), uDVN = smem_u32(s.DVN);
  const uint32_t uTI = smem_u32(s.TI);

  // =========================== phase A: state-dependent products ====================================
  float dqa[4][2][4], dwa[4][2][4], dkn[4][2][4], dAq[4][4];
#pragma unroll
  for (int m = 0; m < 4; ++m) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      dqa[m][0][e] = dqa[m][1][e] = dwa[m][0][e] = dwa[m][1][e] = dkn[m][0][e] = dkn[m][1][e] = 0.f;
      dAq[m][e] = 0.f;
    }
  }
#pragma unroll 1
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t bh[4], bd[4];
    ldsm_x4_t(bh, uHS + vk_off(ks * 16 + trow, n0 + tcol));      // B[k=v][n=kk] = h[kk][v]
    ldsm_x4_t(bd, uDH + vk_off(ks * 16 + trow, n0 + tcol));      // B[k=v][n=kk] = dh'[kk][v]
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      uint32_t a[4];
      ldsm_x4(a, smem_u32(&s.dO[(mt * 16 + arow) * QS + ks * 16 + acol]));             // dO[t][v]
      mma16816(dqa[mt][0], a, bh[0], bh[1]);
      mma16816(dqa[mt][1], a, bh[2], bh[3]);
      ldsm_x4_t(a, uDVN + swz<128>(ks * 16 + atrow, mt * 16 + atcol));                 // dv_new[t][v] from [v][t]
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] ^= 0x80008000u;
      mma16816(dwa[mt][0], a, bh[0], bh[1]);
      mma16816(dwa[mt][1], a, bh[2], bh[3]);
      ldsm_x4_t(a, uVN + swz<128>(ks * 16 + atrow, mt * 16 + atcol));                  // v_new[t][v] from [v][t]
      mma16816(dkn[mt][0], a, bd[0], bd[1]);
      mma16816(dkn[mt][1], a, bd[2], bd[3]);
    }
  }
#pragma unroll 1
  for (int ks2 = 0; ks2 < 4; ++ks2) {
    uint32_t b[4];
    ldsm_x4_t(b, uVN + swz<128>(ks2 * 32 + lane, j0));             // B[k=v][n=j] = v_new[j][v]
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      uint32_t a[4];
      ldsm_x4(a, smem_u32(&s.dO[(mt * 16 + arow) * QS + (2 * ks2) * 16 + acol]));
      mma16816(dAq[mt], a, b[0], b[1]);
      ldsm_x4(a, smem_u32(&s.dO[(mt * 16 + arow) * QS + (2 * ks2 + 1) * 16 + acol]));
      mma16816(dAq[mt], a, b[2], b[3]);
    }
  }
  {  // sum over v of h * dh' (feeds the gradient of G at the chunk's last row)
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
  cp_async_wait<0>();
  __syncthreads();   // (1) HS, DH, VN, dO are dead from here on; q, k, v, g have landed
  KDA_DBG_CLOCK(dbg, 2);
  {  // G = cumsum(g) * log2(e): two half-columns per column, then the carry
    const int col = tid & 127, half = tid >> 7;
    float gv[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) gv[i] = s.G[(half * 32 + i) * GS + col];
    float run = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      run += gv[i];
      gv[i] = run;
    }
    if (half == 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i) s.G[i * GS + col] = gv[i] * LOG2E;
    }
    __syncthreads();
    if (half == 1) {
      const float carry = s.G[31 * GS + col];
#pragma unroll
      for (int i = 0; i < 32; ++i) s.G[(32 + i) * GS + col] = carry + gv[i] * LOG2E;
    }
    if (!mbar_wait(&s.bar2, it & 1) && tid == 0) atomicOr(p.status, 16u);
    __syncthreads();
  }

  // ---- re-use of the dead regions --------------------------------------------------------------------
  __nv_bfloat16* sKG = reinterpret_cast<__nv_bfloat16*>(s.HS);                    // k * Gam      [64][QS]
  __nv_bfloat16* sDT = reinterpret_cast<__nv_bfloat16*>(s.HS + C * QS * 2);       // dTm          [64][TS]
  __nv_bfloat16* sDW = reinterpret_cast<__nv_bfloat16*>(s.DH);                    // dw           [64][QS]
  __nv_bfloat16* sDAK = reinterpret_cast<__nv_bfloat16*>(s.DH + C * QS * 2);      // beta dAkk    [64][TS]
  __nv_bfloat16* sDAQ = reinterpret_cast<__nv_bfloat16*>(s.VN);                   // dAqk         [64][TS]
  __nv_bfloat16* sX = s.dO;                                                       // dTm Tm^T     [64][TS]

  {
    // dw -> shared (bf16); dq(a) = scale Gam dqg; dk-(a) = dkg exp2(G_last - G); column sums of k dk_end
    float cs[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int col = n0 + nt * 8 + tig * 2;
        const float2 Gl = *reinterpret_cast<const float2*>(&s.G[(C - 1) * GS + col]);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int row = mt * 16 + gid + hh * 8;
          const float2 Gr = *reinterpret_cast<const float2*>(&s.G[row * GS + col]);
          const float2 kk = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[row * QS + col]));
          *reinterpret_cast<uint32_t*>(&sDW[row * QS + col]) = pack_bf16(dwa[mt][nt][2 * hh], dwa[mt][nt][2 * hh + 1]);
          dqa[mt][nt][2 * hh] *= p.scale * ex2(Gr.x);
          dqa[mt][nt][2 * hh + 1] *= p.scale * ex2(Gr.y);
          dkn[mt][nt][2 * hh] *= ex2(Gl.x - Gr.x);
          dkn[mt][nt][2 * hh + 1] *= ex2(Gl.y - Gr.y);
          cs[nt][0] += kk.x * dkn[mt][nt][2 * hh];
          cs[nt][1] += kk.y * dkn[mt][nt][2 * hh + 1];
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float x = cs[nt][e];
        x += __shfl_xor_sync(0xffffffffu, x, 4);
        x += __shfl_xor_sync(0xffffffffu, x, 8);
        x += __shfl_xor_sync(0xffffffffu, x, 16);
        if (gid == 0) {
          const int col = n0 + nt * 8 + tig * 2 + e;
          const float hd = s.hdh[0][col] + s.hdh[1][col] + s.hdh[2][col] + s.hdh[3][col];
          s.dgl[col] = x + ex2(s.G[(C - 1) * GS + col]) * hd;
        }
      }
    }
    // dAqk: keep j <= t; bf16 copy for the off-diagonal products, diagonal 16x16 blocks in fp32 to global
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8, col = j0 + tig * 2;
        const float x0 = (col <= row) ? dAq[mt][2 * hh] : 0.f;
        const float x1 = (col + 1 <= row) ? dAq[mt][2 * hh + 1] : 0.f;
        *reinterpret_cast<uint32_t*>(&sDAQ[row * TS + col]) = pack_bf16(x0, x1);
        if ((warp >> 1) == mt) {
          s.Ad[mt][gid + hh * 8][col & 15].x = p.scale * x0;      // scale folded in for phase D
          s.Ad[mt][gid + hh * 8][(col & 15) + 1].x = p.scale * x1;
        }
      }
    }
    // k * Gam
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const uint4 kr = *reinterpret_cast<const uint4*>(&s.k[r * QS + pc * 8]);
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[r * GS + pc * 8]);
      const float4 Gb = *reinterpret_cast<const float4*>(&s.G[r * GS + pc * 8 + 4]);
      const float2 k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y), k2 = unpack_bf16(kr.z), k3 = unpack_bf16(kr.w);
      *reinterpret_cast<uint4*>(&sKG[r * QS + pc * 8]) =
          make_uint4(pack_bf16(k0.x * ex2(Ga.x), k0.y * ex2(Ga.y)), pack_bf16(k1.x * ex2(Ga.z), k1.y * ex2(Ga.w)),
                     pack_bf16(k2.x * ex2(Gb.x), k2.y * ex2(Gb.y)), pack_bf16(k3.x * ex2(Gb.z), k3.y * ex2(Gb.w)));
    }
  }
  __syncthreads();   // (2)
  KDA_DBG_CLOCK(dbg, 3);

  // =========================== phase B: through Tm = (I + Akk)^-1 =====================================
  float pb[4][2];    // dbeta partial row sums: rows mt*16 + gid (+8)
#pragma unroll
  for (int m = 0; m < 4; ++m) pb[m][0] = pb[m][1] = 0.f;
  {
    // dTm = du (beta v)^T + dw (beta k Gam)^T        (this warp: columns j0..j0+7)
    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
#pragma unroll 1
    for (int ks2 = 0; ks2 < 4; ++ks2) {
      uint32_t bv[4], bk[4];
      ldsm_x4(bv, smem_u32(&s.v[(j0 + (lane & 7)) * QS + ks2 * 32 + (lane >> 3) * 8]));     // B[k=v][n=j] = v[j][v]
      ldsm_x4(bk, smem_u32(&sKG[(j0 + (lane & 7)) * QS + ks2 * 32 + (lane >> 3) * 8]));     // B[k=kk][n=j] = kG[j][kk]
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t a[4];
        ldsm_x4_t(a, uDVN + swz<128>((2 * ks2) * 16 + atrow, mt * 16 + atcol));
        mma16816(acc[mt], a, bv[0], bv[1]);
        ldsm_x4_t(a, uDVN + swz<128>((2 * ks2 + 1) * 16 + atrow, mt * 16 + atcol));
        mma16816(acc[mt], a, bv[2], bv[3]);
        ldsm_x4(a, smem_u32(&sDW[(mt * 16 + arow) * QS + (2 * ks2) * 16 + acol]));
        mma16816(acc[mt], a, bk[0], bk[1]);
        ldsm_x4(a, smem_u32(&sDW[(mt * 16 + arow) * QS + (2 * ks2 + 1) * 16 + acol]));
        mma16816(acc[mt], a, bk[2], bk[3]);
      }
    }
    const float2 bj = *reinterpret_cast<const float2*>(&s.beta[j0 + tig * 2]);
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8;
        *reinterpret_cast<uint32_t*>(&sDT[row * TS + j0 + tig * 2]) = pack_bf16(acc[mt][2 * hh] * bj.x, acc[mt][2 * hh + 1] * bj.y);
      }
    }
  }
  __syncthreads();   // (3)
  KDA_DBG_CLOCK(dbg, 4);
  {
    // X = dTm Tm^T
    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
#pragma unroll
    for (int ks2 = 0; ks2 < 2; ++ks2) {
      uint32_t b[4];
      ldsm_x4(b, uTI + swz<128>(j0 + (lane & 7), ks2 * 32 + (lane >> 3) * 8));               // B[k=m][n=j] = Tm[j][m]
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t a[4];
        ldsm_x4(a, smem_u32(&sDT[(mt * 16 + arow) * TS + (2 * ks2) * 16 + acol]));
        mma16816(acc[mt], a, b[0], b[1]);
        ldsm_x4(a, smem_u32(&sDT[(mt * 16 + arow) * TS + (2 * ks2 + 1) * 16 + acol]));
        mma16816(acc[mt], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8;
        *reinterpret_cast<uint32_t*>(&sX[row * TS + j0 + tig * 2]) = pack_bf16(acc[mt][2 * hh], acc[mt][2 * hh + 1]);
      }
    }
  }
  __syncthreads();   // (4)
  KDA_DBG_CLOCK(dbg, 5);
  // Tm^T as A fragments: A[m=i][k=m'] = Tm[m'][i]
  uint32_t tA[4][4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) ldsm_x4_t(tA[mt][ks], uTI + swz<128>(ks * 16 + atrow, mt * 16 + atcol));
  }
  {
    // dAkk = -(Tm^T X), strictly lower; dbeta += <dAkk, raw kk>; beta_t dAkk -> shared / diagonal blocks
    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
#pragma unroll
    for (int ks2 = 0; ks2 < 2; ++ks2) {
      uint32_t b[4];
      ldsm_x4_t(b, smem_u32(&sX[(ks2 * 32 + lane) * TS + j0]));                             // B[k=m'][n=j] = X[m'][j]
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        mma16816(acc[mt], tA[mt][2 * ks2], b[0], b[1]);
        mma16816(acc[mt], tA[mt][2 * ks2 + 1], b[2], b[3]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8, col = j0 + tig * 2;
        const float x0 = (col < row) ? -acc[mt][2 * hh] : 0.f;
        const float x1 = (col + 1 < row) ? -acc[mt][2 * hh + 1] : 0.f;
        const float2 raw = unpack_bf16(*reinterpret_cast<const uint32_t*>(s.RKK + swz<128>(row, col)));
        pb[mt][hh] += x0 * raw.x + x1 * raw.y;
        const float br = s.beta[row];
        *reinterpret_cast<uint32_t*>(&sDAK[row * TS + col]) = pack_bf16(br * x0, br * x1);
        if ((warp >> 1) == mt) {
          s.Ad[mt][gid + hh * 8][col & 15].y = br * x0;
          s.Ad[mt][gid + hh * 8][(col & 15) + 1].y = br * x1;
        }
      }
    }
  }
  float dkp[4][2][4];
  {
    // dv = beta (Tm^T du);   dk+(a) = Gam beta (Tm^T dw)
    float acc[4][2][4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][0][e] = acc[m][1][e] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t b[4];
      ldsm_x4(b, uDVN + swz<128>(n0 + (lane & 7) + ((lane >> 4) << 3), ks * 16 + (((lane >> 3) & 1) << 3)));   // B[k=t][n=v] = du[t][v]
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        mma16816(acc[mt][0], tA[mt][ks], b[0], b[1]);
        mma16816(acc[mt][1], tA[mt][ks], b[2], b[3]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8;
        const float br = s.beta[row];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = n0 + nt * 8 + tig * 2;
          const float2 vv = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.v[row * QS + col]));
          pb[mt][hh] += acc[mt][nt][2 * hh] * vv.x + acc[mt][nt][2 * hh + 1] * vv.y;
          if (row < len)
            *reinterpret_cast<uint32_t*>(p.dv + (static_cast<size_t>(ci.tok0 + row) * p.H + h) * VD + col) =
                pack_bf16(br * acc[mt][nt][2 * hh], br * acc[mt][nt][2 * hh + 1]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
#pragma unroll
      for (int e = 0; e < 4; ++e) dkp[m][0][e] = dkp[m][1][e] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t b[4];
      ldsm_x4_t(b, smem_u32(&sDW[(ks * 16 + trow) * QS + n0 + tcol]));                       // B[k=t][n=kk] = dw[t][kk]
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        mma16816(dkp[mt][0], tA[mt][ks], b[0], b[1]);
        mma16816(dkp[mt][1], tA[mt][ks], b[2], b[3]);
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int row = mt * 16 + gid + hh * 8;
        const float br = s.beta[row];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int col = n0 + nt * 8 + tig * 2;
          const float2 kg = unpack_bf16(*reinterpret_cast<const uint32_t*>(&sKG[row * QS + col]));
          const float2 Gr = *reinterpret_cast<const float2*>(&s.G[row * GS + col]);
          pb[mt][hh] += dkp[mt][nt][2 * hh] * kg.x + dkp[mt][nt][2 * hh + 1] * kg.y;
          dkp[mt][nt][2 * hh] *= br * ex2(Gr.x);
          dkp[mt][nt][2 * hh + 1] *= br * ex2(Gr.y);
        }
      }
    }
  }
  __syncthreads();   // (5) dAq / dAk (bf16) complete
  KDA_DBG_CLOCK(dbg, 6);

  // =========================== phase C: off-diagonal 16x16 blocks of the intra-chunk terms ============
  // decay factored around the first row r0 = 16 I of row block I (both factors <= 1), as in the forward
#pragma unroll 1
  for (int I = 1; I < 4; ++I) {
    const int r0 = 16 * I;
    float Lf[2][2][2];                // Lf[nt][hh][e]: exp2(G[t] - G[r0]) at the accumulator positions
    float accq[2][4], acck[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) accq[nt][0] = accq[nt][1] = accq[nt][2] = accq[nt][3] = acck[nt][0] = acck[nt][1] = acck[nt][2] = acck[nt][3] = 0.f;
    float Rb[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) Rb[nt] = s.G[r0 * GS + n0 + nt * 8 + gid];
#pragma unroll 1
    for (int ksj = 0; ksj < I; ++ksj) {
      uint32_t aq[4], ak[4];
      ldsm_x4(aq, smem_u32(&sDAQ[(r0 + arow) * TS + ksj * 16 + acol]));
      ldsm_x4(ak, smem_u32(&sDAK[(r0 + arow) * TS + ksj * 16 + acol]));
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int n = n0 + nt * 8 + gid;
        const int ja = ksj * 16 + tig * 2;
        float kr[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = ja + (e & 1) + ((e >> 1) << 3);
          kr[e] = __bfloat162float(s.k[j * QS + n]) * ex2(Rb[nt] - s.G[j * GS + n]);
        }
        const uint32_t b0 = pack_bf16(kr[0], kr[1]), b1 = pack_bf16(kr[2], kr[3]);
        mma16816(accq[nt], aq, b0, b1);
        mma16816(acck[nt], ak, b0, b1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int col = n0 + nt * 8 + tig * 2;
      const float2 Rc = *reinterpret_cast<const float2*>(&s.G[r0 * GS + col]);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const float2 Gr = *reinterpret_cast<const float2*>(&s.G[(r0 + gid + hh * 8) * GS + col]);
        Lf[nt][hh][0] = ex2(Gr.x - Rc.x);
        Lf[nt][hh][1] = ex2(Gr.y - Rc.y);
      }
    }
    // dq, dk+ of row block I  (static register indexing: select the block with a switch)
#define KDA_ADD_ROWBLOCK(II)                                                       \
  _Pragma("unroll") for (int nt = 0; nt < 2; ++nt) {                               \
    _Pragma("unroll") for (int e = 0; e < 4; ++e) {                                \
      dqa[II][nt][e] += p.scale * Lf[nt][e >> 1][e & 1] * accq[nt][e];             \
      dkp[II][nt][e] += Lf[nt][e >> 1][e & 1] * acck[nt][e];                       \
    }                                                                              \
  }
    if (I == 1) { KDA_ADD_ROWBLOCK(1) } else if (I == 2) { KDA_ADD_ROWBLOCK(2) } else { KDA_ADD_ROWBLOCK(3) }
#undef KDA_ADD_ROWBLOCK
    // dk- of the column blocks J < I:  B[k=t][n=kk] = (scale q_t | k_t) exp2(G_t - G_r0),  t in block I
    uint32_t bq[2][2], bk[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int n = n0 + nt * 8 + gid;
      float qv[4], kv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = r0 + tig * 2 + (e & 1) + ((e >> 1) << 3);
        const float f = ex2(s.G[t * GS + n] - Rb[nt]);
        qv[e] = p.scale * __bfloat162float(s.q[t * QS + n]) * f;
        kv[e] = __bfloat162float(s.k[t * QS + n]) * f;
      }
      bq[nt][0] = pack_bf16(qv[0], qv[1]); bq[nt][1] = pack_bf16(qv[2], qv[3]);
      bk[nt][0] = pack_bf16(kv[0], kv[1]); bk[nt][1] = pack_bf16(kv[2], kv[3]);
    }
#pragma unroll
    for (int J = 0; J < 3; ++J) {
      if (J < I) {
        uint32_t aq[4], ak[4];
        ldsm_x4_t(aq, smem_u32(&sDAQ[(r0 + atrow) * TS + J * 16 + atcol]));      // A[m=j][k=t] = dAqk[t][j]
        ldsm_x4_t(ak, smem_u32(&sDAK[(r0 + atrow) * TS + J * 16 + atcol]));
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816(acc, aq, bq[nt][0], bq[nt][1]);
          mma16816(acc, ak, bk[nt][0], bk[nt][1]);
          const int col = n0 + nt * 8 + tig * 2;
          const float2 Rc = *reinterpret_cast<const float2*>(&s.G[r0 * GS + col]);
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const float2 Gj = *reinterpret_cast<const float2*>(&s.G[(J * 16 + gid + hh * 8) * GS + col]);
            dkn[J][nt][2 * hh] += ex2(Rc.x - Gj.x) * acc[2 * hh];
            dkn[J][nt][2 * hh + 1] += ex2(Rc.y - Gj.y) * acc[2 * hh + 1];
          }
        }
      }
    }
  }

  KDA_DBG_CLOCK(dbg, 7);
  __syncthreads();   // (6) every shared-memory operand of phase C has been read: the regions become staging
  // ---- stage the fp32 partial dq / dk+ / dk- as [64][FS] matrices; dbeta partial row sums --------------
  float* stq = reinterpret_cast<float*>(s.dO);
  float* stp = stq + C * FS;
  float* stn = stp + C * FS;
  {
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int o = (mt * 16 + gid + hh * 8) * FS + n0 + nt * 8 + tig * 2;
          *reinterpret_cast<float2*>(stq + o) = make_float2(dqa[mt][nt][2 * hh], dqa[mt][nt][2 * hh + 1]);
          *reinterpret_cast<float2*>(stp + o) = make_float2(dkp[mt][nt][2 * hh], dkp[mt][nt][2 * hh + 1]);
          *reinterpret_cast<float2*>(stn + o) = make_float2(dkn[mt][nt][2 * hh], dkn[mt][nt][2 * hh + 1]);
        }
      }
    }
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float x = pb[mt][hh];
        x += __shfl_xor_sync(0xffffffffu, x, 1);
        x += __shfl_xor_sync(0xffffffffu, x, 2);
        if (tig == 0) s.red[warp][mt * 16 + gid + hh * 8] = x;
      }
    }
  }
  __syncthreads();   // (7)
  KDA_DBG_CLOCK(dbg, 8);
  if (tid < len) {
    float x = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) x += s.red[w][tid];
    p.dbeta[static_cast<size_t>(ci.tok0 + tid) * p.H + h] = x;
  }

  // =========================== phase D: diagonal 16x16 blocks pairwise + epilogue =======================
  // One thread per PAIR of key columns and 16-row block, all arithmetic in packed fp32x2 (sm_100 FFMA2).
  // The decay between rows of a block is the running product of the per-row factors
  // lam_s = exp2(G_s - G_{s-1}) <= 1 (range-safe, no exp per pair).
  // dG = q dq + k (dk+ - dk-), dg = reverse cumsum over the chunk, final dq / dk / dg.
  {
    const int kp = tid & 63, b = tid >> 6, kk = 2 * kp;
    float4* sAd4 = reinterpret_cast<float4*>(s.TI);          // (a1, a1, a2, a2) per (block, t, j): TI, RKK are dead
    static_assert(4 * 16 * 16 * sizeof(float4) <= 2 * TILE_TT, "duplicated diagonal blocks must fit TI + RKK");
    for (int i = tid; i < 1024; i += 256) {
      const float2 a = (&s.Ad[0][0][0])[i];
      sAd4[i] = make_float4(a.x, a.x, a.y, a.y);
    }
    float2 cq[16], cp[16], cn[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int t = b * 16 + i;
      cq[i] = *reinterpret_cast<const float2*>(&stq[t * FS + kk]);
      cp[i] = *reinterpret_cast<const float2*>(&stp[t * FS + kk]);
      cn[i] = *reinterpret_cast<const float2*>(&stn[t * FS + kk]);
    }
    fence_proxy_async();
    __syncthreads();   // (8) the staging regions are free again: fetch the next tile's phase-A operands
    if (next_idx < total_tiles) {
      if (tid == 0) fetch_state(next_idx);
      fetch_do(next_idx);
    }
    KDA_DBG_CLOCK(dbg, 10);
    float2 lam[16], qv[16], kv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int t = b * 16 + i;
      const float2 Gt = *reinterpret_cast<const float2*>(&s.G[t * GS + kk]);
      const float2 Gp = (i > 0) ? *reinterpret_cast<const float2*>(&s.G[(t - 1) * GS + kk]) : Gt;
      lam[i] = make_float2(ex2(Gt.x - Gp.x), ex2(Gt.y - Gp.y));
      qv[i] = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[t * QS + kk]));
      kv[i] = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[t * QS + kk]));
    }
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      float2 D = make_float2(1.f, 1.f);
#pragma unroll
      for (int j = t; j >= 0; --j) {
        const float4 a = sAd4[(b * 16 + t) * 16 + j];
        const float2 a1 = make_float2(a.x, a.y), a2 = make_float2(a.z, a.w);
        const float2 kd = __fmul2_rn(kv[j], D);
        cq[t] = __ffma2_rn(a1, kd, cq[t]);
        cp[t] = __ffma2_rn(a2, kd, cp[t]);
        const float2 tmp = __ffma2_rn(a2, kv[t], __fmul2_rn(a1, qv[t]));
        cn[j] = __ffma2_rn(D, tmp, cn[j]);
        D = __fmul2_rn(D, lam[j]);      // decay from row j-1 to row t
      }
    }
    KDA_DBG_CLOCK(dbg, 11);
    // dq, dk replace this thread's own q, k elements in shared memory (nobody else reads them any more)
    float2 dGv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int t = b * 16 + i;
      const float2 dkk = make_float2(cp[i].x + cn[i].x, cp[i].y + cn[i].y);
      dGv[i] = make_float2(qv[i].x * cq[i].x + kv[i].x * (cp[i].x - cn[i].x), qv[i].y * cq[i].y + kv[i].y * (cp[i].y - cn[i].y));
      *reinterpret_cast<uint32_t*>(&s.q[t * QS + kk]) = pack_bf16(cq[i].x, cq[i].y);
      *reinterpret_cast<uint32_t*>(&s.k[t * QS + kk]) = pack_bf16(dkk.x, dkk.y);
    }
    if (b == 3) {
      dGv[15].x += s.dgl[kk];
      dGv[15].y += s.dgl[kk + 1];
    }
    float* carry = &s.red[0][0];          // [4][128]; the dbeta partials in it were consumed before sync (8)
    {
      float2 run = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 15; i >= 0; --i) {
        run.x += dGv[i].x;
        run.y += dGv[i].y;
        dGv[i] = run;
      }
      *reinterpret_cast<float2*>(&carry[b * KD + kk]) = run;
    }
    __syncthreads();
    {
      float2 add = make_float2(0.f, 0.f);
#pragma unroll
      for (int bb = 1; bb < 4; ++bb) {
        if (bb > b) {
          const float2 cb = *reinterpret_cast<const float2*>(&carry[bb * KD + kk]);
          add.x += cb.x;
          add.y += cb.y;
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i)
        *reinterpret_cast<float2*>(&s.G[(b * 16 + i) * GS + kk]) = make_float2(dGv[i].x + add.x, dGv[i].y + add.y);   // dg replaces G
    }
    __syncthreads();
    // coalesced 16-byte stores of dq, dk (bf16) and dg (fp32) rows
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      if (r < len) {
        const size_t row = (static_cast<size_t>(ci.tok0 + r) * p.H + h) * KD + pc * 8;
        *reinterpret_cast<uint4*>(p.dq + row) = *reinterpret_cast<const uint4*>(&s.q[r * QS + pc * 8]);
        *reinterpret_cast<uint4*>(p.dk + row) = *reinterpret_cast<const uint4*>(&s.k[r * QS + pc * 8]);
      }
    }
    for (int i = tid; i < C * 32; i += 256) {
      const int r = i >> 5, pc = i & 31;
      if (r < len) {
        const size_t row = (static_cast<size_t>(ci.tok0 + r) * p.H + h) * KD + pc * 4;
        *reinterpret_cast<float4*>(p.dg + row) = *reinterpret_cast<const float4*>(&s.G[r * GS + pc * 4]);
      }
    }
  }
  KDA_DBG_CLOCK(dbg, 9);
  __syncthreads();   // (9) q, k, G, beta, Ad, dgl, carry may be overwritten by the next tile
  }  // tile loop
}

// =================================================================================================
// q/k L2 normalisation around the backward (use_qk_l2norm): y = x rsqrt(sum x^2 + eps)
// =================================================================================================
__global__ void __launch_bounds__(256) kda_l2norm_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                             __nv_bfloat16* __restrict__ qn, __nv_bfloat16* __restrict__ kn,
                                                             float* __restrict__ rstd, long long rows) {
  const long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  uint2 qr = *reinterpret_cast<const uint2*>(q + r * KD + lane * 4);
  uint2 kr = *reinterpret_cast<const uint2*>(k + r * KD + lane * 4);
  float2 q0 = unpack_bf16(qr.x), q1 = unpack_bf16(qr.y), k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y);
  const float sq = warp_sum(q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y);
  const float sk = warp_sum(k0.x * k0.x + k0.y * k0.y + k1.x * k1.x + k1.y * k1.y);
  const float rq = rsqrtf(sq + L2NORM_EPS), rk = rsqrtf(sk + L2NORM_EPS);
  qr.x = pack_bf16(q0.x * rq, q0.y * rq); qr.y = pack_bf16(q1.x * rq, q1.y * rq);
  kr.x = pack_bf16(k0.x * rk, k0.y * rk); kr.y = pack_bf16(k1.x * rk, k1.y * rk);
  *reinterpret_cast<uint2*>(qn + r * KD + lane * 4) = qr;
  *reinterpret_cast<uint2*>(kn + r * KD + lane * 4) = kr;
  if (lane == 0) {
    rstd[r] = rq;
    rstd[rows + r] = rk;
  }
}

// dx = rstd (dy - y <y, dy>), in place on dq / dk (fla/modules/l2norm.py:190-240)
__global__ void __launch_bounds__(256) kda_l2norm_bwd_kernel(const __nv_bfloat16* __restrict__ qn, const __nv_bfloat16* __restrict__ kn,
                                                             const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dq,
                                                             __nv_bfloat16* __restrict__ dk, long long rows) {
  const long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* y = which ? kn : qn;
    __nv_bfloat16* d = which ? dk : dq;
    const uint2 yr = *reinterpret_cast<const uint2*>(y + r * KD + lane * 4);
    uint2 dr = *reinterpret_cast<const uint2*>(d + r * KD + lane * 4);
    const float2 y0 = unpack_bf16(yr.x), y1 = unpack_bf16(yr.y);
    float2 d0 = unpack_bf16(dr.x), d1 = unpack_bf16(dr.y);
    const float dot = warp_sum(y0.x * d0.x + y0.y * d0.y + y1.x * d1.x + y1.y * d1.y);
    const float rs = rstd[which * rows + r];
    dr.x = pack_bf16(rs * (d0.x - y0.x * dot), rs * (d0.y - y0.y * dot));
    dr.y = pack_bf16(rs * (d1.x - y1.x * dot), rs * (d1.y - y1.y * dot));
    *reinterpret_cast<uint2*>(d + r * KD + lane * 4) = dr;
  }
}

// one persistent CTA per SM (the kernel needs a whole SM's shared memory), never more CTAs than tiles
static int main_grid(int max_chunks, int H) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = static_cast<long long>(max_chunks) * H;
  return static_cast<int>(tiles < sms ? (tiles > 0 ? tiles : 1) : sms);
}

static std::once_flag g_battr_once;
static cudaError_t g_battr_err = cudaSuccess;
static cudaError_t set_bwd_attrs() {
  std::call_once(g_battr_once, [] {
    cudaError_t e = cudaFuncSetAttribute(kda_chunk_bwd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(RScanSmem)));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(kda_chunk_bwd_main_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(sizeof(MainSmem)));
    g_battr_err = e;
  });
  return g_battr_err;
}

}  // namespace kda

extern "C" size_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V, int32_t use_qk_l2norm) {
  (void)K; (void)V;
  return kda::carve_ws(nullptr, nullptr, tokens, N, H, true, use_qk_l2norm != 0).bwd_bytes;
}

extern "C" int kda_chunk_bwd(const kda_chunk_args* args, void* stream) {
  using namespace kda;
  if (!args) return KDA_E_NULL;
  const kda_chunk_args& a = *args;
  int rc = validate_chunk_args(a, true);
  if (rc != KDA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.N == 0) return KDA_OK;
  if (a.tokens == 0) {
    if (a.dh0) {
      const size_t bytes = static_cast<size_t>(a.N) * a.H * KD * VD * sizeof(float);
      return static_cast<int>(a.d_ht ? cudaMemcpyAsync(a.dh0, a.d_ht, bytes, cudaMemcpyDeviceToDevice, st)
                                     : cudaMemsetAsync(a.dh0, 0, bytes, st));
    }
    return KDA_OK;
  }
  const bool l2 = a.use_qk_l2norm != 0;
  ChunkWs w = carve_ws(static_cast<unsigned char*>(a.workspace), static_cast<unsigned char*>(a.bwd_workspace), a.tokens, a.N,
                       a.H, true, l2);
  if (a.workspace_bytes < w.fwd_bytes || a.bwd_workspace_bytes < w.bwd_bytes) return KDA_E_WORKSPACE;
  cudaError_t e = set_bwd_attrs();
  if (e != cudaSuccess) return static_cast<int>(e);
  const int NTmax = static_cast<int>(a.tokens / C + a.N);
  const long long rows = static_cast<long long>(a.tokens) * a.H;
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* k = static_cast<const __nv_bfloat16*>(a.k);
  ProfCall* prof = prof_begin(st);
  if (l2) {
    kda_l2norm_fwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(q, k, w.QN, w.KN, w.RSTD, rows);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
    prof_mark(prof, KDA_STAGE_L2NORM, st);
    q = w.QN;
    k = w.KN;
  }

  RScanParams rp{};
  rp.cu = a.cu_seqlens; rp.seq_chunk_off = w.seq_chunk_off; rp.chunk_seq = w.chunk_seq;
  rp.W = w.W; rp.KG = w.KG; rp.QG = w.QG; rp.AQK = w.AQK; rp.GL = w.GL;
  rp.DH = w.DH; rp.DVNEWT = w.DVNEWT;
  rp.d_o = static_cast<const __nv_bfloat16*>(a.d_o); rp.d_ht = a.d_ht; rp.dh0 = a.dh0; rp.status = w.status;
  rp.N = a.N; rp.H = a.H;
  kda_chunk_bwd_scan_kernel<<<a.N * a.H, RS_THREADS, sizeof(RScanSmem), st>>>(rp);
  if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  prof_mark(prof, KDA_STAGE_BWD_SCAN, st);

  MainParams mp{};
  mp.q = q; mp.k = k; mp.v = static_cast<const __nv_bfloat16*>(a.v); mp.d_o = static_cast<const __nv_bfloat16*>(a.d_o);
  mp.g = a.g; mp.beta = a.beta; mp.cu = a.cu_seqlens; mp.seq_chunk_off = w.seq_chunk_off; mp.chunk_seq = w.chunk_seq;
  mp.TI = w.TI; mp.RKK = w.RKK; mp.HS = w.HS; mp.VNEWT = w.VNEWT; mp.DH = w.DH; mp.DVNEWT = w.DVNEWT;
  mp.dv = static_cast<__nv_bfloat16*>(a.dv); mp.dq = static_cast<__nv_bfloat16*>(a.dq); mp.dk = static_cast<__nv_bfloat16*>(a.dk);
  mp.dbeta = a.dbeta; mp.dg = a.dg; mp.status = w.status; mp.dbg = g_dbg_clocks;
  mp.N = a.N; mp.H = a.H; mp.scale = a.scale;
  if ((e = launch_bwd_main_tc(mp, main_grid(NTmax, a.H), st)) != cudaSuccess) return static_cast<int>(e);
  prof_mark(prof, KDA_STAGE_BWD_MAIN, st);

  if (l2) {
    kda_l2norm_bwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(w.QN, w.KN, w.RSTD, mp.dq, mp.dk, rows);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
    prof_mark(prof, KDA_STAGE_L2NORM, st);
  }
  return KDA_OK;
}
