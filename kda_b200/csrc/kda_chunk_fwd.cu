// Chunked KDA forward for sm_100a: chunk tables, per-chunk preparation, and the state scan.
//
//  kda_chunk_tables_kernel   cu_seqlens -> (first chunk of each sequence, sequence of each chunk); device only,
//                            so that variable-length calls need no device->host copy.
//  kda_chunk_prepare_kernel  one CTA per (chunk, head): everything that does not depend on the state:
//                            G = cumsum(g), Aqk, Akk, Tm = (I+Akk)^-1, w, u, qg, kg  -> tiles in the workspace.
//  kda_chunk_scan_tc_kernel  (kda_chunk_scan_tc.cu) one CTA per (sequence, head): walks the chunks in order with
//                            the fp32 state in tensor memory, products on tcgen05.
//                            v_new = u - w h;  o = qg h + Aqk v_new;  h = Diag(Gam_last) h + kg^T v_new.
#include <mutex>

#include "kda_chunk.cuh"
#include "kda_device.cuh"
#include "kda_scan.cuh"

namespace kda {

// =================================================================================================
// chunk tables
// =================================================================================================
// A cu_seqlens that does not describe `tokens` tokens (a negative first entry, a negative length, more tokens than the
// tensors hold, or more chunks than the workspace was sized for) would send every later kernel past the end of the
// workspace.  The tables kernel checks it on the device: it then sets KDA_STATUS_BAD_CU_SEQLENS in the status word
// and writes empty tables (zero chunks for every sequence), so that prepare, the scans and the backward kernels do
// nothing; no device->host synchronisation is needed for the check.
__global__ void __launch_bounds__(1024) kda_chunk_tables_kernel(const int* __restrict__ cu, int N, long long tokens, int max_chunks,
                                                                int* __restrict__ seq_chunk_off, int* __restrict__ chunk_seq,
                                                                unsigned* __restrict__ status) {
  __shared__ int part[1024];
  const int tid = threadIdx.x;
  const int per = (N + 1023) / 1024;
  const int n0 = min(N, tid * per), n1 = min(N, n0 + per);
  int sum = 0;
  bool bad = (tid == 0) && (cu[0] < 0 || static_cast<long long>(cu[N]) > tokens);
  for (int n = n0; n < n1; ++n) {
    const int len = cu[n + 1] - cu[n];
    bad |= len < 0;
    // a partial sum that would overflow is certainly beyond max_chunks; saturate instead of wrapping
    const int nc = (len > 0) ? (len + C - 1) / C : 0;
    sum = (sum > max_chunks || nc > max_chunks) ? max_chunks + 1 : sum + nc;
  }
  part[tid] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {   // inclusive Hillis-Steele scan (saturating)
    int x = (tid >= off) ? part[tid - off] : 0;
    __syncthreads();
    const int y = part[tid] + x;
    part[tid] = (y > max_chunks || y < 0) ? max_chunks + 1 : y;
    __syncthreads();
  }
  bad |= part[tid] > max_chunks;
  bad = __syncthreads_or(bad) != 0;
  if (tid < 4) status[tid] = (tid == 0 && bad) ? KDA_STATUS_BAD_CU_SEQLENS : 0u;
  if (bad) {
    for (int n = n0; n < n1; ++n) seq_chunk_off[n] = 0;
    if (tid == 1023) seq_chunk_off[N] = 0;
    return;
  }
  int run = part[tid] - sum;   // exclusive prefix
  for (int n = n0; n < n1; ++n) {
    const int len = cu[n + 1] - cu[n];
    const int nc = (len > 0) ? (len + C - 1) / C : 0;
    seq_chunk_off[n] = run;
    for (int c = 0; c < nc; ++c) chunk_seq[run + c] = n;
    run += nc;
  }
  if (tid == 1023) seq_chunk_off[N] = part[1023];
}

// =================================================================================================
// per-chunk preparation
// =================================================================================================
constexpr int QS = 136;   // bf16 elements per padded row of the q/k/v tiles (272 B: ldmatrix rows hit distinct banks)
constexpr int GS = 136;   // floats per padded row of G
constexpr int AS = 68;    // floats per padded row of the fp32 64x64 matrix
constexpr int TS = 72;    // bf16 elements per padded row of the bf16 64x64 matrix (144 B)

// 113,920 bytes: two CTAs per SM.
struct PrepSmem {
  __nv_bfloat16 q[C * QS];   // q; from P5a on k * Gam
  __nv_bfloat16 k[C * QS];
  __nv_bfloat16 v[C * QS];
  float G[C * GS];           // log2-domain inclusive cumsum of g; at the very end the staged UT and W tiles
  float Akk[C * AS];         // raw <k_t D, k_j>, then beta_t * raw, then Tm = (I + Akk)^-1
  __nv_bfloat16 Aqk[C * TS]; // scale <q_t D, k_j>, lower triangle incl. diagonal; after P5a the scratch X of P4
  float beta[C];
  float rq[C], rk[C];        // reciprocal norms of the q, k rows (use_l2norm)
};
static_assert(TILE_VT + TILE_TK <= C * GS * 4, "staged tiles must fit the G buffer");

struct PrepParams {
  const __nv_bfloat16 *q, *k, *v;
  const float *g, *beta;
  const int* cu;
  const int *seq_chunk_off, *chunk_seq;
  unsigned char *W, *UT, *KG, *QG, *AQK, *GL, *TI, *RKK;   // TI, RKK may be NULL
  long long* dbg;
  int N, H;
  int use_l2norm;
  float scale;
  int HQ, grp;      // q/k heads and value heads per q/k head (grouped value heads); H counts value heads
  __nv_bfloat16 *QN, *KN;   // [tokens][HQ][128]: the normalised q, k kept for the backward (use_l2norm, training), or NULL
  float* RSTD;              // [2][tokens * HQ] reciprocal norms of q, k
  long long qrows;          // tokens * HQ
};

// Sum over the 32 lanes of 32 per-lane values at once: afterwards lane L holds the total of slot L.
// 31 shuffles instead of 32 x 5.
__device__ __forceinline__ float butterfly32(float (&v)[32], int lane) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {
      const float mine = up ? v[i + o] : v[i];
      const float other = up ? v[i] : v[i + o];
      v[i] = mine + __shfl_xor_sync(0xffffffffu, other, o);
    }
  }
  return v[0];
}

// ---- diagonal 8x8 blocks of Aqk / Akk ------------------------------------------------------------------------
// Pairwise decay is needed only where no row lies between j and t that both factors could be taken around; with
// the lower-left 8x8 quarter of every 16x16 diagonal block factored around the block's row 8 (tensor cores, see the
// kernel), what remains pairwise are the eight 8x8 diagonal blocks.
// A warp takes one 16-row block b and one half of the key columns; a lane owns two adjacent key columns.  Inside an
// 8x8 block the rows are walked upwards while E_j = k_j 2^(G_t - G_j) is carried per column j as a running product
// of lam_t = 2^(G_t - G_{t-1}) (every factor <= 1: range-safe, one ex2 per row instead of one per pair).
// Row t contributes t+1 values of q_t.E_j and t values of k_t.E_j: slot t*t + j, resp. t*t + t+1 + j, 64 slots per
// 8x8 block = two groups of 32 that butterfly32 sums over the lanes (lane L ends up with the total of slot L).
constexpr int DIAG_GROUPS = 4;      // per warp: two 8x8 blocks x two groups

__device__ __forceinline__ void prep_diag_half(const PrepSmem& s, const int b, const int hh, const int lane, float (&res)[DIAG_GROUPS]) {
  const int kk = hh * 64 + 2 * lane;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int r0 = 16 * b + 8 * u;
    float2 E[8];
    float val0[32], val1[32];
#define KDA_DIAG_VAL(sl) ((sl) < 32 ? val0[(sl) & 31] : val1[(sl) & 31])
    float2 Gprev = make_float2(0.f, 0.f);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const float2 Gt = *reinterpret_cast<const float2*>(&s.G[(r0 + t) * GS + kk]);
      const float2 qt = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[(r0 + t) * QS + kk]));
      const float2 kt = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[(r0 + t) * QS + kk]));
      if (t > 0) {
        const float lx = ex2(Gt.x - Gprev.x), ly = ex2(Gt.y - Gprev.y);
#pragma unroll
        for (int j = 0; j < t; ++j) {
          E[j].x *= lx;
          E[j].y *= ly;
        }
      }
      Gprev = Gt;
      E[t] = kt;
#pragma unroll
      for (int j = 0; j <= t; ++j) KDA_DIAG_VAL(t * t + j) = fmaf(qt.y, E[j].y, qt.x * E[j].x);
#pragma unroll
      for (int j = 0; j < t; ++j) KDA_DIAG_VAL(t * t + t + 1 + j) = fmaf(kt.y, E[j].y, kt.x * E[j].x);
      if (t == 5) res[2 * u] = butterfly32(val0, lane);      // slots 0..31 are complete (row 5 ends at slot 35)
    }
    res[2 * u + 1] = butterfly32(val1, lane);
#undef KDA_DIAG_VAL
  }
}

// Which (row, column, matrix) of the 16x16 block the value of lane L in group g is.
__device__ __forceinline__ void diag_decode(const int g, const int L, int& row, int& col, bool& is_kk) {
  const int u = g >> 1, sl = 32 * (g & 1) + L;
  const int t = (sl >= 49) ? 7 : (sl >= 36) ? 6 : (sl >= 25) ? 5 : (sl >= 16) ? 4 : (sl >= 9) ? 3 : (sl >= 4) ? 2 : (sl >= 1) ? 1 : 0;
  const int off = sl - t * t;
  is_kk = off > t;
  row = 8 * u + t;
  col = 8 * u + (is_kk ? off - t - 1 : off);
}

// One 16 x 16 block of Aqk / Akk on tensor cores: rows row0 .. row0 + 15, columns col0 .. col0 + 15, the decay factored
// around row `ref`:  2^(G_t - G_ref) on the row side, 2^(G_ref - G_j) on the column side.  Off-diagonal blocks take ref = row0
// (both factors <= 1: safe for any gate).  DIAG: a diagonal block (col0 == row0) with ref = its middle row -- only valid when
// the caller has promised bounded gates (safe_gate: at least -5 per token), which keeps both factors within 2^58.
template <bool DIAG>
__device__ __forceinline__ void prep_block16(PrepSmem& s, const float scale, const int row0, const int col0, const int ref, const int lane) {
const int gid = lane >> 2, tig = lane & 3;
const int ta = row0 + gid, tb = ta + 8;
const int ja = col0 + gid, jb = ja + 8;
const int r0 = ref;
  float cq[2][4], ck[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n) cq[n][0] = cq[n][1] = cq[n][2] = cq[n][3] = ck[n][0] = ck[n][1] = ck[n][2] = ck[n][3] = 0.f;
#pragma unroll 2
  for (int ks = 0; ks < 8; ++ks) {
    const int k0 = ks * 16 + tig * 2, k1 = k0 + 8;
    const float2 R0 = *reinterpret_cast<const float2*>(&s.G[r0 * GS + k0]);
    const float2 R1 = *reinterpret_cast<const float2*>(&s.G[r0 * GS + k1]);
    const float2 Ga0 = *reinterpret_cast<const float2*>(&s.G[ta * GS + k0]);
    const float2 Ga1 = *reinterpret_cast<const float2*>(&s.G[ta * GS + k1]);
    const float2 Gb0 = *reinterpret_cast<const float2*>(&s.G[tb * GS + k0]);
    const float2 Gb1 = *reinterpret_cast<const float2*>(&s.G[tb * GS + k1]);
    const float ea0x = ex2(Ga0.x - R0.x), ea0y = ex2(Ga0.y - R0.y), ea1x = ex2(Ga1.x - R1.x), ea1y = ex2(Ga1.y - R1.y);
    const float eb0x = ex2(Gb0.x - R0.x), eb0y = ex2(Gb0.y - R0.y), eb1x = ex2(Gb1.x - R1.x), eb1y = ex2(Gb1.y - R1.y);
    const float2 qa0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[ta * QS + k0]));
    const float2 qa1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[ta * QS + k1]));
    const float2 qb0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[tb * QS + k0]));
    const float2 qb1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[tb * QS + k1]));
    const float2 ka0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ta * QS + k0]));
    const float2 ka1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ta * QS + k1]));
    const float2 kb0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[tb * QS + k0]));
    const float2 kb1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[tb * QS + k1]));
    uint32_t aq[4], ak[4];
    aq[0] = pack_bf16(qa0.x * ea0x, qa0.y * ea0y); aq[1] = pack_bf16(qb0.x * eb0x, qb0.y * eb0y);
    aq[2] = pack_bf16(qa1.x * ea1x, qa1.y * ea1y); aq[3] = pack_bf16(qb1.x * eb1x, qb1.y * eb1y);
    ak[0] = pack_bf16(ka0.x * ea0x, ka0.y * ea0y); ak[1] = pack_bf16(kb0.x * eb0x, kb0.y * eb0y);
    ak[2] = pack_bf16(ka1.x * ea1x, ka1.y * ea1y); ak[3] = pack_bf16(kb1.x * eb1x, kb1.y * eb1y);
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const int j = n ? jb : ja;
      const float2 Gj0 = *reinterpret_cast<const float2*>(&s.G[j * GS + k0]);
      const float2 Gj1 = *reinterpret_cast<const float2*>(&s.G[j * GS + k1]);
      const float2 kj0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[j * QS + k0]));
      const float2 kj1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[j * QS + k1]));
      const uint32_t b0 = pack_bf16(kj0.x * ex2(R0.x - Gj0.x), kj0.y * ex2(R0.y - Gj0.y));
      const uint32_t b1 = pack_bf16(kj1.x * ex2(R1.x - Gj1.x), kj1.y * ex2(R1.y - Gj1.y));
      mma16816(cq[n], aq, b0, b1);
      mma16816(ck[n], ak, b0, b1);
    }
  }
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int col = col0 + n * 8 + tig * 2;
    if (DIAG) {      // a diagonal block: Aqk keeps j <= t, the raw k-k products j < t, the rest is zero
      cq[n][0] = (col <= ta) ? cq[n][0] : 0.f; cq[n][1] = (col + 1 <= ta) ? cq[n][1] : 0.f;
      cq[n][2] = (col <= tb) ? cq[n][2] : 0.f; cq[n][3] = (col + 1 <= tb) ? cq[n][3] : 0.f;
      ck[n][0] = (col < ta) ? ck[n][0] : 0.f; ck[n][1] = (col + 1 < ta) ? ck[n][1] : 0.f;
      ck[n][2] = (col < tb) ? ck[n][2] : 0.f; ck[n][3] = (col + 1 < tb) ? ck[n][3] : 0.f;
    }
    *reinterpret_cast<uint32_t*>(&s.Aqk[ta * TS + col]) = pack_bf16(scale * cq[n][0], scale * cq[n][1]);
    *reinterpret_cast<uint32_t*>(&s.Aqk[tb * TS + col]) = pack_bf16(scale * cq[n][2], scale * cq[n][3]);
    *reinterpret_cast<float2*>(&s.Akk[ta * AS + col]) = make_float2(ck[n][0], ck[n][1]);
    *reinterpret_cast<float2*>(&s.Akk[tb * AS + col]) = make_float2(ck[n][2], ck[n][3]);
  }
}

// KEEP_QN: also leave the L2-normalised q, k and their reciprocal norms in the workspace (training with use_l2norm).
// SAFE: the caller promises bounded gates (safe_gate); the diagonal 16 x 16 blocks then go to the tensor cores as well.
template <bool KEEP_QN, bool SAFE>
__global__ void __launch_bounds__(256, 2) kda_chunk_prepare_kernel(const PrepParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PrepSmem& s = *reinterpret_cast<PrepSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, tig = lane & 3;
  const int c = blockIdx.x, h = blockIdx.y;
  if (c >= p.seq_chunk_off[p.N]) return;
  const ChunkInfo ci = chunk_info(p.seq_chunk_off, p.chunk_seq, p.cu, c);
  const int len = ci.len;
  const size_t tile = static_cast<size_t>(c) * p.H + h;
  KDA_DBG_CLOCK(p.dbg, 16);

  // ---- P1: stage q, k, g, beta (v follows after P3a); rows >= len are zero-filled -----------------------------------
  // g goes first and alone in its copy group: the cumsum starts as soon as it is there, while q and k still arrive.
  {
    for (int i = tid; i < C * 32; i += 256) {
      const int r = i >> 5, pc = i & 31;
      const bool ok = r < len;
      const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 4;
      cp_async16(&s.G[r * GS + pc * 4], p.g + row, ok);
    }
    cp_async_commit();
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const bool ok = r < len;
      const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.HQ + h / p.grp) * KD + pc * 8;
      cp_async16(&s.q[r * QS + pc * 8], p.q + row, ok);
      cp_async16(&s.k[r * QS + pc * 8], p.k + row, ok);
    }
    cp_async_commit();
    if (tid < C) s.beta[tid] = (tid < len) ? __ldg(p.beta + static_cast<size_t>(ci.tok0 + tid) * p.H + h) : 0.f;
    for (int i = tid; i < C * AS; i += 256) s.Akk[i] = 0.f;
    for (int i = tid; i < C * TS / 2; i += 256) reinterpret_cast<uint32_t*>(s.Aqk)[i] = 0u;
    cp_async_wait<1>();
    __syncthreads();
  }

  KDA_DBG_CLOCK(p.dbg, 17);
  // ---- P2: G = cumsum(g) * log2(e): two half-columns per column, then the carry ----------------------
  {
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
    __syncthreads();   // row 31 of the first half is final
    if (half == 1) {
      const float carry = s.G[31 * GS + col];          // already in the log2 domain
#pragma unroll
      for (int i = 0; i < 32; ++i) s.G[(32 + i) * GS + col] = carry + gv[i] * LOG2E;
    }
  }
  cp_async_wait<0>();   // q, k
  __syncthreads();
  // ---- P1b: optional L2 normalisation of q and k rows (result rounded to bf16, as the unfused op does)
  if (p.use_l2norm) {
    for (int r = warp; r < C; r += 8) {
      uint2 qr = *reinterpret_cast<uint2*>(&s.q[r * QS + lane * 4]);
      uint2 kr = *reinterpret_cast<uint2*>(&s.k[r * QS + lane * 4]);
      float2 q0 = unpack_bf16(qr.x), q1 = unpack_bf16(qr.y), k0 = unpack_bf16(kr.x), k1 = unpack_bf16(kr.y);
      float sq = warp_sum(q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y);
      float sk = warp_sum(k0.x * k0.x + k0.y * k0.y + k1.x * k1.x + k1.y * k1.y);
      const float rq = rsqrtf(sq + L2NORM_EPS), rk = rsqrtf(sk + L2NORM_EPS);
      qr.x = pack_bf16(q0.x * rq, q0.y * rq); qr.y = pack_bf16(q1.x * rq, q1.y * rq);
      kr.x = pack_bf16(k0.x * rk, k0.y * rk); kr.y = pack_bf16(k1.x * rk, k1.y * rk);
      *reinterpret_cast<uint2*>(&s.q[r * QS + lane * 4]) = qr;
      *reinterpret_cast<uint2*>(&s.k[r * QS + lane * 4]) = kr;
      if (KEEP_QN && lane == 0) {
        s.rq[r] = rq;
        s.rk[r] = rk;
      }
    }
  }
  if (p.use_l2norm) __syncthreads();

  KDA_DBG_CLOCK(p.dbg, 18);
  // ---- P3a: diagonal 8x8 blocks, pairwise decay as running products (never a factorisation there: range-safe).
  // Warp = (block, key half).  The halves meet in the v buffer, whose load is issued only afterwards.
  {
    if constexpr (!SAFE) {
    const int b = warp & 3, hh = warp >> 2, r0 = 16 * b;
    float res[DIAG_GROUPS];
    prep_diag_half(s, b, hh, lane, res);
    float* const scratch = reinterpret_cast<float*>(s.v) + b * (DIAG_GROUPS * 32);
    if (hh == 1) {
#pragma unroll
      for (int g = 0; g < DIAG_GROUPS; ++g) scratch[g * 32 + lane] = res[g];
    }
    __syncthreads();
    if (hh == 0) {
#pragma unroll
      for (int g = 0; g < DIAG_GROUPS; ++g) {
        int row, col;
        bool is_kk;
        diag_decode(g, lane, row, col, is_kk);
        const float x = res[g] + scratch[g * 32 + lane];
        {
          if (is_kk) s.Akk[(r0 + row) * AS + r0 + col] = x;                            // raw; beta_t is applied later
          else s.Aqk[(r0 + row) * TS + r0 + col] = __float2bfloat16_rn(p.scale * x);
        }
      }
    }
    __syncthreads();
    }      // !SAFE
    for (int i = tid; i < C * 16; i += 256) {       // v: needed by the last phase only
      const int r = i >> 4, pc = i & 15;
      const bool ok = r < len;
      const size_t row = (static_cast<size_t>(ci.tok0 + (ok ? r : 0)) * p.H + h) * KD + pc * 8;
      cp_async16(&s.v[r * QS + pc * 8], p.v + row, ok);
    }
    cp_async_commit();
  }

  KDA_DBG_CLOCK(p.dbg, 19);
  // ---- P3b: off-diagonal 16x16 blocks on tensor cores.  For row block I the decay is factored around
  // the block's first row r0 = 16 I:  exp2(G_t - G_r0) * exp2(G_r0 - G_j), both factors <= 1 for j < r0 <= t.
  // Six units (I, 16 columns j): I=1 -> 1, I=2 -> 2, I=3 -> 3; warps 0..5 take one each.  Warps 6 and 7 take the
  // lower-left 8x8 quarters of the four diagonal blocks (rows 16b+8.., columns 16b..16b+7, factored around row 16b+8).
  if (warp < 6) {
    const int I = (warp < 1) ? 1 : (warp < 3 ? 2 : 3);
    const int np = (warp < 1) ? 0 : (warp < 3 ? warp - 1 : warp - 3);
    prep_block16<false>(s, p.scale, 16 * I, 16 * np, 16 * I, lane);
  } else if constexpr (SAFE) {
    // bounded gates: the four diagonal blocks whole, factored around their middle row (no pairwise phase at all)
#pragma unroll 1
    for (int bb = 0; bb < 2; ++bb) {
      const int b = 2 * (warp - 6) + bb;
      prep_block16<true>(s, p.scale, 16 * b, 16 * b, 16 * b + 8, lane);
    }
  } else {
#pragma unroll 1
    for (int bb = 0; bb < 2; ++bb) {
      const int b = 2 * (warp - 6) + bb;
      const int r0 = 16 * b + 8, ta = r0 + gid, ja = 16 * b + gid;      // m16 tile: rows gid real, rows gid + 8 a copy
      float cq[4] = {0.f, 0.f, 0.f, 0.f}, ck[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int ks = 0; ks < 8; ++ks) {
        const int k0 = ks * 16 + tig * 2, k1 = k0 + 8;
        const float2 R0 = *reinterpret_cast<const float2*>(&s.G[r0 * GS + k0]);
        const float2 R1 = *reinterpret_cast<const float2*>(&s.G[r0 * GS + k1]);
        const float2 Ga0 = *reinterpret_cast<const float2*>(&s.G[ta * GS + k0]);
        const float2 Ga1 = *reinterpret_cast<const float2*>(&s.G[ta * GS + k1]);
        const float ea0x = ex2(Ga0.x - R0.x), ea0y = ex2(Ga0.y - R0.y), ea1x = ex2(Ga1.x - R1.x), ea1y = ex2(Ga1.y - R1.y);
        const float2 qa0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[ta * QS + k0]));
        const float2 qa1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.q[ta * QS + k1]));
        const float2 ka0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ta * QS + k0]));
        const float2 ka1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ta * QS + k1]));
        uint32_t aq[4], ak[4];
        aq[0] = aq[1] = pack_bf16(qa0.x * ea0x, qa0.y * ea0y);
        aq[2] = aq[3] = pack_bf16(qa1.x * ea1x, qa1.y * ea1y);
        ak[0] = ak[1] = pack_bf16(ka0.x * ea0x, ka0.y * ea0y);
        ak[2] = ak[3] = pack_bf16(ka1.x * ea1x, ka1.y * ea1y);
        const float2 Gj0 = *reinterpret_cast<const float2*>(&s.G[ja * GS + k0]);
        const float2 Gj1 = *reinterpret_cast<const float2*>(&s.G[ja * GS + k1]);
        const float2 kj0 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ja * QS + k0]));
        const float2 kj1 = unpack_bf16(*reinterpret_cast<const uint32_t*>(&s.k[ja * QS + k1]));
        const uint32_t b0 = pack_bf16(kj0.x * ex2(R0.x - Gj0.x), kj0.y * ex2(R0.y - Gj0.y));
        const uint32_t b1 = pack_bf16(kj1.x * ex2(R1.x - Gj1.x), kj1.y * ex2(R1.y - Gj1.y));
        mma16816(cq, aq, b0, b1);
        mma16816(ck, ak, b0, b1);
      }
      const int col = 16 * b + tig * 2;
      *reinterpret_cast<uint32_t*>(&s.Aqk[ta * TS + col]) = pack_bf16(p.scale * cq[0], p.scale * cq[1]);
      *reinterpret_cast<float2*>(&s.Akk[ta * AS + col]) = make_float2(ck[0], ck[1]);
    }
  }
  __syncthreads();

  KDA_DBG_CLOCK(p.dbg, 20);
  // ---- P3c: keep the raw k-k products for the backward (dbeta), then Akk = beta_t * raw;
  // ---- P5a: elementwise tiles straight to global in their swizzled images: QG, KG, AQK, GL ------------
  {
    unsigned char* gR = p.RKK ? p.RKK + tile * TILE_TT : nullptr;
    unsigned char* gA = p.AQK + tile * TILE_TT;
    for (int i = tid; i < C * 8; i += 256) {
      const int r = i >> 3, pc = i & 7;
      float4 a0 = *reinterpret_cast<const float4*>(&s.Akk[r * AS + pc * 8]);
      float4 a1 = *reinterpret_cast<const float4*>(&s.Akk[r * AS + pc * 8 + 4]);
      const uint32_t off = swz<128>(r, pc * 8);
      if (gR)
        *reinterpret_cast<uint4*>(gR + off) =
            make_uint4(pack_bf16(a0.x, a0.y), pack_bf16(a0.z, a0.w), pack_bf16(a1.x, a1.y), pack_bf16(a1.z, a1.w));
      const float b = s.beta[r];
      a0.x *= b; a0.y *= b; a0.z *= b; a0.w *= b; a1.x *= b; a1.y *= b; a1.z *= b; a1.w *= b;
      *reinterpret_cast<float4*>(&s.Akk[r * AS + pc * 8]) = a0;
      *reinterpret_cast<float4*>(&s.Akk[r * AS + pc * 8 + 4]) = a1;
      *reinterpret_cast<uint4*>(gA + off) = *reinterpret_cast<const uint4*>(&s.Aqk[r * TS + pc * 8]);
    }
    KDA_DBG_CLOCK(p.dbg, 25);
    unsigned char* gQG = p.QG + tile * TILE_TK;
    unsigned char* gKG = p.KG + tile * TILE_TK;
    const bool keep_qn = p.QN != nullptr && h % p.grp == 0;      // once per q/k head
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, pc = i & 15;
      const uint4 qr = *reinterpret_cast<const uint4*>(&s.q[r * QS + pc * 8]);
      const uint4 kr = *reinterpret_cast<const uint4*>(&s.k[r * QS + pc * 8]);
      if (KEEP_QN && keep_qn && r < len) {      // the normalised q, k (and their reciprocal norms) stay for the backward
        const long long grow = static_cast<long long>(ci.tok0 + r) * p.HQ + h / p.grp;
        *reinterpret_cast<uint4*>(p.QN + grow * KD + pc * 8) = qr;
        *reinterpret_cast<uint4*>(p.KN + grow * KD + pc * 8) = kr;
        if (pc == 0) {
          p.RSTD[grow] = s.rq[r];
          p.RSTD[p.qrows + grow] = s.rk[r];
        }
      }
      const float4 Ga = *reinterpret_cast<const float4*>(&s.G[r * GS + pc * 8]);
      const float4 Gb = *reinterpret_cast<const float4*>(&s.G[r * GS + pc * 8 + 4]);
      const float4 La = *reinterpret_cast<const float4*>(&s.G[(C - 1) * GS + pc * 8]);
      const float4 Lb = *reinterpret_cast<const float4*>(&s.G[(C - 1) * GS + pc * 8 + 4]);
      const float g8[8] = {Ga.x, Ga.y, Ga.z, Ga.w, Gb.x, Gb.y, Gb.z, Gb.w};
      const float l8[8] = {La.x, La.y, La.z, La.w, Lb.x, Lb.y, Lb.z, Lb.w};
      const uint32_t qw[4] = {qr.x, qr.y, qr.z, qr.w}, kw[4] = {kr.x, kr.y, kr.z, kr.w};
      uint32_t oq[4], ok[4], og[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 qq = unpack_bf16(qw[e]), kk = unpack_bf16(kw[e]);
        const float e0 = ex2(g8[2 * e]), e1 = ex2(g8[2 * e + 1]);
        oq[e] = pack_bf16(p.scale * qq.x * e0, p.scale * qq.y * e1);
        ok[e] = pack_bf16(kk.x * ex2(l8[2 * e] - g8[2 * e]), kk.y * ex2(l8[2 * e + 1] - g8[2 * e + 1]));
        og[e] = pack_bf16(kk.x * e0, kk.y * e1);
      }
      const uint32_t off = tk_off(r, pc * 8);
      *reinterpret_cast<uint4*>(gQG + off) = make_uint4(oq[0], oq[1], oq[2], oq[3]);
      *reinterpret_cast<uint4*>(gKG + off) = make_uint4(ok[0], ok[1], ok[2], ok[3]);
      // k * Gam takes the place of this thread's own q piece (no other thread reads it in this phase)
      *reinterpret_cast<uint4*>(&s.q[r * QS + pc * 8]) = make_uint4(og[0], og[1], og[2], og[3]);
    }
    KDA_DBG_CLOCK(p.dbg, 26);
    if (tid < KD) reinterpret_cast<float*>(p.GL + tile * TILE_GL)[tid] = ex2(s.G[(C - 1) * GS + tid]);
  }
  __syncthreads();   // s.q now holds k * Gam; s.Aqk has been copied out and becomes the scratch X
  KDA_DBG_CLOCK(p.dbg, 21);

  // ---- P4: Tm = (I + Akk)^-1.  16x16 diagonal blocks by fp32 forward substitution (one column per thread,
  // in registers); the two levels of block merges  T21 = -T22 A21 T11  run on tensor cores with every fp32
  // operand split into bf16 hi + lo (three MMAs per product: about 16 bits of mantissa, better than TF32).
  {
    constexpr int XS = 36;                                   // floats per row of the scratch X
    float* sX = reinterpret_cast<float*>(s.Aqk);
    static_assert(32 * XS * 4 <= C * TS * 2, "X must fit the Aqk buffer");
    float x[16];
    if (tid < 64) {
      const int b = tid >> 4, cc = tid & 15;
      const float* A = &s.Akk[(16 * b) * AS + 16 * b];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = (i == cc) ? 1.f : 0.f;
#pragma unroll
        for (int m = 0; m < i; ++m) acc -= A[i * AS + m] * x[m];
        x[i] = acc;
      }
    }
    __syncthreads();
    if (tid < 64) {
      const int b = tid >> 4, cc = tid & 15;
      float* A = &s.Akk[(16 * b) * AS + 16 * b];
#pragma unroll
      for (int i = 0; i < 16; ++i) A[i * AS + cc] = x[i];
    }
    __syncthreads();
    KDA_DBG_CLOCK(p.dbg, 27);
    // c += A[ar.., ac..](16x16, stride AS, from Akk) * B[br.., bc..](16x8, row stride bs)
    auto mma_split = [&](float (&c)[4], int ar, int ac, const float* Bm, int bs, int br, int bc) {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 v2 = *reinterpret_cast<const float2*>(&s.Akk[(ar + gid + (e & 1) * 8) * AS + ac + tig * 2 + (e >> 1) * 8]);
        ah[e] = pack_bf16(v2.x, v2.y);
        const float2 hi = unpack_bf16(ah[e]);
        al[e] = pack_bf16(v2.x - hi.x, v2.y - hi.y);
      }
      uint32_t bh[2], bl[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float y0 = Bm[(br + tig * 2 + e * 8) * bs + bc + gid];
        const float y1 = Bm[(br + tig * 2 + 1 + e * 8) * bs + bc + gid];
        bh[e] = pack_bf16(y0, y1);
        const float2 hi = unpack_bf16(bh[e]);
        bl[e] = pack_bf16(y0 - hi.x, y1 - hi.y);
      }
      mma16816(c, ah, bh[0], bh[1]);
      mma16816(c, ah, bl[0], bl[1]);
      mma16816(c, al, bh[0], bh[1]);
    };
    // level 1: pairs (rows 16..31 | cols 0..15) and (rows 48..63 | cols 32..47); warps 0..3: (pair, 8 columns)
    {
      const int pr = (warp >> 1) & 1, nt = warp & 1, base = 32 * pr;
      float c1[4] = {0.f, 0.f, 0.f, 0.f};
      if (warp < 4) {
        mma_split(c1, base + 16, base, s.Akk, AS, base, base + nt * 8);                 // X = A21 T11
        float* X = sX + pr * 16 * XS;
        *reinterpret_cast<float2*>(&X[gid * XS + nt * 8 + tig * 2]) = make_float2(c1[0], c1[1]);
        *reinterpret_cast<float2*>(&X[(gid + 8) * XS + nt * 8 + tig * 2]) = make_float2(c1[2], c1[3]);
      }
      __syncthreads();
      if (warp < 4) {
        float c2[4] = {0.f, 0.f, 0.f, 0.f};
        mma_split(c2, base + 16, base + 16, sX + pr * 16 * XS, XS, 0, nt * 8);          // T22 X
        float* A21 = &s.Akk[(base + 16) * AS + base + nt * 8 + tig * 2];
        *reinterpret_cast<float2*>(&A21[gid * AS]) = make_float2(-c2[0], -c2[1]);
        *reinterpret_cast<float2*>(&A21[(gid + 8) * AS]) = make_float2(-c2[2], -c2[3]);
      }
      __syncthreads();
    }
    // level 2: rows 32..63 | cols 0..31; warp = (16-row tile mt, 8-column tile nt)
    {
      const int mt = warp >> 2, nt = warp & 3;
      float c1[4] = {0.f, 0.f, 0.f, 0.f};
      mma_split(c1, 32 + 16 * mt, 0, s.Akk, AS, 0, nt * 8);                             // X = A21 T11
      mma_split(c1, 32 + 16 * mt, 16, s.Akk, AS, 16, nt * 8);
      *reinterpret_cast<float2*>(&sX[(16 * mt + gid) * XS + nt * 8 + tig * 2]) = make_float2(c1[0], c1[1]);
      *reinterpret_cast<float2*>(&sX[(16 * mt + gid + 8) * XS + nt * 8 + tig * 2]) = make_float2(c1[2], c1[3]);
      __syncthreads();
      float c2[4] = {0.f, 0.f, 0.f, 0.f};
      mma_split(c2, 32 + 16 * mt, 32, sX, XS, 0, nt * 8);                               // T22 X
      mma_split(c2, 32 + 16 * mt, 48, sX, XS, 16, nt * 8);
      float* A21 = &s.Akk[(32 + 16 * mt) * AS + nt * 8 + tig * 2];
      *reinterpret_cast<float2*>(&A21[gid * AS]) = make_float2(-c2[0], -c2[1]);
      *reinterpret_cast<float2*>(&A21[(gid + 8) * AS]) = make_float2(-c2[2], -c2[3]);
      __syncthreads();
    }
  }

  KDA_DBG_CLOCK(p.dbg, 22);
  // ---- P5b: Tm (bf16) to global for the backward ---------------------------------------------------------
  if (p.TI) {
    unsigned char* gT = p.TI + tile * TILE_TT;
    for (int i = tid; i < C * 8; i += 256) {
      const int r = i >> 3, pc = i & 7;
      const float4 t0 = *reinterpret_cast<const float4*>(&s.Akk[r * AS + pc * 8]);
      const float4 t1 = *reinterpret_cast<const float4*>(&s.Akk[r * AS + pc * 8 + 4]);
      *reinterpret_cast<uint4*>(gT + swz<128>(r, pc * 8)) =
          make_uint4(pack_bf16(t0.x, t0.y), pack_bf16(t0.z, t0.w), pack_bf16(t1.x, t1.y), pack_bf16(t1.z, t1.w));
    }
  }
  cp_async_wait<0>();   // v
  __syncthreads();   // G is dead from here on: its buffer stages the UT and W tiles
  KDA_DBG_CLOCK(p.dbg, 23);

  // ---- P5c: u = (Tm beta) v,  w = (Tm beta) kGam on tensor cores.  Warp = (row tile mt, column half nh).
  // The accumulators are written into swizzled tile images in shared memory and leave with two TMA bulk stores.
  {
    unsigned char* stUT = reinterpret_cast<unsigned char*>(s.G);
    unsigned char* stW = stUT + TILE_VT;
    const int mt = warp & 3, nh = warp >> 2;
    uint32_t a[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const int ra = mt * 16 + gid, rb = ra + 8, c0 = ks * 16 + tig * 2, c1 = c0 + 8;
      const float2 b0 = *reinterpret_cast<const float2*>(&s.beta[c0]);
      const float2 b1 = *reinterpret_cast<const float2*>(&s.beta[c1]);
      const float2 t00 = *reinterpret_cast<const float2*>(&s.Akk[ra * AS + c0]);
      const float2 t10 = *reinterpret_cast<const float2*>(&s.Akk[rb * AS + c0]);
      const float2 t01 = *reinterpret_cast<const float2*>(&s.Akk[ra * AS + c1]);
      const float2 t11 = *reinterpret_cast<const float2*>(&s.Akk[rb * AS + c1]);
      a[ks][0] = pack_bf16(t00.x * b0.x, t00.y * b0.y);
      a[ks][1] = pack_bf16(t10.x * b0.x, t10.y * b0.y);
      a[ks][2] = pack_bf16(t01.x * b1.x, t01.y * b1.y);
      a[ks][3] = pack_bf16(t11.x * b1.x, t11.y * b1.y);
    }
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const __nv_bfloat16* Bs = which ? s.q : s.v;   // kGam or v, [token j][column]
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          const int krow = ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ncol = nh * 64 + np * 16 + ((lane >> 4) << 3);
          uint32_t b[4];
          ldsm_x4_t(b, smem_u32(&Bs[krow * QS + ncol]));
          mma16816(acc[2 * np], a[ks], b[0], b[1]);
          mma16816(acc[2 * np + 1], a[ks], b[2], b[3]);
        }
      }
      const int ta = mt * 16 + gid, tb = ta + 8;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const int col = nh * 64 + n * 8 + tig * 2;
        if (which) {   // W tile [t][k]
          *reinterpret_cast<uint32_t*>(stW + tk_off(ta, col)) = pack_bf16(acc[n][0], acc[n][1]);
          *reinterpret_cast<uint32_t*>(stW + tk_off(tb, col)) = pack_bf16(acc[n][2], acc[n][3]);
        } else {       // UT tile [v][t]
          *reinterpret_cast<__nv_bfloat16*>(stUT + swz<128>(col, ta)) = __float2bfloat16_rn(acc[n][0]);
          *reinterpret_cast<__nv_bfloat16*>(stUT + swz<128>(col + 1, ta)) = __float2bfloat16_rn(acc[n][1]);
          *reinterpret_cast<__nv_bfloat16*>(stUT + swz<128>(col, tb)) = __float2bfloat16_rn(acc[n][2]);
          *reinterpret_cast<__nv_bfloat16*>(stUT + swz<128>(col + 1, tb)) = __float2bfloat16_rn(acc[n][3]);
        }
      }
    }
    fence_proxy_async();   // the staged tiles (generic-proxy writes) are read next by the bulk-copy engine
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(p.UT + tile * TILE_VT, stUT, TILE_VT);
      bulk_s2g(p.W + tile * TILE_TK, stW, TILE_TK);
      bulk_commit();
      bulk_wait_read<0>();   // shared memory must stay valid until the engine has read it
    }
    KDA_DBG_CLOCK(p.dbg, 24);
  }
}

static DeviceOnce g_prepare_once;

static int set_attrs() {      // KDA_OK, a negative KDA_E_* or a positive cudaError_t
  return g_prepare_once.run([] {
    cudaError_t e = cudaSuccess;
    for (auto fn : {kda_chunk_prepare_kernel<false, false>, kda_chunk_prepare_kernel<true, false>, kda_chunk_prepare_kernel<false, true>,
                    kda_chunk_prepare_kernel<true, true>}) {
      if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(PrepSmem)));
      if (e == cudaSuccess) e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    return e;
  });
}

int validate_chunk_args(const kda_chunk_args& a, bool backward);
int validate_chunk_args(const kda_chunk_args& a, bool backward) {
  if (a.tokens < 0 || a.N < 0 || a.H <= 0) return KDA_E_SHAPE;
  if (a.HQ < 0 || (a.HQ > 0 && (a.HQ > a.H || a.H % a.HQ != 0))) return KDA_E_SHAPE;
  if (a.K != KD || a.V != VD) return KDA_E_SHAPE;
  if (a.scan_slices != 0 && a.scan_slices != 1 && a.scan_slices != 4) return KDA_E_SHAPE;
  if (a.io_dtype != KDA_BF16) return KDA_E_DTYPE;
  if (a.tokens / C + a.N > 0x3fffffffLL) return KDA_E_SHAPE;
  if (a.tokens == 0 || a.N == 0) return KDA_OK;
  if (!a.q || !a.k || !a.v || !a.g || !a.beta || !a.cu_seqlens || !a.workspace) return KDA_E_NULL;
  if (!backward && !a.o) return KDA_E_NULL;
  uintptr_t bits = reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k) | reinterpret_cast<uintptr_t>(a.v) |
                   reinterpret_cast<uintptr_t>(a.g) | reinterpret_cast<uintptr_t>(a.o) | reinterpret_cast<uintptr_t>(a.h0) |
                   reinterpret_cast<uintptr_t>(a.ht);
  if (backward) {
    if (!a.d_o || !a.dq || !a.dk || !a.dv || !a.dg || !a.dbeta || !a.bwd_workspace) return KDA_E_NULL;
    bits |= reinterpret_cast<uintptr_t>(a.d_o) | reinterpret_cast<uintptr_t>(a.dq) | reinterpret_cast<uintptr_t>(a.dk) |
            reinterpret_cast<uintptr_t>(a.dv) | reinterpret_cast<uintptr_t>(a.dg) | reinterpret_cast<uintptr_t>(a.d_ht) |
            reinterpret_cast<uintptr_t>(a.dh0) | (reinterpret_cast<uintptr_t>(a.bwd_workspace) & 255u);
  }
  if (bits & 15u) return KDA_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(a.workspace) & 255u) return KDA_E_ALIGN;
  return KDA_OK;
}

}  // namespace kda

extern "C" int64_t kda_chunk_max_chunks(int64_t tokens, int32_t N) { return tokens / kda::C + N; }

extern "C" size_t kda_chunk_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V, int32_t save) {
  (void)K; (void)V;
  return kda::carve_ws(nullptr, nullptr, tokens, N, H, (save & 1) != 0, true, false, (save & 2) != 0).fwd_bytes;
}

extern "C" int kda_chunk_fwd(const kda_chunk_args* args, void* stream) {
  using namespace kda;
  if (!args) return KDA_E_NULL;
  const kda_chunk_args& a = *args;
  int rc = validate_chunk_args(a, false);
  if (rc != KDA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a.N == 0) return KDA_OK;
  if (a.tokens == 0) {
    if (a.ht && a.ht != a.h0) {
      const size_t bytes = static_cast<size_t>(a.N) * a.H * KD * VD * sizeof(float);
      return static_cast<int>(a.h0 ? cudaMemcpyAsync(a.ht, a.h0, bytes, cudaMemcpyDeviceToDevice, st)
                                   : cudaMemsetAsync(a.ht, 0, bytes, st));
    }
    return KDA_OK;
  }
  const bool save = (a.save_for_backward & 1) != 0;
  const bool keep_qn = save && (a.save_for_backward & 2) != 0 && a.use_qk_l2norm != 0;
  ChunkWs w = carve_ws(static_cast<unsigned char*>(a.workspace), nullptr, a.tokens, a.N, a.H, save, true, false,
                       (a.save_for_backward & 2) != 0);
  if (a.workspace_bytes < w.fwd_bytes) return KDA_E_WORKSPACE;
  rc = set_attrs();
  if (rc != KDA_OK) return rc;
  cudaError_t e = cudaSuccess;
  const int NTmax = static_cast<int>(a.tokens / C + a.N);

  ProfCall* prof = prof_begin(st);
  kda_chunk_tables_kernel<<<1, 1024, 0, st>>>(a.cu_seqlens, a.N, a.tokens, NTmax, w.seq_chunk_off, w.chunk_seq, w.status);
  if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  prof_mark(prof, KDA_STAGE_TABLES, st);

  PrepParams pp{};
  pp.q = static_cast<const __nv_bfloat16*>(a.q);
  pp.k = static_cast<const __nv_bfloat16*>(a.k);
  pp.v = static_cast<const __nv_bfloat16*>(a.v);
  pp.g = a.g; pp.beta = a.beta; pp.cu = a.cu_seqlens;
  pp.seq_chunk_off = w.seq_chunk_off; pp.chunk_seq = w.chunk_seq;
  pp.W = w.W; pp.UT = w.UT; pp.KG = w.KG; pp.QG = w.QG; pp.AQK = w.AQK; pp.GL = w.GL; pp.TI = save ? w.TI : nullptr; pp.RKK = save ? w.RKK : nullptr;
  pp.dbg = g_dbg_clocks; pp.N = a.N; pp.H = a.H; pp.use_l2norm = a.use_qk_l2norm; pp.scale = a.scale;
  pp.HQ = a.HQ > 0 ? a.HQ : a.H; pp.grp = a.H / pp.HQ;
  pp.QN = keep_qn ? w.QN : nullptr; pp.KN = keep_qn ? w.KN : nullptr; pp.RSTD = keep_qn ? w.RSTD : nullptr;
  pp.qrows = static_cast<long long>(a.tokens) * pp.HQ;
  const dim3 pgrid(NTmax, a.H);
  if (a.safe_gate) {
    if (keep_qn) kda_chunk_prepare_kernel<true, true><<<pgrid, 256, sizeof(PrepSmem), st>>>(pp);
    else kda_chunk_prepare_kernel<false, true><<<pgrid, 256, sizeof(PrepSmem), st>>>(pp);
  } else {
    if (keep_qn) kda_chunk_prepare_kernel<true, false><<<pgrid, 256, sizeof(PrepSmem), st>>>(pp);
    else kda_chunk_prepare_kernel<false, false><<<pgrid, 256, sizeof(PrepSmem), st>>>(pp);
  }
  if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  prof_mark(prof, KDA_STAGE_PREPARE, st);

  ScanParams sp{};
  sp.cu = a.cu_seqlens; sp.seq_chunk_off = w.seq_chunk_off; sp.chunk_seq = w.chunk_seq;
  sp.W = w.W; sp.UT = w.UT; sp.KG = w.KG; sp.QG = w.QG; sp.AQK = w.AQK; sp.GL = w.GL;
  sp.HS = save ? w.HS : nullptr; sp.VNEWT = save ? w.VNEWT : nullptr;
  sp.h0 = a.h0; sp.ht = a.ht; sp.o = static_cast<__nv_bfloat16*>(a.o); sp.status = w.status; sp.dbg = g_dbg_clocks;
  sp.N = a.N; sp.H = a.H;
  const int slices = scan_slices_for(a.N * a.H, a.scan_slices);
  if ((rc = slices > 1 ? launch_scan_vs(sp, a.N * a.H, st) : launch_scan_tc(sp, a.N * a.H, st)) != KDA_OK) return rc;
  prof_mark(prof, KDA_STAGE_SCAN, st);
  return KDA_OK;
}

// =================================================================================================
// forward without any allocation: the workspace is a fixed array inside the library's device image
// =================================================================================================
// The name below is a device symbol.  In host code it is only a handle: its device address has to be
// asked for with cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_noalloc_scratch[KDA_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = kda::kMaxDeviceOrdinals;
std::mutex g_noalloc_mu;
unsigned char* g_noalloc_addr[kMaxDevices] = {};   // device address of g_noalloc_scratch, per device ordinal
}  // namespace

// Forward-only variant of kda_chunk_fwd for callers that cannot allocate device memory (a server whose
// memory pool is frozen after start-up, a thread inside a no-allocation region, a C caller without an
// allocator).  Inputs and outputs are the caller's; the per-chunk tiles live in g_noalloc_scratch.
// The first call on a device resolves the array's address (do it at start-up, before stream capture).
// Calls that overlap on one GPU share the array and race; the array keeps the previous call's bytes,
// which is harmless because every call rewrites all it reads.
extern "C" int kda_chunk_fwd_noalloc(const kda_chunk_args* args, void* stream) {
  if (!args) return KDA_E_NULL;
  if (args->save_for_backward != 0) return KDA_E_SHAPE;
  if (args->tokens < 0 || args->N < 0 || args->H <= 0) return KDA_E_SHAPE;
  const size_t need = kda::carve_ws(nullptr, nullptr, args->tokens, args->N, args->H, false).fwd_bytes;
  if (need > static_cast<size_t>(KDA_NOALLOC_SCRATCH_BYTES)) return KDA_E_LIMIT;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return KDA_E_LIMIT;
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_addr[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess) return static_cast<int>(e);
      g_noalloc_addr[dev] = static_cast<unsigned char*>(p);
    }
    scratch = g_noalloc_addr[dev];
  }
  kda_chunk_args a = *args;
  a.workspace = scratch;
  a.workspace_bytes = KDA_NOALLOC_SCRATCH_BYTES;
  a.bwd_workspace = nullptr;
  a.bwd_workspace_bytes = 0;
  return kda_chunk_fwd(&a, stream);
}

// Status word of the chunked kernels (see the header): copies it to the host, which waits for the device.
extern "C" int kda_chunk_status(const void* workspace, uint32_t* host_out) {
  if (!host_out) return KDA_E_NULL;
  *host_out = 0;
  const unsigned char* base = static_cast<const unsigned char*>(workspace);
  if (!base) {      // the array kda_chunk_fwd_noalloc uses on the current device; never used there: nothing to report
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return KDA_E_LIMIT;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    base = g_noalloc_addr[dev];
    if (!base) return KDA_OK;
  }
  const kda::ChunkWs w = kda::carve_ws(const_cast<unsigned char*>(base), nullptr, 0, 0, 1, false);
  unsigned v = 0;
  const cudaError_t e = cudaMemcpy(&v, w.status, sizeof(v), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  *host_out = v;
  return KDA_OK;
}
