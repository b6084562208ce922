// Chunked KDA backward for sm_100a.  Two kernels, both reading the tiles the forward left behind:
//
//  kda_chunk_bwd_scan_kernel   one CTA per (sequence, head): chunks in REVERSE order with the fp32 state
//                              gradient in registers (transposed, one warp per 16 value columns):
//                                 dv_new = Aqk^T dO + kg dh';   dh = Diag(Gam_last) dh' + qg^T dO - w^T dv_new
//                              stores dh' (gradient w.r.t. the state at the chunk's end) and dv_new per chunk.
//  kda_chunk_bwd_main_tc_kernel (kda_chunk_bwd_tc.cu)  persistent CTAs over (chunk, head) tiles: every matrix
//                              product of the chunk's backward on tcgen05 with TMEM accumulators, then, one thread
//                              per key column, the diagonal 16x16 blocks pairwise (range-safe), dg = reverse
//                              cumsum, and the final dq, dk, dv, dg, dbeta.
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
        ldsm_x4(b, kbase + tk_off(np * 16 + brow, ks * 16 + bcol));       // B[k=kk][n=j] = kg[j][kk]
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
        ldsm_x4_t(b, qbase + tk_off(ks * 16 + trow, np * 16 + tcol));     // B[k=t][n=kk] = qg[t][kk]
        mma16816(dhT[2 * np], doA[ks], b[0], b[1]);
        mma16816(dhT[2 * np + 1], doA[ks], b[2], b[3]);
        ldsm_x4_t(b, wbase + tk_off(ks * 16 + trow, np * 16 + tcol));     // B[k=j][n=kk] = w[j][kk]
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
  if (make_rows_tmap(&mp.tm_q, q, false, a.tokens, a.H, KD, KD, C, false) || make_rows_tmap(&mp.tm_k, k, false, a.tokens, a.H, KD, KD, C, false) ||
      make_rows_tmap(&mp.tm_g, a.g, true, a.tokens, a.H, KD, KD, C, false) ||
      make_rows_tmap(&mp.tm_v, a.v, false, a.tokens, a.H, VD, 64, C, true) ||
      make_rows_tmap(&mp.tm_do, a.d_o, false, a.tokens, a.H, VD, 64, C, true))
    return KDA_E_DEVICE;
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
