// Chunked KDA backward for sm_100a.  Two kernels, both reading the tiles the forward left behind:
//
//  kda_chunk_bwd_scan_tc_kernel (kda_chunk_bwd_scan_tc.cu)  one CTA per (sequence, head): chunks in REVERSE order
//                              with the fp32 state gradient in tensor memory, products on tcgen05:
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
#include "kda_chunk.cuh"
#include "kda_chunk_bwd.cuh"
#include "kda_scan.cuh"

namespace kda {

int validate_chunk_args(const kda_chunk_args& a, bool backward);

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

}  // namespace kda

namespace kda {
// Grouped value heads: dq, dk [tokens, HQ, 128] = sum over the grp value heads of a group of the per-value-head
// gradients [tokens, HQ * grp, 128] (fp32 sum, one rounding).  One thread per 16-byte piece of an output row.
__global__ void __launch_bounds__(256) kda_group_sum_kernel(const __nv_bfloat16* __restrict__ dqh, const __nv_bfloat16* __restrict__ dkh,
                                                            __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk, long long pieces,
                                                            int grp) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= pieces) return;
  const long long row = i / (KD / 8);
  const int pc = static_cast<int>(i % (KD / 8));
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = (which ? dkh : dqh) + row * grp * KD + pc * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < grp; ++j) {
      const uint4 r = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(j) * KD);
      const float2 a = unpack_bf16(r.x), b = unpack_bf16(r.y), c = unpack_bf16(r.z), d = unpack_bf16(r.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    *reinterpret_cast<uint4*>((which ? dk : dq) + row * KD + pc * 8) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}
}  // namespace kda

extern "C" size_t kda_chunk_bwd_workspace_bytes(int64_t tokens, int32_t N, int32_t H, int32_t K, int32_t V, int32_t use_qk_l2norm) {
  (void)K; (void)V;
  return kda::carve_ws(nullptr, nullptr, tokens, N, H, true, (use_qk_l2norm & 1) != 0, (use_qk_l2norm & 2) != 0, (use_qk_l2norm & 4) != 0).bwd_bytes;
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
  const int HQ = a.HQ > 0 ? a.HQ : a.H, grp = a.H / HQ;
  const bool kept_qn = l2 && (a.save_for_backward & 2) != 0;      // the forward left the normalised q, k in its workspace
  ChunkWs w = carve_ws(static_cast<unsigned char*>(a.workspace), static_cast<unsigned char*>(a.bwd_workspace), a.tokens, a.N,
                       a.H, true, l2, grp > 1, (a.save_for_backward & 2) != 0);
  if (a.workspace_bytes < w.fwd_bytes || a.bwd_workspace_bytes < w.bwd_bytes) return KDA_E_WORKSPACE;
  cudaError_t e = cudaSuccess;
  const int NTmax = static_cast<int>(a.tokens / C + a.N);
  const long long rows = static_cast<long long>(a.tokens) * HQ;      // rows of q and k
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* k = static_cast<const __nv_bfloat16*>(a.k);
  ProfCall* prof = prof_begin(st);
  if (l2) {
    if (!kept_qn) {
      kda_l2norm_fwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(q, k, w.QN, w.KN, w.RSTD, rows);
      if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
      prof_mark(prof, KDA_STAGE_L2NORM, st);
    }
    q = w.QN;
    k = w.KN;
  }

  RScanParams rp{};
  rp.cu = a.cu_seqlens; rp.seq_chunk_off = w.seq_chunk_off; rp.chunk_seq = w.chunk_seq;
  rp.W = w.W; rp.KG = w.KG; rp.QG = w.QG; rp.AQK = w.AQK; rp.GL = w.GL;
  rp.DH = w.DH; rp.DVNEWT = w.DVNEWT;
  rp.d_o = static_cast<const __nv_bfloat16*>(a.d_o); rp.d_ht = a.d_ht; rp.dh0 = a.dh0; rp.status = w.status; rp.dbg = g_dbg_clocks;
  rp.N = a.N; rp.H = a.H;
  if (make_rows_tmap(&rp.tm_do, a.d_o, false, a.tokens, a.H, VD, 64, C, true)) return KDA_E_TMAP;
  const int slices = scan_slices_for(a.N * a.H, a.scan_slices);
  if ((rc = slices > 1 ? launch_bwd_scan_vs(rp, a.N * a.H, st) : launch_bwd_scan_tc(rp, a.N * a.H, st)) != KDA_OK) return rc;
  prof_mark(prof, KDA_STAGE_BWD_SCAN, st);

  MainParams mp{};
  mp.q = q; mp.k = k; mp.v = static_cast<const __nv_bfloat16*>(a.v); mp.d_o = static_cast<const __nv_bfloat16*>(a.d_o);
  mp.g = a.g; mp.beta = a.beta; mp.cu = a.cu_seqlens; mp.seq_chunk_off = w.seq_chunk_off; mp.chunk_seq = w.chunk_seq;
  mp.TI = w.TI; mp.RKK = w.RKK; mp.HS = w.HS; mp.VNEWT = w.VNEWT; mp.DH = w.DH; mp.DVNEWT = w.DVNEWT;
  mp.dv = static_cast<__nv_bfloat16*>(a.dv);
  // grouped value heads: every value head writes its own dq, dk; a second kernel sums each group
  mp.dq = grp > 1 ? w.DQH : static_cast<__nv_bfloat16*>(a.dq);
  mp.dk = grp > 1 ? w.DKH : static_cast<__nv_bfloat16*>(a.dk);
  mp.dbeta = a.dbeta; mp.dg = a.dg; mp.status = w.status; mp.dbg = g_dbg_clocks;
  if (make_rows_tmap(&mp.tm_q, q, false, a.tokens, HQ, KD, KD, C, false) || make_rows_tmap(&mp.tm_k, k, false, a.tokens, HQ, KD, KD, C, false) ||
      make_rows_tmap(&mp.tm_g, a.g, true, a.tokens, a.H, KD, KD, C, false) ||
      make_rows_tmap(&mp.tm_v, a.v, false, a.tokens, a.H, VD, 64, C, true) ||
      make_rows_tmap(&mp.tm_do, a.d_o, false, a.tokens, a.H, VD, 64, C, true))
    return KDA_E_TMAP;
  mp.N = a.N; mp.H = a.H; mp.scale = a.scale; mp.grp = grp;
  // without grouped heads the normalisation's backward is applied by bwd_main's own epilogue
  const bool fused_l2 = l2 && grp == 1;
  mp.rstd = fused_l2 ? w.RSTD : nullptr; mp.qrows = rows;
  if ((rc = launch_bwd_main_tc(mp, main_grid(NTmax, a.H), st)) != KDA_OK) return rc;
  if (grp > 1) {
    const long long pieces = rows * (KD / 8);
    kda_group_sum_kernel<<<static_cast<unsigned>((pieces + 255) / 256), 256, 0, st>>>(w.DQH, w.DKH, static_cast<__nv_bfloat16*>(a.dq),
                                                                                       static_cast<__nv_bfloat16*>(a.dk), pieces, grp);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  }
  prof_mark(prof, KDA_STAGE_BWD_MAIN, st);

  if (l2 && !fused_l2) {
    kda_l2norm_bwd_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(w.QN, w.KN, w.RSTD, static_cast<__nv_bfloat16*>(a.dq),
                                                                                  static_cast<__nv_bfloat16*>(a.dk), rows);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
    prof_mark(prof, KDA_STAGE_L2NORM, st);
  }
  return KDA_OK;
}
