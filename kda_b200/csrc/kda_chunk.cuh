// Shared definitions of the chunked KDA kernels: workspace carving and per-(chunk, head) tile formats.
//
// Every intermediate that travels between kernels is a per-(chunk, head) TILE that is contiguous in
// global memory and already holds the XOR-swizzled image the consumer wants in shared memory, so a
// consumer fetches a tile with one 1-D bulk (TMA) copy and hands it to tcgen05.mma as a 128-byte-swizzled
// operand tile (the same image is conflict-free for ldmatrix).  Tile index = chunk * H + head.  Formats (bf16 unless noted):
//   W, QG, KG : [64 tokens][128 k]   two [64 t][64 k] sub-tiles of 128-byte rows (tk_off)
//                                    w = Tm (beta k Gam), qg = scale q Gam, kg = k exp(G_last - G)
//   AQK, TI, RKK : [64 t][64 j]      128-byte rows      Aqk (lower incl. diagonal), Tm = (I + Akk)^-1, raw <k_t D, k_j>
//   UT        : [128 v][64 t]        128-byte rows      u^T,  u = Tm (beta v)
//   GL        : fp32 [128]                              Gam_last = exp(G_last)
//   HS, DH    : [128 v][128 k]       two [128 v][64 k] spans of 128-byte rows (vk_off): transposed state at chunk
//                                    start / its gradient at chunk end; each span is a tcgen05 SW128 operand tile
//   VNEWT, DVNEWT : [128 v][64 t]    128-byte rows      v_new^T and its gradient
#pragma once

#include "kda_common.cuh"

namespace kda {

constexpr int KD = 128;   // key head dim served by the chunked kernels
constexpr int VD = 128;   // value head dim

constexpr size_t TILE_TK = size_t(C) * KD * 2;    // 16 KiB
constexpr size_t TILE_TT = size_t(C) * C * 2;     //  8 KiB
constexpr size_t TILE_VT = size_t(VD) * C * 2;    // 16 KiB
constexpr size_t TILE_VK = size_t(VD) * KD * 2;   // 32 KiB
constexpr size_t TILE_GL = size_t(KD) * 4;        // 512 B

struct ChunkWs {
  int* seq_chunk_off;   // [N+1] first chunk of each sequence; [N] = total chunks
  int* chunk_seq;       // [max_chunks] sequence of each chunk
  unsigned* status;     // [4] device status word (first bytes of the workspace): KDA_STATUS_* bits, 0 = nothing to report
  unsigned char *W, *UT, *KG, *QG, *AQK, *GL;          // always
  unsigned char *TI, *RKK, *HS, *VNEWT;                // save_for_backward only
  unsigned char *DH, *DVNEWT;                          // backward scratch (bf16 tiles)
  __nv_bfloat16 *DQH, *DKH;                            // [tokens][H][128] per-value-head dq, dk (grouped value heads only)
  __nv_bfloat16 *QN, *KN;                              // [tokens][H][128] normalised q, k (use_qk_l2norm only)
  float *RSTD;                                         // [2][tokens][H]
  size_t fwd_bytes, bwd_bytes;
};

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Lays the workspace out.  base may be NULL (sizes only).  bwd_base: separate backward scratch.
// keep_qn: the forward keeps the L2-normalised q, k and their reciprocal norms in its workspace (then the backward
// does not recompute them and they are not carved from the backward scratch).
inline ChunkWs carve_ws(unsigned char* base, unsigned char* bwd_base, int64_t tokens, int N, int H, bool save,
                        bool l2norm = true, bool gva = false, bool keep_qn = false) {
  ChunkWs w{};
  const size_t NTmax = static_cast<size_t>(tokens / C + N);
  const size_t tiles = NTmax * static_cast<size_t>(H);
  size_t off = 0;
  auto take = [&](size_t bytes) { unsigned char* p = base ? base + off : nullptr; off += align_up(bytes); return p; };
  w.status = reinterpret_cast<unsigned*>(take(16));      // first, so that its address does not depend on the sizes
  w.seq_chunk_off = reinterpret_cast<int*>(take(sizeof(int) * (static_cast<size_t>(N) + 1)));
  w.chunk_seq = reinterpret_cast<int*>(take(sizeof(int) * (NTmax + 1)));
  w.W = take(tiles * TILE_TK);
  w.UT = take(tiles * TILE_VT);
  w.KG = take(tiles * TILE_TK);
  w.QG = take(tiles * TILE_TK);
  w.AQK = take(tiles * TILE_TT);
  w.GL = take(tiles * TILE_GL);
  if (save) {
    w.TI = take(tiles * TILE_TT);
    w.RKK = take(tiles * TILE_TT);
    w.HS = take(tiles * TILE_VK);
    w.VNEWT = take(tiles * TILE_VT);
    if (keep_qn) {
      w.QN = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(tokens) * H * KD * 2));
      w.KN = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(tokens) * H * KD * 2));
      w.RSTD = reinterpret_cast<float*>(take(static_cast<size_t>(tokens) * H * 2 * 4));
    }
  }
  w.fwd_bytes = off;
  size_t boff = 0;
  auto takeb = [&](size_t bytes) { unsigned char* p = bwd_base ? bwd_base + boff : nullptr; boff += align_up(bytes); return p; };
  w.DH = takeb(tiles * TILE_VK);
  w.DVNEWT = takeb(tiles * TILE_VT);
  if (l2norm && !(save && keep_qn)) {
    w.QN = reinterpret_cast<__nv_bfloat16*>(takeb(static_cast<size_t>(tokens) * H * KD * 2));
    w.KN = reinterpret_cast<__nv_bfloat16*>(takeb(static_cast<size_t>(tokens) * H * KD * 2));
    w.RSTD = reinterpret_cast<float*>(takeb(static_cast<size_t>(tokens) * H * 2 * 4));
  }
  if (gva) {
    w.DQH = reinterpret_cast<__nv_bfloat16*>(takeb(static_cast<size_t>(tokens) * H * KD * 2));
    w.DKH = reinterpret_cast<__nv_bfloat16*>(takeb(static_cast<size_t>(tokens) * H * KD * 2));
  }
  w.bwd_bytes = boff;
  return w;
}

// Chunk geometry read from the tables: which sequence, first token, valid rows.
struct ChunkInfo {
  int seq;
  long long tok0;
  int len;
};
__device__ __forceinline__ ChunkInfo chunk_info(const int* seq_chunk_off, const int* chunk_seq, const int* cu, int c) {
  ChunkInfo ci;
  ci.seq = chunk_seq[c];
  const int cis = c - seq_chunk_off[ci.seq];
  ci.tok0 = static_cast<long long>(cu[ci.seq]) + static_cast<long long>(cis) * C;
  const long long rem = static_cast<long long>(cu[ci.seq + 1]) - ci.tok0;
  ci.len = rem < C ? static_cast<int>(rem) : C;
  return ci;
}

// byte offset of element (v, k) of a [128 v][128 k] state tile: span k/64, then the 128-byte-row swizzle
__device__ __forceinline__ uint32_t vk_off(int v, int k) { return (static_cast<uint32_t>(k >> 6) << 14) + swz<128>(v, k & 63); }

// byte offset of element (t, k) of a [64 t][128 k] tile: sub-tile k/64, then the 128-byte-row swizzle
__device__ __forceinline__ uint32_t tk_off(int t, int k) { return (static_cast<uint32_t>(k >> 6) << 13) + swz<128>(t, k & 63); }

// ---- development aid: phase clocks of one CTA (x = 0, y = half the grid: a steady-state one), written when a buffer has been registered; compiled in
// only with -DKDA_PHASE_CLOCKS (python -m kda_b200.build --clocks), otherwise the marks vanish ----------------
extern long long* g_dbg_clocks;   // device pointer or NULL
#ifdef KDA_PHASE_CLOCKS
#define KDA_DBG_CLOCK(ptr, idx)                                                        \
  do {                                                                                 \
    if ((ptr) != nullptr && blockIdx.x == 0 && blockIdx.y == (gridDim.y >> 1) && threadIdx.x == 0) (ptr)[idx] = clock64(); \
  } while (0)
#else
#define KDA_DBG_CLOCK(ptr, idx) \
  do {                          \
    (void)(ptr);                \
  } while (0)
#endif

// ---- optional per-kernel timing (host side, see kda_b200_profile_* in the public header) ------------
struct ProfCall;                                  // one call's worth of events
ProfCall* prof_begin(cudaStream_t st);            // NULL when profiling is off
void prof_mark(ProfCall* pc, int stage, cudaStream_t st);   // records "stage finished"

}  // namespace kda
