// Parameters shared by the per-chunk backward kernels.
#pragma once

#include "kda_chunk.cuh"
#include "kda_tma.cuh"

namespace kda {

struct MainParams {
  const __nv_bfloat16 *q, *k, *v, *d_o;
  const float *g, *beta;
  const int* cu;
  const int *seq_chunk_off, *chunk_seq;
  const unsigned char *TI, *RKK, *HS, *VNEWT, *DH, *DVNEWT;
  __nv_bfloat16 *dv, *dq, *dk;
  float *dbeta, *dg;
  unsigned* status;
  long long* dbg;
  int N, H;
  float scale;
  int grp;          // value heads per q/k head (grouped value heads): the q, k maps have H / grp heads
  const float* rstd;    // [2][qrows] reciprocal norms of the q, k rows, or NULL.  Not NULL (only with grp == 1): q, k are the
  long long qrows;      // L2-normalised rows and the kernel applies the normalisation's backward to dq, dk before storing them
  // tiled-load maps of the [tokens, H, 128] operator tensors (64-token boxes of one head)
  alignas(64) CUtensorMap tm_q, tm_k, tm_g;   // plain row-major boxes [64][128]
  alignas(64) CUtensorMap tm_v, tm_do;        // 64-column boxes in the 128-byte-swizzled operand layout
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
  long long* dbg;       // development aid: phase clocks
  int N, H;
  alignas(64) CUtensorMap tm_do;   // 64-column boxes of dO in the 128-byte-swizzled operand layout
};

int launch_bwd_scan_tc(const RScanParams& p, int blocks, cudaStream_t st);
// four CTAs per (sequence, head) unit, one per slice of 32 value columns (kda_chunk_bwd_scan_vs.cu)
int launch_bwd_scan_vs(const RScanParams& p, int units, cudaStream_t st);

// both return KDA_OK, a negative KDA_E_* or a positive cudaError_t
// tcgen05 / TMEM version of the per-chunk backward kernel (kda_chunk_bwd_tc.cu)
int launch_bwd_main_tc(const MainParams& p, int grid, cudaStream_t st);

}  // namespace kda
