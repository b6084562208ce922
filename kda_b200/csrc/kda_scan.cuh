// Parameters of the forward state-scan kernels.
#pragma once

#include "kda_chunk.cuh"

namespace kda {

struct ScanParams {
  const int* cu;
  const int *seq_chunk_off, *chunk_seq;
  const unsigned char *W, *UT, *KG, *QG, *AQK, *GL;
  unsigned char *HS, *VNEWT;    // NULL unless saving for backward
  const float* h0;
  float* ht;
  __nv_bfloat16* o;
  unsigned* status;
  int N, H;
};

// tcgen05 / TMEM version (kda_chunk_scan_tc.cu); returns KDA_OK, a negative KDA_E_* or a positive cudaError_t
int launch_scan_tc(const ScanParams& p, int blocks, cudaStream_t st);

}  // namespace kda
