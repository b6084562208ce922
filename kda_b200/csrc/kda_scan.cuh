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
  long long* dbg;       // development aid: phase clocks (NULL unless built with the clock marks and a buffer is registered)
  int N, H;
};

// tcgen05 / TMEM version (kda_chunk_scan_tc.cu); returns KDA_OK, a negative KDA_E_* or a positive cudaError_t
int launch_scan_tc(const ScanParams& p, int blocks, cudaStream_t st);

// The same scan with four CTAs per (sequence, head) unit, one per slice of 32 value columns (kda_chunk_scan_vs.cu): for
// calls with so few units that one CTA's chunk-to-chunk chain sets the time.
int launch_scan_vs(const ScanParams& p, int units, cudaStream_t st);

// How many CTAs per unit the two state scans use: `requested` (1 or 4) if the caller chose, otherwise four while the
// grid stays within one CTA per SM of the current device.  (Two slices of 64 columns were built and measured: slower
// than one CTA per unit at every size, because the chain's cost is latency, not the width of its products.)
inline int scan_slices_for(int units, int requested) {
  if (requested == 1 || requested == 4) return requested;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return units * 4 <= sms ? 4 : 1;
}

}  // namespace kda
