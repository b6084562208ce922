// Intermediate states for inference engines: chunk_kda(..., return_intermediate_states=True) returns the state at the
// start of every chunk as h [chunks, H, K, V] in bf16.  The forward scan already leaves exactly that, transposed and
// swizzled, in the HS tiles of a workspace written with save_for_backward != 0; this kernel turns one tile per CTA into
// the plain row-major layout.  HBM-bound: 32 KiB read and 32 KiB written per (chunk, head).
#include "kda_chunk.cuh"

namespace kda {

__global__ void __launch_bounds__(256) kda_chunk_export_states_kernel(const unsigned char* __restrict__ HS, const int* __restrict__ seq_chunk_off,
                                                                      int N, int H, __nv_bfloat16* __restrict__ h_out) {
  __shared__ __align__(16) unsigned char tile[TILE_VK];
  const int c = blockIdx.x, h = blockIdx.y;
  if (c >= seq_chunk_off[N]) return;
  const size_t t = static_cast<size_t>(c) * H + h;
  const uint4* src = reinterpret_cast<const uint4*>(HS + t * TILE_VK);
  for (int i = threadIdx.x; i < static_cast<int>(TILE_VK / 16); i += 256) reinterpret_cast<uint4*>(tile)[i] = __ldcs(src + i);
  __syncthreads();
  __nv_bfloat16* dst = h_out + t * KD * VD;
  // a thread gathers eight consecutive value columns of one key row: the eight source rows differ in (v & 7), so the
  // swizzle spreads them over eight bank groups
  for (int i = threadIdx.x; i < KD * VD / 8; i += 256) {
    const int k = i >> 4, v0 = (i & 15) * 8;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint16_t lo = *reinterpret_cast<const uint16_t*>(tile + vk_off(v0 + 2 * e, k));
      const uint16_t hi = *reinterpret_cast<const uint16_t*>(tile + vk_off(v0 + 2 * e + 1, k));
      w[e] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    __stcs(reinterpret_cast<uint4*>(dst + k * VD + v0), make_uint4(w[0], w[1], w[2], w[3]));
  }
}

}  // namespace kda

extern "C" int kda_chunk_export_states(const void* workspace, size_t workspace_bytes, int64_t tokens, int32_t N, int32_t H, void* h_out,
                                       void* stream) {
  using namespace kda;
  if (!workspace || !h_out) return KDA_E_NULL;
  if (tokens < 0 || N < 0 || H <= 0 || tokens / C + N > 0x3fffffffLL) return KDA_E_SHAPE;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || (reinterpret_cast<uintptr_t>(h_out) & 15u)) return KDA_E_ALIGN;
  if (tokens == 0 || N == 0) return KDA_OK;
  const ChunkWs w = carve_ws(static_cast<unsigned char*>(const_cast<void*>(workspace)), nullptr, tokens, N, H, true);
  if (workspace_bytes < w.fwd_bytes) return KDA_E_WORKSPACE;
  const int NTmax = static_cast<int>(tokens / C + N);
  kda_chunk_export_states_kernel<<<dim3(NTmax, H), 256, 0, static_cast<cudaStream_t>(stream)>>>(w.HS, w.seq_chunk_off, N, H,
                                                                                                 static_cast<__nv_bfloat16*>(h_out));
  return static_cast<int>(cudaGetLastError());
}
