// Chunked KDA backward (placeholder until the kernels land: reports an unsupported-shape error).
#include "kda_chunk.cuh"

extern "C" int kda_chunk_bwd(const kda_chunk_args* args, void* stream) {
  (void)args; (void)stream;
  return KDA_E_SHAPE;
}
