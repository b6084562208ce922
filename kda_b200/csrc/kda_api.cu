// Library-level entry points: ABI version and error text.
#include <cuda_runtime.h>

#include "kda_b200.h"

extern "C" int kda_b200_abi_version(void) { return KDA_B200_ABI_VERSION; }

extern "C" const char* kda_b200_strerror(int code) {
  switch (code) {
    case KDA_OK: return "ok";
    case KDA_E_NULL: return "a required pointer is NULL";
    case KDA_E_SHAPE: return "unsupported or inconsistent sizes";
    case KDA_E_DTYPE: return "unsupported io_dtype for this entry point";
    case KDA_E_ALIGN: return "a pointer is not 16-byte aligned";
    case KDA_E_WORKSPACE: return "workspace too small";
    case KDA_E_DEVICE: return "the current device is not sm_100 (compute capability 10.x)";
    case KDA_E_LIMIT: return "size beyond a documented fixed maximum";
    case KDA_E_TMAP: return "the driver refused to encode a TMA tensor map";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown kda_b200 error code";
}

extern "C" int kda_copy_rows_async(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width_bytes, size_t rows, void* stream) {
  if (!dst || !src) return KDA_E_NULL;
  if (rows == 0 || width_bytes == 0) return KDA_OK;
  if (dpitch < width_bytes || spitch < width_bytes) return KDA_E_SHAPE;
  return static_cast<int>(cudaMemcpy2DAsync(dst, dpitch, src, spitch, width_bytes, rows, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}

// ---- per-kernel timing ------------------------------------------------------------------------------
#include <mutex>
#include <vector>

#include "kda_chunk.cuh"

namespace kda {

long long* g_dbg_clocks = nullptr;

constexpr int PROF_RING = 256;          // calls kept between two reads
constexpr int PROF_MARKS = 6;           // marks per call (a forward uses 3, a backward up to 5)

struct ProfCall {
  cudaEvent_t start;
  cudaEvent_t mark[PROF_MARKS];
  int stage[PROF_MARKS];
  int nmarks;
};

static std::mutex g_prof_mu;
static bool g_prof_on = false;
static std::vector<ProfCall> g_prof_ring;
static int g_prof_used = 0;

ProfCall* prof_begin(cudaStream_t st) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!g_prof_on || g_prof_used >= PROF_RING) return nullptr;
  ProfCall* pc = &g_prof_ring[g_prof_used++];
  pc->nmarks = 0;
  cudaEventRecord(pc->start, st);
  return pc;
}

void prof_mark(ProfCall* pc, int stage, cudaStream_t st) {
  if (!pc || pc->nmarks >= PROF_MARKS) return;
  pc->stage[pc->nmarks] = stage;
  cudaEventRecord(pc->mark[pc->nmarks], st);
  pc->nmarks++;
}

}  // namespace kda

extern "C" int kda_b200_profile_enable(int on) {
  using namespace kda;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (on && g_prof_ring.empty()) {
    g_prof_ring.resize(PROF_RING);
    for (auto& pc : g_prof_ring) {
      cudaError_t e = cudaEventCreate(&pc.start);
      for (int i = 0; i < PROF_MARKS && e == cudaSuccess; ++i) e = cudaEventCreate(&pc.mark[i]);
      if (e != cudaSuccess) {
        g_prof_ring.clear();
        return static_cast<int>(e);
      }
    }
  }
  g_prof_on = on != 0;
  return KDA_OK;
}

extern "C" int kda_b200_profile_read(float* stage_ms, int* stage_launches, int reset) {
  using namespace kda;
  if (!stage_ms || !stage_launches) return KDA_E_NULL;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (int i = 0; i < KDA_NUM_STAGES; ++i) {
    stage_ms[i] = 0.f;
    stage_launches[i] = 0;
  }
  for (int c = 0; c < g_prof_used; ++c) {
    ProfCall& pc = g_prof_ring[c];
    cudaEvent_t prev = pc.start;
    for (int m = 0; m < pc.nmarks; ++m) {
      cudaError_t e = cudaEventSynchronize(pc.mark[m]);
      float ms = 0.f;
      if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, prev, pc.mark[m]);
      if (e != cudaSuccess) return static_cast<int>(e);
      stage_ms[pc.stage[m]] += ms;
      stage_launches[pc.stage[m]] += 1;
      prev = pc.mark[m];
    }
  }
  if (reset) g_prof_used = 0;
  return KDA_OK;
}

#ifdef KDA_PHASE_CLOCKS
// development aid, only in builds made with `python -m kda_b200.build --clocks` (not part of the public header): device
// buffer of >= 64 long long for the phase clocks
extern "C" __attribute__((visibility("default"))) void kda_b200_debug_clocks(void* device_buffer) {
  kda::g_dbg_clocks = static_cast<long long*>(device_buffer);
}
#endif
