// Library identification and the optional per-kernel event timing of the C ABI.
#include <mutex>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../../include/kda_b200.h"
#include "kda_timing.cuh"

namespace kda {

static const char* kStageNames[kStageCount] = {
    "prepare", "state_fwd", "state_bwd", "bwd_chunk", "recurrent",
    "gate_fwd", "gate_bwd", "l2norm", "conv", "chunk_offsets", "state_affine",
    "epilogue"};

// Every kernel launch of the library sits in an NVTX range (a few nanoseconds when no tool is
// attached), named after the reference's profiler ranges for the stages the kernel fuses
// (fwd/cute/chunk_kda_fwd.py:94-119, bwd/cute/chunk_kda_bwd.py:58-129, kda/utils.py:269), so a
// timeline of this library reads like one of the reference.
static const char* kStageTraceNames[kStageCount] = {
    "kda/fused/chunk_kda_fwd_intra",                        // gating, pairwise products, solve, w / u
    "kda/fused/inter_chunk_state+output_composition",
    "kda/fused/backward_dav+delta_h",
    "kda/fused/backward_wy_dqkg+intra",
    "kda/fused/recurrent",
    "kda/fused/gate_cumsum_fwd", "kda/fused/gate_cumsum_bwd", "kda/fused/l2norm", "kda/fused/short_conv",
    "kda/fused/chunk_offsets", "kda/fused/state_affine", "kda/fused/output_gate_norm"};

struct Pair { cudaEvent_t a, b; int device; };
constexpr int kMaxDevices = 64;
static bool g_enabled = false;
static std::mutex g_mu;
static std::vector<Pair> g_pairs[kStageCount];
static std::vector<cudaEvent_t> g_free[kMaxDevices];   // an event belongs to the device it was created on

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
  return dev;
}

static cudaEvent_t get_event(int dev) {
  if (!g_free[dev].empty()) { cudaEvent_t e = g_free[dev].back(); g_free[dev].pop_back(); return e; }
  cudaEvent_t e;
  cudaEventCreate(&e);
  return e;
}

void stage_begin(int stage, cudaStream_t s) {
  nvtxRangePushA(kStageTraceNames[stage]);
  if (!g_enabled) return;
  std::lock_guard<std::mutex> lock(g_mu);
  const int dev = current_device();
  Pair p{get_event(dev), get_event(dev), dev};
  cudaEventRecord(p.a, s);
  g_pairs[stage].push_back(p);
}
void stage_end(int stage, cudaStream_t s) {
  nvtxRangePop();
  if (!g_enabled) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_pairs[stage].empty()) cudaEventRecord(g_pairs[stage].back().b, s);
}

}  // namespace kda

extern "C" int kda_b200_version(void) { return 100; }

extern "C" int kda_stage_count(void) { return kda::kStageCount; }

extern "C" const char* kda_stage_name(int stage) {
  return (stage >= 0 && stage < kda::kStageCount) ? kda::kStageNames[stage] : "";
}

extern "C" int kda_stage_timing_enable(int on) {
  std::lock_guard<std::mutex> lock(kda::g_mu);
  kda::g_enabled = on != 0;
  return KDA_OK;
}

extern "C" int kda_stage_timing_read(int64_t* launches, float* total_ms, int reset) {
  if (!launches || !total_ms) return KDA_ERR_ARG;
  std::lock_guard<std::mutex> lock(kda::g_mu);
  for (int st = 0; st < kda::kStageCount; ++st) {
    launches[st] = 0;
    total_ms[st] = 0.f;
    for (auto& p : kda::g_pairs[st]) {
      float ms = 0.f;
      if (cudaEventSynchronize(p.b) == cudaSuccess && cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) {
        launches[st] += 1;
        total_ms[st] += ms;
      }
    }
    if (reset) {
      for (auto& p : kda::g_pairs[st]) {
        kda::g_free[p.device].push_back(p.a);
        kda::g_free[p.device].push_back(p.b);
      }
      kda::g_pairs[st].clear();
    }
  }
  return KDA_OK;
}
