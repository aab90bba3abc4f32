// Optional per-kernel timing with CUDA events on the launching stream.
//
// Off by default and free when off.  When enabled (kda_stage_timing_enable), every kernel launch of
// the library is bracketed by two events recorded on the caller's stream; kda_stage_timing_read
// synchronises those events and returns, per stage, the number of launches and the summed device
// time.  This is how a benchmark attributes a step's time to kernels without a profiler.
#pragma once
#include <cuda_runtime.h>

namespace kda {

enum Stage {
  kStagePrepare = 0, kStageStateFwd, kStageStateBwd, kStageBwdChunk,
  kStageRecurrent, kStageGateFwd, kStageGateBwd, kStageL2norm, kStageConv, kStageOffsets,
  kStageAffine, kStageEpilogue, kStageCount
};

void stage_begin(int stage, cudaStream_t s);
void stage_end(int stage, cudaStream_t s);

struct StageScope {
  int stage; cudaStream_t s;
  StageScope(int st, cudaStream_t str) : stage(st), s(str) { stage_begin(stage, s); }
  ~StageScope() { stage_end(stage, s); }
};

}  // namespace kda
