// Per-kernel timing scopes (see profile.cu). Usage at a launch site:  { ProfScope ps(kProfSgFwd, stream); launch; }
#pragma once
#include <cuda_runtime.h>

namespace jla {

enum {
  kProfTables = 0, kProfGates, kProfL2Norm, kProfKktInv, kProfSgFwd, kProfSgBwdState, kProfSgChunkGrads,
  kProfFinalize, kProfRecFwd, kProfRecBwd, kProfKdaPrep, kProfKdaIntra, kProfKdaFwd, kProfKdaBwdState,
  kProfKdaChunkGrads, kProfCpCorrection, kProfSgGradsQ, kProfSgGradsK, kProfKernels
};

class ProfScope {
 public:
  ProfScope(int id, cudaStream_t stream);
  ~ProfScope();
  ProfScope(const ProfScope&) = delete;
  ProfScope& operator=(const ProfScope&) = delete;

 private:
  int id_;
  cudaStream_t stream_;
  cudaEvent_t begin_;
};

}  // namespace jla
