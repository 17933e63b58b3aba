#include "common.cuh"
namespace jla {
const char* chunked_unsupported(const jla_problem&) { return "chunked path not built yet"; }
size_t chunked_residual_bytes(const jla_problem&) { return 0; }
size_t chunked_fwd_scratch_bytes(const jla_problem&) { return 0; }
size_t chunked_bwd_scratch_bytes(const jla_problem&) { return 0; }
int chunked_fwd(const jla_problem&, const jla_fwd_io&, cudaStream_t) { return JLA_ERR_UNSUPPORTED; }
int chunked_bwd(const jla_problem&, const jla_bwd_io&, cudaStream_t) { return JLA_ERR_UNSUPPORTED; }
}
