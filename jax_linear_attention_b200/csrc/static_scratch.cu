// Forward entry point for callers that cannot hand over scratch memory and must not allocate any.
//
// A host that runs inside somebody else's executor -- an XLA custom call that did not reserve a scratch result,
// a serving loop whose memory pool is frozen after start-up -- has no buffer to give jla_linear_attention_fwd and
// may not call cudaMalloc (it would synchronise the device behind the executor's back, and the executor owns the
// memory budget). For them the library carries its own scratch: one fixed array in device global memory,
// kStaticScratchBytes long, that every GPU which loads the library holds from load until exit.
//
// The array is shared by all calls on a device and keeps whatever the last call left in it. The forward rewrites
// every word it later reads (chunk table, gate sums, run ids, T0), so nothing has to be cleared between calls; but
// two such calls that overlap on the GPU (different streams) would overwrite each other's scratch: issue them on
// one stream, or order them with events.
#include <mutex>

#include "chunked.cuh"

namespace jla {
int chunked_fwd(const jla_problem& p, const jla_fwd_io& io, cudaStream_t stream);
size_t chunked_fwd_scratch_bytes(const jla_problem& p);
const char* chunked_unsupported(const jla_problem& p);

namespace {

constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle here; kernels need its device address. It is looked up once per
// device, with that device current, and cached. Not an allocation: the array already exists in the loaded module.
int static_scratch(void** out) {
  int dev = -1;
  JLA_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device index %d out of range", dev);
    return JLA_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    JLA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return JLA_OK;
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" {

size_t jla_noalloc_scratch_limit(void) { return kStaticScratchBytes; }

int jla_linear_attention_fwd_noalloc(const jla_problem* p, void* o, float* final_state, jla_stream_t stream) {
  if (!p || ((long)p->B * p->T > 0 && !o)) {
    set_error("null problem or output");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (p->flags & JLA_FLAG_SAVE_RESIDUALS) {
    set_error("the no-allocation entry point runs the forward only: clear JLA_FLAG_SAVE_RESIDUALS");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (p->flags & JLA_FLAG_PREP_DONE) {
    set_error("the no-allocation entry point shares its scratch with every other call on the device: "
              "JLA_FLAG_PREP_DONE cannot be honoured, clear it");
    return JLA_ERR_BAD_ARGUMENT;
  }
  jla_fwd_io io{};
  io.o = o;
  io.final_state = final_state;
  const size_t need = jla_fwd_scratch_bytes(p);
  if (need > kStaticScratchBytes) {
    set_error("this call needs %zu bytes of scratch, more than the %zu bytes the library holds per GPU: "
              "use jla_linear_attention_fwd with a caller-provided buffer", need, kStaticScratchBytes);
    return JLA_ERR_WORKSPACE;
  }
  if (need > 0) {
    void* ptr = nullptr;
    if (int rc = static_scratch(&ptr)) return rc;
    io.scratch = ptr;
    io.scratch_bytes = kStaticScratchBytes;
  }
  return jla_linear_attention_fwd(p, &io, stream);
}

}  // extern "C"
