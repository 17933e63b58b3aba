// Optional per-kernel timing: when switched on, every kernel launch of the library is bracketed by two CUDA
// events recorded on the launch stream. Recording costs no synchronisation; reading the totals synchronises
// on the recorded events. Off by default.
#include <mutex>
#include <vector>

#include "common.cuh"
#include "profile.cuh"

namespace jla {
namespace {

struct Span {
  int id;
  cudaEvent_t begin, end;
};

std::mutex g_mu;
bool g_on = false;
std::vector<Span> g_open;            // recorded, not yet folded into the totals
std::vector<cudaEvent_t> g_pool;     // recycled events
double g_total_ms[kProfKernels] = {};
int g_launches[kProfKernels] = {};

const char* const kNames[kProfKernels] = {
    "build_tables", "prep_gates", "l2norm_fwd", "kkt_inv", "sg_fwd", "sg_bwd_state", "sg_chunk_grads",
    "finalize_key_grad", "rec_fwd", "rec_bwd", "kda_prep", "kda_intra", "kda_fwd", "kda_bwd_state", "kda_chunk_grads",
    "cp_correction", "sg_grads_q", "sg_grads_k"};

cudaEvent_t take_event() {
  if (!g_pool.empty()) {
    cudaEvent_t e = g_pool.back();
    g_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}

void fold() {
  for (const Span& s : g_open) {
    float ms = 0.f;
    if (cudaEventSynchronize(s.end) == cudaSuccess && cudaEventElapsedTime(&ms, s.begin, s.end) == cudaSuccess) {
      g_total_ms[s.id] += ms;
      g_launches[s.id] += 1;
    }
    g_pool.push_back(s.begin);
    g_pool.push_back(s.end);
  }
  g_open.clear();
}

}  // namespace

ProfScope::ProfScope(int id, cudaStream_t stream) : id_(id), stream_(stream), begin_(nullptr) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_on) return;
  begin_ = take_event();
  if (begin_) cudaEventRecord(begin_, stream_);
}

ProfScope::~ProfScope() {
  if (!begin_) return;
  std::lock_guard<std::mutex> lock(g_mu);
  cudaEvent_t end = take_event();
  if (end) cudaEventRecord(end, stream_);
  g_open.push_back(Span{id_, begin_, end});
}

}  // namespace jla

using namespace jla;

extern "C" {

int jla_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_on = on != 0;
  return JLA_OK;
}

int jla_profile_reset(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  fold();
  for (int i = 0; i < kProfKernels; ++i) {
    g_total_ms[i] = 0.0;
    g_launches[i] = 0;
  }
  return JLA_OK;
}

const char* jla_profile_kernel_name(int kernel_id) {
  return (kernel_id >= 0 && kernel_id < kProfKernels) ? kNames[kernel_id] : nullptr;
}

int jla_profile_read(int kernel_id, double* total_ms, int* launches) {
  if (kernel_id < 0 || kernel_id >= kProfKernels || !total_ms || !launches) return JLA_ERR_BAD_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_mu);
  fold();
  *total_ms = g_total_ms[kernel_id];
  *launches = g_launches[kernel_id];
  return JLA_OK;
}

}  // extern "C"
