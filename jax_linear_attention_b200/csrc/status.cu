// Device status word of the tensor-core kernels, and the host's view of it.
//
// Every wait inside the tcgen05 kernels (on an mbarrier that a TMA copy, an MMA commit or another warp role
// completes) is bounded: when it runs out the kernel stops waiting, lets its copies in flight land, frees its
// TMEM, stores a non-zero code in this word and returns normally, so the context stays usable. The results of
// that launch are then garbage; jla_device_status() is how a host finds out.
//
// The word is a __device__ variable of this module, i.e. one instance per GPU that loads the library. Host code
// cannot pass the variable's name to a kernel; the device address is looked up once per device (with that device
// current) and cached under a mutex, so a process that drives several GPUs hands each kernel its own GPU's word.
#include <mutex>

#include "chunked.cuh"
#include "umma.cuh"

namespace jla {

__device__ int g_device_status = 0;

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int* g_status_ptr[kMaxDevices] = {};

// One CTA of 32 threads: a wait on an mbarrier nobody ever arrives on, with a caller-chosen spin limit. The wait
// gives up, the kernel records code `kStatusSelftest` and exits normally: the path a lost arrival takes.
constexpr int kStatusSelftest = 9;

__global__ void bounded_wait_selftest_kernel(uint32_t spin_limit, int* status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    umma::mbar_init(&bar, 1);
    umma::mbar_init_fence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t addr = umma::smem_addr(&bar);
    bool done = false;
    for (uint32_t spin = 0; spin < spin_limit && !done; ++spin) {
      uint32_t ok;
      asm volatile(
          "{\n.reg .pred p;\n"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
          "selp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(ok)
          : "r"(addr), "r"(0u)
          : "memory");
      done = ok != 0;
    }
    if (!done) atomicExch(status, kStatusSelftest);
  }
}

}  // namespace

// Device address of the status word on the current device, or nullptr when the lookup fails.
int* tc_status_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_status_ptr[dev]) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_device_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<int*>(q);
  }
  return g_status_ptr[dev];
}

}  // namespace jla

using namespace jla;

extern "C" {

int jla_device_status(int* out, jla_stream_t stream) {
  if (!out) {
    set_error("null status output");
    return JLA_ERR_BAD_ARGUMENT;
  }
  int* ptr = tc_status_ptr();
  if (!ptr) {
    set_error("the status word of the current device could not be located");
    return JLA_ERR_CUDA;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int value = 0;
  JLA_CUDA_OK(cudaMemcpyAsync(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost, s));
  JLA_CUDA_OK(cudaMemsetAsync(ptr, 0, sizeof(int), s));
  JLA_CUDA_OK(cudaStreamSynchronize(s));
  *out = value;
  return JLA_OK;
}

int jla_selftest_bounded_wait(uint32_t spin_limit, jla_stream_t stream) {
  int* ptr = tc_status_ptr();
  if (!ptr) {
    set_error("the status word of the current device could not be located");
    return JLA_ERR_CUDA;
  }
  if (spin_limit == 0 || spin_limit > (1u << 20)) {
    set_error("spin_limit must be in 1 .. 2^20");
    return JLA_ERR_BAD_ARGUMENT;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(spin_limit, ptr);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // extern "C"
