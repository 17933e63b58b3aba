// Shared device/host helpers of the sm_100a kernels: dtype conversion, the row table that maps
// batches / packed sequences to token ranges, and launch-error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/jla_b200.h"

namespace jla {

constexpr int kChunk = 64;  // tokens per chunk of the chunked kernels (the reference fixes 64 too:
                            // src/jla/ops/mosaic_gpu/_common.py:33)

// ---- dtype conversion -------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// One-instruction approximations for the element-wise kernels (relative error about 2^-22: far below the rounding of
// 16-bit outputs and inside the 1e-5 their float32 paths are held to); the IEEE-rounded reciprocal, the division and
// the library exp / log cost ten to thirty instructions each.
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_exp(float x) {  // one multiply and one ex2, no range fix-up
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
__device__ __forceinline__ float fast_log(float x) {  // x > 0; absolute error about 1e-7 near x = 1
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y * 0.6931471805599453f;
}
__device__ __forceinline__ float fast_rsqrt(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Asynchronous copy of one thread's row (BYTES = 8, 16 or 32) from global to shared memory; `valid` false writes
// zeros without reading. One commit per group of rows, cp_async_wait_groups<N> leaves the N newest groups in flight.
template <int BYTES>
__device__ __forceinline__ void cp_async_row(void* smem, const void* gmem, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int n = valid ? (BYTES < 16 ? BYTES : 16) : 0;
  if constexpr (BYTES == 8) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(gmem), "r"(n));
  } else {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(d + 16 * i),
                   "l"(static_cast<const char*>(gmem) + 16 * i), "r"(n));
    }
  }
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_groups() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Groups in a thread's ring of asynchronous copies: one being worked on, the others in flight (two where a row is 32
// bytes, so that the widest blocks still fit their shared memory).
__host__ __device__ constexpr int ring_stages(int row_bytes) { return row_bytes >= 32 ? 2 : 3; }

// ---- rows ----------------------------------------------------------------------------------------
// A "row" is a stretch of tokens whose state starts from its own initial state and ends in its own
// final state: one batch element, or one sequence of cu_seqlens (reference.py:170-203). Tokens are
// indexed flat over [B * T]. Inside a row, segment_ids may restart the state from zero.
struct Rows {
  int B, T, num_seqs;
  const int32_t* cu;   // [num_seqs + 1] or nullptr
  const int32_t* seg;  // [B * T] or nullptr

  __host__ __device__ int count() const { return cu ? num_seqs : B; }
  __device__ __forceinline__ void range(int r, int& tok0, int& len) const {
    if (cu) {  // device data: a range that is not inside [0, B * T] counts as an empty row, never as an address
      const int a = cu[r], b = cu[r + 1];
      const bool good = a >= 0 && b >= a && b <= B * T;
      tok0 = good ? a : 0;
      len = good ? b - a : 0;
    } else {
      tok0 = r * T;
      len = T;
    }
  }
  // True when token `tok` (flat index, not the first token of its row) starts a new document.
  __device__ __forceinline__ bool resets(int tok, int row_tok0) const {
    return seg != nullptr && tok > row_tok0 && seg[tok] != seg[tok - 1];
  }
};

inline Rows make_rows(const jla_problem& p) {
  Rows r;
  r.B = p.B;
  r.T = p.T;
  r.num_seqs = p.num_seqs;
  r.cu = p.cu_seqlens;
  r.seg = p.segment_ids;
  return r;
}

// ---- errors ----------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);  // api.cu: stores the text returned by jla_last_error()

#define JLA_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      ::jla::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return JLA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

#define JLA_LAUNCH_OK()                                                                \
  do {                                                                                 \
    cudaError_t _e = cudaGetLastError();                                               \
    if (_e != cudaSuccess) {                                                           \
      ::jla::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
      return JLA_ERR_CUDA;                                                             \
    }                                                                                  \
  } while (0)

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Carves aligned sub-buffers out of a caller-provided workspace; with base == nullptr it only sizes.
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* b) : base(static_cast<char*>(b)) {}
  template <typename T> T* take(size_t count) {
    off = align_up(off);
    T* ptr = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return ptr;
  }
  size_t bytes() const { return align_up(off); }
};

// ---- entry points of the translation units (all enqueue on `stream`, return jla_status) -------------
int recurrent_fwd(const jla_problem& p, const jla_fwd_io& io, cudaStream_t stream);
int recurrent_bwd(const jla_problem& p, const jla_bwd_io& io, cudaStream_t stream);
size_t recurrent_bwd_scratch_bytes(const jla_problem& p);

// dq/dk epilogue shared by both paths: sums per-value-head fp32 gradients over each key group, applies the
// L2-norm backward when the op normalised q/k itself, rounds to the tensor dtype.
//   acc [B*T, H, K] f32 -> out [B*T, Hk, K] dtype ; raw = the un-normalised input (or nullptr)
int finalize_key_grad(const float* acc, const void* raw, void* out, int dtype, long tokens, int H, int Hk, int K,
                      bool l2norm, cudaStream_t stream);

}  // namespace jla
