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
