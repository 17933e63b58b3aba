// Element-wise glue of Gated DeltaNet-2 around the KDA kernels (reference: the erase gate b multiplies the key where
// it reads the state, the write gate w multiplies the value; src/jla/ops/reference.py:152-154; the reference's
// kernels take the gates rounded to 16 bits, src/jla/ops/mosaic_gpu/gdn2.py:11-12):
//
//   forward    k_read = k * b          v_gated = v * w                    (fp32 product, rounded once to the dtype)
//   backward   dk = dk_read * b        db = dk_read * k                   (dk: the read side's share; the kernels'
//              dv = dv_gated * w       dw = dv_gated * v                   own dk is the write side's)
//
// Both tensor pairs are flat arrays of the same dtype (n_k and n_v elements, multiples of 8); one thread moves 8
// elements of each tensor with 16-byte loads and stores. HBM-bound: every tensor is read or written once.
#include "common.cuh"

namespace jla {
namespace {

constexpr int kThreads = 256;

// 8 adjacent elements as 16-byte accesses: one for the 16-bit types, two for float
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  constexpr int kVecs = sizeof(T) * 8 / 16;
  uint4 u[kVecs];
#pragma unroll
  for (int i = 0; i < kVecs; ++i) u[i] = reinterpret_cast<const uint4*>(p)[i];
  const T* e = reinterpret_cast<const T*>(u);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  constexpr int kVecs = sizeof(T) * 8 / 16;
  uint4 u[kVecs];
  T* e = reinterpret_cast<T*>(u);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(f[i]);
#pragma unroll
  for (int i = 0; i < kVecs; ++i) reinterpret_cast<uint4*>(p)[i] = u[i];
}

// out[i] = x[i] * gate[i] over n elements (the forward, and the x-side gradient with x = upstream gradient)
template <typename T>
__device__ __forceinline__ void product8(const T* x, const T* gate, T* out, long i) {
  float a[8], b[8], r[8];
  load8<T>(x + i, a);
  load8<T>(gate + i, b);
#pragma unroll
  for (int e = 0; e < 8; ++e) r[e] = a[e] * b[e];
  store8<T>(out + i, r);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) gdn2_fwd_kernel(long n_k, long n_v, const T* k, const T* b, const T* v,
                                                            const T* w, T* k_read, T* v_gated) {
  const long stride = (long)gridDim.x * kThreads * 8;
  for (long i = ((long)blockIdx.x * kThreads + threadIdx.x) * 8; i < n_k + n_v; i += stride) {
    if (i < n_k) product8<T>(k, b, k_read, i);
    else product8<T>(v, w, v_gated, i - n_k);
  }
}

// d_x = d_out * gate, d_gate = d_out * x
template <typename T>
__device__ __forceinline__ void grads8(const T* x, const T* gate, const T* d_out, T* d_x, T* d_gate, long i) {
  float a[8], b[8], d[8], rx[8], rg[8];
  load8<T>(x + i, a);
  load8<T>(gate + i, b);
  load8<T>(d_out + i, d);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    rx[e] = d[e] * b[e];
    rg[e] = d[e] * a[e];
  }
  store8<T>(d_x + i, rx);
  store8<T>(d_gate + i, rg);
}

template <typename T>
__global__ void __launch_bounds__(kThreads) gdn2_bwd_kernel(long n_k, long n_v, const T* k, const T* b, const T* v,
                                                            const T* w, const T* dk_read, const T* dv_gated, T* dk, T* db,
                                                            T* dv, T* dw) {
  const long stride = (long)gridDim.x * kThreads * 8;
  for (long i = ((long)blockIdx.x * kThreads + threadIdx.x) * 8; i < n_k + n_v; i += stride) {
    if (i < n_k) grads8<T>(k, b, dk_read, dk, db, i);
    else grads8<T>(v, w, dv_gated, dv, dw, i - n_k);
  }
}

int grid_for(long n) {
  const long blocks = (n / 8 + kThreads - 1) / kThreads;
  return (int)(blocks < 148L * 16 ? (blocks > 0 ? blocks : 1) : 148L * 16);  // a few waves of grid-stride blocks
}

bool bad_sizes(long n_k, long n_v) { return n_k < 0 || n_v < 0 || n_k % 8 || n_v % 8; }

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_gdn2_inputs_fwd(int dtype, int64_t n_k, int64_t n_v, const void* k, const void* b, const void* v,
                                   const void* w, void* k_read, void* v_gated, jla_stream_t stream) {
  if (bad_sizes(n_k, n_v) || (n_k + n_v > 0 && (!k || !b || !v || !w || !k_read || !v_gated))) {
    set_error("gdn2 inputs: null tensor, or sizes that are not multiples of 8 (n_k = %ld, n_v = %ld)", (long)n_k, (long)n_v);
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (n_k + n_v == 0) return JLA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n_k + n_v);
  switch (dtype) {
    case JLA_DTYPE_BF16:
      gdn2_fwd_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(
          n_k, n_v, static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(b),
          static_cast<const __nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(k_read),
          static_cast<__nv_bfloat16*>(v_gated));
      break;
    case JLA_DTYPE_F16:
      gdn2_fwd_kernel<__half><<<grid, kThreads, 0, s>>>(n_k, n_v, static_cast<const __half*>(k), static_cast<const __half*>(b),
                                                        static_cast<const __half*>(v), static_cast<const __half*>(w),
                                                        static_cast<__half*>(k_read), static_cast<__half*>(v_gated));
      break;
    case JLA_DTYPE_F32:
      gdn2_fwd_kernel<float><<<grid, kThreads, 0, s>>>(n_k, n_v, static_cast<const float*>(k), static_cast<const float*>(b),
                                                       static_cast<const float*>(v), static_cast<const float*>(w),
                                                       static_cast<float*>(k_read), static_cast<float*>(v_gated));
      break;
    default:
      set_error("gdn2 inputs: unknown dtype %d", dtype);
      return JLA_ERR_BAD_ARGUMENT;
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

extern "C" int jla_gdn2_inputs_bwd(int dtype, int64_t n_k, int64_t n_v, const void* k, const void* b, const void* v,
                                   const void* w, const void* dk_read, const void* dv_gated, void* dk, void* db, void* dv,
                                   void* dw, jla_stream_t stream) {
  if (bad_sizes(n_k, n_v) ||
      (n_k + n_v > 0 && (!k || !b || !v || !w || !dk_read || !dv_gated || !dk || !db || !dv || !dw))) {
    set_error("gdn2 inputs backward: null tensor, or sizes that are not multiples of 8 (n_k = %ld, n_v = %ld)", (long)n_k,
              (long)n_v);
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (n_k + n_v == 0) return JLA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n_k + n_v);
#define JLA_GDN2_BWD(T)                                                                                                \
  gdn2_bwd_kernel<T><<<grid, kThreads, 0, s>>>(n_k, n_v, static_cast<const T*>(k), static_cast<const T*>(b),             \
                                               static_cast<const T*>(v), static_cast<const T*>(w),                       \
                                               static_cast<const T*>(dk_read), static_cast<const T*>(dv_gated),          \
                                               static_cast<T*>(dk), static_cast<T*>(db), static_cast<T*>(dv),            \
                                               static_cast<T*>(dw))
  switch (dtype) {
    case JLA_DTYPE_BF16: JLA_GDN2_BWD(__nv_bfloat16); break;
    case JLA_DTYPE_F16: JLA_GDN2_BWD(__half); break;
    case JLA_DTYPE_F32: JLA_GDN2_BWD(float); break;
    default:
      set_error("gdn2 inputs backward: unknown dtype %d", dtype);
      return JLA_ERR_BAD_ARGUMENT;
  }
#undef JLA_GDN2_BWD
  JLA_LAUNCH_OK();
  return JLA_OK;
}
