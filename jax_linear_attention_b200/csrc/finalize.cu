// HBM-bound epilogue / prologue kernels shared by both paths: key-gradient group sums with the L2-norm
// backward, and the forward L2 norm of q and k.
#include "common.cuh"
#include "profile.cuh"

namespace jla {
namespace {

// One warp per (token, key head) row. acc [tokens, H, K] f32 holds d(q or k) per VALUE head; the key head's
// gradient is the fp32 sum over its group's heads (the reference sums grouped key gradients in fp32 too:
// src/jla/ops/mosaic_gpu/scalar_gate.py:351-354). With the in-op L2 norm y = x * rsqrt(sum x^2 + eps), the
// gradient of the raw tensor is inv * (dy - y * <y, dy>).
template <typename T>
__global__ void finalize_key_grad_kernel(const float* __restrict__ acc, const T* __restrict__ raw, T* __restrict__ out,
                                         long rows, int H, int Hk, int K, int l2norm) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long tok = row / Hk;
  const int hk = (int)(row - tok * Hk);
  const int group = H / Hk;
  float dy[8], x[8];  // K <= 256
  float sumsq = 0.f;
  const bool vec4 = (K & 3) == 0;  // a lane owns channels 4 * lane .. + 3 (and 128 + those): 16-byte loads
#pragma unroll
  for (int i = 0; i < 8; ++i) dy[i] = x[i] = 0.f;
  if (vec4) {
    // the heads of the group are walked four at a time with all their loads in flight before the first add (the
    // per-head accumulators of a large call do not fit L2: the sum is bound by how many bytes a warp keeps in flight)
    const float* base = acc + (tok * H + (long)hk * group) * K;
    for (int h0 = 0; h0 < group; h0 += 4) {
      float4 v[4][2];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c = 4 * lane + 128 * half;
          v[j][half] = (h0 + j < group && c < K) ? *reinterpret_cast<const float4*>(base + (long)(h0 + j) * K + c)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          dy[4 * half] += v[j][half].x, dy[4 * half + 1] += v[j][half].y;
          dy[4 * half + 2] += v[j][half].z, dy[4 * half + 3] += v[j][half].w;
        }
      }
    }
    if (l2norm) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = 4 * lane + 128 * half;
        if (c < K) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            x[4 * half + j] = to_f32(raw[row * K + c + j]);
            sumsq += x[4 * half + j] * x[4 * half + j];
          }
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = lane + 32 * i;
      if (c < K) {
        for (int hh = 0; hh < group; ++hh) dy[i] += acc[(tok * H + hk * group + hh) * K + c];
        if (l2norm) {
          x[i] = to_f32(raw[row * K + c]);
          sumsq += x[i] * x[i];
        }
      }
    }
  }
  if (l2norm) {
    for (int off = 16; off > 0; off >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, off);
    const float inv = rsqrtf(sumsq + 1e-6f);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += x[i] * inv * dy[i];
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
    for (int i = 0; i < 8; ++i) dy[i] = inv * (dy[i] - x[i] * inv * dot);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = vec4 ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i;
    if (c < K) out[row * K + c] = from_f32<T>(dy[i]);
  }
}

// y = x * rsqrt(sum x^2 + 1e-6), fp32 math, rounded to the tensor dtype (reference.py:65-69). One warp per row.
template <typename T>
__global__ void l2norm_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long rows, int K) {
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float v[8];
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    v[i] = c < K ? to_f32(x[row * K + c]) : 0.f;
    sumsq += v[i] * v[i];
  }
  for (int off = 16; off > 0; off >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, off);
  const float inv = rsqrtf(sumsq + 1e-6f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = lane + 32 * i;
    if (c < K) y[row * K + c] = from_f32<T>(v[i] * inv);
  }
}

template <typename T>
int finalize_t(const float* acc, const void* raw, void* out, long rows, int H, int Hk, int K, bool l2norm,
               cudaStream_t stream) {
  if (rows == 0) return JLA_OK;
  const int warps = 8;
  const long blocks = (rows + warps - 1) / warps;
  {
    ProfScope ps(kProfFinalize, stream);
    finalize_key_grad_kernel<T><<<(unsigned)blocks, warps * 32, 0, stream>>>(
        acc, static_cast<const T*>(raw), static_cast<T*>(out), rows, H, Hk, K, l2norm ? 1 : 0);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <typename T>
int l2norm_t(const void* x, void* y, long rows, int K, cudaStream_t stream) {
  if (rows == 0) return JLA_OK;
  const int warps = 8;
  const long blocks = (rows + warps - 1) / warps;
  {
    ProfScope ps(kProfL2Norm, stream);
    l2norm_fwd_kernel<T><<<(unsigned)blocks, warps * 32, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(y),
                                                                       rows, K);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

int finalize_key_grad(const float* acc, const void* raw, void* out, int dtype, long tokens, int H, int Hk, int K,
                      bool l2norm, cudaStream_t stream) {
  const long rows = tokens * Hk;
  switch (dtype) {
    case JLA_DTYPE_BF16: return finalize_t<__nv_bfloat16>(acc, raw, out, rows, H, Hk, K, l2norm, stream);
    case JLA_DTYPE_F16: return finalize_t<__half>(acc, raw, out, rows, H, Hk, K, l2norm, stream);
    case JLA_DTYPE_F32: return finalize_t<float>(acc, raw, out, rows, H, Hk, K, l2norm, stream);
  }
  set_error("unknown dtype %d", dtype);
  return JLA_ERR_BAD_ARGUMENT;
}

int l2norm_fwd(const void* x, void* y, int dtype, long rows, int K, cudaStream_t stream) {
  switch (dtype) {
    case JLA_DTYPE_BF16: return l2norm_t<__nv_bfloat16>(x, y, rows, K, stream);
    case JLA_DTYPE_F16: return l2norm_t<__half>(x, y, rows, K, stream);
    case JLA_DTYPE_F32: return l2norm_t<float>(x, y, rows, K, stream);
  }
  set_error("unknown dtype %d", dtype);
  return JLA_ERR_BAD_ARGUMENT;
}

}  // namespace jla
