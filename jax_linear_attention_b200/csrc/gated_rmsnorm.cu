// Gated RMS norm behind the linear-attention kernels, forward and backward in one pass each
// (src/jla/layers/norm.py:60-112 `GatedRMSNorm`, the output norm of the mixers in
// src/jla/layers/linear_attention.py and, with norm_before_gate = false, the Mamba-2 norm of src/jla/layers/ssm.py):
//
//   gate = silu(z) or sigmoid(z)                      x, z, y [rows, dim] dtype; weight [dim] f32
//   u = x            (norm_before_gate)   or   x * gate
//   n = u * rsqrt(mean_group(u^2) + eps)              groups of `group` consecutive channels
//   y = n * weight * gate   (norm_before_gate)   or   n * weight
//
//   dn = dy * weight (* gate);  du = r (dn - n mean_group(dn n));  dweight = sum_rows dy n (* gate)
//   norm_before_gate:  dx = du,  dz = (dy n weight) act'(z);   else:  dx = du gate,  dz = (du x) act'(z)
//
// HBM-bound. A thread owns eight adjacent channels (16-byte loads) and walks rows; a group's mean is a butterfly
// over the group's threads (inside a warp for groups up to 256 channels, through shared memory for wider groups, in
// which case a block is exactly one group). The weight gradient is summed in registers over the rows a thread walks,
// then over the block's row lanes in shared memory, and leaves the block as one atomic per channel.
#include "common.cuh"

namespace jla {
namespace {

constexpr int THREADS = 512;

struct NormParams {
  long rows;
  int dim, group;
  const void *x, *z;
  const float* w;
  float eps;
  int sigmoid_gate, norm_before_gate;
  void* y;
  const void* dy;
  void *dx, *dz;
  float* dw;
  int rows_per_lane;  // rows one thread walks
  int cols;           // column threads of a block (8 channels each); the other threads are row lanes
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(p[i]);
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 u;
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(f[i]);
    *reinterpret_cast<uint4*>(p) = u;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = from_f32<T>(f[i]);
  }
}

// Sum over the `lanes` threads of a group. lanes <= 32: an aligned butterfly inside the warp. Wider: the block is one
// group (blockDim.x == lanes); every thread of the block must call this.
__device__ __forceinline__ float group_sum(float v, int lanes, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {  // five predicated butterflies, no loop
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    if (off < lanes) v += o;
  }
  if (lanes <= 32) return v;
  const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();  // the previous use of red is over
  if ((threadIdx.x & 31) == 0) red[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < nw; ++w) total += red[w];
  return total;
}

template <typename T, bool BWD, int MAXT>
__global__ void __launch_bounds__(MAXT) gated_rmsnorm_kernel(NormParams p) {
  __shared__ float red[32];
  extern __shared__ __align__(16) float dw_red[];  // backward: [row lanes][cols * 8]; then the ring of row copies
  const int cv = p.dim / 8;                 // 8-channel vectors per row
  const int lanes = p.group / 8;            // threads per group
  const int cols = p.cols;                  // column threads of this block
  const int lanes_r = blockDim.x / cols;    // row lanes
  const int ct = threadIdx.x % cols, lr = threadIdx.x / cols;
  const int vec = blockIdx.x * cols + ct;
  const bool live = vec < cv && lr < lanes_r;
  const int col = (live ? vec : 0) * 8;
  const long tile = (long)p.rows_per_lane * lanes_r;
  const long r0 = (long)blockIdx.y * tile;
  const long r1 = r0 + tile < p.rows ? r0 + tile : p.rows;
  float w[8], dw[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = p.w[col + i];
    dw[i] = 0.f;
  }
  const T* __restrict__ x = static_cast<const T*>(p.x);
  const T* __restrict__ z = static_cast<const T*>(p.z);
  const float inv_group = 1.f / (float)p.group;
  // The rows arrive through a ring of asynchronous copies in shared memory, private to the thread (behind the
  // weight-gradient fold buffer): STAGES - 1 rows of x, z (and dy) in flight while one is worked on; a plain loop of
  // loads left the kernel waiting on memory for most of its time at one or two blocks per SM.
  constexpr int RB = 8 * (int)sizeof(T), STAGES = ring_stages(RB), NTENS = BWD ? 3 : 2;
  unsigned char* ring = reinterpret_cast<unsigned char*>(dw_red) + (BWD ? (size_t)blockDim.x * 8 * sizeof(float) : 0);
  auto slot = [&](int n, int st) { return ring + ((size_t)(n * STAGES + st) * blockDim.x + threadIdx.x) * RB; };
  const int n_it = (int)((r1 - r0 + lanes_r - 1) / lanes_r);
  auto request = [&](int it) {
    const long r = r0 + (long)it * lanes_r + lr;
    const long idx = ((live && r < r1) ? r : r0) * p.dim + col;  // rows nobody owns read the tile's first row
    cp_async_row<RB>(slot(0, it % STAGES), x + idx, true);
    cp_async_row<RB>(slot(1, it % STAGES), z + idx, true);
    if constexpr (BWD) cp_async_row<RB>(slot(2, it % STAGES), static_cast<const T*>(p.dy) + idx, true);
    cp_async_commit_group();
  };
#pragma unroll
  for (int it = 0; it < STAGES - 1; ++it) request(it);
  // every thread of the block runs the same number of iterations (group_sum may synchronise the block)
  for (int it = 0; it < n_it; ++it) {
    const long r = r0 + (long)it * lanes_r + lr;
    const bool on = live && r < r1;
    const long idx = (on ? r : r0) * p.dim + col;
    request(it + STAGES - 1);
    cp_async_wait_groups<STAGES - 1>();
    float xv[8], zv[8], gate[8], u[8];
    load8<T>(reinterpret_cast<const T*>(slot(0, it % STAGES)), xv);
    load8<T>(reinterpret_cast<const T*>(slot(1, it % STAGES)), zv);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = fast_rcp(1.f + fast_exp(-zv[i]));
      gate[i] = p.sigmoid_gate ? sg : zv[i] * sg;
      u[i] = p.norm_before_gate ? xv[i] : xv[i] * gate[i];
      ss += u[i] * u[i];
    }
    if (!on) ss = 0.f;
    const float rstd = fast_rsqrt(group_sum(ss, lanes, red) * inv_group + p.eps);
    if (!BWD) {
      float out[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = u[i] * rstd * w[i] * (p.norm_before_gate ? gate[i] : 1.f);
      if (on) store8<T>(static_cast<T*>(p.y) + idx, out);
    } else {
      float dyv[8], n[8], dn[8];
      load8<T>(reinterpret_cast<const T*>(slot(2, it % STAGES)), dyv);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        n[i] = u[i] * rstd;
        dn[i] = dyv[i] * w[i] * (p.norm_before_gate ? gate[i] : 1.f);
        dot += dn[i] * n[i];
      }
      if (!on) dot = 0.f;
      const float mean_dot = group_sum(dot, lanes, red) * inv_group;
      float dxv[8], dzv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float du = rstd * (dn[i] - n[i] * mean_dot);
        const float sg = fast_rcp(1.f + fast_exp(-zv[i]));
        const float dact = p.sigmoid_gate ? sg * (1.f - sg) : sg * (1.f + zv[i] * (1.f - sg));  // d gate / d z
        if (p.norm_before_gate) {
          dxv[i] = du;
          dzv[i] = dyv[i] * n[i] * w[i] * dact;
          if (on) dw[i] += dyv[i] * n[i] * gate[i];
        } else {
          dxv[i] = du * gate[i];
          dzv[i] = du * xv[i] * dact;
          if (on) dw[i] += dyv[i] * n[i];
        }
      }
      if (on) {
        store8<T>(static_cast<T*>(p.dx) + idx, dxv);
        store8<T>(static_cast<T*>(p.dz) + idx, dzv);
      }
    }
  }
  cp_async_wait_groups<0>();  // the trailing groups of the ring
  if (BWD) {
    if (lanes_r > 1) {  // fold the row lanes first: one atomic per channel and block
#pragma unroll
      for (int i = 0; i < 8; ++i) dw_red[(lr * cols + ct) * 8 + i] = dw[i];
      __syncthreads();
      if (lr == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = 0.f;
          for (int l = 0; l < lanes_r; ++l) t += dw_red[(l * cols + ct) * 8 + i];
          dw[i] = t;
        }
      }
    }
    if (live && lr == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(p.dw + col + i, dw[i]);
    }
  }
}

template <bool BWD>
int launch(int dtype, NormParams np, cudaStream_t s) {
  const int lanes = np.group / 8;
  if (np.rows < 0 || np.dim <= 0 || np.group <= 0 || np.dim % np.group || np.group % 8 || (lanes & (lanes - 1)) ||
      lanes > 1024) {
    set_error("gated rms norm: group (%d) must divide dim (%d) and be 8 times a power of two, at most 8192", np.group,
              np.dim);
    return JLA_ERR_UNSUPPORTED;
  }
  if (BWD) JLA_CUDA_OK(cudaMemsetAsync(np.dw, 0, sizeof(float) * np.dim, s));
  if (np.rows == 0) return JLA_OK;
  const int cv = np.dim / 8;
  int threads, cols;
  long per_lane;
  if (lanes > 32) {
    threads = cols = lanes;  // a block is one group
    per_lane = np.rows / 1024;
    per_lane = per_lane < 1 ? 1 : (per_lane > 16 ? 16 : per_lane);
  } else {
    // a warp covers 32 adjacent column vectors of one row (512 contiguous bytes); the block's other warps are row
    // lanes, so that many rows fold into one set of weight-gradient atomics
    cols = cv < 32 ? cv : 32;
    threads = cols * (512 / cols);
    per_lane = np.rows / ((threads / cols) * 64);
    per_lane = per_lane < 1 ? 1 : (per_lane > 16 ? 16 : per_lane);
  }
  np.cols = cols;
  const long lanes_r = threads / cols;
  np.rows_per_lane = (int)per_lane;
  const long tile = per_lane * lanes_r;
  const long tiles = (np.rows + tile - 1) / tile;
  if (tiles > 65535) {
    set_error("gated rms norm: more than %ld rows per call", 65535 * tile);
    return JLA_ERR_UNSUPPORTED;
  }
  const size_t row_bytes = 8 * (dtype == JLA_DTYPE_F32 ? 4 : 2);
  const size_t smem = (BWD ? sizeof(float) * threads * 8 : 0) +
                      (size_t)(BWD ? 3 : 2) * ring_stages((int)row_bytes) * threads * row_bytes;
  const dim3 grid((cv + cols - 1) / cols, (unsigned)tiles);
  cudaError_t attr = cudaSuccess;
  auto go = [&](auto kern) {
    attr = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr == cudaSuccess) kern<<<grid, threads, smem, s>>>(np);
  };
  const bool wide = threads > 512;
  switch (dtype) {
    case JLA_DTYPE_BF16:
      wide ? go(gated_rmsnorm_kernel<__nv_bfloat16, BWD, 1024>) : go(gated_rmsnorm_kernel<__nv_bfloat16, BWD, THREADS>);
      break;
    case JLA_DTYPE_F16:
      wide ? go(gated_rmsnorm_kernel<__half, BWD, 1024>) : go(gated_rmsnorm_kernel<__half, BWD, THREADS>);
      break;
    case JLA_DTYPE_F32:
      wide ? go(gated_rmsnorm_kernel<float, BWD, 1024>) : go(gated_rmsnorm_kernel<float, BWD, THREADS>);
      break;
    default: set_error("gated rms norm: unknown dtype %d", dtype); return JLA_ERR_BAD_ARGUMENT;
  }
  JLA_CUDA_OK(attr);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_gated_rmsnorm_fwd(int dtype, int64_t rows, int dim, int group, const void* x, const void* z,
                                     const float* weight, float eps, int sigmoid_gate, int norm_before_gate, void* y,
                                     jla_stream_t stream) {
  if (!x || !z || !weight || !y) return JLA_ERR_BAD_ARGUMENT;
  NormParams np{};
  np.rows = rows, np.dim = dim, np.group = group, np.x = x, np.z = z, np.w = weight, np.eps = eps;
  np.sigmoid_gate = sigmoid_gate, np.norm_before_gate = norm_before_gate, np.y = y;
  return launch<false>(dtype, np, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_gated_rmsnorm_bwd(int dtype, int64_t rows, int dim, int group, const void* x, const void* z,
                                     const float* weight, float eps, int sigmoid_gate, int norm_before_gate,
                                     const void* dy, void* dx, void* dz, float* dweight, jla_stream_t stream) {
  if (!x || !z || !weight || !dy || !dx || !dz || !dweight) return JLA_ERR_BAD_ARGUMENT;
  NormParams np{};
  np.rows = rows, np.dim = dim, np.group = group, np.x = x, np.z = z, np.w = weight, np.eps = eps;
  np.sigmoid_gate = sigmoid_gate, np.norm_before_gate = norm_before_gate, np.dy = dy, np.dx = dx, np.dz = dz;
  np.dw = dweight;
  return launch<true>(dtype, np, static_cast<cudaStream_t>(stream));
}
