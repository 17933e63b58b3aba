// Element-wise glue of the Mamba-2 SSD layer around the simple_gla kernels, fused so that each tensor of
// [tokens, H, P] is read and written once (the reference computes these in XLA fusions next to its kernels,
// src/jla/layers/ssm.py:207-229):
//
//   inputs   v = (x * dt) rounded to the activation dtype,  g = dt * A                      (fp32 g)
//            dx = dv * dt,  ddt = sum_p dv * x + dg * A,  dA = sum_{tokens} dg * dt
//   output   y = o + D * x   (fp32 sum, rounded once)
//            do = dy (the same tensor),  dx = D * dy,  dD = sum_{tokens, p} dy * x
//   layer    both transposes in one pass when the layer has a D term: dx = dv * dt + D * dy with ddt, dA, dD as
//            above (x, dv, dy read once, dx written once, instead of two partial dx tensors and their sum)
//
// HBM-bound: a thread owns 8 adjacent channels (one 16-byte load per tensor) of one head and walks a tile of
// tokens, so the per-head sums dA, dD stay in registers and leave the block as one atomic per head.
#include "common.cuh"

namespace jla {
namespace {

constexpr int THREADS = 256;
constexpr int TOKENS_PER_BLOCK = 64;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
  uint4 u;
  T* e = reinterpret_cast<T*>(&u);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(f[i]);
  *reinterpret_cast<uint4*>(p) = u;
}

// sum over the `lanes` (power of two <= 32) adjacent lanes that share a head
__device__ __forceinline__ float group_sum(float x, int lanes) {
  for (int off = lanes >> 1; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

struct GlueParams {
  long tokens;
  int H, P;
  const void *x, *other;  // other: dv (inputs_bwd, layer_bwd), o (output_fwd), dy (output_bwd)
  const void* dy;         // layer_bwd only
  const float *dt, *a, *dg;
  const float* d;         // layer_bwd only: the skip weights D [H]
  void* out;              // v, dx, y
  float *g, *ddt, *hsum;  // hsum: dA or dD [H]
  float* dd;              // layer_bwd only: dD [H] (hsum is dA)
};

enum Mode { kInputsFwd, kInputsBwd, kOutputFwd, kOutputBwd, kLayerBwd };

template <typename T, int MODE>
__global__ void __launch_bounds__(THREADS) ssd_glue_kernel(GlueParams p) {
  const int col = (blockIdx.x * THREADS + threadIdx.x) * 8;  // channel offset inside the token's [H * P] row
  const int HP = p.H * p.P;
  const bool live = col < HP;
  const int h = live ? col / p.P : 0;
  const int lanes = p.P / 8;                    // threads per head
  const bool pow2 = lanes <= 32 && (lanes & (lanes - 1)) == 0;
  const bool head_lead = (col % p.P) == 0;
  const long t0 = (long)blockIdx.y * TOKENS_PER_BLOCK;
  const long t1 = t0 + TOKENS_PER_BLOCK < p.tokens ? t0 + TOKENS_PER_BLOCK : p.tokens;
  const float coef = live && (MODE == kOutputFwd || MODE == kOutputBwd) ? p.a[h] : 0.f;  // D for the output side
  const float ah = live && (MODE == kInputsFwd || MODE == kInputsBwd || MODE == kLayerBwd) ? p.a[h] : 0.f;
  const float dh = live && MODE == kLayerBwd ? p.d[h] : 0.f;
  float hacc = 0.f, dacc = 0.f;
  for (long t = t0; t < t1; ++t) {
    const long row = t * p.H + h;
    const long off = t * HP + col;
    float xv[8] = {}, ov[8] = {}, res[8];
    if (live) {
      load8<T>(static_cast<const T*>(p.x) + off, xv);
      if (MODE != kInputsFwd) load8<T>(static_cast<const T*>(p.other) + off, ov);
    }
    float yv[8] = {};
    if (MODE == kLayerBwd && live) load8<T>(static_cast<const T*>(p.dy) + off, yv);
    if (MODE == kInputsFwd) {
      const float dt = live ? p.dt[row] : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = xv[i] * dt;
      if (live && head_lead) p.g[row] = dt * ah;
    } else if (MODE == kInputsBwd || MODE == kLayerBwd) {
      const float dt = live ? p.dt[row] : 0.f;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // the two-kernel form rounds dv * dt and D * dy to the activation dtype before their sum; here one rounding
        res[i] = MODE == kLayerBwd ? fmaf(dh, yv[i], ov[i] * dt) : ov[i] * dt;
        dot += ov[i] * xv[i];
        if (MODE == kLayerBwd) dacc += yv[i] * xv[i];
      }
      const float dg = live ? p.dg[row] : 0.f;
      if (pow2) {
        dot = group_sum(dot, lanes);
        if (live && head_lead) p.ddt[row] = dot + dg * ah;
      } else if (live) {
        atomicAdd(p.ddt + row, dot + (head_lead ? dg * ah : 0.f));  // ddt zeroed by the launcher in this case
      }
      if (head_lead) hacc += dg * dt;
    } else if (MODE == kOutputFwd) {
#pragma unroll
      for (int i = 0; i < 8; ++i) res[i] = ov[i] + coef * xv[i];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        res[i] = coef * ov[i];
        hacc += ov[i] * xv[i];
      }
    }
    if (live) store8<T>(static_cast<T*>(p.out) + off, res);
  }
  if (MODE == kInputsBwd || MODE == kLayerBwd) {
    if (live && head_lead) atomicAdd(p.hsum + h, hacc);
    if (MODE == kLayerBwd) {
      if (pow2) {
        dacc = group_sum(dacc, lanes);
        if (live && head_lead) atomicAdd(p.dd + h, dacc);
      } else if (live) {
        atomicAdd(p.dd + h, dacc);
      }
    }
  } else if (MODE == kOutputBwd) {
    if (pow2) {
      hacc = group_sum(hacc, lanes);
      if (live && head_lead) atomicAdd(p.hsum + h, hacc);
    } else if (live) {
      atomicAdd(p.hsum + h, hacc);
    }
  }
}

template <int MODE>
int launch(int dtype, const GlueParams& gp, cudaStream_t s) {
  if (gp.tokens < 0 || gp.H <= 0 || gp.P <= 0 || gp.P % 8 != 0) {
    set_error("ssd glue: need H > 0 and P a positive multiple of 8 (got H=%d, P=%d)", gp.H, gp.P);
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (dtype != JLA_DTYPE_BF16 && dtype != JLA_DTYPE_F16) {
    set_error("ssd glue: 16-bit activations only");
    return JLA_ERR_UNSUPPORTED;
  }
  if (gp.tokens == 0) return JLA_OK;
  const int lanes = gp.P / 8;
  const bool pow2 = lanes <= 32 && (lanes & (lanes - 1)) == 0;
  if (MODE == kInputsBwd || MODE == kOutputBwd || MODE == kLayerBwd) {
    JLA_CUDA_OK(cudaMemsetAsync(gp.hsum, 0, sizeof(float) * gp.H, s));
    if (MODE == kLayerBwd) JLA_CUDA_OK(cudaMemsetAsync(gp.dd, 0, sizeof(float) * gp.H, s));
    if (MODE != kOutputBwd && !pow2) JLA_CUDA_OK(cudaMemsetAsync(gp.ddt, 0, sizeof(float) * gp.tokens * gp.H, s));
  }
  const long tiles = (gp.tokens + TOKENS_PER_BLOCK - 1) / TOKENS_PER_BLOCK;
  if (tiles > 65535) {
    set_error("ssd glue: more than %d tokens per call", 65535 * TOKENS_PER_BLOCK);
    return JLA_ERR_UNSUPPORTED;
  }
  const dim3 grid((gp.H * gp.P / 8 + THREADS - 1) / THREADS, (unsigned)tiles);
  if (dtype == JLA_DTYPE_BF16) ssd_glue_kernel<__nv_bfloat16, MODE><<<grid, THREADS, 0, s>>>(gp);
  else ssd_glue_kernel<__half, MODE><<<grid, THREADS, 0, s>>>(gp);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_ssd_inputs_fwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a,
                                  void* v, float* g, jla_stream_t stream) {
  if (!x || !dt || !a || !v || !g) return JLA_ERR_BAD_ARGUMENT;
  GlueParams gp{};
  gp.tokens = tokens, gp.H = H, gp.P = P, gp.x = x, gp.dt = dt, gp.a = a, gp.out = v, gp.g = g;
  return launch<kInputsFwd>(dtype, gp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_ssd_inputs_bwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a,
                                  const void* dv, const float* dg, void* dx, float* ddt, float* da, jla_stream_t stream) {
  if (!x || !dt || !a || !dv || !dg || !dx || !ddt || !da) return JLA_ERR_BAD_ARGUMENT;
  GlueParams gp{};
  gp.tokens = tokens, gp.H = H, gp.P = P, gp.x = x, gp.other = dv, gp.dt = dt, gp.a = a, gp.dg = dg, gp.out = dx;
  gp.ddt = ddt, gp.hsum = da;
  return launch<kInputsBwd>(dtype, gp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_ssd_output_fwd(int dtype, int64_t tokens, int H, int P, const void* o, const void* x, const float* d,
                                  void* y, jla_stream_t stream) {
  if (!o || !x || !d || !y) return JLA_ERR_BAD_ARGUMENT;
  GlueParams gp{};
  gp.tokens = tokens, gp.H = H, gp.P = P, gp.x = x, gp.other = o, gp.a = d, gp.out = y;
  return launch<kOutputFwd>(dtype, gp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_ssd_output_bwd(int dtype, int64_t tokens, int H, int P, const void* dy, const void* x, const float* d,
                                  void* dx, float* dd, jla_stream_t stream) {
  if (!dy || !x || !d || !dx || !dd) return JLA_ERR_BAD_ARGUMENT;
  GlueParams gp{};
  gp.tokens = tokens, gp.H = H, gp.P = P, gp.x = x, gp.other = dy, gp.a = d, gp.out = dx, gp.hsum = dd;
  return launch<kOutputBwd>(dtype, gp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_ssd_layer_bwd(int dtype, int64_t tokens, int H, int P, const void* x, const float* dt, const float* a,
                                 const float* d, const void* dv, const float* dg, const void* dy, void* dx, float* ddt,
                                 float* da, float* dd, jla_stream_t stream) {
  if (!x || !dt || !a || !d || !dv || !dg || !dy || !dx || !ddt || !da || !dd) return JLA_ERR_BAD_ARGUMENT;
  GlueParams gp{};
  gp.tokens = tokens, gp.H = H, gp.P = P, gp.x = x, gp.other = dv, gp.dy = dy, gp.dt = dt, gp.a = a, gp.d = d, gp.dg = dg;
  gp.out = dx, gp.ddt = ddt, gp.hsum = da, gp.dd = dd;
  return launch<kLayerBwd>(dtype, gp, static_cast<cudaStream_t>(stream));
}
