// Gate activations in front of the linear-attention kernels, fused forward and backward
// (src/jla/layers/linear_attention.py:84-86 `_mamba_gate`, :159-162 `_write_strength`; used by the Gated DeltaNet
// mixer :295-297 and the KDA mixer :324-328):
//
//   g    = -exp(A_log[h]) * softplus(a + dt_bias)        a [tokens, H, C] (C = 1: one decay per head; C = K: KDA),
//                                                        dt_bias [H, C], A_log [H]; g float32
//   beta = m * sigmoid(b),  m = 2 if allow_neg_eigval else 1      b [tokens, H]; beta float32
//
//   da = dg * (-exp(A_log)) * sigmoid(a + dt_bias);  dA_log[h] = sum dg * g;  ddt_bias[h, c] = sum_tokens da
//   db = dbeta * beta * (1 - beta / m)
//
// HBM-bound element-wise work. A thread owns eight adjacent (h, c) columns and walks a tile of tokens, so the
// parameter gradients are summed in registers and leave the thread as one atomic per output.
#include "common.cuh"

namespace jla {
namespace {

constexpr int THREADS = 512;

struct GateParams {
  long tokens;
  int H, C;
  const void *a, *b;            // activations (dtype), b may be null
  const float *a_log, *dt_bias;
  float mult;                   // 1 or 2
  int tokens_per_lane;          // tokens one thread walks (set by the launcher)
  int cols;                     // column threads of a block; the other threads are token lanes
  float *g, *beta;              // forward outputs
  const float *dg, *dbeta;      // backward inputs
  void *da, *db;                // backward outputs (dtype)
  float *da_log, *ddt_bias;     // [H], [H * C], accumulated with atomics (zeroed by the launcher)
};

// softplus(x) = max(x, 0) + log1p(e), e = exp(-|x|) in (0, 1]. log1p(e) = 2 atanh(s) with s = e / (2 + e) <= 1/3, as
// the odd series up to s^13 (the next term is 1.4e-8 of the result): relative error about 1e-7 for every e, small
// ones included, in a third of the instructions of the library's log1pf.
__device__ __forceinline__ float softplus(float x) {
  const float e = fast_exp(-fabsf(x));
  const float s = e * fast_rcp(2.f + e), z = s * s;
  float poly = 1.f / 13.f;
  poly = fmaf(poly, z, 1.f / 11.f);
  poly = fmaf(poly, z, 1.f / 9.f);
  poly = fmaf(poly, z, 1.f / 7.f);
  poly = fmaf(poly, z, 1.f / 5.f);
  poly = fmaf(poly, z, 1.f / 3.f);
  poly = fmaf(poly, z, 1.f);
  return fmaxf(x, 0.f) + 2.f * s * poly;
}
__device__ __forceinline__ float sigmoid(float x) { return fast_rcp(1.f + fast_exp(-x)); }

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[VEC]) {
  if constexpr (VEC == 8 && sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
  } else if constexpr (VEC == 8) {
    const float4 x = *reinterpret_cast<const float4*>(p), y = *reinterpret_cast<const float4*>(p + 4);
    f[0] = to_f32(x.x), f[1] = to_f32(x.y), f[2] = to_f32(x.z), f[3] = to_f32(x.w);
    f[4] = to_f32(y.x), f[5] = to_f32(y.y), f[6] = to_f32(y.z), f[7] = to_f32(y.w);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = to_f32(p[i]);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[VEC]) {
  if constexpr (VEC == 8 && sizeof(T) == 2) {
    uint4 u;
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(f[i]);
    *reinterpret_cast<uint4*>(p) = u;
  } else if constexpr (VEC == 8) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = from_f32<T>(f[i]);
  }
}

// A thread owns VEC adjacent (h, c) columns (one 16-byte load of 16-bit activations) and walks every `lanes_t`-th token
// of its block's tile. Block layout: min(H * C / VEC, THREADS) column threads x the remaining threads as token lanes.
template <typename T, bool BWD, int VEC>
__global__ void __launch_bounds__(THREADS, 2) gate_kernel(GateParams p) {
  const int HC = p.H * p.C;
  const int groups = HC / VEC;
  const int cols = p.cols;
  const int lanes_t = blockDim.x / cols;
  const int ct = (int)(threadIdx.x % cols);
  const int grp = blockIdx.x * cols + ct;
  const int lt = threadIdx.x / cols;
  const bool active = lt < lanes_t && grp < groups;
  const int col = active ? grp * VEC : 0;
  const long tile = (long)p.tokens_per_lane * lanes_t;
  const long t0 = (long)blockIdx.y * tile;
  const long t1 = t0 + tile < p.tokens ? t0 + tile : p.tokens;
  float neg_a[VEC], bias[VEC], s_alog[VEC], s_bias[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    neg_a[i] = -expf(p.a_log[(col + i) / p.C]);
    bias[i] = p.dt_bias[col + i];
    s_alog[i] = s_bias[i] = 0.f;
  }
  const T* __restrict__ a = static_cast<const T*>(p.a);
  const T* __restrict__ b = static_cast<const T*>(p.b);
  unsigned beta_cols = 0;  // bit i: column col + i is the first of its head
  int beta_head[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    beta_head[i] = (col + i) / p.C;
    if (b && (col + i) % p.C == 0) beta_cols |= 1u << i;
  }
  // VEC = 8: the rows of a (and dg) arrive through a ring of asynchronous copies in shared memory, private to the
  // thread, STAGES - 1 tokens in flight while one is worked on (a plain loop of loads waits on memory most of the
  // time at one or two blocks per SM). Tokens past the thread's range are zero-filled and never used.
  constexpr bool RING = VEC == 8;
  constexpr int RA = VEC * (int)sizeof(T), RG = VEC * (int)sizeof(float), STAGES = 3;
  extern __shared__ __align__(16) unsigned char ring[];
  auto slot_a = [&](int st) { return ring + ((size_t)st * blockDim.x + threadIdx.x) * RA; };
  auto slot_g = [&](int st) {
    return ring + (size_t)STAGES * blockDim.x * RA + ((size_t)st * blockDim.x + threadIdx.x) * RG;
  };
  auto request = [&](int it) {
    if constexpr (RING) {
      const long t = t0 + lt + (long)it * lanes_t;
      const bool valid = active && t < t1;
      const long idx = valid ? t * HC + col : 0;
      cp_async_row<RA>(slot_a(it % STAGES), a + idx, valid);
      if constexpr (BWD) cp_async_row<RG>(slot_g(it % STAGES), p.dg + idx, valid);
      cp_async_commit_group();
    }
  };
#pragma unroll
  for (int it = 0; it < STAGES - 1; ++it) request(it);
  int it = 0;
  for (long t = t0 + lt; active && t < t1; t += lanes_t, ++it) {
    const long idx = t * HC + col;
    float x[VEC], out[VEC];
    if constexpr (RING) {
      request(it + STAGES - 1);
      cp_async_wait_groups<STAGES - 1>();
      load_vec<T, VEC>(reinterpret_cast<const T*>(slot_a(it % STAGES)), x);
    } else {
      load_vec<T, VEC>(a + idx, x);
    }
    if (!BWD) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) out[i] = neg_a[i] * softplus(x[i] + bias[i]);
      store_vec<float, VEC>(p.g + idx, out);
    } else {
      float dg[VEC];
      if constexpr (RING) load_vec<float, VEC>(reinterpret_cast<const float*>(slot_g(it % STAGES)), dg);
      else load_vec<float, VEC>(p.dg + idx, dg);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        // one exponential serves the sigmoid and the softplus; the softplus only enters the sum dA_log, where the
        // one-instruction logarithm's absolute error of 1e-7 disappears
        const float xi = x[i] + bias[i];
        const float e = fast_exp(-fabsf(xi));  // in (0, 1]
        const float r = fast_rcp(1.f + e);
        const float ga = dg[i] * neg_a[i];
        out[i] = ga * (xi >= 0.f ? r : e * r);
        s_bias[i] += out[i];
        s_alog[i] += ga * (fmaxf(xi, 0.f) + fast_log(1.f + e));
      }
      store_vec<T, VEC>(static_cast<T*>(p.da) + idx, out);
    }
    // the thread that owns column c = 0 of a head handles that head's beta (which of its columns those are was
    // worked out once, before the loop: a division by the runtime C per column and token costs more than the gate)
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (!(beta_cols >> i & 1)) continue;
      const long bi = t * p.H + beta_head[i];
      const float beta = p.mult * sigmoid(to_f32(b[bi]));
      if (!BWD) p.beta[bi] = beta;
      else static_cast<T*>(p.db)[bi] = from_f32<T>(p.dbeta[bi] * beta * (1.f - beta / p.mult));
    }
  }
  if constexpr (RING) cp_async_wait_groups<0>();  // the trailing (empty) groups of the ring
  if (BWD) {
    // parameter gradients: first over the block's token lanes in shared memory, then one atomic per column and block
    __shared__ float red_bias[THREADS * VEC], red_alog[THREADS * VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      red_bias[threadIdx.x * VEC + i] = s_bias[i];
      red_alog[threadIdx.x * VEC + i] = s_alog[i];
    }
    __syncthreads();
    if (active && lt == 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float sb = 0.f, sa = 0.f;
        for (int l = 0; l < lanes_t; ++l) {
          sb += red_bias[(l * cols + ct) * VEC + i];
          sa += red_alog[(l * cols + ct) * VEC + i];
        }
        s_bias[i] = sb;
        s_alog[i] = sa;
        atomicAdd(p.ddt_bias + col + i, sb);
      }
      if (p.C % VEC == 0) {  // the thread's columns share one head
        float sa = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) sa += s_alog[i];
        atomicAdd(p.da_log + col / p.C, sa);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) atomicAdd(p.da_log + (col + i) / p.C, s_alog[i]);
      }
    }
  }
}

template <bool BWD, int VEC>
int launch_vec(int dtype, const GateParams& gp, cudaStream_t s) {
  const int groups = gp.H * gp.C / VEC;
  // a warp covers up to 32 adjacent column groups of one token; the block's other warps are token lanes, so that
  // many tokens fold into one set of parameter-gradient atomics
  const int cols = groups < 32 ? groups : 32;
  if (groups % cols != 0 || THREADS % cols != 0) {
    set_error("gate prologue: H * C / %d = %d must divide 32 or be a multiple of it", VEC, groups);
    return JLA_ERR_UNSUPPORTED;
  }
  const long lanes_t = THREADS / cols;
  long per_lane = gp.tokens / (lanes_t * 64);
  // up to 16 tokens per thread (4 measured slower: the fixed cost of a block, its ring's first copies and its atomics,
  // outweighs the better fill of the last round of blocks)
  per_lane = per_lane < 1 ? 1 : (per_lane > 16 ? 16 : per_lane);
  const long tile = per_lane * lanes_t;
  const long tiles = (gp.tokens + tile - 1) / tile;
  if (tiles > 65535) {
    set_error("gate prologue: more than %ld tokens per call", 65535 * tile);
    return JLA_ERR_UNSUPPORTED;
  }
  GateParams q = gp;
  q.tokens_per_lane = (int)per_lane;
  q.cols = cols;
  const dim3 grid(groups / cols, (unsigned)tiles);
  // the ring of row copies (VEC = 8): three stages of a, and of dg in the backward, per thread
  const size_t es = dtype == JLA_DTYPE_F32 ? 4 : 2;
  const size_t smem = VEC == 8 ? (size_t)3 * THREADS * (VEC * es + (BWD ? VEC * sizeof(float) : 0)) : 0;
  cudaError_t attr = cudaSuccess;
  auto go = [&](auto kern) {
    attr = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (attr == cudaSuccess) kern<<<grid, THREADS, smem, s>>>(q);
  };
  switch (dtype) {
    case JLA_DTYPE_BF16: go(gate_kernel<__nv_bfloat16, BWD, VEC>); break;
    case JLA_DTYPE_F16: go(gate_kernel<__half, BWD, VEC>); break;
    case JLA_DTYPE_F32: go(gate_kernel<float, BWD, VEC>); break;
    default: set_error("gate prologue: unknown dtype %d", dtype); return JLA_ERR_BAD_ARGUMENT;
  }
  JLA_CUDA_OK(attr);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <bool BWD>
int launch(int dtype, const GateParams& gp, cudaStream_t s) {
  if (gp.tokens < 0 || gp.H <= 0 || gp.C <= 0) {
    set_error("gate prologue: need H > 0 and C > 0 (got H=%d, C=%d)", gp.H, gp.C);
    return JLA_ERR_BAD_ARGUMENT;
  }
  if (BWD) {
    JLA_CUDA_OK(cudaMemsetAsync(gp.da_log, 0, sizeof(float) * gp.H, s));
    JLA_CUDA_OK(cudaMemsetAsync(gp.ddt_bias, 0, sizeof(float) * gp.H * gp.C, s));
  }
  if (gp.tokens == 0) return JLA_OK;
  return (gp.H * gp.C) % 8 == 0 ? launch_vec<BWD, 8>(dtype, gp, s) : launch_vec<BWD, 1>(dtype, gp, s);
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_gate_prologue_fwd(int dtype, int64_t tokens, int H, int C, const void* a, const float* a_log,
                                     const float* dt_bias, const void* b, int allow_neg_eigval, float* g, float* beta,
                                     jla_stream_t stream) {
  if (!a || !a_log || !dt_bias || !g || (b && !beta)) return JLA_ERR_BAD_ARGUMENT;
  GateParams gp{};
  gp.tokens = tokens, gp.H = H, gp.C = C, gp.a = a, gp.b = b, gp.a_log = a_log, gp.dt_bias = dt_bias;
  gp.mult = allow_neg_eigval ? 2.f : 1.f, gp.g = g, gp.beta = beta;
  return launch<false>(dtype, gp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_gate_prologue_bwd(int dtype, int64_t tokens, int H, int C, const void* a, const float* a_log,
                                     const float* dt_bias, const void* b, int allow_neg_eigval, const float* dg,
                                     const float* dbeta, void* da, void* db, float* da_log, float* ddt_bias,
                                     jla_stream_t stream) {
  if (!a || !a_log || !dt_bias || !dg || !da || !da_log || !ddt_bias || (b && (!dbeta || !db))) return JLA_ERR_BAD_ARGUMENT;
  GateParams gp{};
  gp.tokens = tokens, gp.H = H, gp.C = C, gp.a = a, gp.b = b, gp.a_log = a_log, gp.dt_bias = dt_bias;
  gp.mult = allow_neg_eigval ? 2.f : 1.f, gp.dg = dg, gp.dbeta = dbeta, gp.da = da, gp.db = db;
  gp.da_log = da_log, gp.ddt_bias = ddt_bias;
  return launch<true>(dtype, gp, static_cast<cudaStream_t>(stream));
}
