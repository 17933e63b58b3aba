// Short causal depthwise convolution + SiLU + per-head L2 norm, the q / k prologue of the delta-rule mixers, forward
// and backward in one pass each (src/jla/layers/conv.py:97-142 `ShortConv.__call__`,
// src/jla/ops/mosaic_gpu/short_conv_l2norm.py:5-20, src/jla/ops/reference.py:65-69 `l2norm`):
//
//   pre_t = bias + sum_{i < K} w[:, i] * x_ext[t + i],  x_ext = [state (K - 1 rows) ; x],  taps that reach into an
//           earlier document (segment_ids differ; state rows count as the first token's document) contribute zero
//   y_t   = silu(pre_t)  (activation)          n_t = y_t * rsqrt(sum over the head's channels of y_t^2 + 1e-6)
//
//   dy = inv (dn - n sum_head(dn n));  dpre = dy silu'(pre);  dx_ext[s] = sum_i w[:, i] dpre[s - i + K - 1] (same
//   document);  dw[:, i] = sum dpre_t x_ext[t + i];  dbias = sum dpre_t
//
// HBM-bound. The conv output stays in float32 until the norm has been applied and is rounded once. (Block and
// thread layout: see the kernel.)
#include "common.cuh"

namespace jla {
namespace {

constexpr int THREADS = 256;
constexpr int KMAX = 4;
constexpr float kL2Eps = 1e-6f;

struct ConvParams {
  int B, T, C, K, head_dim, activation;
  const void* x;
  const float *w, *bias;
  const int32_t* seg;
  const void* state;
  void* y;
  const void* dy;
  void* dx;
  float *dw, *dbias;
  void* dstate;
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

__device__ __forceinline__ float head_sum(float v, int lanes) {
  for (int off = lanes >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// A block owns TT consecutive tokens of one batch row and 32 adjacent channel vectors (256 channels: one or several
// whole heads). The inputs it needs (the tile plus K - 1 rows in front, in the backward also K - 1 behind) are staged
// once in shared memory; a warp then handles one token at a time (lane = channel vector), so the head sums are warp
// butterflies and nothing is walked serially.
constexpr int TT = 64;
constexpr int COLS = 32;
constexpr int ROW_LANES = THREADS / COLS;  // 8 tokens in flight per block

struct Tile {
  int b, t0, t1;
};

__device__ __forceinline__ int seg_at(const ConvParams& p, int b, int t) {
  if (!p.seg) return 0;
  return p.seg[(long)b * p.T + (t < 0 ? 0 : (t >= p.T ? p.T - 1 : t))];
}

// Stages rows [r0, r0 + rows) of x_ext (state rows for t < 0, zeros outside) as float32: xs[row][COLS * 8], and their
// document ids (state rows: the first token's).
template <typename T>
__device__ __forceinline__ void stage_rows(const ConvParams& p, int b, int r0, int rows, int col0, int cv, int vec0,
                                           float* xs, int* ss) {
  for (int idx = threadIdx.x; idx < rows * COLS; idx += THREADS) {
    const int r = idx / COLS, c = idx % COLS, t = r0 + r;
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = 0.f;
    if (vec0 + c < cv && t < p.T) {
      if (t >= 0) load8<T>(static_cast<const T*>(p.x) + ((long)b * p.T + t) * p.C + col0 + c * 8, f);
      else if (p.state && t >= -(p.K - 1))
        load8<T>(static_cast<const T*>(p.state) + ((long)b * (p.K - 1) + (p.K - 1 + t)) * p.C + col0 + c * 8, f);
    }
    float4* dst = reinterpret_cast<float4*>(xs + (size_t)r * COLS * 8 + c * 8);
    dst[0] = make_float4(f[0], f[1], f[2], f[3]);
    dst[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
  for (int r = threadIdx.x; r < rows; r += THREADS) ss[r] = seg_at(p, b, r0 + r);
}

// Pre-activation, activation and norm of the token whose window starts at staged row `r` (rows r .. r + K - 1, the
// last one being the token itself). y is normalised when head_dim > 0.
struct TokenOut {
  float y[8], pre[8], sg[8], inv;  // sg = sigmoid(pre) when the activation is on
};

template <int K>
__device__ __forceinline__ void conv_token(const ConvParams& p, const float (&w)[KMAX][8], const float (&bias)[8],
                                           const float* xs, const int* ss, int r, int ct, int lanes, TokenOut& o) {
  const int sc = ss[r + K - 1];
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = bias[c];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    if (j == K - 1 || ss[r + j] == sc) {
      const float4* src = reinterpret_cast<const float4*>(xs + (size_t)(r + j) * COLS * 8 + ct * 8);
      const float4 a = src[0], b4 = src[1];
      const float v[8] = {a.x, a.y, a.z, a.w, b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += w[j][c] * v[c];
    }
  }
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    o.pre[c] = acc[c];
    o.sg[c] = __frcp_rn(1.f + __expf(-acc[c]));
    const float y = p.activation ? acc[c] * o.sg[c] : acc[c];
    o.y[c] = y;
    sq += y * y;
  }
  o.inv = 1.f;
  if (p.head_dim > 0) {
    o.inv = rsqrtf(head_sum(sq, lanes) + kL2Eps);
#pragma unroll
    for (int c = 0; c < 8; ++c) o.y[c] *= o.inv;
  }
}

template <typename T, bool BWD, int K>
__global__ void __launch_bounds__(THREADS) short_conv_kernel(ConvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int cv = p.C / 8;
  const int ct = threadIdx.x % COLS, lr = threadIdx.x / COLS;
  const int vec0 = blockIdx.x * COLS;
  const bool live = vec0 + ct < cv;
  const int col0 = vec0 * 8, col = (live ? vec0 + ct : 0) * 8;
  const int lanes = p.head_dim > 0 ? p.head_dim / 8 : 1;
  const int tiles_per_row = (p.T + TT - 1) / TT;
  const int b = blockIdx.y / tiles_per_row;
  const int t0 = (blockIdx.y % tiles_per_row) * TT;
  const int t1 = t0 + TT < p.T ? t0 + TT : p.T;
  float w[KMAX][8], bias[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    bias[c] = p.bias ? p.bias[col + c] : 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) w[j][c] = j < K ? p.w[(long)(col + c) * K + j] : 0.f;
  }

  if constexpr (!BWD) {
    constexpr int ROWS = TT + K - 1;  // staged rows: tokens t0 - (K - 1) .. t1 - 1
    float* xs = reinterpret_cast<float*>(smem_raw);
    int* ss = reinterpret_cast<int*>(xs + ROWS * COLS * 8);
    stage_rows<T>(p, b, t0 - (K - 1), ROWS, col0, cv, vec0, xs, ss);
    __syncthreads();
    for (int i = lr; i < TT; i += ROW_LANES) {  // token t0 + i: its window starts at staged row i
      TokenOut o;
      conv_token<K>(p, w, bias, xs, ss, i, ct, lanes, o);
      if (live && t0 + i < t1) store8<T>(static_cast<T*>(p.y) + ((long)b * p.T + t0 + i) * p.C + col, o.y);
    }
  } else {
    // staged inputs: tokens t0 - (K - 1) .. t1 + (K - 1) - 1 (the K - 1 tokens behind the tile are recomputed: their
    // pre-activation gradients reach back into the tile); dps[i] = dpre of token t0 + i, i < TT + K - 1
    constexpr int ROWS = TT + 2 * (K - 1), DROWS = TT + K - 1;
    float* xs = reinterpret_cast<float*>(smem_raw);
    float* dps = xs + ROWS * COLS * 8;
    float* fold = xs;  // [ROW_LANES][COLS * 8 * (K + 1)], over the staged rows once they are dead
    static_assert(ROW_LANES * (K + 1) <= ROWS + DROWS, "the fold buffer fits over the staged rows");
    int* ss = reinterpret_cast<int*>(dps + DROWS * COLS * 8);
    stage_rows<T>(p, b, t0 - (K - 1), ROWS, col0, cv, vec0, xs, ss);
    __syncthreads();
    float dwacc[KMAX][8], dbacc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      dbacc[c] = 0.f;
#pragma unroll
      for (int j = 0; j < KMAX; ++j) dwacc[j][c] = 0.f;
    }
    for (int i = lr; i < DROWS; i += ROW_LANES) {  // a warp handles one token at a time (i depends on the warp only)
      const int t = t0 + i;
      const bool token = t < p.T;
      TokenOut o;
      conv_token<K>(p, w, bias, xs, ss, i, ct, lanes, o);
      float dnv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) dnv[c] = 0.f;
      if (token && live) load8<T>(static_cast<const T*>(p.dy) + ((long)b * p.T + t) * p.C + col, dnv);
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) dot += dnv[c] * o.y[c];
      if (p.head_dim > 0) dot = head_sum(dot, lanes);
      float dpre[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float dy = p.head_dim > 0 ? o.inv * (dnv[c] - o.y[c] * dot) : dnv[c];
        const float sg = o.sg[c];
        dpre[c] = !token ? 0.f : (p.activation ? dy * sg * (1.f + o.pre[c] * (1.f - sg)) : dy);
      }
      float4* dst = reinterpret_cast<float4*>(dps + (size_t)i * COLS * 8 + ct * 8);
      dst[0] = make_float4(dpre[0], dpre[1], dpre[2], dpre[3]);
      dst[1] = make_float4(dpre[4], dpre[5], dpre[6], dpre[7]);
      if (t < t1) {  // inside the tile: this token's share of the parameter gradients
        const int sc = ss[i + K - 1];
#pragma unroll
        for (int j = 0; j < K; ++j) {
          if (j == K - 1 || ss[i + j] == sc) {
            const float4* src = reinterpret_cast<const float4*>(xs + (size_t)(i + j) * COLS * 8 + ct * 8);
            const float4 a = src[0], b4 = src[1];
            const float v[8] = {a.x, a.y, a.z, a.w, b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) dwacc[j][c] += dpre[c] * v[c];
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) dbacc[c] += dpre[c];
      }
    }
    __syncthreads();
    // dx_ext[s] = sum_{l < K} w[:, K - 1 - l] dpre[s + l] over the later tokens of the same document (l = 0: the token
    // itself). Rows s = t0 .. t1 - 1, and for the row's first tile also the K - 1 state rows in front.
    const int first = (t0 == 0 && p.dstate) ? -(K - 1) : 0;
    for (int i = first + lr; i < TT; i += ROW_LANES) {
      const int srow = t0 + i;
      if (srow >= t1 || !live) continue;
      const int sc = ss[i + K - 1];  // staged row of token t0 + i is i + K - 1
      float acc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = 0.f;
#pragma unroll
      for (int l = 0; l < K; ++l) {
        const int u = i + l;  // dps index of token srow + l
        if (u < 0 || u >= DROWS) continue;
        if (l == 0 ? srow >= 0 : ss[u + K - 1] == sc) {
          const float4* src = reinterpret_cast<const float4*>(dps + (size_t)u * COLS * 8 + ct * 8);
          const float4 a = src[0], b4 = src[1];
          const float v[8] = {a.x, a.y, a.z, a.w, b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] += w[K - 1 - l][c] * v[c];
        }
      }
      if (srow >= 0) store8<T>(static_cast<T*>(p.dx) + ((long)b * p.T + srow) * p.C + col, acc);
      else store8<T>(static_cast<T*>(p.dstate) + ((long)b * (K - 1) + (K - 1 + srow)) * p.C + col, acc);
    }
    __syncthreads();  // every warp is done with the staged rows: the fold buffer takes their place
    // parameter gradients: fold the block's token lanes, then one atomic per entry and block
    constexpr int PER = 8 * (K + 1);
    float* mine_f = fold + (size_t)(lr * COLS + ct) * PER;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      mine_f[c] = dbacc[c];
#pragma unroll
      for (int j = 0; j < K; ++j) mine_f[8 * (j + 1) + c] = dwacc[j][c];
    }
    __syncthreads();
    if (lr == 0 && live) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float sb = 0.f;
        for (int l = 0; l < ROW_LANES; ++l) sb += fold[(size_t)(l * COLS + ct) * PER + c];
        if (p.dbias) atomicAdd(p.dbias + col + c, sb);
#pragma unroll
        for (int j = 0; j < K; ++j) {
          float sw_ = 0.f;
          for (int l = 0; l < ROW_LANES; ++l) sw_ += fold[(size_t)(l * COLS + ct) * PER + 8 * (j + 1) + c];
          atomicAdd(p.dw + (long)(col + c) * K + j, sw_);
        }
      }
    }
  }
}

template <bool BWD>
int launch(int dtype, ConvParams cp, cudaStream_t s) {
  if (cp.B < 0 || cp.T < 0 || cp.C <= 0 || cp.C % 8 || cp.K < 1 || cp.K > KMAX) {
    set_error("short conv: need C a positive multiple of 8 and 1 <= K <= %d (got C=%d, K=%d)", KMAX, cp.C, cp.K);
    return JLA_ERR_UNSUPPORTED;
  }
  const int lanes = cp.head_dim > 0 ? cp.head_dim / 8 : 1;
  if (cp.head_dim < 0 || (cp.head_dim > 0 && (cp.head_dim % 8 || cp.C % cp.head_dim || lanes > 32 || (lanes & (lanes - 1))))) {
    set_error("short conv: head_dim (%d) must divide C (%d) and be 8 times a power of two, at most 256", cp.head_dim, cp.C);
    return JLA_ERR_UNSUPPORTED;
  }
  if (BWD) {
    JLA_CUDA_OK(cudaMemsetAsync(cp.dw, 0, sizeof(float) * cp.C * cp.K, s));
    if (cp.dbias) JLA_CUDA_OK(cudaMemsetAsync(cp.dbias, 0, sizeof(float) * cp.C, s));
  }
  if (cp.B == 0 || cp.T == 0) return JLA_OK;
  const int cv = cp.C / 8;
  const dim3 grid((cv + COLS - 1) / COLS, 1, 1);
  const int K = cp.K;
  const size_t smem = BWD ? sizeof(float) * COLS * 8 * ((TT + 2 * (K - 1)) + (TT + K - 1)) + sizeof(int) * (TT + 2 * (K - 1))
                          : sizeof(float) * COLS * 8 * (TT + K - 1) + sizeof(int) * (TT + K - 1);
  auto go = [&](auto kern) -> int {
    if (smem > 48 * 1024) JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // the token-tile index lives in gridDim.y (<= 65535): larger problems go in slices of batch rows
    const int tiles_per_row = (cp.T + TT - 1) / TT;
    const int rows_per_launch = tiles_per_row > 65535 ? 0 : 65535 / tiles_per_row;
    if (rows_per_launch == 0) {
      set_error("short conv: more than %d tokens per batch row", 65535 * TT);
      return JLA_ERR_UNSUPPORTED;
    }
    for (int b0 = 0; b0 < cp.B; b0 += rows_per_launch) {
      ConvParams q = cp;
      const int nb = cp.B - b0 < rows_per_launch ? cp.B - b0 : rows_per_launch;
      const size_t es = dtype == JLA_DTYPE_F32 ? 4 : 2;
      auto adv = [&](const void* ptr, size_t per_row) {
        return ptr ? static_cast<const void*>(static_cast<const char*>(ptr) + (size_t)b0 * per_row) : nullptr;
      };
      q.B = nb;
      q.x = adv(cp.x, (size_t)cp.T * cp.C * es);
      q.y = const_cast<void*>(adv(cp.y, (size_t)cp.T * cp.C * es));
      q.dy = adv(cp.dy, (size_t)cp.T * cp.C * es);
      q.dx = const_cast<void*>(adv(cp.dx, (size_t)cp.T * cp.C * es));
      q.state = adv(cp.state, (size_t)(K - 1) * cp.C * es);
      q.dstate = const_cast<void*>(adv(cp.dstate, (size_t)(K - 1) * cp.C * es));
      q.seg = static_cast<const int32_t*>(adv(cp.seg, (size_t)cp.T * sizeof(int32_t)));
      kern<<<dim3(grid.x, (unsigned)(nb * tiles_per_row)), THREADS, smem, s>>>(q);
      JLA_LAUNCH_OK();
    }
    return JLA_OK;
  };
  auto by_k = [&](auto tag) -> int {
    using T = decltype(tag);
    switch (cp.K) {
      case 1: return go(short_conv_kernel<T, BWD, 1>);
      case 2: return go(short_conv_kernel<T, BWD, 2>);
      case 3: return go(short_conv_kernel<T, BWD, 3>);
      default: return go(short_conv_kernel<T, BWD, 4>);
    }
  };
  switch (dtype) {
    case JLA_DTYPE_BF16: return by_k(__nv_bfloat16{});
    case JLA_DTYPE_F16: return by_k(__half{});
    case JLA_DTYPE_F32: return by_k(float{});
    default: set_error("short conv: unknown dtype %d", dtype); return JLA_ERR_BAD_ARGUMENT;
  }
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_short_conv_fwd(int dtype, int B, int T, int C, int K, int head_dim, int activation, const void* x,
                                  const float* weight, const float* bias, const int32_t* segment_ids, const void* state,
                                  void* y, jla_stream_t stream) {
  if (!x || !weight || !y) return JLA_ERR_BAD_ARGUMENT;
  ConvParams cp{};
  cp.B = B, cp.T = T, cp.C = C, cp.K = K, cp.head_dim = head_dim, cp.activation = activation, cp.x = x, cp.w = weight;
  cp.bias = bias, cp.seg = segment_ids, cp.state = state, cp.y = y;
  return launch<false>(dtype, cp, static_cast<cudaStream_t>(stream));
}

extern "C" int jla_short_conv_bwd(int dtype, int B, int T, int C, int K, int head_dim, int activation, const void* x,
                                  const float* weight, const float* bias, const int32_t* segment_ids, const void* state,
                                  const void* dy, void* dx, float* dweight, float* dbias, void* dstate,
                                  jla_stream_t stream) {
  if (!x || !weight || !dy || !dx || !dweight) return JLA_ERR_BAD_ARGUMENT;
  ConvParams cp{};
  cp.B = B, cp.T = T, cp.C = C, cp.K = K, cp.head_dim = head_dim, cp.activation = activation, cp.x = x, cp.w = weight;
  cp.bias = bias, cp.seg = segment_ids, cp.state = state, cp.dy = dy, cp.dx = dx, cp.dw = dweight, cp.dbias = dbias;
  cp.dstate = dstate;
  return launch<true>(dtype, cp, static_cast<cudaStream_t>(stream));
}
