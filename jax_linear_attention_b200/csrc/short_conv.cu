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
// HBM-bound. A thread owns eight adjacent channels and a tile of consecutive tokens of one batch row and slides a
// window of the last K - 1 inputs (forward) or of the next K - 1 pre-activation gradients (backward, walking the
// tile from its end; the K - 1 tokens behind the tile are recomputed) through registers, so every input row is
// loaded once per tile. A head's sum is a butterfly over the head_dim / 8 threads that hold it. The conv output
// stays in float32 until the norm has been applied and is rounded once.
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
  int cols, tile;  // column threads per block (8 channels each); tokens per thread
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

// Row t of x_ext's token axis for batch row b: t >= 0 reads x, t < 0 the carried state (zeros without one).
template <typename T>
__device__ __forceinline__ void load_row(const ConvParams& p, int b, int t, int col, bool live, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = 0.f;
  if (!live || t >= p.T) return;
  if (t >= 0) {
    load8<T>(static_cast<const T*>(p.x) + ((long)b * p.T + t) * p.C + col, f);
  } else if (p.state && t >= -(p.K - 1)) {
    load8<T>(static_cast<const T*>(p.state) + ((long)b * (p.K - 1) + (p.K - 1 + t)) * p.C + col, f);
  }
}

__device__ __forceinline__ int seg_at(const ConvParams& p, int b, int t) {
  if (!p.seg) return 0;
  return p.seg[(long)b * p.T + (t < 0 ? 0 : (t >= p.T ? p.T - 1 : t))];
}

// Pre-activation, activation and norm of one token from its window (win[j] = x_ext token t - (K - 1) + j, j < K).
// Returns the quantities the backward needs: y (normalised when head_dim > 0), sig = sigmoid(pre), inv.
struct TokenOut {
  float y[8], pre[8], inv;
};

template <int K>
__device__ __forceinline__ void conv_token(const ConvParams& p, const float (&w)[KMAX][8], const float (&bias)[8],
                                           const float (&win)[KMAX][8], const int (&sw)[KMAX], int lanes, TokenOut& o) {
  const int sc = sw[K - 1];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float acc = bias[c];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < K && (j == K - 1 || sw[j] == sc)) acc += w[j][c] * win[j][c];
    }
    o.pre[c] = acc;
    const float y = p.activation ? acc / (1.f + __expf(-acc)) : acc;
    o.y[c] = y;
    ss += y * y;
  }
  o.inv = 1.f;
  if (p.head_dim > 0) {
    o.inv = rsqrtf(head_sum(ss, lanes) + kL2Eps);
#pragma unroll
    for (int c = 0; c < 8; ++c) o.y[c] *= o.inv;
  }
}

template <typename T, bool BWD, int K>
__global__ void __launch_bounds__(THREADS) short_conv_kernel(ConvParams p) {
  extern __shared__ float fold[];  // backward: [row lanes][cols * 8 * (K + 1)]
  const int cv = p.C / 8;
  const int cols = p.cols, lanes_r = blockDim.x / cols;
  const int ct = threadIdx.x % cols, lr = threadIdx.x / cols;
  const int vec = blockIdx.x * cols + ct;
  const bool live = vec < cv;
  const int col = (live ? vec : 0) * 8;
  const int lanes = p.head_dim > 0 ? p.head_dim / 8 : 1;
  const int tiles_per_row = (p.T + p.tile - 1) / p.tile;
  const long tile_id = (long)blockIdx.y * lanes_r + lr;
  const bool has_tile = tile_id < (long)p.B * tiles_per_row;
  const int b = has_tile ? (int)(tile_id / tiles_per_row) : 0;
  const int t0 = has_tile ? (int)(tile_id % tiles_per_row) * p.tile : 0;
  const int t1 = has_tile ? (t0 + p.tile < p.T ? t0 + p.tile : p.T) : 0;
  float w[KMAX][8], bias[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    bias[c] = p.bias ? p.bias[col + c] : 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) w[j][c] = j < K ? p.w[(long)(col + c) * K + j] : 0.f;
  }

  if constexpr (!BWD) {
    float win[KMAX][8];
    int sw[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {  // tokens t0 - (K - 1) + j, j < K - 1, sit in win[j]; win[K - 1] is the token itself
      if (j < K - 1) {
        load_row<T>(p, b, t0 - (K - 1) + j, col, live && has_tile, win[j]);
        sw[j] = seg_at(p, b, t0 - (K - 1) + j);
      } else {
        sw[j] = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) win[j][c] = 0.f;
      }
    }
    for (int t = t0; t < t0 + p.tile; ++t) {  // uniform trip count: the head sums shuffle across the warp
      const bool on = live && has_tile && t < t1;
      load_row<T>(p, b, t, col, on, win[K - 1]);
      sw[K - 1] = seg_at(p, b, t);
      TokenOut o;
      conv_token<K>(p, w, bias, win, sw, lanes, o);
      if (on) store8<T>(static_cast<T*>(p.y) + ((long)b * p.T + t) * p.C + col, o.y);
#pragma unroll
      for (int j = 0; j < KMAX - 1; ++j) {
        if (j < K - 1) {
          sw[j] = sw[j + 1];
#pragma unroll
          for (int c = 0; c < 8; ++c) win[j][c] = win[j + 1][c];
        }
      }
    }
  } else {
  // ---------------------------------------------------------------------------------------------- backward
  float dwacc[KMAX][8], dbacc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    dbacc[c] = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) dwacc[j][c] = 0.f;
  }
  // dp[l - 1] = dpre of token t + l (l = 1 .. K - 1) while the walk stands at token t; sp its document id
  float dp[KMAX][8];
  int sp[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    sp[j] = -1;
#pragma unroll
    for (int c = 0; c < 8; ++c) dp[j][c] = 0.f;
  }
  // the walk starts K - 1 tokens behind the tile (their dpre feed the tile's dx) and ends K - 1 rows into the state
  const int t_hi = t1 + (K - 1) - 1;                      // first token visited
  const int t_lo = (t0 == 0 && p.dstate) ? -(K - 1) : t0;  // last row visited (state rows only for the row's first tile)
  float win[KMAX][8];
  int sw[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < K) {
      load_row<T>(p, b, t_hi - (K - 1) + j, col, live && has_tile, win[j]);
      sw[j] = seg_at(p, b, t_hi - (K - 1) + j);
    } else {
      sw[j] = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) win[j][c] = 0.f;
    }
  }
  const int steps = p.tile + 2 * (K - 1);  // uniform trip count
  for (int s = 0; s < steps; ++s) {
    const int t = t_hi - s;
    const bool visit = has_tile && t >= t_lo;
    const bool token = visit && t >= 0 && t < p.T;       // a real token: it has a dpre of its own
    const bool mine = token && t >= t0 && t < t1;        // inside the tile: dx, dw, dbias are this thread's to write
    float dpre[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) dpre[c] = 0.f;
    TokenOut o;
    conv_token<K>(p, w, bias, win, sw, lanes, o);        // every thread of the warp takes part in the head sums
    float dnv[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) dnv[c] = 0.f;
    if (token && live) load8<T>(static_cast<const T*>(p.dy) + ((long)b * p.T + t) * p.C + col, dnv);
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) dot += dnv[c] * o.y[c];
    if (p.head_dim > 0) dot = head_sum(dot, lanes);
    if (token && live) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float dy = p.head_dim > 0 ? o.inv * (dnv[c] - o.y[c] * dot) : dnv[c];
        const float sg = 1.f / (1.f + __expf(-o.pre[c]));
        dpre[c] = p.activation ? dy * sg * (1.f + o.pre[c] * (1.f - sg)) : dy;
      }
    }
    const int sc = sw[K - 1];  // document of row t (state rows: the first token's)
    if (visit && live && (mine || t < 0)) {
      // dx_ext[t] = w[:, K - 1] dpre_t + sum_l w[:, K - 1 - l] dpre_{t + l} for later tokens of the same document
      float dxv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float acc = w[K - 1][c] * dpre[c];
#pragma unroll
        for (int l = 1; l < KMAX; ++l) {
          if (l < K && sp[l - 1] == sc) acc += w[K - 1 - l][c] * dp[l - 1][c];
        }
        dxv[c] = acc;
      }
      if (t >= 0) store8<T>(static_cast<T*>(p.dx) + ((long)b * p.T + t) * p.C + col, dxv);
      else store8<T>(static_cast<T*>(p.dstate) + ((long)b * (K - 1) + (K - 1 + t)) * p.C + col, dxv);
    }
    if (mine && live) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        dbacc[c] += dpre[c];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
          if (j < K && (j == K - 1 || sw[j] == sc)) dwacc[j][c] += dpre[c] * win[j][c];
        }
      }
    }
    // slide: dpre_t becomes the nearest later token; the input window moves one row down
#pragma unroll
    for (int l = KMAX - 1; l > 0; --l) {
      sp[l] = sp[l - 1];
#pragma unroll
      for (int c = 0; c < 8; ++c) dp[l][c] = dp[l - 1][c];
    }
    sp[0] = token ? sc : -1;
#pragma unroll
    for (int c = 0; c < 8; ++c) dp[0][c] = dpre[c];
#pragma unroll
    for (int j = KMAX - 1; j > 0; --j) {
      if (j < K) {
        sw[j] = sw[j - 1];
#pragma unroll
        for (int c = 0; c < 8; ++c) win[j][c] = win[j - 1][c];
      }
    }
    load_row<T>(p, b, t - 1 - (K - 1), col, live && has_tile && s + 1 < steps, win[0]);
    sw[0] = seg_at(p, b, t - 1 - (K - 1));
  }
  // parameter gradients: fold the block's row lanes, then one atomic per entry and block
  const int per = 8 * (KMAX + 1);
  float* mine_f = fold + (size_t)(lr * cols + ct) * per;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    mine_f[c] = dbacc[c];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) mine_f[8 * (j + 1) + c] = dwacc[j][c];
  }
  __syncthreads();
  if (lr == 0 && live) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float sb = 0.f;
      for (int l = 0; l < lanes_r; ++l) sb += fold[(size_t)(l * cols + ct) * per + c];
      if (p.dbias) atomicAdd(p.dbias + col + c, sb);
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (j >= K) continue;
        float sw_ = 0.f;
        for (int l = 0; l < lanes_r; ++l) sw_ += fold[(size_t)(l * cols + ct) * per + 8 * (j + 1) + c];
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
  int cols = cv < 32 ? cv : 32;
  if (cols % lanes) cols = lanes;  // a head never straddles two blocks' column ranges
  if (cv % cols) {
    set_error("short conv: C / 8 = %d must be a multiple of %d", cv, cols);
    return JLA_ERR_UNSUPPORTED;
  }
  const int threads = cols * (THREADS / cols);
  const int lanes_r = threads / cols;
  cp.cols = cols;
  // tokens per thread: long enough to amortise the K - 1 recomputed tokens and 2 (K - 1) extra steps of the backward
  cp.tile = cp.T >= 1024 ? 64 : (cp.T >= 256 ? 32 : 16);
  const long tiles = (long)cp.B * ((cp.T + cp.tile - 1) / cp.tile);
  const long gy = (tiles + lanes_r - 1) / lanes_r;
  if (gy > 65535) {
    set_error("short conv: more than %ld token tiles per call", 65535L * lanes_r);
    return JLA_ERR_UNSUPPORTED;
  }
  const dim3 grid(cv / cols, (unsigned)gy);
  const size_t smem = BWD ? sizeof(float) * threads * 8 * (KMAX + 1) : 0;
  auto go = [&](auto kern) -> int {
    if (smem > 48 * 1024) JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, threads, smem, s>>>(cp);
    JLA_LAUNCH_OK();
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
