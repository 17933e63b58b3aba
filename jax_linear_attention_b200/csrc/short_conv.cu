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
// The conv output stays in float32 until the norm has been applied and is rounded once. Bound by instruction issue
// (about 130 instructions per token and four channels forward, 300 backward), not by HBM: what the kernel does about
// it is said at the thread layout below.
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

// VEC adjacent channels of one token, as loaded (16-bit types: VEC / 2 words, float: VEC words).
template <typename T, int VEC>
struct alignas(VEC * sizeof(T) >= 16 ? 16 : VEC * sizeof(T)) Packed {
  static constexpr int W = VEC * (int)sizeof(T) / 4;
  uint32_t r[W];
};

template <typename T, int VEC>
__device__ __forceinline__ Packed<T, VEC> zero_row() {
  Packed<T, VEC> o;
#pragma unroll
  for (int i = 0; i < Packed<T, VEC>::W; ++i) o.r[i] = 0u;  // all-zero bits are 0.0 in every dtype
  return o;
}

template <typename T, int VEC>
__device__ __forceinline__ Packed<T, VEC> load_row(const T* p) {
  Packed<T, VEC> o;
  constexpr int W = Packed<T, VEC>::W;
  if constexpr (W == 2) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    o.r[0] = u.x, o.r[1] = u.y;
  } else {
#pragma unroll
    for (int i = 0; i < W / 4; ++i) {
      const uint4 u = reinterpret_cast<const uint4*>(p)[i];
      o.r[4 * i] = u.x, o.r[4 * i + 1] = u.y, o.r[4 * i + 2] = u.z, o.r[4 * i + 3] = u.w;
    }
  }
  return o;
}

template <typename T, int VEC>
__device__ __forceinline__ void unpack(const Packed<T, VEC>& in, float (&f)[VEC]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = __uint_as_float(in.r[i]);
  } else {
    const T* e = reinterpret_cast<const T*>(in.r);
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = to_f32(e[i]);
  }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_row(T* p, const float (&f)[VEC]) {
  Packed<T, VEC> o;
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.r[i] = __float_as_uint(f[i]);
  } else {
    T* e = reinterpret_cast<T*>(o.r);
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = from_f32<T>(f[i]);
  }
  constexpr int W = Packed<T, VEC>::W;
  if constexpr (W == 2) {
    *reinterpret_cast<uint2*>(p) = make_uint2(o.r[0], o.r[1]);
  } else {
#pragma unroll
    for (int i = 0; i < W / 4; ++i) reinterpret_cast<uint4*>(p)[i] = make_uint4(o.r[4 * i], o.r[4 * i + 1], o.r[4 * i + 2], o.r[4 * i + 3]);
  }
}

// Sum over the `lanes` (a power of two <= 32) adjacent lanes of a head: five predicated butterflies, no loop.
__device__ __forceinline__ float head_sum(float v, int lanes) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    if (off < lanes) v += o;
  }
  return v;
}

// A thread owns VEC adjacent channels and walks TT (TT_FWD or TT_BWD) consecutive tokens of one batch row in time
// order, with the K - 1 rows in front of the current token (and, backward, the K - 1 pre-activation gradients behind
// it) in registers as float32. Its rows of x (and of the upstream gradient) come through a ring of asynchronous
// copies in shared memory that only this thread reads: groups of UNROLL tokens, two groups in flight while one is
// worked on, no block-wide barrier (plain loads in the loop, even written a group ahead in the source, left the
// kernel waiting on memory: the compiler is free to move them next to their use). Every row is fetched once per
// thread, plus K - 1 rows of overlap per walk. The 32 lanes of a warp hold adjacent channel vectors of the same
// tokens, so a head's sums (head_dim / VEC lanes) are warp butterflies and a token's document id is one shuffle. A
// block is 32 lanes x SUB walks over adjacent token ranges; backward, the SUB walks' parameter gradients are summed
// in shared memory before one atomic per entry.
constexpr int COLS = 32;
constexpr int SUB = THREADS / COLS;
// Tokens per walk (16-token walks in the forward, to fill the last round of blocks better, measured slower: the
// fixed cost of a walk, its first rows and its weights, weighs more).
constexpr int TT_FWD = 32, TT_BWD = 32;
constexpr int UNROLL_FWD = 4, UNROLL_BWD = 4;  // tokens per group (the backward holds twice the rows per token)
static_assert(UNROLL_BWD >= KMAX - 1 && UNROLL_FWD >= KMAX - 1, "the window slides by whole groups");

__device__ __forceinline__ int seg_at(const ConvParams& p, int b, int t) {
  if (!p.seg) return 0;
  return p.seg[(long)b * p.T + (t < 0 ? 0 : (t >= p.T ? p.T - 1 : t))];
}

// Row t of x_ext for this thread's channels: x for 0 <= t < T, the carried state for -(K - 1) <= t < 0, zero elsewhere.
template <typename T, int VEC>
__device__ __forceinline__ Packed<T, VEC> fetch_x(const ConvParams& p, int b, int t, int col, bool live) {
  if (!live || t >= p.T) return zero_row<T, VEC>();
  if (t >= 0) return load_row<T, VEC>(static_cast<const T*>(p.x) + ((long)b * p.T + t) * p.C + col);
  if (p.state && t >= -(p.K - 1)) {
    return load_row<T, VEC>(static_cast<const T*>(p.state) + ((long)b * (p.K - 1) + (p.K - 1 + t)) * p.C + col);
  }
  return zero_row<T, VEC>();
}

// Pre-activation, activation and norm of one token from its window of K rows (the last one being the token itself);
// taps into an earlier document are skipped. y is normalised when head_dim > 0.
template <int VEC>
struct TokenOut {
  float y[VEC], pre[VEC], sg[VEC], inv;  // sg = sigmoid(pre) when the activation is on
};

template <int K, int VEC>
__device__ __forceinline__ void conv_token(const ConvParams& p, const float (&w)[KMAX][VEC], const float (&bias)[VEC],
                                           const float (*rows)[VEC], const int* segs, int lanes, TokenOut<VEC>& o) {
  const int sc = segs[K - 1];
  float acc[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) acc[c] = bias[c];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    if (j == K - 1 || segs[j] == sc) {
#pragma unroll
      for (int c = 0; c < VEC; ++c) acc[c] += w[j][c] * rows[j][c];
    }
  }
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    o.pre[c] = acc[c];
    o.sg[c] = fast_rcp(1.f + fast_exp(-acc[c]));
    const float y = p.activation ? acc[c] * o.sg[c] : acc[c];
    o.y[c] = y;
    sq += y * y;
  }
  o.inv = 1.f;
  if (p.head_dim > 0) {
    o.inv = fast_rsqrt(head_sum(sq, lanes) + kL2Eps);
#pragma unroll
    for (int c = 0; c < VEC; ++c) o.y[c] *= o.inv;
  }
}

template <typename T, bool BWD, int K, int VEC>
__global__ void __launch_bounds__(THREADS, BWD ? (VEC == 4 ? 2 : 1) : (VEC == 4 ? 3 : 1)) short_conv_kernel(ConvParams p) {
  constexpr int UNROLL = BWD ? UNROLL_BWD : UNROLL_FWD;
  constexpr int TT = BWD ? TT_BWD : TT_FWD;
  constexpr int RB = VEC * (int)sizeof(T);       // bytes of one row of this thread
  constexpr int STAGES = ring_stages(RB);        // groups in the ring: one worked on, the others in flight
  extern __shared__ __align__(16) unsigned char ring_raw[];
  // slot of (tensor n, stage s, token u of the group) for this thread; adjacent threads are adjacent in memory
  auto slot = [&](int n, int s_, int u) {
    return ring_raw + ((size_t)((n * STAGES + s_) * UNROLL + u) * THREADS + threadIdx.x) * RB;
  };
  const int lane = threadIdx.x % COLS, lr = threadIdx.x / COLS;
  const int vec = blockIdx.x * COLS + lane;
  const bool live = vec < p.C / VEC;
  const int col = (live ? vec : 0) * VEC;
  const int lanes = p.head_dim > 0 ? p.head_dim / VEC : 1;
  const int tiles_per_row = (p.T + SUB * TT - 1) / (SUB * TT);
  const int b = blockIdx.y / tiles_per_row;
  const int ta = (blockIdx.y % tiles_per_row) * (SUB * TT) + lr * TT;  // this walk: tokens ta .. tb - 1
  const int tb = ta + TT < p.T ? ta + TT : p.T;
  // The walk's rows arrive through a ring of asynchronous copies in shared memory, private to the thread: groups of
  // UNROLL tokens, STAGES - 1 groups in flight while one is worked on. Tokens of the walk itself are never state
  // rows: row t of this thread's channels is xrow + t * C (lanes past the last channel read channel 0's rows and
  // never store: no lane-dependent branch around the copies). Rows from `tend` on read as zero.
  const int tend = !BWD ? tb : (ta < tb ? tb + (K - 1) : ta);  // backward: K - 1 tokens past the range, see below
  const int tload = tend < p.T ? tend : p.T;
  const T* xrow = static_cast<const T*>(p.x) + (long)b * p.T * p.C + col;
  const T* dyrow = BWD ? static_cast<const T*>(p.dy) + (long)b * p.T * p.C + col : nullptr;
  auto request = [&](int g) {  // group g: tokens ta + g * UNROLL ...
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int tn = ta + g * UNROLL + u;
      const bool valid = tn < tload;
      const long off = (long)(valid ? tn : 0) * p.C;
      cp_async_row<RB>(slot(0, g % STAGES, u), xrow + off, valid);
      if constexpr (BWD) cp_async_row<RB>(slot(1, g % STAGES, u), dyrow + off, valid);
    }
    cp_async_commit_group();
  };
#pragma unroll
  for (int g = 0; g < STAGES - 1; ++g) request(g);

  float w[KMAX][VEC], bias[VEC];
#pragma unroll
  for (int c = 0; c < VEC; ++c) {
    bias[c] = p.bias ? p.bias[col + c] : 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) w[j][c] = j < K ? p.w[(long)(col + c) * K + j] : 0.f;
  }
  // document ids: lane i of the warp holds that of token ta + i (and of ta + 32 + i for the overhang of a 32-token walk);
  // a token's id is one shuffle
  static_assert(TT + KMAX - 1 <= 32 || TT == 32, "one document id per lane of the walk's warp, two for the overhang");
  static_assert(COLS == 32, "a walk is one warp");
  const int32_t* srow = p.seg ? p.seg + (long)b * p.T : nullptr;
  auto seg_of = [&](int t) { return srow ? srow[t < p.T ? t : p.T - 1] : 0; };
  const int seg_walk = seg_of(ta + lane);
  const int seg_over = BWD && lane < K - 1 ? seg_of(ta + 32 + lane) : 0;
  auto seg_tok = [&](int i) { return __shfl_sync(0xffffffffu, i < 32 ? seg_walk : seg_over, i & 31); };
  // rows[0 .. K - 2]: the K - 1 rows in front of the group; rows[K - 1 + u]: token t + u of the group (float32: a
  // row is converted once and used by K tokens)
  float rows[K - 1 + UNROLL][VEC];
  int segs[K - 1 + UNROLL];
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    unpack<T, VEC>(ta < tb ? fetch_x<T, VEC>(p, b, ta - (K - 1) + j, col, live) : zero_row<T, VEC>(), rows[j]);
    segs[j] = seg_at(p, b, ta - (K - 1) + j);
  }
  const int ngroups = (tend - ta + UNROLL - 1) / UNROLL;

  if constexpr (!BWD) {
    T* yrow = static_cast<T*>(p.y) + (long)b * p.T * p.C + col;
    for (int g = 0; g < ngroups; ++g) {
      const int t = ta + g * UNROLL;
      request(g + STAGES - 1);
      cp_async_wait_groups<STAGES - 1>();
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        unpack<T, VEC>(*reinterpret_cast<const Packed<T, VEC>*>(slot(0, g % STAGES, u)), rows[K - 1 + u]);
        segs[K - 1 + u] = seg_tok(g * UNROLL + u);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        TokenOut<VEC> o;
        conv_token<K, VEC>(p, w, bias, rows + u, segs + u, lanes, o);
        if (live && t + u < tb) store_row<T, VEC>(yrow + (long)(t + u) * p.C, o.y);
      }
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
#pragma unroll
        for (int c = 0; c < VEC; ++c) rows[j][c] = rows[j + UNROLL][c];
        segs[j] = segs[j + UNROLL];
      }
    }
    cp_async_wait_groups<0>();  // the trailing (empty) groups of the ring
  } else {
    // The walk runs K - 1 tokens past its range: their pre-activation gradients (recomputed here, owned by the next
    // walk) reach back into it. dp[l] = dpre of token s + l where s = t - (K - 1) is the row whose dx is complete once
    // token t is done: dx_ext[s] = sum_l w[:, K - 1 - l] dpre[s + l] over the later tokens of the same document
    // (l = 0: the token itself). The row's first walk also produces the K - 1 state rows in front.
    float dwacc[KMAX][VEC], dbacc[VEC], dp[K][VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      dbacc[c] = 0.f;
#pragma unroll
      for (int j = 0; j < KMAX; ++j) dwacc[j][c] = 0.f;
#pragma unroll
      for (int l = 0; l < K; ++l) dp[l][c] = 0.f;
    }
    const int s_lo = (ta == 0 && p.dstate) ? -(K - 1) : ta;
    T* dxrow = static_cast<T*>(p.dx) + (long)b * p.T * p.C + col;
    for (int g = 0; g < ngroups; ++g) {
      const int t = ta + g * UNROLL;
      request(g + STAGES - 1);
      cp_async_wait_groups<STAGES - 1>();
      Packed<T, VEC> dnr[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        unpack<T, VEC>(*reinterpret_cast<const Packed<T, VEC>*>(slot(0, g % STAGES, u)), rows[K - 1 + u]);
        dnr[u] = *reinterpret_cast<const Packed<T, VEC>*>(slot(1, g % STAGES, u));
        segs[K - 1 + u] = seg_tok(g * UNROLL + u);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int tok = t + u;
        const bool token = tok < p.T && tok < tend;
        TokenOut<VEC> o;
        conv_token<K, VEC>(p, w, bias, rows + u, segs + u, lanes, o);
        float dnv[VEC];
        unpack<T, VEC>(dnr[u], dnv);
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < VEC; ++c) dot += dnv[c] * o.y[c];
        if (p.head_dim > 0) dot = head_sum(dot, lanes);
#pragma unroll
        for (int l = 0; l + 1 < K; ++l) {
#pragma unroll
          for (int c = 0; c < VEC; ++c) dp[l][c] = dp[l + 1][c];
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          const float dy = p.head_dim > 0 ? o.inv * (dnv[c] - o.y[c] * dot) : dnv[c];
          const float sg = o.sg[c];
          dp[K - 1][c] = !token ? 0.f : (p.activation ? dy * sg * (1.f + o.pre[c] * (1.f - sg)) : dy);
        }
        if (tok < tb) {  // inside the range: this token's share of the parameter gradients
          const int sc = segs[u + K - 1];
#pragma unroll
          for (int j = 0; j < K; ++j) {
            if (j == K - 1 || segs[u + j] == sc) {
#pragma unroll
              for (int c = 0; c < VEC; ++c) dwacc[j][c] += dp[K - 1][c] * rows[u + j][c];
            }
          }
#pragma unroll
          for (int c = 0; c < VEC; ++c) dbacc[c] += dp[K - 1][c];
        }
        const int srow = tok - (K - 1);  // its document id is segs[u], that of srow + l is segs[u + l]
        if (live && srow >= s_lo && srow < tb) {
          float acc[VEC];
#pragma unroll
          for (int c = 0; c < VEC; ++c) acc[c] = 0.f;
#pragma unroll
          for (int l = 0; l < K; ++l) {
            if (l == 0 ? srow >= 0 : segs[u + l] == segs[u]) {
#pragma unroll
              for (int c = 0; c < VEC; ++c) acc[c] += w[K - 1 - l][c] * dp[l][c];
            }
          }
          if (srow >= 0) store_row<T, VEC>(dxrow + (long)srow * p.C, acc);
          else store_row<T, VEC>(static_cast<T*>(p.dstate) + ((long)b * (K - 1) + (K - 1 + srow)) * p.C + col, acc);
        }
      }
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
#pragma unroll
        for (int c = 0; c < VEC; ++c) rows[j][c] = rows[j + UNROLL][c];
        segs[j] = segs[j + UNROLL];
      }
    }
    cp_async_wait_groups<0>();  // the trailing (empty) groups of the ring
    // parameter gradients: sum the block's SUB walks, then one atomic per entry and block
    constexpr int PER = VEC * (K + 1);
    __shared__ float fold[SUB * COLS * PER];
    float* mine = fold + (size_t)(lr * COLS + lane) * PER;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      mine[c] = dbacc[c];
#pragma unroll
      for (int j = 0; j < K; ++j) mine[VEC * (j + 1) + c] = dwacc[j][c];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < COLS * PER; e += THREADS) {
      const int ln = e / PER, k = e % PER, j = k / VEC, c = k % VEC;
      const int ch = (blockIdx.x * COLS + ln) * VEC + c;
      if (ch >= p.C) continue;
      float sum = 0.f;
#pragma unroll
      for (int l = 0; l < SUB; ++l) sum += fold[(size_t)(l * COLS + ln) * PER + k];
      if (j == 0) {
        if (p.dbias) atomicAdd(p.dbias + ch, sum);
      } else {
        atomicAdd(p.dw + (long)ch * K + (j - 1), sum);
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
  const int K = cp.K;
  // channels per thread: four (eight-byte loads of 16-bit tensors; fewer registers, more walks in flight) while a
  // head's lanes then still fit a warp, else eight
  const int vec = cp.head_dim > 4 * 32 ? 8 : 4;
  const int cv = cp.C / vec;
  const dim3 grid((cv + COLS - 1) / COLS, 1, 1);
  const size_t es = dtype == JLA_DTYPE_F32 ? 4 : 2;
  const size_t smem = (size_t)(BWD ? 2 : 1) * ring_stages((int)(vec * es)) * (BWD ? UNROLL_BWD : UNROLL_FWD) * THREADS * vec * es;
  auto go = [&](auto kern) -> int {
    // always: the backward adds a static array, and the sum of the two is what the 48 KB default limits
    JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // the token-tile index lives in gridDim.y (<= 65535): larger problems go in slices of batch rows
    constexpr int TT = BWD ? TT_BWD : TT_FWD;
    const int tiles_per_row = (cp.T + SUB * TT - 1) / (SUB * TT);
    const int rows_per_launch = tiles_per_row > 65535 ? 0 : 65535 / tiles_per_row;
    if (rows_per_launch == 0) {
      set_error("short conv: more than %d tokens per batch row", 65535 * SUB * TT);
      return JLA_ERR_UNSUPPORTED;
    }
    for (int b0 = 0; b0 < cp.B; b0 += rows_per_launch) {
      ConvParams q = cp;
      const int nb = cp.B - b0 < rows_per_launch ? cp.B - b0 : rows_per_launch;
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
    if (vec == 8) {
      switch (cp.K) {
        case 1: return go(short_conv_kernel<T, BWD, 1, 8>);
        case 2: return go(short_conv_kernel<T, BWD, 2, 8>);
        case 3: return go(short_conv_kernel<T, BWD, 3, 8>);
        default: return go(short_conv_kernel<T, BWD, 4, 8>);
      }
    }
    switch (cp.K) {
      case 1: return go(short_conv_kernel<T, BWD, 1, 4>);
      case 2: return go(short_conv_kernel<T, BWD, 2, 4>);
      case 3: return go(short_conv_kernel<T, BWD, 3, 4>);
      default: return go(short_conv_kernel<T, BWD, 4, 4>);
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
