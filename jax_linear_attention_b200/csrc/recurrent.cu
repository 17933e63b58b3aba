// fp32 token-scan kernels: the exact path of the library (JLA_PATH_RECURRENT).
//
// They walk the tokens in the order of the reference's scan step (src/jla/ops/reference.py:140-157):
// reset, decay, delta write, read; with cu_seqlens every sequence is a row with its own initial and
// final state (reference.py:170-203). Arithmetic is fp32 FMA on CUDA cores whatever the storage dtype,
// so this path serves the fp32 configuration (relative L2 error <= 1e-5 against the fp32 reference) and
// is the on-device cross-check of the tensor-core kernels. It is latency-bound by design: one CTA per
// (row, head), the K x V state distributed over the CTA's registers.
//
// Thread layout: thread = (ks, v) with v the value column and ks one of KS = K / KPT key slices; a thread
// owns state entries S[ks*KPT .. ks*KPT+KPT-1][v]. Reductions over keys go through shared memory (KS
// partials per column); reductions over value columns use warp shuffles (V is a power of two).
#include <stdio.h>

#include "common.cuh"
#include "profile.cuh"

namespace jla {
namespace {

constexpr int TB = 16;  // tokens staged in shared memory per block

struct RecParams {
  Rows rows;
  int H, Hk, K, V;
  int gate;  // 0 none, 1 scalar, 2 per key channel
  int delta, l2norm;
  float scale;
  const void *q, *k, *v;
  const void* k_read;  // optional [B*T, H, K]: the recall reads the state with it (k still writes); nullptr = k
  const float *g, *beta, *h0;
  void* o;
  float* final_state;
  const void* d_o;
  const float* d_final;
  float *dq_acc, *dk_acc;  // [B*T, H, K] f32
  float* dkr_acc;          // [B*T, H, K] f32: gradient of k_read (with k_read only)
  void* dv;
  float *dg, *dbeta, *dh0;
  float* ckpt;  // [H][total_blocks][K*V]
  float* spre;  // [rows*H][TB][K*V]
  long total_blocks;
};

struct Smem {
  float *qs, *ks, *kr, *vs, *eg, *bs, *inv, *part, *dos, *us, *es, *red;  // kr: the read key (= ks without k_read)
  int* rs;
};

__host__ __device__ inline size_t smem_floats(int K, int V, int KS, bool bwd) {
  size_t n = 3 * TB * K + TB * V + TB * K + TB + 2 * TB + TB /*rs*/ + 3 * (size_t)KS * V;
  if (bwd) n += 3 * TB * V + 2 * (size_t)(4 * 8 * K + 64);
  return n;
}

__device__ inline Smem carve(float* base, int K, int V, int KS, bool bwd) {
  Smem s;
  s.qs = base;
  s.ks = s.qs + TB * K;
  s.kr = s.ks + TB * K;
  s.vs = s.kr + TB * K;
  s.eg = s.vs + TB * V;
  s.bs = s.eg + TB * K;
  s.inv = s.bs + TB;
  s.rs = reinterpret_cast<int*>(s.inv + 2 * TB);
  s.part = reinterpret_cast<float*>(s.rs + TB);
  s.dos = s.part + 3 * KS * V;
  s.us = s.dos + TB * V;
  s.es = s.us + TB * V;
  s.red = s.es + TB * V;
  return s;
}

// Stage `nb` tokens starting at flat token `tok` into shared memory as fp32 (q, k of key head hk; v, gates
// of head h), including the in-op L2 norm of q and k (reference.py:128-129) and the per-token reset flags.
template <typename T>
__device__ void load_block(const RecParams& p, const Smem& s, int tok, int nb, int row_tok0, int h, int hk,
                           bool with_do) {
  const int K = p.K, V = p.V, NT = blockDim.x, tid = threadIdx.x;
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  for (int idx = tid; idx < nb * K; idx += NT) {
    const int j = idx / K, c = idx - j * K;
    const long src = ((long)(tok + j) * p.Hk + hk) * K + c;
    s.qs[idx] = to_f32(q[src]);
    s.ks[idx] = to_f32(k[src]);
    if (p.k_read) s.kr[idx] = to_f32(static_cast<const T*>(p.k_read)[((long)(tok + j) * p.H + h) * K + c]);
    if (p.gate == 2) s.eg[idx] = expf(p.g[((long)(tok + j) * p.H + h) * K + c]);
  }
  for (int idx = tid; idx < nb * V; idx += NT) {
    const int j = idx / V, c = idx - j * V;
    const long src = ((long)(tok + j) * p.H + h) * V + c;
    s.vs[idx] = to_f32(v[src]);
    if (with_do) s.dos[idx] = to_f32(static_cast<const T*>(p.d_o)[src]);
  }
  if (tid < nb) {
    const long src = (long)(tok + tid) * p.H + h;
    if (p.gate == 1) s.eg[tid] = expf(p.g[src]);
    s.bs[tid] = p.delta ? p.beta[src] : 1.f;
    s.rs[tid] = p.rows.resets(tok + tid, row_tok0) ? 1 : 0;
  }
  __syncthreads();
  if (p.l2norm) {
    if (tid < 2 * nb) {
      const int which = tid / nb, j = tid - which * nb;
      const float* x = (which ? s.ks : s.qs) + j * K;
      float acc = 0.f;
      for (int c = 0; c < K; ++c) acc += x[c] * x[c];
      s.inv[which * TB + j] = rsqrtf(acc + 1e-6f);
    }
    __syncthreads();
    for (int idx = tid; idx < nb * K; idx += NT) {
      const int j = idx / K;
      // the reference rounds the normalised tensors to the input dtype (reference.py:69)
      s.qs[idx] = to_f32(from_f32<T>(s.qs[idx] * s.inv[j]));
      s.ks[idx] = to_f32(from_f32<T>(s.ks[idx] * s.inv[TB + j]));
    }
    __syncthreads();
  }
  if (!p.k_read) {  // the write key is also the read key (after its normalisation)
    for (int idx = tid; idx < nb * K; idx += NT) s.kr[idx] = s.ks[idx];
    __syncthreads();
  }
}

// One forward token: reset, decay, (delta) recall and write. Returns the written value u_v; *resid gets
// v_v - r_v. Contains one __syncthreads() when delta is set.
template <int KPT>
__device__ __forceinline__ float forward_token(const RecParams& p, const Smem& s, float (&S)[KPT], int j, int ks,
                                               int v, int KS, float* resid, float* pre /*global or nullptr*/) {
  const int K = p.K, V = p.V;
  if (s.rs[j]) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) S[i] = 0.f;
  }
  if (p.gate == 1) {
    const float d = s.eg[j];
#pragma unroll
    for (int i = 0; i < KPT; ++i) S[i] *= d;
  } else if (p.gate == 2) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) S[i] *= s.eg[j * K + ks * KPT + i];
  }
  if (pre) {
#pragma unroll
    for (int i = 0; i < KPT; ++i) pre[(long)(ks * KPT + i) * V + v] = S[i];
  }
  float u = s.vs[j * V + v];
  if (p.delta) {
    float partial = 0.f;
#pragma unroll
    for (int i = 0; i < KPT; ++i) partial += s.kr[j * K + ks * KPT + i] * S[i];
    float* part_r = s.part + 2 * KS * V;
    part_r[ks * V + v] = partial;
    __syncthreads();
    float r = 0.f;
    for (int t = 0; t < KS; ++t) r += part_r[t * V + v];
    *resid = u - r;
    u = s.bs[j] * (u - r);
  }
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] += s.ks[j * K + ks * KPT + i] * u;
  return u;
}

template <typename T, int KPT>
__global__ void __launch_bounds__(512) rec_fwd_kernel(RecParams p) {
  extern __shared__ float smem_raw[];
  const int h = blockIdx.x, r = blockIdx.y;
  const int K = p.K, V = p.V, tid = threadIdx.x;
  const int v = tid % V, ks = tid / V, KS = K / KPT;
  const int hk = h / (p.H / p.Hk);
  const Smem s = carve(smem_raw, K, V, KS, false);
  int tok0, len;
  p.rows.range(r, tok0, len);

  float S[KPT];
  const float* h0 = p.h0 ? p.h0 + ((long)r * p.H + h) * K * V : nullptr;
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] = h0 ? h0[(long)(ks * KPT + i) * V + v] : 0.f;

  T* o = static_cast<T*>(p.o);
  for (int t0 = 0; t0 < len; t0 += TB) {
    const int nb = min(TB, len - t0);
    __syncthreads();
    load_block<T>(p, s, tok0 + t0, nb, tok0, h, hk, false);
    for (int j = 0; j < nb; ++j) {
      float resid;
      forward_token<KPT>(p, s, S, j, ks, v, KS, &resid, nullptr);
      float po = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) po += s.qs[j * K + ks * KPT + i] * S[i];
      float* part_o = s.part + (j & 1) * KS * V;
      part_o[ks * V + v] = po;
      __syncthreads();
      if (ks == 0) {
        float acc = 0.f;
        for (int t = 0; t < KS; ++t) acc += part_o[t * V + v];
        o[((long)(tok0 + t0 + j) * p.H + h) * V + v] = from_f32<T>(p.scale * acc);
      }
    }
  }
  if (p.final_state) {
    float* f = p.final_state + ((long)r * p.H + h) * K * V;
#pragma unroll
    for (int i = 0; i < KPT; ++i) f[(long)(ks * KPT + i) * V + v] = S[i];
  }
}

// Sum val[i] over the value columns of this key slice; lane v % 32 == 0 of every warp writes its partial to
// red[(v / 32) * K + key]. V is a power of two, so a shuffle tree of width min(V, 32) stays inside the slice.
template <int KPT>
__device__ __forceinline__ void reduce_over_v(const float (&val)[KPT], float* red, int K, int V, int ks, int v) {
  const int width = V < 32 ? V : 32;
#pragma unroll
  for (int i = 0; i < KPT; ++i) {
    float x = val[i];
    for (int off = width >> 1; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    if ((v & (width - 1)) == 0) red[(v >> 5) * K + ks * KPT + i] = x;
  }
}

// Backward of the token scan. Phase A re-runs the forward and checkpoints the state entering every TB-token
// block; phase B walks the blocks in reverse, re-materialises the post-decay states S'_t of one block into
// `spre` (each thread writes and later reads only its own entries) and then walks its tokens backwards:
//   dS += scale q_t^T do_t;  dq_t = scale S_t do_t;  du_t = k_t dS;  dk_t = dS u_t (+ S'_t dr_t);
//   delta: dbeta_t = du_t . (v_t - r_t), dv_t = beta_t du_t, dr_t = -beta_t du_t, dS' = dS + k_t^T dr_t;
//   dg_t = <dS', S'_t> (per channel for vector gates);  dS_{t-1} = exp(g_t) dS' (zero across a reset).
template <typename T, int KPT>
__global__ void __launch_bounds__(512) rec_bwd_kernel(RecParams p) {
  extern __shared__ float smem_raw[];
  const int h = blockIdx.x, r = blockIdx.y;
  const int K = p.K, V = p.V, tid = threadIdx.x;
  const int v = tid % V, ks = tid / V, KS = K / KPT;
  const int hk = h / (p.H / p.Hk);
  const int VW = V < 32 ? 1 : V / 32;
  const Smem s = carve(smem_raw, K, V, KS, true);
  int tok0, len;
  p.rows.range(r, tok0, len);
  const int nblk = (len + TB - 1) / TB;
  float* ckpt = p.ckpt + ((long)h * p.total_blocks + tok0 / TB + r) * K * V;
  float* spre = p.spre + ((long)r * p.H + h) * TB * K * V;

  float S[KPT];
  const float* h0 = p.h0 ? p.h0 + ((long)r * p.H + h) * K * V : nullptr;
#pragma unroll
  for (int i = 0; i < KPT; ++i) S[i] = h0 ? h0[(long)(ks * KPT + i) * V + v] : 0.f;

  // ---- phase A: checkpoints
  for (int b = 0; b < nblk; ++b) {
    const int t0 = b * TB, nb = min(TB, len - t0);
#pragma unroll
    for (int i = 0; i < KPT; ++i) ckpt[(long)b * K * V + (long)(ks * KPT + i) * V + v] = S[i];
    if (b == nblk - 1) break;
    __syncthreads();
    load_block<T>(p, s, tok0 + t0, nb, tok0, h, hk, false);
    for (int j = 0; j < nb; ++j) {
      float resid;
      forward_token<KPT>(p, s, S, j, ks, v, KS, &resid, nullptr);
      if (!p.delta) continue;
      __syncthreads();  // part_r is rewritten by the next token
    }
  }

  // ---- phase B
  float dS[KPT];
  const float* dfin = p.d_final ? p.d_final + ((long)r * p.H + h) * K * V : nullptr;
#pragma unroll
  for (int i = 0; i < KPT; ++i) dS[i] = dfin ? dfin[(long)(ks * KPT + i) * V + v] : 0.f;

  T* dv = static_cast<T*>(p.dv);
  for (int b = nblk - 1; b >= 0; --b) {
    const int t0 = b * TB, nb = min(TB, len - t0);
#pragma unroll
    for (int i = 0; i < KPT; ++i) S[i] = ckpt[(long)b * K * V + (long)(ks * KPT + i) * V + v];
    __syncthreads();
    load_block<T>(p, s, tok0 + t0, nb, tok0, h, hk, true);
    for (int j = 0; j < nb; ++j) {
      float resid = 0.f;
      const float u = forward_token<KPT>(p, s, S, j, ks, v, KS, &resid, spre + (long)j * K * V);
      if (ks == 0) {
        s.us[j * V + v] = u;
        s.es[j * V + v] = resid;
      }
      if (p.delta) __syncthreads();
    }
    __syncthreads();

    for (int j = nb - 1; j >= 0; --j) {
      const long tok = tok0 + t0 + j;
      float* red = s.red + (j & 1) * (4 * 8 * K + 64);
      float* red_q = red;
      float* red_k = red + 8 * K;
      float* red_g = red + 16 * K;
      float* red_s = red + 24 * K;  // [0..31] dbeta partials, [32..63] scalar dg partials (per warp, <= 16 warps)
      float* red_kr = red + 24 * K + 64;
      float Sp[KPT], tmp[KPT];
      const float u = s.us[j * V + v];
      const float dov = s.dos[j * V + v];
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const float ki = s.ks[j * K + ks * KPT + i];
        Sp[i] = spre[(long)j * K * V + (long)(ks * KPT + i) * V + v];
        tmp[i] = (Sp[i] + ki * u) * dov;                      // S_t[k, v] do_v
        dS[i] += p.scale * s.qs[j * K + ks * KPT + i] * dov;  // o_t = scale q_t S_t
      }
      reduce_over_v<KPT>(tmp, red_q, K, V, ks, v);
      float partial = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) partial += s.ks[j * K + ks * KPT + i] * dS[i];
      float* part_r = s.part + 2 * KS * V;
      part_r[ks * V + v] = partial;
      __syncthreads();  // #1
      float du = 0.f;
      for (int t = 0; t < KS; ++t) du += part_r[t * V + v];
      const float beta = s.bs[j];
      const float dr = p.delta ? -beta * du : 0.f;
      float tmpr[KPT];  // the read key's gradient S'_t dr_t; added to dk when the write key is also the read key
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        tmpr[i] = Sp[i] * dr;
        tmp[i] = dS[i] * u + (p.k_read ? 0.f : tmpr[i]);
      }
      reduce_over_v<KPT>(tmp, red_k, K, V, ks, v);
      if (p.k_read) reduce_over_v<KPT>(tmpr, red_kr, K, V, ks, v);
      if (ks == 0) dv[(tok * p.H + h) * V + v] = from_f32<T>(p.delta ? beta * du : du);
      if (p.delta) {  // dbeta_t = sum_v du_v (v_v - r_v): reduce over the ks == 0 threads (warps 0 .. VW-1)
        float x = ks == 0 ? du * s.es[j * V + v] : 0.f;
        for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
        if ((tid & 31) == 0 && tid < V) red_s[tid >> 5] = x;
      }
      float gsum = 0.f;
#pragma unroll
      for (int i = 0; i < KPT; ++i) {
        const float dSp = dS[i] + s.kr[j * K + ks * KPT + i] * dr;  // gradient of S'_t
        tmp[i] = dSp * Sp[i];
        gsum += tmp[i];
        const float decay = p.gate == 1 ? s.eg[j] : (p.gate == 2 ? s.eg[j * K + ks * KPT + i] : 1.f);
        dS[i] = s.rs[j] ? 0.f : decay * dSp;
      }
      if (p.gate == 2) reduce_over_v<KPT>(tmp, red_g, K, V, ks, v);
      if (p.gate == 1) {
        for (int off = 16; off > 0; off >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, off);
        if ((tid & 31) == 0) red_s[32 + (tid >> 5)] = gsum;
      }
      __syncthreads();  // #2
      if (tid < K) {
        float aq = 0.f, ak = 0.f, ag = 0.f, akr = 0.f;
        for (int w = 0; w < VW; ++w) {
          aq += red_q[w * K + tid];
          ak += red_k[w * K + tid];
          if (p.gate == 2) ag += red_g[w * K + tid];
          if (p.k_read) akr += red_kr[w * K + tid];
        }
        p.dq_acc[(tok * p.H + h) * K + tid] = p.scale * aq;
        p.dk_acc[(tok * p.H + h) * K + tid] = ak;
        if (p.k_read) p.dkr_acc[(tok * p.H + h) * K + tid] = akr;
        if (p.gate == 2) p.dg[(tok * p.H + h) * K + tid] = ag;
      }
      if (tid == 0) {
        if (p.delta) {
          float x = 0.f;
          for (int w = 0; w < VW; ++w) x += red_s[w];
          p.dbeta[tok * p.H + h] = x;
        }
        if (p.gate == 1) {
          float x = 0.f;
          for (int w = 0; w < (int)(blockDim.x >> 5); ++w) x += red_s[32 + w];
          p.dg[tok * p.H + h] = x;
        }
      }
    }
  }
  if (p.dh0) {
    float* out = p.dh0 + ((long)r * p.H + h) * K * V;
#pragma unroll
    for (int i = 0; i < KPT; ++i) out[(long)(ks * KPT + i) * V + v] = dS[i];
  }
}

int pick_kpt(int K, int V) {
  for (int kpt = 1; kpt <= 128; kpt *= 2) {
    if (K % kpt) continue;
    const long nt = (long)V * (K / kpt);
    if (nt <= 512 && nt % 32 == 0) return kpt;
  }
  return 0;
}

RecParams base_params(const jla_problem& p) {
  RecParams r{};
  r.rows = make_rows(p);
  r.H = p.H; r.Hk = p.Hk; r.K = p.K; r.V = p.V;
  r.gate = p.kind == JLA_KIND_DELTANET ? 0 : (p.kind == JLA_KIND_KDA ? 2 : 1);
  r.delta = p.kind != JLA_KIND_SIMPLE_GLA;
  r.l2norm = (p.flags & JLA_FLAG_QK_L2NORM) != 0;
  r.scale = p.scale;
  r.q = p.q; r.k = p.k; r.v = p.v; r.g = p.g; r.beta = p.beta; r.h0 = p.h0;
  r.k_read = p.k_read;
  return r;
}

template <typename T, int KPT>
int launch(const RecParams& rp, bool bwd, int rows, cudaStream_t stream) {
  const int KS = rp.K / KPT;
  const size_t smem = smem_floats(rp.K, rp.V, KS, bwd) * sizeof(float);
  auto* kern = bwd ? rec_bwd_kernel<T, KPT> : rec_fwd_kernel<T, KPT>;
  if (smem > 48 * 1024) JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(rp.H, rows), block(rp.V * KS);
  {
    ProfScope ps(bwd ? kProfRecBwd : kProfRecFwd, stream);
    kern<<<grid, block, smem, stream>>>(rp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <typename T>
int launch_kpt(const RecParams& rp, int kpt, bool bwd, int rows, cudaStream_t stream) {
  switch (kpt) {
    case 1: return launch<T, 1>(rp, bwd, rows, stream);
    case 2: return launch<T, 2>(rp, bwd, rows, stream);
    case 4: return launch<T, 4>(rp, bwd, rows, stream);
    case 8: return launch<T, 8>(rp, bwd, rows, stream);
    case 16: return launch<T, 16>(rp, bwd, rows, stream);
    case 32: return launch<T, 32>(rp, bwd, rows, stream);
    case 64: return launch<T, 64>(rp, bwd, rows, stream);
    case 128: return launch<T, 128>(rp, bwd, rows, stream);
  }
  set_error("recurrent path: no thread layout for K=%d V=%d", rp.K, rp.V);
  return JLA_ERR_UNSUPPORTED;
}

int launch_dtype(const RecParams& rp, int dtype, int kpt, bool bwd, int rows, cudaStream_t stream) {
  switch (dtype) {
    case JLA_DTYPE_BF16: return launch_kpt<__nv_bfloat16>(rp, kpt, bwd, rows, stream);
    case JLA_DTYPE_F16: return launch_kpt<__half>(rp, kpt, bwd, rows, stream);
    case JLA_DTYPE_F32: return launch_kpt<float>(rp, kpt, bwd, rows, stream);
  }
  set_error("unknown dtype %d", dtype);
  return JLA_ERR_BAD_ARGUMENT;
}

struct BwdScratch {
  float *dq_acc, *dk_acc, *dkr_acc, *ckpt, *spre;
  long total_blocks;
  size_t bytes;
};

BwdScratch carve_bwd(const jla_problem& p, void* base) {
  Carver c(base);
  BwdScratch s;
  const long tokens = (long)p.B * p.T;
  const int rows = p.cu_seqlens || p.num_seqs ? p.num_seqs : p.B;
  s.total_blocks = tokens / TB + rows + 1;
  s.dq_acc = c.take<float>((size_t)tokens * p.H * p.K);
  s.dk_acc = c.take<float>((size_t)tokens * p.H * p.K);
  s.dkr_acc = c.take<float>(p.k_read ? (size_t)tokens * p.H * p.K : 0);
  s.ckpt = c.take<float>((size_t)p.H * s.total_blocks * p.K * p.V);
  s.spre = c.take<float>((size_t)rows * p.H * TB * p.K * p.V);
  s.bytes = c.bytes();
  return s;
}

}  // namespace

const char* recurrent_unsupported(const jla_problem& p) {
  if (p.K > 256 || p.V > 256 || p.K % 8) return "recurrent path: K must be a multiple of 8 and K, V <= 256";
  if (p.V < 8 || (p.V & (p.V - 1))) return "recurrent path: V must be a power of two in [8, 256]";
  if (!pick_kpt(p.K, p.V)) return "recurrent path: no thread layout for this K, V";
  return nullptr;
}

size_t recurrent_bwd_scratch_bytes(const jla_problem& p) { return carve_bwd(p, nullptr).bytes; }

int recurrent_fwd(const jla_problem& p, const jla_fwd_io& io, cudaStream_t stream) {
  RecParams rp = base_params(p);
  rp.o = io.o;
  rp.final_state = io.final_state;
  const int rows = p.cu_seqlens ? p.num_seqs : p.B;
  if (rows == 0 || p.H == 0) return JLA_OK;
  return launch_dtype(rp, p.dtype, pick_kpt(p.K, p.V), false, rows, stream);
}

int recurrent_bwd(const jla_problem& p, const jla_bwd_io& io, cudaStream_t stream) {
  RecParams rp = base_params(p);
  const BwdScratch s = carve_bwd(p, io.scratch);
  if (io.scratch_bytes < s.bytes) {
    set_error("backward scratch too small: %zu < %zu bytes", io.scratch_bytes, s.bytes);
    return JLA_ERR_WORKSPACE;
  }
  rp.d_o = io.d_o; rp.d_final = io.d_final;
  rp.dq_acc = s.dq_acc; rp.dk_acc = s.dk_acc; rp.dkr_acc = s.dkr_acc;
  rp.dv = io.dv; rp.dg = io.dg; rp.dbeta = io.dbeta; rp.dh0 = io.dh0;
  rp.ckpt = s.ckpt; rp.spre = s.spre; rp.total_blocks = s.total_blocks;
  const int rows = p.cu_seqlens ? p.num_seqs : p.B;
  const long tokens = (long)p.B * p.T;
  if (rows > 0 && p.H > 0) {
    const int rc = launch_dtype(rp, p.dtype, pick_kpt(p.K, p.V), true, rows, stream);
    if (rc != JLA_OK) return rc;
  }
  const bool l2 = (p.flags & JLA_FLAG_QK_L2NORM) != 0;
  int rc = finalize_key_grad(s.dq_acc, p.q, io.dq, p.dtype, tokens, p.H, p.Hk, p.K, l2, stream);
  if (rc != JLA_OK) return rc;
  if (p.k_read) {  // one row per value head, used as passed: no group sum, no norm to differentiate through
    rc = finalize_key_grad(s.dkr_acc, nullptr, io.dk_read, p.dtype, tokens, p.H, p.H, p.K, false, stream);
    if (rc != JLA_OK) return rc;
  }
  return finalize_key_grad(s.dk_acc, p.k, io.dk, p.dtype, tokens, p.H, p.Hk, p.K, l2, stream);
}

}  // namespace jla
