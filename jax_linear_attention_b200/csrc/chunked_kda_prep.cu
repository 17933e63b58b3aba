// Prologue of the chunked KDA forward (per-channel gates, reference: src/jla/ops/mosaic_gpu/vector_gate.py:226-303
// cumsum, :559-769 intra-chunk scores, :849-870 solve, :873-949 gate-folded operands). One CTA per (chunk, head).
//
// With G_i[c] the chunk-local cumulative log decay of channel c (token i sees exp(G_i) of the entering state), the
// chunk step of the delta rule is
//   Aqk_ij = sum_c q_ic k_jc exp(G_ic - G_jc)  (j <= i)        Akk_ij = beta_i sum_c k_ic k_jc exp(G_ic - G_jc)  (j < i)
//   T = (I + Akk)^-1,  Ag = T beta_j,  W = V - (k exp(G)) S,  Vn = Ag W,
//   O = scale [(q exp(G)) S + Aqk Vn],  S+ = diag(exp(G_63)) S + (k exp(G_63 - G))^T Vn.
// Everything that touches a gate is done here, in parallel over the chunks, so that the serial state pass
// (sg_fwd_tc_kernel, VG variant) is a gate-free delta rule on folded operands:
//   qs = cin   * q exp(G)          [64 x K]  reads the entering state        (cin: token still sees it)
//   kr = cin   * k exp(G)          [64 x K]  recalls from the entering state
//   kw = tail  * k exp(G_63 - G)   [64 x K]  writes into the leaving state   (tail: token reaches it)
//   d  = keep  * exp(G_63)         [K]       decay of the entering state
//   P  = Aqk, Ag                   [64 x 64] with the document mask applied
// All exponents above are <= 0, so these never overflow. The two score matrices need exp(G_i - G_j) per channel
// inside a contraction; they are factored through the per-channel mid point R = G_63 / 2,
//   (q exp(G - R)) (k exp(R - G))^T,   |G - R| <= |G_63| / 2,
// and run on the tensor cores when no channel decays by more than exp(-kda_bounded_log<T>()) over the chunk. Chunks with a
// stronger decay take the exact fp32 loop over (i, j, c) instead, so the result never depends on the bound.
//
// With a separate read key (jla_problem.k_read, Gated DeltaNet-2: S = S' + k^T (v - k_read S')) the key has two roles:
// wherever a token READS the state or the earlier tokens of its chunk -- the rows of Akk and the operand kr -- the
// read key stands for k; wherever it WRITES -- the columns of Akk and Aqk, the operand kw -- k itself does. The RK
// variant reads the read key from global memory where it folds the operands (its factored form takes the place of
// the raw k tile, which is dead by then); the exact path stages it in the tile of the factored write key, which that
// path does not build, and holds its score results in registers until the tile is free.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tri_inverse.cuh"

namespace jla {
namespace {

constexpr int KD = 128;

struct KdaPrepParams {
  const ChunkMeta* meta;
  const void *q, *k;   // [tokens, Hk, K] (after the optional L2 norm)
  const void* k_read;  // [tokens, H, K] or nullptr
  const float* g;      // [tokens, H, K]
  const float* gates;  // per (chunk, head): G[64] (zero here), beta[64]
  const unsigned char* runs;
  void *qs, *kr, *kw;  // [slot][64][K]
  void *ptile, *ag;    // [slot][64][64]
  void* t0;            // [slot][64][64] T itself, for the backward
  float* dvec;         // [slot][K]
  int H, Hk;
};

template <typename T, bool RK>
__global__ void __launch_bounds__(256, 2) kda_prep_kernel(KdaPrepParams p) {
  constexpr int LDK = KD + 8, LDA = kTriLda, LDM = kTriLdm, LDP = 72, NT = 256;
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long slot = (long)c * p.H + h;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tq = reinterpret_cast<T*>(smem_raw);        // q, then q exp(G - R); the inverse X takes its place afterwards
  T* tk = tq + 64 * LDK;                         // k, then k exp(G - R)
  T* tb = tk + 64 * LDK;                         // k exp(R - G); later the staged P tile [64][LDP]
  float* Gm = reinterpret_cast<float*>(tb + 64 * LDK);  // [64][KD]
  float* A = Gm + 64 * KD;                       // [64][LDA]
  float* M = A + 64 * LDA;                       // [32][LDM]
  float* betas = M + 32 * LDM;                   // [64]
  float* Glast = betas + 64;                     // [KD]
  int* run = reinterpret_cast<int*>(Glast + KD); // [64]
  T* tr = tk;  // factored path: read key exp(G - R) takes the raw k tile's place
  float* X = reinterpret_cast<float*>(smem_raw);
  static_assert(64 * LDK * sizeof(T) >= 64 * LDA * sizeof(float), "X overlays the q tile");
  T* pst = tb;

  const long kstride = (long)p.Hk * KD;
  load_tile_async<T, 64, KD>(tq, LDK, static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * KD, kstride, m.len, tid, NT);
  load_tile_async<T, 64, KD>(tk, LDK, static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * KD, kstride, m.len, tid, NT);
  const T* krg = RK ? static_cast<const T*>(p.k_read) + ((long)m.tok0 * p.H + h) * KD : nullptr;  // read key rows
  const long krstride = (long)p.H * KD;
  cp_async_commit();
  if (tid < 64) {
    betas[tid] = p.gates[slot * 128 + 64 + tid];
    run[tid] = p.runs[(long)c * 64 + tid];
  }
  // ---- cumulative log decay per channel: two threads per channel, 32 tokens each, then the second half is offset;
  // padding tokens add nothing
  int unbounded;
  {
    const int ch = tid & (KD - 1), hh = tid >> 7;
    const float* gp = p.g + ((long)m.tok0 * p.H + h) * KD + ch;
    const long gstride = (long)p.H * KD;
    float acc = 0.f;
#pragma unroll
    for (int i0 = 32 * hh; i0 < 32 * hh + 32; i0 += 16) {
      float gv[16];  // sixteen loads in flight before the first add
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) gv[ii] = (i0 + ii < m.len) ? gp[(i0 + ii) * gstride] : 0.f;
#pragma unroll
      for (int ii = 0; ii < 16; ++ii) {
        acc += gv[ii];
        Gm[(i0 + ii) * KD + ch] = acc;
      }
    }
    if (hh == 0) M[ch] = acc;  // scratch of the inverse, free until then
    cp_async_wait<0>();
    __syncthreads();
    float total = acc;
    if (hh == 1) {
      const float off = M[ch];
      for (int i = 32; i < 64; ++i) Gm[i * KD + ch] += off;
      total = acc + off;
      Glast[ch] = total;
    }
    unbounded = __syncthreads_or(hh == 1 && !(fabsf(total) <= kda_bounded_log<T>()));
  }
  const bool entering = !(m.flags & 1);
  const int run_last = run[63];

  T* qs = static_cast<T*>(p.qs) + slot * 64 * KD;
  T* kr = static_cast<T*>(p.kr) + slot * 64 * KD;
  T* kw = static_cast<T*>(p.kw) + slot * 64 * KD;
  if (tid < KD) p.dvec[slot * KD + tid] = (entering && run_last == 0) ? __expf(Glast[tid]) : 0.f;

  if (!unbounded) {
    // ---- one pass over the tiles: the state-side operands to global memory and the factored operands in place.
    // With d = G - R, R = G_63 / 2 (|d|, |R| <= kda_bounded_log<T>() / 2 here): exp(G) = exp(d) exp(R) and
    // exp(G_63 - G) = exp(-d) exp(R), so two exponentials per element serve all five operands.
    float* eRs = M + KD;  // exp(R) per channel (scratch of the inverse, free until then)
    if (tid < KD) eRs[tid] = __expf(0.5f * Glast[tid]);
    __syncthreads();
    for (int idx = tid; idx < 64 * (KD / 8); idx += NT) {
      const int i = idx >> 4, c8 = (idx & 15) * 8;
      const bool cin = entering && run[i] == 0;
      const bool tail = i < m.len && run[i] == run_last;
      uint4 qv = *reinterpret_cast<const uint4*>(tq + i * LDK + c8);
      uint4 kv = *reinterpret_cast<const uint4*>(tk + i * LDK + c8);
      uint4 rv = kv;  // the read key (tokens past a partial chunk's end read as zero, like the tiles)
      if (RK) rv = i < m.len ? *reinterpret_cast<const uint4*>(krg + i * krstride + c8) : make_uint4(0u, 0u, 0u, 0u);
      uint4 bv, oq, or_, ow;
      uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
      uint32_t* kwd = reinterpret_cast<uint32_t*>(&kv);
      uint32_t* rwd = reinterpret_cast<uint32_t*>(&rv);
      uint32_t* bw = reinterpret_cast<uint32_t*>(&bv);
      uint32_t* oqw = reinterpret_cast<uint32_t*>(&oq);
      uint32_t* orw = reinterpret_cast<uint32_t*>(&or_);
      uint32_t* oww = reinterpret_cast<uint32_t*>(&ow);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 qf = unpack2<T>(qw[e]), kf = unpack2<T>(kwd[e]), rf = unpack2<T>(rwd[e]);
        const float d0 = Gm[i * KD + c8 + 2 * e] - 0.5f * Glast[c8 + 2 * e];
        const float d1 = Gm[i * KD + c8 + 2 * e + 1] - 0.5f * Glast[c8 + 2 * e + 1];
        const float u0 = __expf(d0), u1 = __expf(d1), n0 = __expf(-d0), n1 = __expf(-d1);
        const float r0 = eRs[c8 + 2 * e], r1 = eRs[c8 + 2 * e + 1];
        const float e0 = cin ? u0 * r0 : 0.f, e1 = cin ? u1 * r1 : 0.f;
        const float w0 = tail ? n0 * r0 : 0.f, w1 = tail ? n1 * r1 : 0.f;
        oqw[e] = pack2<T>(qf.x * e0, qf.y * e1);
        orw[e] = pack2<T>(rf.x * e0, rf.y * e1);
        oww[e] = pack2<T>(kf.x * w0, kf.y * w1);
        qw[e] = pack2<T>(qf.x * u0, qf.y * u1);
        rwd[e] = pack2<T>(rf.x * u0, rf.y * u1);
        bw[e] = pack2<T>(kf.x * n0, kf.y * n1);
      }
      *reinterpret_cast<uint4*>(qs + i * KD + c8) = oq;
      *reinterpret_cast<uint4*>(kr + i * KD + c8) = or_;
      *reinterpret_cast<uint4*>(kw + i * KD + c8) = ow;
      *reinterpret_cast<uint4*>(tq + i * LDK + c8) = qv;
      *reinterpret_cast<uint4*>(tr + i * LDK + c8) = rv;  // over the raw k tile, which this thread has just read
      *reinterpret_cast<uint4*>(tb + i * LDK + c8) = bv;
    }
    __syncthreads();
    // warps 0-3: q^ k~^T (the score tile), warps 4-7: k^ k~^T (the solve matrix; k^ from the read key); 16 rows each
    const int rw = warp & 3;
    const bool score = warp < 4;
    float acc[8][4];
    zero_acc(acc);
    warp_gemm<T, 8, KD / 16, A_ROW, B_NK>(acc, (score ? tq : tr) + rw * 16 * LDK, LDK, tb, LDK, lane);
    __syncthreads();  // every warp has read the tiles: X and the staged P may take their place
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int i = rw * 16 + g + 8 * hh, j = nt * 8 + 2 * t;
        const int ri = run[i];
        const bool s0 = ri == run[j], s1 = ri == run[j + 1];
        if (score) {
          const float p0 = (j <= i && s0) ? acc[nt][2 * hh] : 0.f;
          const float p1 = (j + 1 <= i && s1) ? acc[nt][2 * hh + 1] : 0.f;
          *reinterpret_cast<uint32_t*>(pst + i * LDP + j) = pack2<T>(p0, p1);
        } else {
          const float bi = betas[i];
          float2 v;
          v.x = (j < i && s0) ? bi * acc[nt][2 * hh] : 0.f;
          v.y = (j + 1 < i && s1) ? bi * acc[nt][2 * hh + 1] : 0.f;
          *reinterpret_cast<float2*>(A + i * LDA + j) = v;
        }
      }
    }
  } else {
    // ---- exact path. The state-side operands with their own (always non-positive) exponents:
    T* te = RK ? tb : tk;  // the raw read key of this path (tb holds no factored tile here)
    if (RK) {
      load_tile_async<T, 64, KD>(te, LDK, krg, krstride, m.len, tid, NT);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
    }
    for (int idx = tid; idx < 64 * (KD / 8); idx += NT) {
      const int i = idx >> 4, c8 = (idx & 15) * 8;
      const bool cin = entering && run[i] == 0;
      const bool tail = i < m.len && run[i] == run_last;
      const uint4 qv = *reinterpret_cast<const uint4*>(tq + i * LDK + c8);
      const uint4 kv = *reinterpret_cast<const uint4*>(tk + i * LDK + c8);
      const uint4 rv = *reinterpret_cast<const uint4*>(te + i * LDK + c8);
      const uint32_t* qw = reinterpret_cast<const uint32_t*>(&qv);
      const uint32_t* kwd = reinterpret_cast<const uint32_t*>(&kv);
      const uint32_t* rwd = reinterpret_cast<const uint32_t*>(&rv);
      uint4 oq, or_, ow;
      uint32_t* oqw = reinterpret_cast<uint32_t*>(&oq);
      uint32_t* orw = reinterpret_cast<uint32_t*>(&or_);
      uint32_t* oww = reinterpret_cast<uint32_t*>(&ow);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 qf = unpack2<T>(qw[e]), kf = unpack2<T>(kwd[e]), rf = unpack2<T>(rwd[e]);
        const float g0 = Gm[i * KD + c8 + 2 * e], g1 = Gm[i * KD + c8 + 2 * e + 1];
        const float e0 = cin ? __expf(g0) : 0.f, e1 = cin ? __expf(g1) : 0.f;
        const float w0 = tail ? __expf(Glast[c8 + 2 * e] - g0) : 0.f, w1 = tail ? __expf(Glast[c8 + 2 * e + 1] - g1) : 0.f;
        oqw[e] = pack2<T>(qf.x * e0, qf.y * e1);
        orw[e] = pack2<T>(rf.x * e0, rf.y * e1);
        oww[e] = pack2<T>(kf.x * w0, kf.y * w1);
      }
      *reinterpret_cast<uint4*>(qs + i * KD + c8) = oq;
      *reinterpret_cast<uint4*>(kr + i * KD + c8) = or_;
      *reinterpret_cast<uint4*>(kw + i * KD + c8) = ow;
    }
    // every pair (i, j <= i) of one document, fp32 with the true exponent per channel
    __syncthreads();
    // one pair's scores: the read row i of the solve matrix (from the read key) and of the score tile (from q)
    auto pair_scores = [&](int i, int j, float& sq, float& sk) {
      sq = 0.f;
      sk = 0.f;
      if (j <= i && run[i] == run[j]) {
        for (int cc = 0; cc < KD; ++cc) {
          const int ch = (cc + lane) & (KD - 1);  // lanes of a warp share i: spread the channels over the banks
          const float e = __expf(Gm[i * KD + ch] - Gm[j * KD + ch]);
          const float kj = to_f32(tk[j * LDK + ch]) * e;
          sq += to_f32(tq[i * LDK + ch]) * kj;
          sk += to_f32(te[i * LDK + ch]) * kj;
        }
      }
    };
    if (!RK) {  // pst (the tile of the factored write key) is free on this path: results go straight into it
      for (int idx = tid; idx < 64 * 64; idx += NT) {
        const int i = idx >> 6, j = idx & 63;
        float sq, sk;
        pair_scores(i, j, sq, sk);
        A[i * LDA + j] = j < i ? betas[i] * sk : 0.f;
        pst[i * LDP + j] = from_f32<T>(sq);
      }
      __syncthreads();  // the raw tiles have been read: X may take their place
    } else {  // the read key sits in that tile: this thread's scores wait in registers until every thread has read it
      T sqv[64 * 64 / NT];
#pragma unroll
      for (int n = 0; n < 64 * 64 / NT; ++n) {
        const int idx = tid + n * NT;
        const int i = idx >> 6, j = idx & 63;
        float sq, sk;
        pair_scores(i, j, sq, sk);
        A[i * LDA + j] = j < i ? betas[i] * sk : 0.f;
        sqv[n] = from_f32<T>(sq);
      }
      __syncthreads();
#pragma unroll
      for (int n = 0; n < 64 * 64 / NT; ++n) {
        const int idx = tid + n * NT;
        pst[(idx >> 6) * LDP + (idx & 63)] = sqv[n];
      }
      // (the barrier after the clearing of X below orders these stores before the tile is read)
    }
  }
  for (int idx = tid; idx < 64 * LDA / 4; idx += NT) reinterpret_cast<float4*>(X)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncthreads();

  invert_unit_lower_64(A, X, M, tid);

  T* outp = static_cast<T*>(p.ptile) + slot * 64 * 64;
  T* outg = static_cast<T*>(p.ag) + slot * 64 * 64;
  T* outt = p.t0 ? static_cast<T*>(p.t0) + slot * 64 * 64 : nullptr;
  for (int idx = tid; idx < 64 * 8; idx += NT) {
    const int r = idx >> 3, c8 = (idx & 7) * 8;
    *reinterpret_cast<uint4*>(outp + r * 64 + c8) = *reinterpret_cast<const uint4*>(pst + r * LDP + c8);
    float a[8], x[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = c8 + e;
      x[e] = (j <= r && run[j] == run[r]) ? X[r * LDA + j] : 0.f;
      a[e] = x[e] * betas[j];
    }
    uint4 v;
    v.x = pack2<T>(a[0], a[1]);
    v.y = pack2<T>(a[2], a[3]);
    v.z = pack2<T>(a[4], a[5]);
    v.w = pack2<T>(a[6], a[7]);
    *reinterpret_cast<uint4*>(outg + r * 64 + c8) = v;
    if (outt) {
      v.x = pack2<T>(x[0], x[1]);
      v.y = pack2<T>(x[2], x[3]);
      v.z = pack2<T>(x[4], x[5]);
      v.w = pack2<T>(x[6], x[7]);
      *reinterpret_cast<uint4*>(outt + r * 64 + c8) = v;
    }
  }
}

template <typename T>
int launch_prep_t(const KdaPrepParams& kp, bool read_key, int blocks, cudaStream_t s) {
  const size_t smem = 3 * 64 * (KD + 8) * sizeof(T) + (64 * KD + 64 * kTriLda + 32 * kTriLdm + 64 + KD) * sizeof(float) +
                      64 * sizeof(int);
  auto* kern = read_key ? kda_prep_kernel<T, true> : kda_prep_kernel<T, false>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    ProfScope ps(kProfKdaPrep, s);
    kern<<<blocks, 256, smem, s>>>(kp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

int launch_kda_prep(const ChunkedCtx& c, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  KdaPrepParams kp{};
  kp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  kp.q = c.q_eff;
  kp.k = c.k_eff;
  kp.k_read = p.k_read;
  kp.g = p.g;
  kp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  kp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  kp.qs = c.res + pl.kda_q;
  kp.kr = c.res + pl.kda_kr;
  kp.kw = c.res + pl.kda_kw;
  kp.ptile = c.res + pl.kda_p;
  kp.ag = c.res + pl.ag;
  kp.t0 = c.res + pl.t0;  // always: a later pass that shares this prologue (JLA_FLAG_PREP_DONE) may be differentiated
  kp.dvec = reinterpret_cast<float*>(c.res + pl.kda_d);
  kp.H = p.H;
  kp.Hk = p.Hk;
  if ((p.dtype != JLA_DTYPE_BF16 && p.dtype != JLA_DTYPE_F16) || p.K != KD) {
    set_error("chunked KDA: bf16 or f16 tensors with K = 128 only");
    return JLA_ERR_UNSUPPORTED;
  }
  return p.dtype == JLA_DTYPE_BF16 ? launch_prep_t<__nv_bfloat16>(kp, p.k_read != nullptr, pl.nc * p.H, s)
                                   : launch_prep_t<__half>(kp, p.k_read != nullptr, pl.nc * p.H, s);
}

}  // namespace jla
