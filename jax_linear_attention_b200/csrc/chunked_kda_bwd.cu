// Chunk-parallel gradients of the chunked KDA path (per-channel gates), after the reverse state pass
// (sg_bwd_state_tc_kernel, VG variant) has produced dS+ per chunk, dVn and dW = dv. Reference:
// src/jla/ops/mosaic_gpu/vector_gate_bwd.py:278-447 (state-side and WY gradients), :450-492 (dAkk), :528-799 (scores).
//
// In the gate-folded form of chunked_kda_prep.cu the chunk step is a gate-free delta rule
//   W = V - Ks S,  Vn = Ag W,  O = scale (Qs S + P Vn),  S+ = diag(d) S + Ku^T Vn,
// so the first kernel needs no gate at all (one CTA per chunk and head, all operands as the forward left them):
//   dQs = scale dO S^T    dKs = -dW S^T    dKu = Vn dS+^T    dP = scale dO Vn^T    dAg = dVn W^T    dd = rowsum(dS+ * S)
// The second kernel takes these back through the triangular solve and the decayed scores and unfolds the gates:
//   dT = dAg beta_j,  dbeta_j += sum_i dAg_ij T_ij,  dA = -strict(T^T dT T^T),  dbeta_i += sum_j dA_ij Akk_ij,
//   dq^ = dP k~,  dk^ = beta_i dA k~,  dk~ = dP^T q^ + dA^T (beta k^)               (q^, k^, k~: mid-point factors)
//   dq = dq^ e^(G-R) + dQs cin e^G          dk = [dk^ e^(G-R) + dKs cin e^G] + [dk~ e^(R-G) + dKu tail e^(G63-G)]
//   dG_i = q dq + k (read-side dk - write-side dk);   dG_63 += sum_i k dKu tail e^(G63-G) + d dd
//   dg_t = sum_(i >= t) dG_i + dG_63        (G is a running sum over the chunk's tokens)
// Chunks whose decay is too strong for the factored scores take exact fp32 loops, as in the forward.
//
// Rounding of dG on the factored path. A pair (i, j) of tokens enters dG twice, +X_ij at row i and -X_ij at row j,
// and a gate parameter's gradient multiplies dG_i by the cumulative decay G_i (dA_log = sum_i dG_i G_i), so the two
// copies must agree far below bf16 precision or their difference is amplified by |G| (the reference met the same
// effect: tests/test_vector_gate_gate_grads.py:1-14). Both copies are therefore formed from the SAME 16-bit operands
// the tensor cores multiply: +X = q^ (dP k~) + (beta k^) (dA k~) and -X = k~ (dP^T q^ + dA^T (beta k^)), with q^, k~
// and beta k^ read back from the rounded tiles, never recomputed from q, k in fp32. Then X+ and X- differ only by the
// order of the fp32 accumulation.
//
// With a separate read key (jla_problem.k_read, Gated DeltaNet-2) the read side of every formula above (k^, the rows
// of Akk, dKs, "read-side dk") belongs to the read key and is returned as dk_read per value head; the write side
// (k~, dKu, "write-side dk") is dk. The RK variant of the second kernel keeps the raw read key in a tile of its own.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"

namespace jla {
namespace {

constexpr int KD = 128, VD = 128;

struct KdaGradParams {
  const ChunkMeta* meta;
  const void *q, *k;   // [tokens, Hk, K]
  const void* k_read;  // [tokens, H, K] or nullptr
  void* dk_read;       // [tokens, H, K] tensor dtype (with k_read)
  const float* g;      // [tokens, H, K]
  const float* gates;  // per (chunk, head): G (zero), beta[64]
  const unsigned char* runs;
  const void *d_o, *dw;              // [tokens, H, V]
  const void *hT, *dhT;              // [slot][V][K]
  const void *vnT, *dvnT, *wT;       // [slot][V][64]
  const void *t0;                    // [slot][64][64]  T = (I + Akk)^-1
  void *dp, *dag;                    // [slot][64][64]
  float *dqs, *dks, *dku;            // [slot][64][K]
  float* dd;                         // [slot][K]
  float *dq_acc, *dk_acc;            // [tokens, H, K] f32, when key heads are grouped or the op normalised q, k
  void *dq, *dk;                     // [tokens, Hk, K] tensor dtype, written directly otherwise (else nullptr)
  float *dg, *dbeta;
  int H, Hk;
  float scale;
};

// ---------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256, 1) kda_state_grads_kernel(KdaGradParams p) {
  constexpr int LDV = VD + 8, LDK = KD + 8, LDC = 72;
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), ch = warp >> 2, kc0 = (KD / 2) * ch, cc0 = 32 * ch;
  const long slot = (long)c * p.H + h;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* dOs = reinterpret_cast<T*>(smem_raw);  // [64][LDV]
  T* dWs = dOs + 64 * LDV;                  // [64][LDV]
  T* hS = dWs + 64 * LDV;                   // [V][LDK]   S^T
  T* dhS = hS + VD * LDK;                   // [V][LDK]   dS+^T
  T* vnS = dhS + VD * LDK;                  // [V][LDC]   Vn^T
  T* dvnS = vnS + VD * LDC;                 // [V][LDC]   dVn^T
  T* wS = dvnS + VD * LDC;                  // [V][LDC]   W^T
  float* ddp = reinterpret_cast<float*>(wS + VD * LDC);  // [2][KD]

  const long vstride = (long)p.H * VD;
  // two load groups: the products of the first run while the second is still in flight
  load_tile_async<T, 64, VD>(dOs, LDV, static_cast<const T*>(p.d_o) + ((long)m.tok0 * p.H + h) * VD, vstride, m.len, tid, 256);
  load_tile_async<T, 64, VD>(dWs, LDV, static_cast<const T*>(p.dw) + ((long)m.tok0 * p.H + h) * VD, vstride, m.len, tid, 256);
  load_tile_async<T, VD, KD>(hS, LDK, static_cast<const T*>(p.hT) + slot * VD * KD, KD, VD, tid, 256);
  load_tile_async<T, VD, 64>(vnS, LDC, static_cast<const T*>(p.vnT) + slot * VD * 64, 64, VD, tid, 256);
  cp_async_commit();
  load_tile_async<T, VD, KD>(dhS, LDK, static_cast<const T*>(p.dhT) + slot * VD * KD, KD, VD, tid, 256);
  load_tile_async<T, VD, 64>(dvnS, LDC, static_cast<const T*>(p.dvnT) + slot * VD * 64, 64, VD, tid, 256);
  load_tile_async<T, VD, 64>(wS, LDC, static_cast<const T*>(p.wT) + slot * VD * 64, 64, VD, tid, 256);
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  auto store_f32 = [&](float* dst, const float (&acc)[8][4], float s) {  // [64][K] tile, this warp's 16 x 64 block
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int col = kc0 + nt * 8 + 2 * t;
      *reinterpret_cast<float2*>(dst + (r0 + g) * KD + col) = make_float2(s * acc[nt][0], s * acc[nt][1]);
      *reinterpret_cast<float2*>(dst + (r0 + g + 8) * KD + col) = make_float2(s * acc[nt][2], s * acc[nt][3]);
    }
  };
  {
    float acc[8][4];
    zero_acc(acc);  // dQs = scale dO S^T
    warp_gemm<T, 8, VD / 16, A_ROW, B_KN>(acc, dOs + r0 * LDV, LDV, hS + kc0, LDK, lane);
    store_f32(p.dqs + slot * 64 * KD, acc, p.scale);
    zero_acc(acc);  // dKs = -dW S^T
    warp_gemm<T, 8, VD / 16, A_ROW, B_KN>(acc, dWs + r0 * LDV, LDV, hS + kc0, LDK, lane);
    store_f32(p.dks + slot * 64 * KD, acc, -1.f);
  }
  {
    float acc[4][4];
    zero_acc(acc);  // dP = scale dO Vn^T
    warp_gemm<T, 4, VD / 16, A_ROW, B_KN>(acc, dOs + r0 * LDV, LDV, vnS + cc0, LDC, lane);
    store_acc<T, 4>(static_cast<T*>(p.dp) + slot * 4096, 64, r0, cc0, acc, lane, p.scale, p.scale);
  }
  cp_async_wait<0>();
  __syncthreads();
  {
    float acc[8][4];
    zero_acc(acc);  // dKu = Vn dS+^T
    warp_gemm<T, 8, VD / 16, A_COL, B_KN>(acc, vnS + r0, LDC, dhS + kc0, LDK, lane);
    store_f32(p.dku + slot * 64 * KD, acc, 1.f);
  }
  {
    float acc[4][4];
    zero_acc(acc);  // dAg = dVn W^T
    warp_gemm<T, 4, VD / 16, A_COL, B_KN>(acc, dvnS + r0, LDC, wS + cc0, LDC, lane);
    store_acc<T, 4>(static_cast<T*>(p.dag) + slot * 4096, 64, r0, cc0, acc, lane);
  }
  {  // dd[c] = sum_v dS+[c][v] S[c][v]
    const int col = tid & (KD - 1), half = tid >> 7;
    float s = 0.f;
    for (int v = 64 * half; v < 64 * half + 64; ++v) s += to_f32(dhS[v * LDK + col]) * to_f32(hS[v * LDK + col]);
    ddp[half * KD + col] = s;
    __syncthreads();
    if (tid < KD) p.dd[slot * KD + tid] = ddp[tid] + ddp[KD + tid];
  }
}


// ---------------------------------------------------------------------------------------------------------------
// sum over the 8 row groups of a warp for one accumulator column pair; valid in lanes 0..3 (t = lane)
__device__ __forceinline__ float col_reduce(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 16);
  return x;
}

template <typename T, bool RK>
__global__ void __launch_bounds__(512, 1) kda_intra_grads_kernel(KdaGradParams p) {
  constexpr int LDK = KD + 8, LDC = 72, NT = 512;
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int rw = warp & 3, cq = warp >> 2;  // row block of 16 tokens; column quarter (of 64 x 64 tiles and of the K channels)
  const int r0 = 16 * rw;
  const long slot = (long)c * p.H + h;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tq = reinterpret_cast<T*>(smem_raw);  // raw q
  T* tk = tq + 64 * LDK;                   // raw k
  T* tqh = tk + 64 * LDK;                  // q exp(G - R)
  T* tkh = tqh + 64 * LDK;                 // beta_i k exp(G - R)
  T* tb = tkh + 64 * LDK;                  // k exp(R - G)
  T* Tt = tb + 64 * LDK;                   // [64][LDC] T
  T* Xd = Tt + 64 * LDC;                   // dT
  T* Xm = Xd + 64 * LDC;                   // dAg, then M1 = dT T^T, then dA
  T* Xp = Xm + 64 * LDC;                   // dP
  float* Gm = reinterpret_cast<float*>(Xp + 64 * LDC);  // [64][KD]
  float* dGt = Gm + 64 * KD;               // [64][KD] per-token dG; the exact path keeps the write-side dk here first
  float* part = dGt + 64 * KD;             // [4][KD] column sums per row block (also scratch of the gate cumsum)
  float* betas = part + 4 * KD;            // [64]
  float* Glast = betas + 64;               // [KD]
  float* dbrow = Glast + KD;               // [4][64] per column quarter
  float* dbcol = dbrow + 256;              // [64]
  int* run = reinterpret_cast<int*>(dbcol + 64);  // [64]
  T* tr = RK ? reinterpret_cast<T*>(run + 64) : tk;  // raw read key (RK: a tile of its own)

  const long kstride = (long)p.Hk * KD;
  load_tile_async<T, 64, KD>(tq, LDK, static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * KD, kstride, m.len, tid, NT);
  load_tile_async<T, 64, KD>(tk, LDK, static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * KD, kstride, m.len, tid, NT);
  if (RK) {
    load_tile_async<T, 64, KD>(tr, LDK, static_cast<const T*>(p.k_read) + ((long)m.tok0 * p.H + h) * KD, (long)p.H * KD,
                               m.len, tid, NT);
  }
  load_tile_async<T, 64, 64>(Tt, LDC, static_cast<const T*>(p.t0) + slot * 4096, 64, 64, tid, NT);
  load_tile_async<T, 64, 64>(Xm, LDC, static_cast<const T*>(p.dag) + slot * 4096, 64, 64, tid, NT);
  load_tile_async<T, 64, 64>(Xp, LDC, static_cast<const T*>(p.dp) + slot * 4096, 64, 64, tid, NT);
  cp_async_commit();
  if (tid < 64) {
    betas[tid] = p.gates[slot * 128 + 64 + tid];
    run[tid] = p.runs[(long)c * 64 + tid];
  }
  // ---- cumulative log decay per channel: four threads per channel, 16 tokens each, then offset by the totals before
  int unbounded;
  {
    const int ch = tid & (KD - 1), hh = tid >> 7;
    const float* gp = p.g + ((long)m.tok0 * p.H + h) * KD + ch;
    const long gstride = (long)p.H * KD;
    float gv[16];  // all sixteen loads in flight before the first add
#pragma unroll
    for (int ii = 0; ii < 16; ++ii) gv[ii] = (16 * hh + ii < m.len) ? gp[(16 * hh + ii) * gstride] : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int ii = 0; ii < 16; ++ii) {
      acc += gv[ii];
      Gm[(16 * hh + ii) * KD + ch] = acc;
    }
    part[hh * KD + ch] = acc;
    cp_async_wait<0>();
    __syncthreads();
    float off = 0.f;
    for (int b = 0; b < hh; ++b) off += part[b * KD + ch];
    if (hh > 0) {
      for (int i = 16 * hh; i < 16 * hh + 16; ++i) Gm[i * KD + ch] += off;
    }
    const float total = acc + off;
    if (hh == 3) Glast[ch] = total;
    unbounded = __syncthreads_or(hh == 3 && !(fabsf(total) <= kda_bounded_log<T>()));
  }
  const bool entering = !(m.flags & 1);
  const int run_last = run[63];

  // ---- dT = dAg beta_j (same document, j <= i); dbeta_j += sum_i dAg_ij T_ij; the same mask on dP
  for (int idx = tid; idx < 64 * 64; idx += NT) {
    const int i = idx >> 6, j = idx & 63;
    const bool ok = j <= i && run[i] == run[j];
    Xd[i * LDC + j] = from_f32<T>(ok ? to_f32(Xm[i * LDC + j]) * betas[j] : 0.f);
    if (!ok) Xp[i * LDC + j] = from_f32<T>(0.f);  // dP arrives unmasked: only pairs of one document with j <= i count
  }
  {  // eight threads per column j, eight rows each
    const int j = tid >> 3, i8 = (tid & 7) * 8;
    float s = 0.f;
#pragma unroll
    for (int ii = 0; ii < 8; ++ii) {
      const int i = i8 + ii;
      if (i >= j && run[i] == run[j]) s += to_f32(Xm[i * LDC + j]) * to_f32(Tt[i * LDC + j]);
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if ((tid & 7) == 0) dbcol[j] = s;
  }
  __syncthreads();
  // ---- dA = -strict(T^T (dT T^T)): this warp's 16 rows x 16 columns
  {
    float accM[2][4], accA[2][4];
    zero_acc(accM);
    warp_gemm<T, 2, 4, A_ROW, B_NK>(accM, Xd + r0 * LDC, LDC, Tt + 16 * cq * LDC, LDC, lane);
    __syncthreads();  // dAg (Xm) and dT (Xd) have been read by every warp
    store_acc<T, 2>(Xm, LDC, r0, 16 * cq, accM, lane);
    __syncthreads();
    zero_acc(accA);
    warp_gemm<T, 2, 4, A_COL, B_KN>(accA, Tt + r0, LDC, Xm + 16 * cq, LDC, lane);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = r0 + g + ((e >> 1) << 3), j = 16 * cq + nt * 8 + 2 * t + (e & 1);
        accA[nt][e] = (j < i && run[i] == run[j]) ? -accA[nt][e] : 0.f;
      }
    }
    __syncthreads();  // M1 (Xm) has been read by every warp
    store_acc<T, 2>(Xm, LDC, r0, 16 * cq, accA, lane);                                      // dA
  }
  const long tokbase = ((long)m.tok0 * p.H + h) * KD;
  const long tstride = (long)p.H * KD;
  T* dq16 = p.dq ? static_cast<T*>(p.dq) + ((long)m.tok0 * p.Hk + hk) * KD : nullptr;  // direct stores (H == Hk)
  T* dk16 = p.dk ? static_cast<T*>(p.dk) + ((long)m.tok0 * p.Hk + hk) * KD : nullptr;
  T* dkr16 = RK ? static_cast<T*>(p.dk_read) + tokbase : nullptr;  // read-side dk, one row per value head
  const float* dqs = p.dqs + slot * 64 * KD;
  const float* dks = p.dks + slot * 64 * KD;
  const float* dku = p.dku + slot * 64 * KD;

  if (!unbounded) {
    // ---- the factored operands
    for (int idx = tid; idx < 64 * (KD / 8); idx += NT) {
      const int i = idx >> 4, c8 = (idx & 15) * 8;
      const float bi = betas[i];
      const uint4 qv = *reinterpret_cast<const uint4*>(tq + i * LDK + c8);
      const uint4 kv = *reinterpret_cast<const uint4*>(tk + i * LDK + c8);
      const uint4 rv = *reinterpret_cast<const uint4*>(tr + i * LDK + c8);
      uint4 oq, ok, ob;
      const uint32_t* qw = reinterpret_cast<const uint32_t*>(&qv);
      const uint32_t* kw = reinterpret_cast<const uint32_t*>(&kv);
      const uint32_t* rw2 = reinterpret_cast<const uint32_t*>(&rv);
      uint32_t* oqw = reinterpret_cast<uint32_t*>(&oq);
      uint32_t* okw = reinterpret_cast<uint32_t*>(&ok);
      uint32_t* obw = reinterpret_cast<uint32_t*>(&ob);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 qf = unpack2<T>(qw[e]), kf = unpack2<T>(kw[e]), rf = unpack2<T>(rw2[e]);
        const float d0 = Gm[i * KD + c8 + 2 * e] - 0.5f * Glast[c8 + 2 * e];
        const float d1 = Gm[i * KD + c8 + 2 * e + 1] - 0.5f * Glast[c8 + 2 * e + 1];
        const float u0 = __expf(d0), u1 = __expf(d1), n0 = __expf(-d0), n1 = __expf(-d1);
        oqw[e] = pack2<T>(qf.x * u0, qf.y * u1);
        okw[e] = pack2<T>(bi * rf.x * u0, bi * rf.y * u1);
        obw[e] = pack2<T>(kf.x * n0, kf.y * n1);
      }
      *reinterpret_cast<uint4*>(tqh + i * LDK + c8) = oq;
      *reinterpret_cast<uint4*>(tkh + i * LDK + c8) = ok;
      *reinterpret_cast<uint4*>(tb + i * LDK + c8) = ob;
    }
    __syncthreads();  // factored tiles and dA (Xm) complete
    float db0 = 0.f, db1 = 0.f;
    const int i0 = r0 + g, i1 = r0 + g + 8;
    const bool cin0 = entering && run[i0] == 0, cin1 = entering && run[i1] == 0;
    const bool tl0 = i0 < m.len && run[i0] == run_last, tl1 = i1 < m.len && run[i1] == run_last;
    const float b0 = betas[i0], b1 = betas[i1];
    const int kc0 = 32 * cq;  // this warp's 32 key channels
    float accU[4][4], accQ[4][4], accW[4][4];
    zero_acc(accU);
    zero_acc(accQ);
    zero_acc(accW);
    // The three fp32 state-side gradient tiles come from global memory in fragment order: the values of the first two
    // column tiles are requested before the products (which hide their latency), those of the other two while the
    // first two are folded.
    float2 sgq[2][2], sgk[2][2], sgu[2][2];  // [nt & 1][hi]
    auto request = [&](int nt) {
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int off = (hi ? i1 : i0) * KD + kc0 + nt * 8 + 2 * t;
        sgq[nt & 1][hi] = *reinterpret_cast<const float2*>(dqs + off);
        sgk[nt & 1][hi] = *reinterpret_cast<const float2*>(dks + off);
        sgu[nt & 1][hi] = *reinterpret_cast<const float2*>(dku + off);
      }
    };
    request(0);
    warp_gemm<T, 4, 4, A_ROW, B_KN>(accU, Xm + r0 * LDC, LDC, tb + kc0, LDK, lane);   // dA k~
    warp_gemm<T, 4, 4, A_ROW, B_KN>(accQ, Xp + r0 * LDC, LDC, tb + kc0, LDK, lane);   // dP k~
    warp_gemm<T, 4, 4, A_COL, B_KN>(accW, Xp + r0, LDC, tqh + kc0, LDK, lane);        // dP^T q^
    warp_gemm<T, 4, 4, A_COL, B_KN>(accW, Xm + r0, LDC, tkh + kc0, LDK, lane);        // + dA^T (beta k^)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float colsum[2] = {0.f, 0.f};
      const float eR[2] = {__expf(0.5f * Glast[kc0 + nt * 8 + 2 * t]), __expf(0.5f * Glast[kc0 + nt * 8 + 2 * t + 1])};
      if (nt + 1 < 4) request(nt + 1);  // into the other half of the buffers
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        const int i = hi ? i1 : i0, col = kc0 + nt * 8 + 2 * t;
        const bool cin = hi ? cin1 : cin0, tail = hi ? tl1 : tl0;
        const float2 qs2 = sgq[nt & 1][hi], ks2 = sgk[nt & 1][hi], ku2 = sgu[nt & 1][hi];
        const float2 qr2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tq + i * LDK + col));
        const float2 kr2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tr + i * LDK + col));  // read key
        const float2 kw2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tk + i * LDK + col));  // write key
        const float2 kh2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tkh + i * LDK + col));  // beta k^
        const float2 qh2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tqh + i * LDK + col));  // q^
        const float2 kt2 = unpack2<T>(*reinterpret_cast<const uint32_t*>(tb + i * LDK + col));   // k~
        float dqv[2], dkv[2], dkrv[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int e = 2 * hi + x;
          const float Gi = Gm[i * KD + col + x], Gl = Glast[col + x];
          const float d = Gi - 0.5f * Gl;
          const float eu = __expf(d), en = __expf(-d);
          // exp(G_i) = exp(d) exp(R) and exp(G_63 - G_i) = exp(-d) exp(R) with R = G_63 / 2 (|R| <= 30 on this path)
          const float eg = cin ? eu * eR[x] : 0.f, ew = tail ? en * eR[x] : 0.f;
          const float khb = x ? kh2.y : kh2.x, qh = x ? qh2.y : qh2.x, kt = x ? kt2.y : kt2.x;
          const float qr = x ? qr2.y : qr2.x, kr = x ? kr2.y : kr2.x, kwr = x ? kw2.y : kw2.x;
          if (hi) db1 += kr * eu * accU[nt][e]; else db0 += kr * eu * accU[nt][e];  // dbeta_i += k^_i . (dA k~)_i
          const float dqs_e = (x ? qs2.y : qs2.x) * eg, dks_e = (x ? ks2.y : ks2.x) * eg;
          const float dq = accQ[nt][e] * eu + dqs_e;
          const float dkr = (hi ? b1 : b0) * accU[nt][e] * eu + dks_e;
          const float kuw = (x ? ku2.y : ku2.x) * ew;
          const float dkw = accW[nt][e] * en + kuw;
          // the pair terms from the rounded operands themselves (see the file header), the state terms in fp32
          dGt[i * KD + col + x] = (qh * accQ[nt][e] + khb * accU[nt][e] - kt * accW[nt][e]) +
                                  (qr * dqs_e + kr * dks_e - kwr * kuw);
          colsum[x] += kwr * kuw;
          dqv[x] = dq;
          dkv[x] = RK ? dkw : dkr + dkw;
          dkrv[x] = dkr;
        }
        if (i < m.len) {
          if (dq16) {
            *reinterpret_cast<uint32_t*>(dq16 + (long)i * kstride + col) = pack2<T>(dqv[0], dqv[1]);
            *reinterpret_cast<uint32_t*>(dk16 + (long)i * kstride + col) = pack2<T>(dkv[0], dkv[1]);
          } else {
            *reinterpret_cast<float2*>(p.dq_acc + tokbase + i * tstride + col) = make_float2(dqv[0], dqv[1]);
            *reinterpret_cast<float2*>(p.dk_acc + tokbase + i * tstride + col) = make_float2(dkv[0], dkv[1]);
          }
          if (RK) *reinterpret_cast<uint32_t*>(dkr16 + (long)i * tstride + col) = pack2<T>(dkrv[0], dkrv[1]);
        }
      }
      const float a = col_reduce(colsum[0]), b = col_reduce(colsum[1]);
      if (lane < 4) {
        part[rw * KD + kc0 + nt * 8 + 2 * lane] = a;
        part[rw * KD + kc0 + nt * 8 + 2 * lane + 1] = b;
      }
    }
    db0 += __shfl_xor_sync(0xffffffffu, db0, 1);
    db0 += __shfl_xor_sync(0xffffffffu, db0, 2);
    db1 += __shfl_xor_sync(0xffffffffu, db1, 1);
    db1 += __shfl_xor_sync(0xffffffffu, db1, 2);
    if (t == 0) {
      dbrow[cq * 64 + i0] = db0;
      dbrow[cq * 64 + i1] = db1;
    }
  } else {
    // ---- exact path: thread = key channel (threads 0..127), fp32 with the true exponent of every pair of one
    // document. The write-side dk accumulates in dGt[j][ch]; q dq + k dk_read and dk_read are parked in the factored
    // tiles, which this path does not build.
    __syncthreads();  // dA (Xm) complete
    const int ch = tid & (KD - 1);
    const bool active = tid < KD;
    float* keep = reinterpret_cast<float*>(tqh);  // [64][KD] fp32 over tqh | tkh
    if (active) {
      for (int i = 0; i < 64; ++i) dGt[i * KD + ch] = 0.f;
      for (int i = 0; i < 64; ++i) {
        const float Gi = Gm[i * KD + ch];
        const float qi = to_f32(tq[i * LDK + ch]), ki = to_f32(tr[i * LDK + ch]);  // ki: the read key of token i
        float dq = 0.f, u = 0.f;
        for (int j = 0; j <= i; ++j) {
          if (run[j] != run[i]) continue;
          const float e = __expf(Gi - Gm[j * KD + ch]);
          const float kj = to_f32(tk[j * LDK + ch]) * e;
          // beta_i dA_ij from the same rounded dA that the row direction sums (u below): the two copies of a pair's
          // term in dG must agree to fp32 rounding (see the file header)
          const float dp = to_f32(Xp[i * LDC + j]), da = to_f32(Xm[i * LDC + j]), dakk = betas[i] * da;
          dq += dp * kj;
          u += da * kj;
          dGt[j * KD + ch] += (dp * qi + dakk * ki) * e;
        }
        float x = ki * u;  // dbeta_i += sum over channels of k_i u_i
        for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
        if (lane == 0) part[warp * KD + i] = x;
        const bool cin = entering && run[i] == 0;
        const float eg = cin ? __expf(Gi) : 0.f;
        const float dqf = dq + dqs[i * KD + ch] * eg;
        const float dkr = betas[i] * u + dks[i * KD + ch] * eg;
        if (i < m.len) {
          if (dq16) dq16[(long)i * kstride + ch] = from_f32<T>(dqf);
          else p.dq_acc[tokbase + i * tstride + ch] = dqf;
        }
        keep[i * KD + ch] = qi * dqf + ki * dkr;
        tb[i * LDK + ch] = from_f32<T>(dkr);  // the read-side dk waits here for the write side (tb is unused on this path)
      }
    }
    __syncthreads();
    if (tid < 64) {
      dbrow[tid] = part[tid] + part[KD + tid] + part[2 * KD + tid] + part[3 * KD + tid];
      dbrow[64 + tid] = dbrow[128 + tid] = dbrow[192 + tid] = 0.f;
    }
    float colsum = 0.f;
    if (active) {
      for (int i = 0; i < 64; ++i) {
        const float Gi = Gm[i * KD + ch];
        const bool tail = i < m.len && run[i] == run_last;
        const float ki = to_f32(tk[i * LDK + ch]);
        const float kuw = dku[i * KD + ch] * (tail ? __expf(Glast[ch] - Gi) : 0.f);
        const float dkw = dGt[i * KD + ch] + kuw;
        dGt[i * KD + ch] = keep[i * KD + ch] - ki * dkw;
        colsum += ki * kuw;
        if (i < m.len) {
          const float dk = RK ? dkw : to_f32(tb[i * LDK + ch]) + dkw;
          if (dk16) dk16[(long)i * kstride + ch] = from_f32<T>(dk);
          else p.dk_acc[tokbase + i * tstride + ch] = dk;
          if (RK) dkr16[(long)i * tstride + ch] = tb[i * LDK + ch];
        }
      }
    }
    __syncthreads();  // part[] has been read
    if (active) {
      part[ch] = colsum;
      part[KD + ch] = part[2 * KD + ch] = part[3 * KD + ch] = 0.f;
    }
  }
  __syncthreads();

  // ---- dg: suffix sums over the chunk's tokens plus the terms that act through G_63; dbeta. Four threads per
  // channel, 16 tokens each: the segment sums go through part[] (whose column sums are read first), then every
  // thread walks its own 16 tokens from the sum of everything behind them.
  {
    const int ch = tid & (KD - 1), seg = tid >> 7;
    const float keep_d = (entering && run_last == 0) ? __expf(Glast[ch]) : 0.f;
    float acc = part[ch] + part[KD + ch] + part[2 * KD + ch] + part[3 * KD + ch] + keep_d * p.dd[slot * KD + ch];
    float own = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) own += dGt[(16 * seg + i) * KD + ch];
    __syncthreads();  // part[] has been read by every thread
    part[seg * KD + ch] = own;
    __syncthreads();
    for (int sg = seg + 1; sg < 4; ++sg) acc += part[sg * KD + ch];
#pragma unroll 4
    for (int i = 16 * seg + 15; i >= 16 * seg; --i) {
      acc += dGt[i * KD + ch];
      if (i < m.len) p.dg[tokbase + i * tstride + ch] = acc;
    }
    if (tid < m.len) {
      p.dbeta[(long)(m.tok0 + tid) * p.H + h] =
          dbrow[tid] + dbrow[64 + tid] + dbrow[128 + tid] + dbrow[192 + tid] + dbcol[tid];
    }
  }
}

template <typename T>
int launch_grads(const KdaGradParams& gp, int blocks, cudaStream_t s) {
  const size_t smem_a = (2 * 64 * (VD + 8) + 2 * VD * (KD + 8) + 3 * VD * 72) * sizeof(T) + 2 * KD * sizeof(float);
  const size_t smem_b = ((gp.k_read ? 6 : 5) * 64 * (KD + 8) + 4 * 64 * 72) * sizeof(T) +
                        (2 * 64 * KD + 4 * KD + 64 + KD + 256 + 64) * sizeof(float) + 64 * sizeof(int);
  auto* ka = kda_state_grads_kernel<T>;
  auto* kb = gp.k_read ? kda_intra_grads_kernel<T, true> : kda_intra_grads_kernel<T, false>;
  JLA_CUDA_OK(cudaFuncSetAttribute(ka, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a));
  JLA_CUDA_OK(cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b));
  {
    ProfScope ps(kProfKdaChunkGrads, s);
    ka<<<blocks, 256, smem_a, s>>>(gp);
  }
  JLA_LAUNCH_OK();
  {
    ProfScope ps(kProfKdaIntra, s);
    kb<<<blocks, 512, smem_b, s>>>(gp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

int launch_kda_grads(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.nc == 0) return JLA_OK;  // no tokens: nothing to differentiate through
  if ((p.dtype != JLA_DTYPE_BF16 && p.dtype != JLA_DTYPE_F16) || p.K != KD || p.V != VD) {
    set_error("chunked KDA backward: bf16 or f16 tensors with K = V = 128 only");
    return JLA_ERR_UNSUPPORTED;
  }
  KdaGradParams gp{};
  gp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  gp.q = c.q_eff;
  gp.k = c.k_eff;
  gp.k_read = p.k_read;
  gp.dk_read = io.dk_read;
  gp.g = p.g;
  gp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  gp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  gp.d_o = io.d_o;
  gp.dw = io.dv;
  gp.hT = c.res + pl.h;
  gp.dhT = scratch + pl.dh;
  gp.vnT = c.res + pl.vn;
  gp.dvnT = scratch + pl.dvn;
  gp.wT = c.res + pl.w;
  gp.t0 = c.res + pl.t0;
  gp.dp = scratch + pl.dp;
  gp.dag = scratch + pl.kda_dag;
  gp.dqs = reinterpret_cast<float*>(scratch + pl.kda_dqs);
  gp.dks = reinterpret_cast<float*>(scratch + pl.kda_dks);
  gp.dku = reinterpret_cast<float*>(scratch + pl.kda_dku);
  gp.dd = reinterpret_cast<float*>(scratch + pl.kda_dd);
  const bool direct = p.H == p.Hk && !pl.l2norm;
  gp.dq_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dq_acc);
  gp.dk_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dk_acc);
  gp.dq = direct ? io.dq : nullptr;
  gp.dk = direct ? io.dk : nullptr;
  gp.dg = io.dg;
  gp.dbeta = io.dbeta;
  gp.H = p.H;
  gp.Hk = p.Hk;
  gp.scale = p.scale;
  return p.dtype == JLA_DTYPE_BF16 ? launch_grads<__nv_bfloat16>(gp, pl.nc * p.H, s)
                                   : launch_grads<__half>(gp, pl.nc * p.H, s);
}

}  // namespace jla
