// Backward of the scalar-gate family, chunk-64: a reverse serial pass per (row, head) that carries dS in fp32
// registers and emits dv, dVn and the per-chunk dS+, then a chunk-parallel kernel for dq, dk, dbeta, dg.
//
//   dVn = scale P^T dO + (tail Gamma_r)(K dS+)       dW = Ag^T dVn = dV
//   dS  = keep gamma dS+ + scale ((cin Gamma) Q)^T dO - ((cin Gamma) K)^T dW
//   dP  = scale (dO Vn^T) D      dQ = scale (cin Gamma)(dO S^T) + dP K
//   dAg = tril(dVn W^T)   dT0 = dAg D beta_j   dA0 = -strict(T0^T dT0 T0^T) same
//   dK  = (tail Gamma_r)(Vn dS+^T) - (cin Gamma)(dW S^T) + dP^T Q + (dA0 beta_i) K + (dA0 beta_i)^T K
// and the gate / beta gradients as row and column sums of the same tiles (the reference's split backward:
// src/jla/ops/mosaic_gpu/gated_delta_rule_bwd.py:303-853; here column sums are shuffle reductions instead of
// second, transposed products).
#include <stdlib.h>

#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"

namespace jla {
namespace {

struct BwdParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;
  const unsigned char* runs;
  const void *q, *k, *v, *t0, *d_o, *h, *vn;
  const float* d_final;
  const float* qk_tab;  // Q K^T and K Q^T per (chunk, key head) in fragment order (qk_table_kernel), or nullptr
  void *dh, *dvn, *dv;
  float* dh0;
  void *dq, *dk;          // tensor dtype, written directly when dq_acc == nullptr
  float *dq_acc, *dk_acc;  // [tokens, H, K] f32 otherwise
  float *dg, *dbeta;
  int H, Hk;
  float scale;
};

// ---------------------------------------------------------------------------------------------------------
// reverse serial pass
template <typename T, int K, int V, bool DELTA>
struct BwdStateSmem {
  static constexpr int LDK = K + 8, LDV = V + 8, LDC = 72;
  static constexpr int kStageElems = 2 * 64 * LDK + 64 * LDV + (DELTA ? 64 * LDC : 0);
  static constexpr int kStageBytes = kStageElems * 2 + 512 + 64;
  // Without the delta rule only the 16-bit dS+ copy lives outside the stages: dv goes to global memory from the
  // accumulators and the scale (cin Gamma) factor of the dS update is applied to the query fragments in registers.
  static constexpr int kBytes = 2 * kStageBytes + (K * LDV + (DELTA ? 3 * 64 * LDV + 64 * LDC : 0)) * 2;
};

// (Two CTAs per SM for the Mamba-2 shape, as in the forward pass: 108 KB of shared memory and <= 128 registers each.)
template <typename T, int K, int V, bool DELTA>
__global__ void __launch_bounds__(256, (!DELTA && V == 64) ? 2 : 1) sg_bwd_state_kernel(BwdParams p) {
  using L = BwdStateSmem<T, K, V, DELTA>;
  constexpr int LDK = L::LDK, LDV = L::LDV, LDC = L::LDC;
  constexpr int WR = K / 16, WC = 8 / WR, SNT = V / 8 / WC, ONT = V / 16;
  const int row = blockIdx.x / p.H, h = blockIdx.x - row * p.H;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), c0 = (V / 2) * (warp >> 2);
  const int sr0 = 16 * (warp % WR), sc0 = (V / WC) * (warp / WR);
  const int2 rc = p.row_chunks[row];

  extern __shared__ __align__(16) unsigned char smem_raw[];
  auto stage_q = [&](int s) { return reinterpret_cast<T*>(smem_raw + s * L::kStageBytes); };
  auto stage_k = [&](int s) { return stage_q(s) + 64 * LDK; };
  auto stage_do = [&](int s) { return stage_k(s) + 64 * LDK; };
  auto stage_t0 = [&](int s) { return stage_do(s) + 64 * LDV; };
  auto stage_g = [&](int s) { return reinterpret_cast<float*>(smem_raw + s * L::kStageBytes + L::kStageElems * 2); };
  auto stage_runs = [&](int s) { return reinterpret_cast<unsigned char*>(stage_g(s) + 128); };
  T* dSb = reinterpret_cast<T*>(smem_raw + 2 * L::kStageBytes);
  T* dVnb = dSb + K * LDV;
  T* dOs = dVnb + 64 * LDV;
  T* dWs = dOs + 64 * LDV;                       // DELTA only
  T* AgT = dWs + 64 * LDV;                       // DELTA only

  auto issue_load = [&](int ci, int s) {
    const int c = rc.x + ci;
    const ChunkMeta m = p.meta[c];
    const T* q = static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * K;
    const T* k = static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * K;
    const T* d_o = static_cast<const T*>(p.d_o) + ((long)m.tok0 * p.H + h) * V;
    load_tile_async<T, 64, K>(stage_q(s), LDK, q, (long)p.Hk * K, m.len, tid, 256);
    load_tile_async<T, 64, K>(stage_k(s), LDK, k, (long)p.Hk * K, m.len, tid, 256);
    load_tile_async<T, 64, V>(stage_do(s), LDV, d_o, (long)p.H * V, m.len, tid, 256);
    if (DELTA) {
      load_tile_async<T, 64, 64>(stage_t0(s), LDC, static_cast<const T*>(p.t0) + ((long)c * p.H + h) * 4096, 64, 64,
                                 tid, 256);
    }
    if (tid < 32) cp_async16(stage_g(s) + tid * 4, p.gates + ((long)c * p.H + h) * 128 + tid * 4);
    if (tid >= 32 && tid < 36) cp_async16(stage_runs(s) + (tid - 32) * 16, p.runs + (long)c * 64 + (tid - 32) * 16);
    cp_async_commit();
  };

  float accD[SNT][4];
  {
    const float* df = p.d_final ? p.d_final + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float2 x = make_float2(0.f, 0.f);
        if (df) x = *reinterpret_cast<const float2*>(df + (long)(sr0 + g + 8 * hh) * V + sc0 + nt * 8 + 2 * t);
        accD[nt][2 * hh] = x.x;
        accD[nt][2 * hh + 1] = x.y;
      }
    }
    store_acc<T, SNT>(dSb, LDV, sr0, sc0, accD, lane);
  }
  if (rc.y > 0) issue_load(rc.y - 1, 0);

  for (int it = 0; it < rc.y; ++it) {
    const int ci = rc.y - 1 - it;
    const int s = it & 1;
    const int c = rc.x + ci;
    cp_async_wait<0>();
    __syncthreads();  // S0
    if (ci > 0) issue_load(ci - 1, s ^ 1);
    const ChunkMeta m = p.meta[c];
    const T* qS = stage_q(s);
    const T* kS = stage_k(s);
    const T* doS = stage_do(s);
    const float* Gs = stage_g(s);
    const float* betas = Gs + 64;
    const unsigned char* runs = stage_runs(s);
    const RowScalars rs0 = row_scalars(Gs, runs, m.flags, r0 + g);
    const RowScalars rs1 = row_scalars(Gs, runs, m.flags, r0 + g + 8);

    store_tile<T, V>(static_cast<T*>(p.dh) + ((long)c * p.H + h) * K * V, V, dSb, LDV, K, tid, 256);
    if (!DELTA) {
      // scale (cin Gamma) per token for the dS update, kept in the (unused) beta half of the gate vectors and
      // applied to the query fragments (ordered before its readers by Sa)
      if (tid < 64) stage_g(s)[64 + tid] = p.scale * row_scalars(Gs, runs, m.flags, tid).gam;
    } else {  // dOs = scale (cin Gamma) dO; AgT[j][i] = Ag_ij
      const int i = tid >> 2, j0 = (tid & 3) * (V / 4);
      const float sg = p.scale * row_scalars(Gs, runs, m.flags, i).gam;
#pragma unroll
      for (int jj = 0; jj < V / 4; jj += 2) {
        const float2 x = unpack2<T>(*reinterpret_cast<const uint32_t*>(doS + i * LDV + j0 + jj));
        *reinterpret_cast<uint32_t*>(dOs + i * LDV + j0 + jj) = pack2<T>(x.x * sg, x.y * sg);
      }
      {
        const T* t0S = stage_t0(s);
        const int c16 = (tid & 3) * 16;
        const float Gi = Gs[i];
        const int runi = runs[i];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          const int j = c16 + jj;
          const float a = to_f32(t0S[i * LDC + j]) * decay_ij(Gs, runs, i, j, Gi, runi) * betas[j];
          AgT[j * LDC + i] = from_f32<T>(a);
        }
      }
    }
    // Pt[j][i] = scale (k_j . q_i) D_ij for this warp's 16 rows j and all 64 columns i
    uint32_t pfrag[4][4];
    {
      float accP[8][4];
      if (p.qk_tab) {  // K Q^T is shared by the value heads of the key head: this warp's fragments from the table
        const float4* src = reinterpret_cast<const float4*>(p.qk_tab + ((long)c * p.Hk + hk) * kQkTabFloats + 4096) +
                            (warp & 3) * 8 * 32 + lane;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const float4 x = __ldg(src + nt * 32);
          accP[nt][0] = x.x, accP[nt][1] = x.y, accP[nt][2] = x.z, accP[nt][3] = x.w;
        }
      } else {
        zero_acc(accP);
        warp_gemm<T, 8, K / 16, A_ROW, B_NK>(accP, kS + r0 * LDK, LDK, qS, LDK, lane);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = r0 + g + ((e >> 1) << 3), i = nt * 8 + 2 * t + (e & 1);
          accP[nt][e] *= p.scale * decay_ij(Gs, runs, i, j, Gs[i], runs[i]);
        }
      }
      acc_to_afrag<T, 4>(pfrag, accP);
    }
    // dVn = (tail Gamma_r)(K dS+) + scale P^T dO
    float acc[ONT][4];
    zero_acc(acc);
    warp_gemm<T, ONT, K / 16, A_ROW, B_KN>(acc, kS + r0 * LDK, LDK, dSb + c0, LDV, lane);
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt) {
      acc[nt][0] *= rs0.gamr;
      acc[nt][1] *= rs0.gamr;
      acc[nt][2] *= rs1.gamr;
      acc[nt][3] *= rs1.gamr;
    }
    warp_gemm_ra<T, ONT, 4, B_KN>(acc, pfrag, doS + c0, LDV, lane);
    T* dv = static_cast<T*>(p.dv) + ((long)m.tok0 * p.H + h) * V;
    if (DELTA) {
      store_acc<T, ONT>(dVnb, LDV, r0, c0, acc, lane);
    } else {  // dV = dVn, straight from the accumulators
#pragma unroll
      for (int nt = 0; nt < ONT; ++nt) {
        const int col = c0 + nt * 8 + 2 * t;
        if (r0 + g < m.len)
          *reinterpret_cast<uint32_t*>(dv + (long)(r0 + g) * p.H * V + col) = pack2<T>(acc[nt][0], acc[nt][1]);
        if (r0 + g + 8 < m.len)
          *reinterpret_cast<uint32_t*>(dv + (long)(r0 + g + 8) * p.H * V + col) = pack2<T>(acc[nt][2], acc[nt][3]);
      }
    }
    __syncthreads();  // Sa: dVnb, dOs, AgT complete; every warp is done reading dSb
    if (DELTA) {
      store_tile<T, V>(static_cast<T*>(p.dvn) + ((long)c * p.H + h) * 64 * V, V, dVnb, LDV, 64, tid, 256);
      zero_acc(acc);
      warp_gemm<T, ONT, 4, A_ROW, B_KN>(acc, AgT + r0 * LDC, LDC, dVnb + c0, LDV, lane);  // dW = Ag^T dVn
#pragma unroll
      for (int nt = 0; nt < ONT; ++nt) {
        const int col = c0 + nt * 8 + 2 * t;
        if (r0 + g < m.len)
          *reinterpret_cast<uint32_t*>(dv + (long)(r0 + g) * p.H * V + col) = pack2<T>(acc[nt][0], acc[nt][1]);
        if (r0 + g + 8 < m.len)
          *reinterpret_cast<uint32_t*>(dv + (long)(r0 + g + 8) * p.H * V + col) = pack2<T>(acc[nt][2], acc[nt][3]);
      }
      store_acc<T, ONT>(dWs, LDV, r0, c0, acc, lane, -rs0.gam, -rs1.gam);
      __syncthreads();  // Sb: dWs complete
    }
    // dS = keep gamma dS+ + Q^T (scale cin Gamma dO) - K^T (cin Gamma dW)
    const float kg = keep_gamma(Gs, runs, m.flags);
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
      accD[nt][0] *= kg;
      accD[nt][1] *= kg;
      accD[nt][2] *= kg;
      accD[nt][3] *= kg;
    }
    if (DELTA) {
      warp_gemm<T, SNT, 4, A_COL, B_KN>(accD, qS + sr0, LDK, dOs + sc0, LDV, lane);
      warp_gemm<T, SNT, 4, A_COL, B_KN>(accD, kS + sr0, LDK, dWs + sc0, LDV, lane);
    } else {
      warp_gemm_scaled_a<T, SNT, 4, B_KN>(accD, qS + sr0, LDK, betas, doS + sc0, LDV, lane);
    }
    store_acc<T, SNT>(dSb, LDV, sr0, sc0, accD, lane);
  }

  if (p.dh0) {
    float* f = p.dh0 + ((long)row * p.H + h) * K * V;
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
      *reinterpret_cast<float2*>(f + (long)(sr0 + g) * V + sc0 + nt * 8 + 2 * t) = make_float2(accD[nt][0], accD[nt][1]);
      *reinterpret_cast<float2*>(f + (long)(sr0 + g + 8) * V + sc0 + nt * 8 + 2 * t) =
          make_float2(accD[nt][2], accD[nt][3]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// chunk-parallel gradients

// Reductions avoid shared-memory float atomics (a compare-and-swap loop): every warp adds into slots that only it
// writes (row sums: one slot array per column half; column sums: one per row quadrant), always from the same lane,
// and the slots are summed once at the end.
// vec[row] += sign * sum over this thread's columns, reduced over the 4 lanes of a quad.
template <int NT>
__device__ __forceinline__ void row_sums_add(const float (&x)[NT][4], float* vec, int r0, int lane, float sign) {
  float a = 0.f, b = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    a += x[nt][0] + x[nt][1];
    b += x[nt][2] + x[nt][3];
  }
  a += __shfl_xor_sync(0xffffffffu, a, 1);
  a += __shfl_xor_sync(0xffffffffu, a, 2);
  b += __shfl_xor_sync(0xffffffffu, b, 1);
  b += __shfl_xor_sync(0xffffffffu, b, 2);
  if ((lane & 3) == 0) {
    vec[r0 + (lane >> 2)] += sign * a;
    vec[r0 + (lane >> 2) + 8] += sign * b;
  }
}

// vec[c0 + col] += sign * sum over the warp's 16 rows.
template <int NT>
__device__ __forceinline__ void col_sums_add(const float (&x)[NT][4], float* vec, int c0, int lane, float sign) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float a = x[nt][0] + x[nt][2], b = x[nt][1] + x[nt][3];
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, off);
      b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    if (lane < 4) {
      vec[c0 + nt * 8 + 2 * lane] += sign * a;
      vec[c0 + nt * 8 + 2 * lane + 1] += sign * b;
    }
  }
}

// sum_k x[i][k] * tile[i][k] for the warp's rows (tile in smem, 16-bit), reduced over the quad.
template <typename T, int NT>
__device__ __forceinline__ void row_dots(const float (&x)[NT][4], const T* tile, int ld, int r0, int c0, int lane,
                                         float& d0, float& d1) {
  const int g = lane >> 2, t = lane & 3;
  d0 = 0.f;
  d1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(tile + (r0 + g) * ld + c0 + nt * 8 + 2 * t));
    const float2 b = unpack2<T>(*reinterpret_cast<const uint32_t*>(tile + (r0 + g + 8) * ld + c0 + nt * 8 + 2 * t));
    d0 += x[nt][0] * a.x + x[nt][1] * a.y;
    d1 += x[nt][2] * b.x + x[nt][3] * b.y;
  }
  d0 += __shfl_xor_sync(0xffffffffu, d0, 1);
  d0 += __shfl_xor_sync(0xffffffffu, d0, 2);
  d1 += __shfl_xor_sync(0xffffffffu, d1, 1);
  d1 += __shfl_xor_sync(0xffffffffu, d1, 2);
}

template <typename T, int K, int V, bool DELTA>
struct GradSmem {
  static constexpr int LDK = K + 8, LDV = V + 8, LDC = 72;
  // k | q | do (q and do contiguous: later reused for dS+) | v (W, then dW) | Vn | S | T0, Xa, Xb, Xc | vectors
  static constexpr int kElems = 2 * 64 * LDK + 2 * 64 * LDV + (DELTA ? 64 * LDV : 0) + K * LDV + 4 * 64 * LDC;
  static constexpr int kBytes = kElems * 2 + (128 + 13 * 64 + 16) * 4 + 64;
  static_assert(K * LDV <= 64 * LDK + 64 * LDV, "dS+ must fit in the q | do region");
};

// (Without the delta rule and with V = 64 -- the Mamba-2 shape -- two CTAs fit the shared memory of an SM; capping the
// registers at 128 lets them, and a second resident CTA hides the first one's load and barrier latencies.)
//
// NH > 1 (grouped key heads only): one CTA walks NH adjacent value heads of one key group for the same chunk and keeps
// their dq and dk sums in its accumulators, so the fp32 partials that finalize_key_grad sums over the group are
// [tokens, H / NH, K] instead of [tokens, H, K] (the reference sums the group inside its kernel as well,
// src/jla/ops/mosaic_gpu/scalar_gate_grouped.py:65-237). Everything else (dv, dg, the gate sums) stays per head.
template <typename T, int K, int V, bool DELTA, int NH>
__global__ void __launch_bounds__(256, (!DELTA && V == 64) ? 2 : 1) sg_chunk_grads_kernel(BwdParams p) {
  using L = GradSmem<T, K, V, DELTA>;
  constexpr int LDK = L::LDK, LDV = L::LDV, LDC = L::LDC;
  constexpr int ONT = V / 16, KNT = K / 16;
  const int hgs = p.H / NH;  // head groups of NH per chunk
  const int c = blockIdx.x / hgs, hg = blockIdx.x - c * hgs;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = (hg * NH) / (p.H / p.Hk);  // NH divides the group size: every head of the walk shares the key head
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), ch = warp >> 2;
  const int c0 = (V / 2) * ch, kc0 = (K / 2) * ch, cc0 = 32 * ch;

  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* kS = reinterpret_cast<T*>(smem_raw);
  T* qS = kS + 64 * LDK;
  T* doS = qS + 64 * LDK;             // dO, later dVn
  T* vS = doS + 64 * LDV;             // V -> W in place, later dW
  T* vnS = DELTA ? vS + 64 * LDV : vS;  // Vn (= V without the delta rule)
  T* SS = vnS + 64 * LDV;
  T* t0S = SS + K * LDV;
  T* Xa = t0S + 64 * LDC;
  T* Xb = Xa + 64 * LDC;
  T* Xc = Xb + 64 * LDC;
  float* Gs = reinterpret_cast<float*>(smem_raw + L::kElems * 2);
  float* betas = Gs + 64;
  float* dGrow = betas + 64;   // [2][64] row-wise dG terms per column half
  float* dGcol = dGrow + 128;  // [4][64] column-wise dG terms per row quadrant
  float* dbrow = dGcol + 256;  // [2][64]
  float* dbcol = dbrow + 128;  // [4][64]
  float* dGv = dbcol + 256;    // [64] folded dG
  float* tot = dGv + 64;       // [8] per warp
  float* sdot = tot + 8;       // [8] per warp
  unsigned char* runs = reinterpret_cast<unsigned char*>(sdot + 8);
  const int quad = warp & 3;
  T* dSS = qS;  // dS+ overlays q | do once both are dead
  float accK[KNT][4];  // dk, 16 rows x K/2 columns per warp; summed over the NH heads of the walk
  float accQ[KNT][4];  // dq likewise
  zero_acc(accK);
  zero_acc(accQ);

#pragma unroll 1
  for (int hi = 0; hi < NH; ++hi) {
  const int h = hg * NH + hi;
  float tot_part = 0.f;
  const long ch_off = (long)c * p.H + h;
  // group 0: k, S, v, T0, gates, runs
  load_tile_async<T, 64, K>(kS, LDK, static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * K, (long)p.Hk * K, m.len,
                            tid, 256);
  load_tile_async<T, K, V>(SS, LDV, static_cast<const T*>(p.h) + ch_off * K * V, V, K, tid, 256);
  load_tile_async<T, 64, V>(vS, LDV, static_cast<const T*>(p.v) + ((long)m.tok0 * p.H + h) * V, (long)p.H * V, m.len,
                            tid, 256);
  if (DELTA) load_tile_async<T, 64, 64>(t0S, LDC, static_cast<const T*>(p.t0) + ch_off * 4096, 64, 64, tid, 256);
  if (tid < 32) cp_async16(Gs + tid * 4, p.gates + ch_off * 128 + tid * 4);
  if (tid >= 32 && tid < 36) cp_async16(runs + (tid - 32) * 16, p.runs + (long)c * 64 + (tid - 32) * 16);
  cp_async_commit();
  // group 1: dO, Vn, q
  load_tile_async<T, 64, V>(doS, LDV, static_cast<const T*>(p.d_o) + ((long)m.tok0 * p.H + h) * V, (long)p.H * V,
                            m.len, tid, 256);
  if (DELTA) load_tile_async<T, 64, V>(vnS, LDV, static_cast<const T*>(p.vn) + ch_off * 64 * V, V, 64, tid, 256);
  load_tile_async<T, 64, K>(qS, LDK, static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * K, (long)p.Hk * K, m.len,
                            tid, 256);
  cp_async_commit();
  for (int idx = tid; idx < 12 * 64; idx += 256) dGrow[idx] = 0.f;
  cp_async_wait<1>();
  __syncthreads();

  const RowScalars rs0 = row_scalars(Gs, runs, m.flags, r0 + g);
  const RowScalars rs1 = row_scalars(Gs, runs, m.flags, r0 + g + 8);

  if (DELTA) {  // 1. W = V - (cin Gamma)(K S), in place over V
    float acc[ONT][4];
    zero_acc(acc);
    warp_gemm<T, ONT, K / 16, A_ROW, B_KN>(acc, kS + r0 * LDK, LDK, SS + c0, LDV, lane);
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt) {
      const int col = c0 + nt * 8 + 2 * t;
      uint32_t* w0 = reinterpret_cast<uint32_t*>(vS + (r0 + g) * LDV + col);
      uint32_t* w1 = reinterpret_cast<uint32_t*>(vS + (r0 + g + 8) * LDV + col);
      const float2 v0 = unpack2<T>(*w0), v1 = unpack2<T>(*w1);
      *w0 = pack2<T>(v0.x - rs0.gam * acc[nt][0], v0.y - rs0.gam * acc[nt][1]);
      *w1 = pack2<T>(v1.x - rs1.gam * acc[nt][2], v1.y - rs1.gam * acc[nt][3]);
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // S1

  {  // 2. dP = scale (dO Vn^T) D ; E = dP (Q K^T)
    float accP[4][4], accE[4][4];
    zero_acc(accP);
    zero_acc(accE);
    warp_gemm<T, 4, V / 16, A_ROW, B_NK>(accP, doS + r0 * LDV, LDV, vnS + cc0 * LDV, LDV, lane);
    if (p.qk_tab) {  // Q K^T of this warp's 16 rows x 32 columns from the table shared by the key head's value heads
      const float4* src = reinterpret_cast<const float4*>(p.qk_tab + ((long)c * p.Hk + hk) * kQkTabFloats) +
                          ((warp & 3) * 8 + 4 * ch) * 32 + lane;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float4 x = __ldg(src + nt * 32);
        accE[nt][0] = x.x, accE[nt][1] = x.y, accE[nt][2] = x.z, accE[nt][3] = x.w;
      }
    } else {
      warp_gemm<T, 4, K / 16, A_ROW, B_NK>(accE, qS + r0 * LDK, LDK, kS + cc0 * LDK, LDK, lane);
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int j = cc0 + nt * 8 + 2 * t;
      accP[nt][0] *= p.scale * decay_ij(Gs, runs, r0 + g, j, rs0.G, rs0.run);
      accP[nt][1] *= p.scale * decay_ij(Gs, runs, r0 + g, j + 1, rs0.G, rs0.run);
      accP[nt][2] *= p.scale * decay_ij(Gs, runs, r0 + g + 8, j, rs1.G, rs1.run);
      accP[nt][3] *= p.scale * decay_ij(Gs, runs, r0 + g + 8, j + 1, rs1.G, rs1.run);
#pragma unroll
      for (int e = 0; e < 4; ++e) accE[nt][e] *= accP[nt][e];
    }
    row_sums_add<4>(accE, dGrow + ch * 64, r0, lane, 1.f);
    col_sums_add<4>(accE, dGcol + quad * 64, cc0, lane, -1.f);
    store_acc<T, 4>(Xa, LDC, r0, cc0, accP, lane);
  }
  {  // 3. dq = scale (cin Gamma)(dO S^T) + dP K
    const float s0 = p.scale * rs0.gam, s1 = p.scale * rs1.gam;
    float d0, d1;
    if (NH == 1) {  // straight into the accumulator
      warp_gemm<T, KNT, V / 16, A_ROW, B_NK>(accQ, doS + r0 * LDV, LDV, SS + kc0 * LDV, LDV, lane);
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        accQ[nt][0] *= s0;
        accQ[nt][1] *= s0;
        accQ[nt][2] *= s1;
        accQ[nt][3] *= s1;
      }
      row_dots<T, KNT>(accQ, qS, LDK, r0, kc0, lane, d0, d1);
    } else {  // this head's term alone is needed for its gate gradient: through a temporary
      float accS[KNT][4];
      zero_acc(accS);
      warp_gemm<T, KNT, V / 16, A_ROW, B_NK>(accS, doS + r0 * LDV, LDV, SS + kc0 * LDV, LDV, lane);
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        accS[nt][0] *= s0;
        accS[nt][1] *= s0;
        accS[nt][2] *= s1;
        accS[nt][3] *= s1;
      }
      row_dots<T, KNT>(accS, qS, LDK, r0, kc0, lane, d0, d1);
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) accQ[nt][e] += accS[nt][e];
      }
    }
    if (t == 0) {
      dGrow[ch * 64 + r0 + g] += d0;
      dGrow[ch * 64 + r0 + g + 8] += d1;
    }
  }
  __syncthreads();  // S2: Xa = dP complete
  warp_gemm<T, KNT, 4, A_ROW, B_KN>(accQ, Xa + r0 * LDC, LDC, kS + kc0, LDK, lane);
  if (hi == NH - 1) {
    const long tok0 = (long)m.tok0 + r0 + g;
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (r0 + g + 8 * hh >= m.len) continue;
        const long tok = tok0 + 8 * hh;
        if (p.dq_acc) {
          *reinterpret_cast<float2*>(p.dq_acc + (tok * hgs + hg) * K + col) = make_float2(accQ[nt][2 * hh], accQ[nt][2 * hh + 1]);
        } else {
          *reinterpret_cast<uint32_t*>(static_cast<T*>(p.dq) + (tok * p.Hk + hk) * K + col) =
              pack2<T>(accQ[nt][2 * hh], accQ[nt][2 * hh + 1]);
        }
      }
    }
  }
  // 4. dk += dP^T Q
  warp_gemm<T, KNT, 4, A_COL, B_KN>(accK, Xa + r0, LDC, qS + kc0, LDK, lane);
  __syncthreads();  // S3: q, dO dead

  if (DELTA) {
    load_tile_async<T, 64, V>(doS, LDV, static_cast<const T*>(p.dvn) + ch_off * 64 * V, V, 64, tid, 256);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();  // S4: dVn landed (in the dO buffer)
    {  // 5. dAg = tril(dVn W^T); F = dAg Ag; dT0 = dAg D beta_j
      float accA[4][4], accF[4][4], accB[4][4];
      zero_acc(accA);
      warp_gemm<T, 4, V / 16, A_ROW, B_NK>(accA, doS + r0 * LDV, LDV, vS + cc0 * LDV, LDV, lane);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = r0 + g + ((e >> 1) << 3), j = cc0 + nt * 8 + 2 * t + (e & 1);
          const RowScalars& rs = (e >> 1) ? rs1 : rs0;
          const float d = decay_ij(Gs, runs, i, j, rs.G, rs.run);
          const float t0v = to_f32(t0S[i * LDC + j]);
          const float dag = accA[nt][e];
          accB[nt][e] = dag * t0v * d;          // -> dbeta_j (column sums)
          accF[nt][e] = accB[nt][e] * betas[j]; // dAg * Ag
          accA[nt][e] = dag * d * betas[j];     // dT0
        }
      }
      row_sums_add<4>(accF, dGrow + ch * 64, r0, lane, 1.f);
      col_sums_add<4>(accF, dGcol + quad * 64, cc0, lane, -1.f);
      col_sums_add<4>(accB, dbcol + quad * 64, cc0, lane, 1.f);
      store_acc<T, 4>(Xb, LDC, r0, cc0, accA, lane);
    }
    __syncthreads();  // S5: Xb = dT0 complete; W and dVn dead
    // prefetch dW (into the W buffer) and dS+ (over q | do)
    load_tile_async<T, 64, V>(vS, LDV, static_cast<const T*>(p.dv) + ((long)m.tok0 * p.H + h) * V, (long)p.H * V, m.len,
                              tid, 256);
    load_tile_async<T, K, V>(dSS, LDV, static_cast<const T*>(p.dh) + ch_off * K * V, V, K, tid, 256);
    cp_async_commit();
    {  // M1 = dT0 T0^T
      float accM[4][4];
      zero_acc(accM);
      warp_gemm<T, 4, 4, A_ROW, B_NK>(accM, Xb + r0 * LDC, LDC, t0S + cc0 * LDC, LDC, lane);
      store_acc<T, 4>(Xc, LDC, r0, cc0, accM, lane);
    }
    __syncthreads();  // S6: Xc = M1 complete, Xb free
    {  // dA0 = -strict(T0^T M1) same ; dbeta_i += sum_j dA0_ij (k_i . k_j)
      float accA0[4][4], accKK[4][4];
      zero_acc(accA0);
      zero_acc(accKK);
      warp_gemm<T, 4, 4, A_COL, B_KN>(accA0, t0S + r0, LDC, Xc + cc0, LDC, lane);
      warp_gemm<T, 4, K / 16, A_ROW, B_NK>(accKK, kS + r0 * LDK, LDK, kS + cc0 * LDK, LDK, lane);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = r0 + g + ((e >> 1) << 3), j = cc0 + nt * 8 + 2 * t + (e & 1);
          const float a = (j < i && runs[j] == runs[i]) ? -accA0[nt][e] : 0.f;
          accKK[nt][e] *= a;
          accA0[nt][e] = a * betas[i];
        }
      }
      row_sums_add<4>(accKK, dbrow + ch * 64, r0, lane, 1.f);
      store_acc<T, 4>(Xb, LDC, r0, cc0, accA0, lane);
    }
    __syncthreads();  // S7: Xb = dA0 beta_i complete
    warp_gemm<T, KNT, 4, A_ROW, B_KN>(accK, Xb + r0 * LDC, LDC, kS + kc0, LDK, lane);
    warp_gemm<T, KNT, 4, A_COL, B_KN>(accK, Xb + r0, LDC, kS + kc0, LDK, lane);
  } else {
    load_tile_async<T, K, V>(dSS, LDV, static_cast<const T*>(p.dh) + ch_off * K * V, V, K, tid, 256);
    cp_async_commit();
  }
  cp_async_wait<0>();
  __syncthreads();  // S8: dW, dS+ landed

  {  // 6. state terms of dk and dG
    float accT[KNT][4];
    float d0, d1;
    if (DELTA) {  // - (cin Gamma)(dW S^T)
      zero_acc(accT);
      warp_gemm<T, KNT, V / 16, A_ROW, B_NK>(accT, vS + r0 * LDV, LDV, SS + kc0 * LDV, LDV, lane);
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        accT[nt][0] *= rs0.gam;
        accT[nt][1] *= rs0.gam;
        accT[nt][2] *= rs1.gam;
        accT[nt][3] *= rs1.gam;
#pragma unroll
        for (int e = 0; e < 4; ++e) accK[nt][e] -= accT[nt][e];
      }
      row_dots<T, KNT>(accT, kS, LDK, r0, kc0, lane, d0, d1);
      if (t == 0) {
        dGrow[ch * 64 + r0 + g] -= d0;
        dGrow[ch * 64 + r0 + g + 8] -= d1;
      }
    }
    zero_acc(accT);  // (tail Gamma_r)(Vn dS+^T)
    warp_gemm<T, KNT, V / 16, A_ROW, B_NK>(accT, vnS + r0 * LDV, LDV, dSS + kc0 * LDV, LDV, lane);
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      accT[nt][0] *= rs0.gamr;
      accT[nt][1] *= rs0.gamr;
      accT[nt][2] *= rs1.gamr;
      accT[nt][3] *= rs1.gamr;
#pragma unroll
      for (int e = 0; e < 4; ++e) accK[nt][e] += accT[nt][e];
    }
    row_dots<T, KNT>(accT, kS, LDK, r0, kc0, lane, d0, d1);
    if (t == 0) {
      dGrow[ch * 64 + r0 + g] -= d0;
      dGrow[ch * 64 + r0 + g + 8] -= d1;
      tot_part += d0 + d1;
    }
    // keep gamma <S, dS+>
    float part = 0.f;
    for (int idx = tid; idx < K * (V / 2); idx += 256) {
      const int r = idx / (V / 2), cidx = (idx - r * (V / 2)) * 2;
      const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(SS + r * LDV + cidx));
      const float2 b = unpack2<T>(*reinterpret_cast<const uint32_t*>(dSS + r * LDV + cidx));
      part += a.x * b.x + a.y * b.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    if (lane == 0) sdot[warp] = part;
    // dk out
    const long tok0 = (long)m.tok0 + r0 + g;
#pragma unroll
    for (int nt = 0; nt < KNT && hi == NH - 1; ++nt) {
      const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (r0 + g + 8 * hh >= m.len) continue;
        const long tok = tok0 + 8 * hh;
        if (p.dk_acc) {
          *reinterpret_cast<float2*>(p.dk_acc + (tok * hgs + hg) * K + col) = make_float2(accK[nt][2 * hh], accK[nt][2 * hh + 1]);
        } else {
          *reinterpret_cast<uint32_t*>(static_cast<T*>(p.dk) + (tok * p.Hk + hk) * K + col) =
              pack2<T>(accK[nt][2 * hh], accK[nt][2 * hh + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) tot_part += __shfl_xor_sync(0xffffffffu, tot_part, off);
  if (lane == 0) tot[warp] = tot_part;
  __syncthreads();  // S9
  if (tid < 64) {
    float dG = dGrow[tid] + dGrow[64 + tid] + dGcol[tid] + dGcol[64 + tid] + dGcol[128 + tid] + dGcol[192 + tid];
    if (tid == 63) {
#pragma unroll
      for (int w = 0; w < 8; ++w) dG += tot[w];
    }
    dGv[tid] = dG;
  }
  __syncthreads();
  if (tid < 64) {  // 7. dg = reverse cumulative sum of dG over the chunk
    float acc = 0.f;
    for (int j = 63; j >= tid; --j) acc += dGv[j];
    // the keep gamma <S, dS+> term belongs to the chunk's last position, so it is part of every suffix sum
    float sd = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) sd += sdot[w];
    acc += keep_gamma(Gs, runs, m.flags) * sd;
    if (tid < m.len) {
      if (p.dg) p.dg[((long)m.tok0 + tid) * p.H + h] = acc;
      if (DELTA) {
        p.dbeta[((long)m.tok0 + tid) * p.H + h] =
            dbrow[tid] + dbrow[64 + tid] + dbcol[tid] + dbcol[64 + tid] + dbcol[128 + tid] + dbcol[192 + tid];
      }
    }
  }
  if (NH > 1) __syncthreads();  // the next head's loads overwrite the tiles and vectors read above
  }  // heads of the walk
}

template <typename T, int K, int V, bool DELTA>
int launch_one(const BwdParams& bp, int rows_blocks, int chunk_blocks, bool legacy_grads, int head_walk, cudaStream_t s) {
  {
    auto* kern = sg_bwd_state_kernel<T, K, V, DELTA>;
    constexpr int smem = BwdStateSmem<T, K, V, DELTA>::kBytes;
    JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    {
      ProfScope ps(kProfSgBwdState, s);
      kern<<<rows_blocks, 256, smem, s>>>(bp);
    }
    JLA_LAUNCH_OK();
  }
  if (legacy_grads) {
    constexpr int smem = GradSmem<T, K, V, DELTA>::kBytes;
    // the Mamba-2 shape with grouped heads: walks of 8, 4 or 2 heads per CTA (see the kernel)
    auto* kern = sg_chunk_grads_kernel<T, K, V, DELTA, 1>;
    if (!DELTA && V == 64 && K == 128 && head_walk == 8) kern = sg_chunk_grads_kernel<T, K, V, DELTA, (!DELTA && V == 64 && K == 128) ? 8 : 1>;
    if (!DELTA && V == 64 && K == 128 && head_walk == 4) kern = sg_chunk_grads_kernel<T, K, V, DELTA, (!DELTA && V == 64 && K == 128) ? 4 : 1>;
    if (!DELTA && V == 64 && K == 128 && head_walk == 2) kern = sg_chunk_grads_kernel<T, K, V, DELTA, (!DELTA && V == 64 && K == 128) ? 2 : 1>;
    JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    {
      ProfScope ps(kProfSgChunkGrads, s);
      kern<<<chunk_blocks / head_walk, 256, smem, s>>>(bp);
    }
    JLA_LAUNCH_OK();
  }
  return JLA_OK;
}

template <typename T, bool DELTA>
int launch_kv(const BwdParams& bp, int K, int V, int rb, int cb, bool legacy, int walk, cudaStream_t s) {
  if (K == 128 && V == 128) return launch_one<T, 128, 128, DELTA>(bp, rb, cb, legacy, walk, s);
  if (K == 128 && V == 64) return launch_one<T, 128, 64, DELTA>(bp, rb, cb, legacy, walk, s);
  if (K == 64 && V == 128) return launch_one<T, 64, 128, DELTA>(bp, rb, cb, legacy, walk, s);
  return launch_one<T, 64, 64, DELTA>(bp, rb, cb, legacy, walk, s);
}

}  // namespace

int launch_sg_bwd(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  const long tokens = (long)p.B * p.T;
  if (pl.rows == 0) return JLA_OK;
  const bool kda = p.kind == JLA_KIND_KDA;
  const bool direct = p.H == p.Hk && !pl.l2norm;
  BwdParams bp{};
  bp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  bp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  bp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  bp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  bp.q = c.q_eff;
  bp.k = c.k_eff;
  bp.v = p.v;
  bp.t0 = c.res + pl.t0;
  bp.d_o = io.d_o;
  bp.h = c.res + pl.h;
  bp.vn = c.res + pl.vn;
  bp.d_final = io.d_final;
  bp.qk_tab = shares_scores(p) ? reinterpret_cast<const float*>(c.res + pl.qk_tab) : nullptr;
  bp.dh = scratch + pl.dh;
  bp.dvn = scratch + pl.dvn;
  bp.dv = io.dv;
  bp.dh0 = io.dh0;
  bp.dq = io.dq;
  bp.dk = io.dk;
  bp.dq_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dq_acc);
  bp.dk_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dk_acc);
  bp.dg = io.dg;
  bp.dbeta = io.dbeta;
  bp.H = p.H;
  bp.Hk = p.Hk;
  bp.scale = p.scale;
  const int rb = pl.rows * p.H, cb = pl.nc * p.H;
  const bool legacy = !use_tc_kernels(p);  // mma.sync chunk gradients (row-major residuals)
  // heads per CTA walk of the legacy gradient kernel (sums dq, dk over them in registers): the Mamba-2 shape with
  // grouped key heads only
  const int group = p.H / p.Hk;
  const int walk = (legacy && !direct && !pl.delta && p.K == 128 && p.V == 64) ? (group % 8 == 0 ? 8 : group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1) : 1;
  int rc;
  if (!legacy) {
    rc = launch_sg_bwd_state_tc(c, io, scratch, s);
  } else if (p.dtype == JLA_DTYPE_BF16) {
    rc = pl.delta ? launch_kv<__nv_bfloat16, true>(bp, p.K, p.V, rb, cb, legacy, walk, s)
                  : launch_kv<__nv_bfloat16, false>(bp, p.K, p.V, rb, cb, legacy, walk, s);
  } else {
    rc = pl.delta ? launch_kv<__half, true>(bp, p.K, p.V, rb, cb, legacy, walk, s)
                  : launch_kv<__half, false>(bp, p.K, p.V, rb, cb, legacy, walk, s);
  }
  if (rc == JLA_OK && !legacy && (p.flags & JLA_FLAG_STATE_GRADS_ONLY)) return rc;
  if (rc == JLA_OK && !legacy) rc = kda ? launch_kda_grads(c, io, scratch, s) : launch_chunk_grads_tc(c, io, scratch, direct, s);
  if (rc != JLA_OK || direct) return rc;
  rc = finalize_key_grad(bp.dq_acc, p.q, io.dq, p.dtype, tokens, p.H / walk, p.Hk, p.K, pl.l2norm, s);
  if (rc != JLA_OK) return rc;
  return finalize_key_grad(bp.dk_acc, p.k, io.dk, p.dtype, tokens, p.H / walk, p.Hk, p.K, pl.l2norm, s);
}

}  // namespace jla
