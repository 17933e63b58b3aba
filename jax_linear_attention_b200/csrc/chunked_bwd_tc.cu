// Chunk-parallel gradients (dq, dk, dbeta, dg) on the Blackwell tensor cores: every product is a tcgen05.mma
// (M = 64 tokens) reading 128-byte-swizzled bf16/f16 tiles straight from shared memory, accumulating in TMEM;
// the tiles arrive by TMA (cp.async.bulk.tensor, one thread issues them, mbarriers count the bytes); sixteen
// warps read the accumulators back in the m16n8 fragment layout for the elementwise work (decay masks, row and
// column sums, rounding of the next operand). Same math as sg_chunk_grads_kernel (chunked_bwd.cu):
//
//   dP  = scale (dO Vn^T) D      dQ = scale (cin Gamma)(dO S^T) + dP K
//   dAg = tril(dVn W^T)   dT0 = dAg D beta_j   dA0 = -strict(T0^T dT0 T0^T) same
//   dK  = (tail Gamma_r)(Vn dS+^T) - (cin Gamma)(dW S^T) + dP^T Q + (dA0 beta_i) K + (dA0 beta_i)^T K
//
// Transposed operands cost nothing: a tile stored [rows][64-element blocks] is read K-major (contraction along
// the contiguous axis) or MN-major (contraction along the rows) by choosing the descriptor.
//
// One CTA per (chunk, head), 512 threads: warp w owns rows 16 (w % 4) .. +15 (its TMEM lane quadrant) and the
// (w / 4)-th quarter of the columns. TMEM columns: [0,128) dq part 1 then Vn dS+^T, [128,256) dk,
// [256,384) K S / dP K / M1 / dW S^T, [384,448) and [448,512) the 64 x 64 tiles.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {

__device__ int g_tc_status = 0;  // set to a non-zero code when a bounded wait gave up

namespace {

using umma::swz_tile;

struct GradTcParams {
  const ChunkMeta* meta;
  const float* gates;
  const unsigned char* runs;
  void *dq, *dk;
  float *dq_acc, *dk_acc;
  float *dg, *dbeta;
  int H, Hk;
  float scale;
};

struct GradTcMaps {
  CUtensorMap q, k, v, d_o, dv, h, dh, vn, dvn, t0;
};

template <int K, int V, bool DELTA>
struct GradTcSmem {
  static constexpr int kK = 0;
  static constexpr int kQ = kK + 64 * K * 2;
  static constexpr int kDo = kQ + 64 * K * 2;          // dO, later dVn
  static constexpr int kV = kDo + 64 * V * 2;          // V -> W in place, later dW
  static constexpr int kVn = DELTA ? kV + 64 * V * 2 : kV;
  static constexpr int kS = kVn + 64 * V * 2;
  static constexpr int kT0 = kS + K * V * 2;
  static constexpr int kXa = kT0 + 8192;               // dP, later M1
  static constexpr int kXb = kXa + 8192;               // dT0, later dA0 beta_i
  static constexpr int kD = kXb + 8192;                // decay matrix D[64][68] f32
  static constexpr int kVec = kD + 64 * 68 * 4;        // G beta gam gamr dG dbeta: [64] f32 each; sdot[4]; runs[64] u8
  static constexpr int kBars = kVec + (6 * 64 + 4) * 4 + 64;
  static constexpr int kBytes = kBars + 12 * 8 + 16 + 1024;  // 12 mbarriers, tmem slot, alignment slack
  static_assert(K * V * 2 <= 64 * K * 2 + 64 * V * 2, "dS+ must fit over q | dO");
  static_assert(kBars % 8 == 0, "mbarrier alignment");
};

constexpr int LDD = 68;

// zero rows [first, 64) of a [64 x COLS] swizzled tile (tokens past the end of a partial chunk)
template <typename T, int COLS>
__device__ __forceinline__ void zero_tail_rows(unsigned char* tile, int first, int tid, int nthreads) {
  T* dst = reinterpret_cast<T*>(tile);
  constexpr int VPR = COLS / 8;
  for (int idx = tid; idx < (64 - first) * VPR; idx += nthreads) {
    const int r = first + idx / VPR, c = (idx % VPR) * 8;
    *reinterpret_cast<uint4*>(dst + swz_tile(64, r, c)) = make_uint4(0, 0, 0, 0);
  }
}

template <typename T, int NT>
__device__ __forceinline__ void store_acc_swz(unsigned char* tile, int rows, int r0, int c0, const float (&acc)[NT][4],
                                              int lane, float s_lo = 1.f, float s_hi = 1.f) {
  T* dst = reinterpret_cast<T*>(tile);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = c0 + nt * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(dst + swz_tile(rows, r0 + g, col)) = pack2<T>(acc[nt][0] * s_lo, acc[nt][1] * s_lo);
    *reinterpret_cast<uint32_t*>(dst + swz_tile(rows, r0 + g + 8, col)) = pack2<T>(acc[nt][2] * s_hi, acc[nt][3] * s_hi);
  }
}

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
    atomicAdd(vec + r0 + (lane >> 2), sign * a);
    atomicAdd(vec + r0 + (lane >> 2) + 8, sign * b);
  }
}

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
      atomicAdd(vec + c0 + nt * 8 + 2 * lane, sign * a);
      atomicAdd(vec + c0 + nt * 8 + 2 * lane + 1, sign * b);
    }
  }
}

// sum_c x[i][c] * tile[i][c] over this warp's columns (swizzled 16-bit tile), reduced over the quad.
template <typename T, int NT>
__device__ __forceinline__ void row_dots_swz(const float (&x)[NT][4], const unsigned char* tile, int rows, int r0,
                                             int c0, int lane, float& d0, float& d1) {
  const T* src = reinterpret_cast<const T*>(tile);
  const int g = lane >> 2, t = lane & 3;
  d0 = 0.f;
  d1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = c0 + nt * 8 + 2 * t;
    const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(src + swz_tile(rows, r0 + g, col)));
    const float2 b = unpack2<T>(*reinterpret_cast<const uint32_t*>(src + swz_tile(rows, r0 + g + 8, col)));
    d0 += x[nt][0] * a.x + x[nt][1] * a.y;
    d1 += x[nt][2] * b.x + x[nt][3] * b.y;
  }
  d0 += __shfl_xor_sync(0xffffffffu, d0, 1);
  d0 += __shfl_xor_sync(0xffffffffu, d0, 2);
  d1 += __shfl_xor_sync(0xffffffffu, d1, 1);
  d1 += __shfl_xor_sync(0xffffffffu, d1, 2);
}

template <typename T, int K, int V, bool DELTA, bool TR>
__global__ void __launch_bounds__(512, 1)
sg_chunk_grads_tc_kernel(const __grid_constant__ GradTcMaps maps, GradTcParams p) {
  using L = GradTcSmem<K, V, DELTA>;
  constexpr int FMT = umma::Fmt<T>::value;
  constexpr int KNT = K / 32, VNT = V / 32;  // n-tiles of this warp's quarter of a K- or V-wide accumulator
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), cq = warp >> 2;
  const int kc0 = (K / 4) * cq, vc0 = (V / 4) * cq, cc0 = 16 * cq;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* kS = base + L::kK;
  unsigned char* qS = base + L::kQ;
  unsigned char* doS = base + L::kDo;
  unsigned char* vS = base + L::kV;
  unsigned char* vnS = base + L::kVn;
  unsigned char* SS = base + L::kS;
  unsigned char* t0S = base + L::kT0;
  unsigned char* Xa = base + L::kXa;
  unsigned char* Xb = base + L::kXb;
  unsigned char* dSS = qS;  // dS+ overlays q | dO once both are dead
  float* Dm = reinterpret_cast<float*>(base + L::kD);
  float* Gs = reinterpret_cast<float*>(base + L::kVec);
  float* betas = Gs + 64;
  float* gam = betas + 64;
  float* gamr = gam + 64;
  float* dGv = gamr + 64;
  float* dbv = dGv + 64;
  float* sdot = dbv + 64;
  unsigned char* runs = reinterpret_cast<unsigned char*>(sdot + 4);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::kBars);  // [0..7] MMA batches, [8..11] TMA loads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  const uint32_t aK = umma::smem_addr(kS), aQ = umma::smem_addr(qS), aDo = umma::smem_addr(doS), aV = umma::smem_addr(vS),
                 aVn = umma::smem_addr(vnS), aS = umma::smem_addr(SS), aT0 = umma::smem_addr(t0S),
                 aXa = umma::smem_addr(Xa), aXb = umma::smem_addr(Xb), adS = umma::smem_addr(dSS);
  const int ch_off = c * p.H + h;
  if (tid == 0) {
    for (int i = 0; i < 12; ++i) umma::mbar_init(bars + i, 1);
    umma::mbar_init_fence();
    // load group 0: k, S, v, T0 ; group 1: dO, Vn, q
    uint32_t bytes = 64 * K * 2 + K * V * 2 + 64 * V * 2 + (DELTA ? 8192 : 0);
    tma::expect_tx(bars + 8, bytes);
    tma::load_tile<64, K>(kS, &maps.k, 0, hk, m.tok0, bars + 8);
    tma::load_tile<K, V>(SS, &maps.h, 0, 0, ch_off * K, bars + 8);
    tma::load_tile<64, V>(vS, &maps.v, 0, h, m.tok0, bars + 8);
    if (DELTA) tma::load_tile<64, 64>(t0S, &maps.t0, 0, 0, ch_off * 64, bars + 8);
    bytes = 64 * V * 2 + 64 * K * 2 + (DELTA ? 64 * V * 2 : 0);
    tma::expect_tx(bars + 9, bytes);
    tma::load_tile<64, V>(doS, &maps.d_o, 0, h, m.tok0, bars + 9);
    if (DELTA && !TR) tma::load_tile<64, V>(vnS, &maps.vn, 0, 0, ch_off * 64, bars + 9);
    if (DELTA && TR) tma::load_tile<V, 64>(vnS, &maps.vn, 0, 0, ch_off * V, bars + 9);
    tma::load_tile<64, K>(qS, &maps.q, 0, hk, m.tok0, bars + 9);
  }
  if (warp == 1) umma::tmem_alloc(tmem_slot, 512);
  if (tid < 64) {
    Gs[tid] = p.gates[(long)ch_off * 128 + tid];
    betas[tid] = p.gates[(long)ch_off * 128 + 64 + tid];
    runs[tid] = p.runs[(long)c * 64 + tid];
    dGv[tid] = 0.f;
    dbv[tid] = 0.f;
    if (tid == 0) sdot[0] = 0.f;
  }
  __syncthreads();
  if (tid < 64) {
    const RowScalars rs = row_scalars(Gs, runs, m.flags, tid);
    gam[tid] = rs.gam;
    gamr[tid] = rs.gamr;
  }
  for (int idx = tid; idx < 64 * 64; idx += 512) {  // D_ij = exp(G_i - G_j) for i >= j in the same run
    const int i = idx >> 6, j = idx & 63;
    Dm[i * LDD + j] = decay_ij(Gs, runs, i, j, Gs[i], runs[i]);
  }
  bool ok = umma::mbar_wait(bars + 8, 0);
  if (m.len < 64) {
    zero_tail_rows<T, K>(kS, m.len, tid, 512);
    zero_tail_rows<T, V>(vS, m.len, tid, 512);
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * (warp & 3)) << 16);  // this warp's lane quadrant
  constexpr uint32_t cQ = 0, cK = 128, cT1 = 256, cP1 = 384, cP2 = 448;

  // ---- batch 1: T1 = K S (for W) -------------------------------------------------------------------------
  if (DELTA && tid == 0 && ok) {
    if (TR) umma::gemm<64, V, K / 16, false, false, FMT>(tmem + cT1, aK, 64, aS, V, false);
    else umma::gemm<64, V, K / 16, false, true, FMT>(tmem + cT1, aK, 64, aS, K, false);
    umma::commit(bars + 0);
  }
  __syncwarp();
  ok = umma::mbar_wait(bars + 9, 0) && ok;
  if (m.len < 64) {
    zero_tail_rows<T, V>(doS, m.len, tid, 512);
    zero_tail_rows<T, K>(qS, m.len, tid, 512);
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  // ---- batch 2: P1 = dO Vn^T, P2 = Q K^T, accQ = dO S^T ------------------------------------------------------
  if (tid == 0 && ok) {
    if (TR && DELTA) umma::gemm<64, 64, V / 16, false, true, FMT>(tmem + cP1, aDo, 64, aVn, V, false);
    else umma::gemm<64, 64, V / 16, false, false, FMT>(tmem + cP1, aDo, 64, aVn, 64, false);
    umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP2, aQ, 64, aK, 64, false);
    if (TR) umma::gemm<64, K, V / 16, false, true, FMT>(tmem + cQ, aDo, 64, aS, V, false);
    else umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cQ, aDo, 64, aS, K, false);
    umma::commit(bars + 1);
  }
  __syncwarp();
  const int i0 = r0 + g, i1 = r0 + g + 8;
  const float gam0 = gam[i0], gam1 = gam[i1], gamr0 = gamr[i0], gamr1 = gamr[i1];

  if (DELTA) {  // epilogue 1: W = V - (cin Gamma)(K S), in place over V
    ok = umma::mbar_wait(bars + 0, 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      float acc[VNT][4];
      umma::ld_16x256b<VNT>(acc, tl + cT1 + vc0);
      umma::wait_ld();
      T* vt = reinterpret_cast<T*>(vS);
#pragma unroll
      for (int nt = 0; nt < VNT; ++nt) {
        const int col = vc0 + nt * 8 + 2 * t;
        uint32_t* w0 = reinterpret_cast<uint32_t*>(vt + swz_tile(64, i0, col));
        uint32_t* w1 = reinterpret_cast<uint32_t*>(vt + swz_tile(64, i1, col));
        const float2 v0 = unpack2<T>(*w0), v1 = unpack2<T>(*w1);
        *w0 = pack2<T>(v0.x - gam0 * acc[nt][0], v0.y - gam0 * acc[nt][1]);
        *w1 = pack2<T>(v1.x - gam1 * acc[nt][2], v1.y - gam1 * acc[nt][3]);
      }
    }
  }
  {  // epilogue 2: dP = scale (dO Vn^T) D ; E = dP (Q K^T)
    ok = umma::mbar_wait(bars + 1, 0) && ok;
    umma::fence_after_sync();
    if (DELTA && tid == 0 && ok) {  // dO is dead: fetch dVn into its buffer
      tma::expect_tx(bars + 10, 64 * V * 2);
      if (TR) tma::load_tile<V, 64>(doS, &maps.dvn, 0, 0, ch_off * V, bars + 10);
      else tma::load_tile<64, V>(doS, &maps.dvn, 0, 0, ch_off * 64, bars + 10);
    }
    __syncwarp();
    if (ok) {
      float accP[2][4], accE[2][4];
      umma::ld_16x256b<2>(accP, tl + cP1 + cc0);
      umma::ld_16x256b<2>(accE, tl + cP2 + cc0);
      umma::wait_ld();
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int j = cc0 + nt * 8 + 2 * t;
        const float2 d0 = *reinterpret_cast<const float2*>(Dm + i0 * LDD + j);
        const float2 d1 = *reinterpret_cast<const float2*>(Dm + i1 * LDD + j);
        accP[nt][0] *= p.scale * d0.x;
        accP[nt][1] *= p.scale * d0.y;
        accP[nt][2] *= p.scale * d1.x;
        accP[nt][3] *= p.scale * d1.y;
#pragma unroll
        for (int e = 0; e < 4; ++e) accE[nt][e] *= accP[nt][e];
      }
      row_sums_add<2>(accE, dGv, r0, lane, 1.f);
      col_sums_add<2>(accE, dGv, cc0, lane, -1.f);
      store_acc_swz<T, 2>(Xa, 64, r0, cc0, accP, lane);
    }
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  // ---- batch 3: T1 = dP K, accK = dP^T Q ---------------------------------------------------------------------
  if (tid == 0 && ok) {
    umma::gemm<64, K, 4, false, true, FMT>(tmem + cT1, aXa, 64, aK, 64, false);
    umma::gemm<64, K, 4, true, true, FMT>(tmem + cK, aXa, 64, aQ, 64, false);
    umma::commit(bars + 2);
  }
  __syncwarp();
  if (DELTA) {
    ok = umma::mbar_wait(bars + 10, 0) && ok;  // dVn landed (whole 64-row tile from the scratch: no tail to clear)
    // ---- batch 3b: P1 = dVn W^T, P2 = K K^T (W was written before the barrier above) ---------------------------
    if (tid == 0 && ok) {
      if (TR) umma::gemm<64, 64, V / 16, true, false, FMT>(tmem + cP1, aDo, V, aV, 64, false);
      else umma::gemm<64, 64, V / 16, false, false, FMT>(tmem + cP1, aDo, 64, aV, 64, false);
      umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP2, aK, 64, aK, 64, false);
      umma::commit(bars + 3);
    }
    __syncwarp();
  }
  {  // epilogue 3: dq = scale (cin Gamma)(dO S^T) + dP K
    ok = umma::mbar_wait(bars + 2, 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      float accQ[KNT][4], accT[KNT][4];
      umma::ld_16x256b<KNT>(accQ, tl + cQ + kc0);
      umma::ld_16x256b<KNT>(accT, tl + cT1 + kc0);
      umma::wait_ld();
      const float s0 = p.scale * gam0, s1 = p.scale * gam1;
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        accQ[nt][0] *= s0;
        accQ[nt][1] *= s0;
        accQ[nt][2] *= s1;
        accQ[nt][3] *= s1;
      }
      float d0, d1;
      row_dots_swz<T, KNT>(accQ, qS, 64, r0, kc0, lane, d0, d1);
      if (t == 0) {
        atomicAdd(dGv + i0, d0);
        atomicAdd(dGv + i1, d1);
      }
      const long tok0 = (long)m.tok0 + i0;
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (i0 + 8 * hh >= m.len) continue;
          const long tok = tok0 + 8 * hh;
          const float x0 = accQ[nt][2 * hh] + accT[nt][2 * hh], x1 = accQ[nt][2 * hh + 1] + accT[nt][2 * hh + 1];
          if (p.dq_acc) {
            *reinterpret_cast<float2*>(p.dq_acc + (tok * p.H + h) * K + col) = make_float2(x0, x1);
          } else {
            *reinterpret_cast<uint32_t*>(static_cast<T*>(p.dq) + (tok * p.Hk + hk) * K + col) = pack2<T>(x0, x1);
          }
        }
      }
    }
  }
  if (DELTA) {
    {  // epilogue 4: dAg = tril(dVn W^T); F = dAg Ag; dT0 = dAg D beta_j
      ok = umma::mbar_wait(bars + 3, 0) && ok;
      umma::fence_after_sync();
      if (ok) {
        float accA[2][4], accF[2][4], accB[2][4];
        umma::ld_16x256b<2>(accA, tl + cP1 + cc0);
        umma::wait_ld();
        const T* t0t = reinterpret_cast<const T*>(t0S);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int j = cc0 + nt * 8 + 2 * t;
          const float2 d0 = *reinterpret_cast<const float2*>(Dm + i0 * LDD + j);
          const float2 d1 = *reinterpret_cast<const float2*>(Dm + i1 * LDD + j);
          const float2 ta = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i0, j)));
          const float2 tb = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i1, j)));
          const float dd[4] = {d0.x, d0.y, d1.x, d1.y};
          const float tt[4] = {ta.x, ta.y, tb.x, tb.y};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float bj = betas[j + (e & 1)];
            const float dag = accA[nt][e];
            accB[nt][e] = dag * tt[e] * dd[e];
            accF[nt][e] = accB[nt][e] * bj;
            accA[nt][e] = dag * dd[e] * bj;
          }
        }
        row_sums_add<2>(accF, dGv, r0, lane, 1.f);
        col_sums_add<2>(accF, dGv, cc0, lane, -1.f);
        col_sums_add<2>(accB, dbv, cc0, lane, 1.f);
        store_acc_swz<T, 2>(Xb, 64, r0, cc0, accA, lane);
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();  // every warp is past its reads of q (epilogue 3); W and dVn were consumed by batch 3b
    umma::fence_after_sync();
    // ---- batch 4: M1 = dT0 T0^T (into T1[0:64]); fetch dW over W and dS+ over q | dO -------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, 64, 4, false, false, FMT>(tmem + cT1, aXb, 64, aT0, 64, false);
      umma::commit(bars + 4);
      tma::expect_tx(bars + 11, 64 * V * 2 + K * V * 2);
      tma::load_tile<64, V>(vS, &maps.dv, 0, h, m.tok0, bars + 11);
      tma::load_tile<K, V>(dSS, &maps.dh, 0, 0, ch_off * K, bars + 11);
    }
    __syncwarp();
    ok = umma::mbar_wait(bars + 4, 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      float accM[2][4];
      umma::ld_16x256b<2>(accM, tl + cT1 + cc0);
      umma::wait_ld();
      store_acc_swz<T, 2>(Xa, 64, r0, cc0, accM, lane);  // dP is dead: M1 takes its tile
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- batch 5: P1 = T0^T M1 -----------------------------------------------------------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, 64, 4, true, true, FMT>(tmem + cP1, aT0, 64, aXa, 64, false);
      umma::commit(bars + 5);
    }
    __syncwarp();
    ok = umma::mbar_wait(bars + 5, 0) && ok;
    umma::fence_after_sync();
    if (ok) {  // epilogue 6: dA0 = -strict(P1) same; dbeta_i += sum_j dA0_ij (k_i . k_j); Xb = dA0 beta_i
      float accA0[2][4], accKK[2][4];
      umma::ld_16x256b<2>(accA0, tl + cP1 + cc0);
      umma::ld_16x256b<2>(accKK, tl + cP2 + cc0);
      umma::wait_ld();
      const float b0 = betas[i0], b1 = betas[i1];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (e >> 1) ? i1 : i0, j = cc0 + nt * 8 + 2 * t + (e & 1);
          const float a = (j < i && Dm[i * LDD + j] != 0.f) ? -accA0[nt][e] : 0.f;  // strictly lower, same run
          accKK[nt][e] *= a;
          accA0[nt][e] = a * ((e >> 1) ? b1 : b0);
        }
      }
      row_sums_add<2>(accKK, dbv, r0, lane, 1.f);
      store_acc_swz<T, 2>(Xb, 64, r0, cc0, accA0, lane);
    }
  } else {
    umma::fence_before_sync();
    __syncthreads();  // every warp is past its reads of q
    umma::fence_after_sync();
    if (tid == 0 && ok) {
      tma::expect_tx(bars + 11, K * V * 2);
      tma::load_tile<K, V>(dSS, &maps.dh, 0, 0, ch_off * K, bars + 11);
    }
    __syncwarp();
  }
  ok = umma::mbar_wait(bars + 11, 0) && ok;
  if (DELTA && m.len < 64) zero_tail_rows<T, V>(vS, m.len, tid, 512);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  // ---- batch 6: accK += dA0b K + dA0b^T K ; T1 = dW S^T ; accQ = Vn dS+^T ------------------------------------------
  if (tid == 0 && ok) {
    if (DELTA) {
      umma::gemm<64, K, 4, false, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
      umma::gemm<64, K, 4, true, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
      if (TR) umma::gemm<64, K, V / 16, false, true, FMT>(tmem + cT1, aV, 64, aS, V, false);
      else umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cT1, aV, 64, aS, K, false);
    }
    if (TR && DELTA) umma::gemm<64, K, V / 16, true, true, FMT>(tmem + cQ, aVn, V, adS, V, false);
    else if (TR) umma::gemm<64, K, V / 16, false, true, FMT>(tmem + cQ, aVn, 64, adS, V, false);
    else umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cQ, aVn, 64, adS, K, false);
    umma::commit(bars + 6);
  }
  __syncwarp();
  {  // keep gamma <S, dS+> while the products run (both tiles share one layout)
    float part = 0.f;
    {
      const uint32_t* a = reinterpret_cast<const uint32_t*>(SS);
      const uint32_t* b = reinterpret_cast<const uint32_t*>(dSS);
      for (int idx = tid; idx < K * V / 2; idx += 512) {
        const float2 x = unpack2<T>(a[idx]), y = unpack2<T>(b[idx]);
        part += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
    if (lane == 0) atomicAdd(sdot, part);
  }
  ok = umma::mbar_wait(bars + 6, 0) && ok;
  umma::fence_after_sync();
  if (ok) {  // epilogue 7: dk and the state terms of dG
    float accK[KNT][4], accT[KNT][4];
    float d0, d1;
    umma::ld_16x256b<KNT>(accK, tl + cK + kc0);
    if (DELTA) {
      umma::ld_16x256b<KNT>(accT, tl + cT1 + kc0);
      umma::wait_ld();
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        accT[nt][0] *= gam0;
        accT[nt][1] *= gam0;
        accT[nt][2] *= gam1;
        accT[nt][3] *= gam1;
#pragma unroll
        for (int e = 0; e < 4; ++e) accK[nt][e] -= accT[nt][e];
      }
      row_dots_swz<T, KNT>(accT, kS, 64, r0, kc0, lane, d0, d1);
      if (t == 0) {
        atomicAdd(dGv + i0, -d0);
        atomicAdd(dGv + i1, -d1);
      }
    }
    umma::ld_16x256b<KNT>(accT, tl + cQ + kc0);
    umma::wait_ld();
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      accT[nt][0] *= gamr0;
      accT[nt][1] *= gamr0;
      accT[nt][2] *= gamr1;
      accT[nt][3] *= gamr1;
#pragma unroll
      for (int e = 0; e < 4; ++e) accK[nt][e] += accT[nt][e];
    }
    row_dots_swz<T, KNT>(accT, kS, 64, r0, kc0, lane, d0, d1);
    if (t == 0) {
      atomicAdd(dGv + i0, -d0);
      atomicAdd(dGv + i1, -d1);
      atomicAdd(dGv + 63, d0 + d1);
    }
    const long tok0 = (long)m.tok0 + i0;
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (i0 + 8 * hh >= m.len) continue;
        const long tok = tok0 + 8 * hh;
        if (p.dk_acc) {
          *reinterpret_cast<float2*>(p.dk_acc + (tok * p.H + h) * K + col) = make_float2(accK[nt][2 * hh], accK[nt][2 * hh + 1]);
        } else {
          *reinterpret_cast<uint32_t*>(static_cast<T*>(p.dk) + (tok * p.Hk + hk) * K + col) =
              pack2<T>(accK[nt][2 * hh], accK[nt][2 * hh + 1]);
        }
      }
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, 512);
  if (!ok) {
    if (tid == 0) atomicExch(&g_tc_status, 1);
    return;
  }
  if (tid < 64) {  // dg = reverse cumulative sum of dG over the chunk
    float acc = 0.f;
    for (int j = 63; j >= tid; --j) acc += dGv[j];
    acc += keep_gamma(Gs, runs, m.flags) * sdot[0];
    if (tid < m.len) {
      if (p.dg) p.dg[((long)m.tok0 + tid) * p.H + h] = acc;
      if (DELTA) p.dbeta[((long)m.tok0 + tid) * p.H + h] = dbv[tid];
    }
  }
}

template <typename T, int K, int V, bool DELTA, bool TR = false>
int launch_one(const GradTcMaps& maps, const GradTcParams& gp, int blocks, cudaStream_t s) {
  auto* kern = sg_chunk_grads_tc_kernel<T, K, V, DELTA, TR>;
  constexpr int smem = GradTcSmem<K, V, DELTA>::kBytes;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  {
    ProfScope ps(kProfSgChunkGrads, s);
    kern<<<blocks, 512, smem, s>>>(maps, gp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <typename T, bool DELTA>
int launch_kv(const GradTcMaps& maps, const GradTcParams& gp, int K, int V, int blocks, bool tr, cudaStream_t s) {
  if (K == 128 && V == 128) return tr ? launch_one<T, 128, 128, DELTA, true>(maps, gp, blocks, s) : launch_one<T, 128, 128, DELTA>(maps, gp, blocks, s);
  if (K == 128 && V == 64) return launch_one<T, 128, 64, DELTA>(maps, gp, blocks, s);
  if (K == 64 && V == 128) return launch_one<T, 64, 128, DELTA>(maps, gp, blocks, s);
  return launch_one<T, 64, 64, DELTA>(maps, gp, blocks, s);
}

}  // namespace

// Same contract as the chunk-gradient half of launch_sg_bwd (chunked_bwd.cu).
int launch_chunk_grads_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, bool direct, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  const uint64_t tokens = (uint64_t)p.B * p.T, slots = (uint64_t)pl.nc * p.H;
  GradTcMaps maps;
  bool ok = tma::encode_3d(&maps.q, c.q_eff, p.K, p.Hk, tokens, 64) && tma::encode_3d(&maps.k, c.k_eff, p.K, p.Hk, tokens, 64) &&
            tma::encode_3d(&maps.v, p.v, p.V, p.H, tokens, 64) && tma::encode_3d(&maps.d_o, io.d_o, p.V, p.H, tokens, 64) &&
            tma::encode_3d(&maps.dv, io.dv, p.V, p.H, tokens, 64) &&
            tma::encode_3d(&maps.h, c.res + pl.h, p.V, 1, slots * p.K, p.K) &&
            tma::encode_3d(&maps.dh, scratch + pl.dh, p.V, 1, slots * p.K, p.K);
  if (ok && pl.delta) {
    const bool trv = use_tc_kernels(p);
    ok = (trv ? tma::encode_3d(&maps.vn, c.res + pl.vn, 64, 1, slots * p.V, p.V)
              : tma::encode_3d(&maps.vn, c.res + pl.vn, p.V, 1, slots * 64, 64)) &&
         (trv ? tma::encode_3d(&maps.dvn, scratch + pl.dvn, 64, 1, slots * p.V, p.V)
              : tma::encode_3d(&maps.dvn, scratch + pl.dvn, p.V, 1, slots * 64, 64)) &&
         tma::encode_3d(&maps.t0, c.res + pl.t0, 64, 1, slots * 64, 64);
  } else if (ok) {
    maps.vn = maps.v;
    maps.dvn = maps.v;
    maps.t0 = maps.v;
  }
  if (!ok) return JLA_ERR_CUDA;
  GradTcParams gp{};
  gp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  gp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  gp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  gp.dq = io.dq;
  gp.dk = io.dk;
  gp.dq_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dq_acc);
  gp.dk_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dk_acc);
  gp.dg = io.dg;
  gp.dbeta = io.dbeta;
  gp.H = p.H;
  gp.Hk = p.Hk;
  gp.scale = p.scale;
  const int blocks = pl.nc * p.H;
  const bool tr = use_tc_kernels(p);
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_kv<__nv_bfloat16, true>(maps, gp, p.K, p.V, blocks, tr, s)
                    : launch_kv<__nv_bfloat16, false>(maps, gp, p.K, p.V, blocks, tr, s);
  }
  return pl.delta ? launch_kv<__half, true>(maps, gp, p.K, p.V, blocks, tr, s)
                  : launch_kv<__half, false>(maps, gp, p.K, p.V, blocks, tr, s);
}

int* tc_status_ptr() {
  static int* ptr = nullptr;
  if (!ptr) {
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_tc_status) != cudaSuccess) return nullptr;
    ptr = static_cast<int*>(q);
  }
  return ptr;
}

int read_tc_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (e != cudaSuccess) return JLA_ERR_CUDA;
  *out = v;
  return JLA_OK;
}

}  // namespace jla
