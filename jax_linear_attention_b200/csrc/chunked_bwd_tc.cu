// Chunk-parallel gradients (dq, dk, dbeta, dg) on the Blackwell tensor cores: every product is a tcgen05.mma
// (M = 64 tokens) reading 128-byte-swizzled bf16/f16 tiles straight from shared memory, accumulating in TMEM;
// eight warps read the accumulators back in the m16n8 fragment layout for the elementwise work (decay masks,
// row/column sums, rounding of the next operand). Same math as sg_chunk_grads_kernel (chunked_bwd.cu):
//
//   dP  = scale (dO Vn^T) D      dQ = scale (cin Gamma)(dO S^T) + dP K
//   dAg = tril(dVn W^T)   dT0 = dAg D beta_j   dA0 = -strict(T0^T dT0 T0^T) same
//   dK  = (tail Gamma_r)(Vn dS+^T) - (cin Gamma)(dW S^T) + dP^T Q + (dA0 beta_i) K + (dA0 beta_i)^T K
//
// Transposed operands cost nothing: a tile stored [rows][64-element blocks] is read K-major (contraction along
// the contiguous axis) or MN-major (contraction along the rows) by choosing the descriptor.
//
// One CTA per (chunk, head), 256 threads. TMEM columns: [0,128) dq part 1 then Vn dS+^T, [128,256) dk,
// [256,384) K S / dP K / M1 / dW S^T, [384,448) and [448,512) the 64 x 64 tiles.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace jla {

__device__ int g_tc_status = 0;  // set to a non-zero code when a bounded wait gave up

namespace {

using umma::swz_tile;

struct GradTcParams {
  const ChunkMeta* meta;
  const float* gates;
  const unsigned char* runs;
  const void *q, *k, *v, *t0, *d_o, *h, *vn, *dh, *dvn, *dv;
  void *dq, *dk;
  float *dq_acc, *dk_acc;
  float *dg, *dbeta;
  int H, Hk;
  float scale;
};

template <int K, int V, bool DELTA>
struct GradTcSmem {
  static constexpr int kK = 0;
  static constexpr int kQ = kK + 64 * K * 2;
  static constexpr int kDo = kQ + 64 * K * 2;
  static constexpr int kV = kDo + 64 * V * 2;
  static constexpr int kVn = DELTA ? kV + 64 * V * 2 : kV;
  static constexpr int kS = kVn + 64 * V * 2;
  static constexpr int kT0 = kS + K * V * 2;
  static constexpr int kXa = kT0 + 8192;
  static constexpr int kXb = kXa + 8192;
  static constexpr int kXc = kXb + 8192;
  static constexpr int kVec = kXc + 8192;             // G[64] beta[64] dG[64] dbeta[64] sdot[4] (f32), runs[64] (u8)
  static constexpr int kBars = kVec + 260 * 4 + 64;   // 8 mbarriers + tmem slot
  static constexpr int kBytes = kBars + 8 * 8 + 16 + 1024;  // + slack for the 1024-byte alignment of the base
  static_assert(K * V * 2 <= 64 * K * 2 + 64 * V * 2, "dS+ must fit over q | dO");
};

// cp.async a [rows_valid x COLS] row-major tile into the swizzled layout (missing rows are zero-filled).
template <typename T, int ROWS, int COLS>
__device__ __forceinline__ void load_tile_swz(unsigned char* tile, const T* src, long gstride, int rows_valid, int tid,
                                              int nthreads) {
  constexpr int VPR = COLS / 8;
  T* dst = reinterpret_cast<T*>(tile);
  for (int idx = tid; idx < ROWS * VPR; idx += nthreads) {
    const int r = idx / VPR, c = (idx - r * VPR) * 8;
    T* d = dst + swz_tile(ROWS, r, c);
    if (r < rows_valid) {
      cp_async16(d, src + r * gstride + c);
    } else {
      *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
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

template <typename T, int K, int V, bool DELTA>
__global__ void __launch_bounds__(256, 1) sg_chunk_grads_tc_kernel(GradTcParams p) {
  using L = GradTcSmem<K, V, DELTA>;
  constexpr int FMT = umma::Fmt<T>::value;
  constexpr int KNT = K / 16, VNT = V / 16;  // n-tiles of this warp's half of a K- or V-wide accumulator
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), ch = warp >> 2;
  const int kc0 = (K / 2) * ch, vc0 = (V / 2) * ch, cc0 = 32 * ch;

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
  unsigned char* Xc = base + L::kXc;
  unsigned char* dSS = qS;  // dS+ overlays q | dO once both are dead
  float* Gs = reinterpret_cast<float*>(base + L::kVec);
  float* betas = Gs + 64;
  float* dGv = betas + 64;
  float* dbv = dGv + 64;
  float* sdot = dbv + 64;
  unsigned char* runs = reinterpret_cast<unsigned char*>(sdot + 4);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  const uint32_t aK = umma::smem_addr(kS), aQ = umma::smem_addr(qS), aDo = umma::smem_addr(doS), aV = umma::smem_addr(vS),
                 aVn = umma::smem_addr(vnS), aS = umma::smem_addr(SS), aT0 = umma::smem_addr(t0S),
                 aXa = umma::smem_addr(Xa), aXb = umma::smem_addr(Xb), aXc = umma::smem_addr(Xc),
                 adS = umma::smem_addr(dSS);

  const long ch_off = (long)c * p.H + h;
  const T* gk = static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * K;
  const T* gq = static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * K;
  const T* gv = static_cast<const T*>(p.v) + ((long)m.tok0 * p.H + h) * V;
  const T* gdo = static_cast<const T*>(p.d_o) + ((long)m.tok0 * p.H + h) * V;
  // group 0: k, S, v, T0, gates, runs
  load_tile_swz<T, 64, K>(kS, gk, (long)p.Hk * K, m.len, tid, 256);
  load_tile_swz<T, K, V>(SS, static_cast<const T*>(p.h) + ch_off * K * V, V, K, tid, 256);
  load_tile_swz<T, 64, V>(vS, gv, (long)p.H * V, m.len, tid, 256);
  if (DELTA) load_tile_swz<T, 64, 64>(t0S, static_cast<const T*>(p.t0) + ch_off * 4096, 64, 64, tid, 256);
  if (tid < 32) cp_async16(Gs + tid * 4, p.gates + ch_off * 128 + tid * 4);
  if (tid >= 32 && tid < 36) cp_async16(runs + (tid - 32) * 16, p.runs + (long)c * 64 + (tid - 32) * 16);
  cp_async_commit();
  // group 1: dO, Vn, q
  load_tile_swz<T, 64, V>(doS, gdo, (long)p.H * V, m.len, tid, 256);
  if (DELTA) load_tile_swz<T, 64, V>(vnS, static_cast<const T*>(p.vn) + ch_off * 64 * V, V, 64, tid, 256);
  load_tile_swz<T, 64, K>(qS, gq, (long)p.Hk * K, m.len, tid, 256);
  cp_async_commit();

  if (tid < 64) {
    dGv[tid] = 0.f;
    dbv[tid] = 0.f;
  }
  if (tid == 0) {
    sdot[0] = 0.f;
    for (int i = 0; i < 8; ++i) umma::mbar_init(bars + i, 1);
    umma::mbar_init_fence();
  }
  if (warp == 0) umma::tmem_alloc(tmem_slot, 512);
  cp_async_wait<1>();
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * (warp & 3)) << 16);  // this warp's lane quadrant
  constexpr uint32_t cQ = 0, cK = 128, cT1 = 256, cP1 = 384, cP2 = 448;
  bool ok = true;

  // ---- batch 1: T1 = K S (for W) -------------------------------------------------------------------------
  if (DELTA && tid == 0) {
    umma::gemm<64, V, K / 16, false, true, FMT>(tmem + cT1, aK, 64, aS, K, false);
    umma::commit(bars + 0);
  }
  cp_async_wait<0>();
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  // ---- batch 2: P1 = dO Vn^T, P2 = Q K^T, accQ = dO S^T ------------------------------------------------------
  if (tid == 0) {
    umma::gemm<64, 64, V / 16, false, false, FMT>(tmem + cP1, aDo, 64, aVn, 64, false);
    umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP2, aQ, 64, aK, 64, false);
    umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cQ, aDo, 64, aS, K, false);
    umma::commit(bars + 1);
  }
  __syncwarp();
  const RowScalars rs0 = row_scalars(Gs, runs, m.flags, r0 + g);
  const RowScalars rs1 = row_scalars(Gs, runs, m.flags, r0 + g + 8);

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
        uint32_t* w0 = reinterpret_cast<uint32_t*>(vt + swz_tile(64, r0 + g, col));
        uint32_t* w1 = reinterpret_cast<uint32_t*>(vt + swz_tile(64, r0 + g + 8, col));
        const float2 v0 = unpack2<T>(*w0), v1 = unpack2<T>(*w1);
        *w0 = pack2<T>(v0.x - rs0.gam * acc[nt][0], v0.y - rs0.gam * acc[nt][1]);
        *w1 = pack2<T>(v1.x - rs1.gam * acc[nt][2], v1.y - rs1.gam * acc[nt][3]);
      }
    }
  }
  {  // epilogue 2: dP = scale (dO Vn^T) D ; E = dP (Q K^T)
    ok = umma::mbar_wait(bars + 1, 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      float accP[4][4], accE[4][4];
      umma::ld_16x256b<4>(accP, tl + cP1 + cc0);
      umma::ld_16x256b<4>(accE, tl + cP2 + cc0);
      umma::wait_ld();
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
      row_sums_add<4>(accE, dGv, r0, lane, 1.f);
      col_sums_add<4>(accE, dGv, cc0, lane, -1.f);
      store_acc_swz<T, 4>(Xa, 64, r0, cc0, accP, lane);
    }
  }
  // dO is dead (batch 2 complete): fetch dVn into its buffer
  if (DELTA) {
    load_tile_swz<T, 64, V>(doS, static_cast<const T*>(p.dvn) + ch_off * 64 * V, V, 64, tid, 256);
    cp_async_commit();
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
    cp_async_wait<0>();
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- batch 3b: P1 = dVn W^T, P2 = K K^T ------------------------------------------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, 64, V / 16, false, false, FMT>(tmem + cP1, aDo, 64, aV, 64, false);
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
      const float s0 = p.scale * rs0.gam, s1 = p.scale * rs1.gam;
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
        atomicAdd(dGv + r0 + g, d0);
        atomicAdd(dGv + r0 + g + 8, d1);
      }
      const long tok0 = (long)m.tok0 + r0 + g;
#pragma unroll
      for (int nt = 0; nt < KNT; ++nt) {
        const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (r0 + g + 8 * hh >= m.len) continue;
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
      // q, dVn and W are dead now: fetch dW (over W) and dS+ (over q | dO)
      load_tile_swz<T, 64, V>(vS, static_cast<const T*>(p.dv) + ((long)m.tok0 * p.H + h) * V, (long)p.H * V, m.len, tid,
                              256);
      load_tile_swz<T, K, V>(dSS, static_cast<const T*>(p.dh) + ch_off * K * V, V, K, tid, 256);
      cp_async_commit();
      if (ok) {
        float accA[4][4], accF[4][4], accB[4][4];
        umma::ld_16x256b<4>(accA, tl + cP1 + cc0);
        umma::wait_ld();
        const T* t0t = reinterpret_cast<const T*>(t0S);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = r0 + g + ((e >> 1) << 3), j = cc0 + nt * 8 + 2 * t + (e & 1);
            const RowScalars& rs = (e >> 1) ? rs1 : rs0;
            const float d = decay_ij(Gs, runs, i, j, rs.G, rs.run);
            const float t0v = to_f32(t0t[swz_tile(64, i, j)]);
            const float dag = accA[nt][e];
            accB[nt][e] = dag * t0v * d;
            accF[nt][e] = accB[nt][e] * betas[j];
            accA[nt][e] = dag * d * betas[j];
          }
        }
        row_sums_add<4>(accF, dGv, r0, lane, 1.f);
        col_sums_add<4>(accF, dGv, cc0, lane, -1.f);
        col_sums_add<4>(accB, dbv, cc0, lane, 1.f);
        store_acc_swz<T, 4>(Xb, 64, r0, cc0, accA, lane);
      }
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- batch 4: M1 = dT0 T0^T (into T1[0:64]) ----------------------------------------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, 64, 4, false, false, FMT>(tmem + cT1, aXb, 64, aT0, 64, false);
      umma::commit(bars + 4);
    }
    __syncwarp();
    ok = umma::mbar_wait(bars + 4, 0) && ok;
    umma::fence_after_sync();
    if (ok) {
      float accM[4][4];
      umma::ld_16x256b<4>(accM, tl + cT1 + cc0);
      umma::wait_ld();
      store_acc_swz<T, 4>(Xc, 64, r0, cc0, accM, lane);
    }
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    // ---- batch 5: P1 = T0^T M1 -----------------------------------------------------------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, 64, 4, true, true, FMT>(tmem + cP1, aT0, 64, aXc, 64, false);
      umma::commit(bars + 5);
    }
    __syncwarp();
    ok = umma::mbar_wait(bars + 5, 0) && ok;
    umma::fence_after_sync();
    if (ok) {  // epilogue 6: dA0 = -strict(P1) same; dbeta_i += sum_j dA0_ij (k_i . k_j); Xb = dA0 beta_i
      float accA0[4][4], accKK[4][4];
      umma::ld_16x256b<4>(accA0, tl + cP1 + cc0);
      umma::ld_16x256b<4>(accKK, tl + cP2 + cc0);
      umma::wait_ld();
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
      row_sums_add<4>(accKK, dbv, r0, lane, 1.f);
      store_acc_swz<T, 4>(Xb, 64, r0, cc0, accA0, lane);
    }
  } else {
    load_tile_swz<T, K, V>(dSS, static_cast<const T*>(p.dh) + ch_off * K * V, V, K, tid, 256);
    cp_async_commit();
  }
  cp_async_wait<0>();
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  // ---- batch 6: accK += dA0b K + dA0b^T K ; T1 = dW S^T ; accQ = Vn dS+^T ------------------------------------------
  if (tid == 0 && ok) {
    if (DELTA) {
      umma::gemm<64, K, 4, false, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
      umma::gemm<64, K, 4, true, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
      umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cT1, aV, 64, aS, K, false);
    }
    umma::gemm<64, K, V / 16, false, false, FMT>(tmem + cQ, aVn, 64, adS, K, false);
    umma::commit(bars + 6);
  }
  __syncwarp();
  {  // keep gamma <S, dS+> while the products run (both tiles share one layout)
    float part = 0.f;
    const uint32_t* a = reinterpret_cast<const uint32_t*>(SS);
    const uint32_t* b = reinterpret_cast<const uint32_t*>(dSS);
    for (int idx = tid; idx < K * V / 2; idx += 256) {
      const float2 x = unpack2<T>(a[idx]), y = unpack2<T>(b[idx]);
      part += x.x * y.x + x.y * y.y;
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
        accT[nt][0] *= rs0.gam;
        accT[nt][1] *= rs0.gam;
        accT[nt][2] *= rs1.gam;
        accT[nt][3] *= rs1.gam;
#pragma unroll
        for (int e = 0; e < 4; ++e) accK[nt][e] -= accT[nt][e];
      }
      row_dots_swz<T, KNT>(accT, kS, 64, r0, kc0, lane, d0, d1);
      if (t == 0) {
        atomicAdd(dGv + r0 + g, -d0);
        atomicAdd(dGv + r0 + g + 8, -d1);
      }
    }
    umma::ld_16x256b<KNT>(accT, tl + cQ + kc0);
    umma::wait_ld();
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      accT[nt][0] *= rs0.gamr;
      accT[nt][1] *= rs0.gamr;
      accT[nt][2] *= rs1.gamr;
      accT[nt][3] *= rs1.gamr;
#pragma unroll
      for (int e = 0; e < 4; ++e) accK[nt][e] += accT[nt][e];
    }
    row_dots_swz<T, KNT>(accT, kS, 64, r0, kc0, lane, d0, d1);
    if (t == 0) {
      atomicAdd(dGv + r0 + g, -d0);
      atomicAdd(dGv + r0 + g + 8, -d1);
      atomicAdd(dGv + 63, d0 + d1);
    }
    const long tok0 = (long)m.tok0 + r0 + g;
#pragma unroll
    for (int nt = 0; nt < KNT; ++nt) {
      const int col = kc0 + nt * 8 + 2 * t;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        if (r0 + g + 8 * hh >= m.len) continue;
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
  if (warp == 0) umma::tmem_dealloc(tmem, 512);
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

template <typename T, int K, int V, bool DELTA>
int launch_one(const GradTcParams& gp, int blocks, cudaStream_t s) {
  auto* kern = sg_chunk_grads_tc_kernel<T, K, V, DELTA>;
  constexpr int smem = GradTcSmem<K, V, DELTA>::kBytes;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  {
    ProfScope ps(kProfSgChunkGrads, s);
    kern<<<blocks, 256, smem, s>>>(gp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <typename T, bool DELTA>
int launch_kv(const GradTcParams& gp, int K, int V, int blocks, cudaStream_t s) {
  if (K == 128 && V == 128) return launch_one<T, 128, 128, DELTA>(gp, blocks, s);
  if (K == 128 && V == 64) return launch_one<T, 128, 64, DELTA>(gp, blocks, s);
  if (K == 64 && V == 128) return launch_one<T, 64, 128, DELTA>(gp, blocks, s);
  return launch_one<T, 64, 64, DELTA>(gp, blocks, s);
}

}  // namespace

// Same contract as the chunk-gradient half of launch_sg_bwd (chunked_bwd.cu).
int launch_chunk_grads_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, bool direct, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  GradTcParams gp{};
  gp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  gp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  gp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  gp.q = c.q_eff;
  gp.k = c.k_eff;
  gp.v = p.v;
  gp.t0 = c.res + pl.t0;
  gp.d_o = io.d_o;
  gp.h = c.res + pl.h;
  gp.vn = c.res + pl.vn;
  gp.dh = scratch + pl.dh;
  gp.dvn = scratch + pl.dvn;
  gp.dv = io.dv;
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
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_kv<__nv_bfloat16, true>(gp, p.K, p.V, blocks, s)
                    : launch_kv<__nv_bfloat16, false>(gp, p.K, p.V, blocks, s);
  }
  return pl.delta ? launch_kv<__half, true>(gp, p.K, p.V, blocks, s) : launch_kv<__half, false>(gp, p.K, p.V, blocks, s);
}

int read_tc_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  if (e != cudaSuccess) return JLA_ERR_CUDA;
  *out = v;
  return JLA_OK;
}

}  // namespace jla
