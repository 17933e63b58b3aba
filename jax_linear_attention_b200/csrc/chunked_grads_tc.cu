// Chunk-parallel gradients (dq, dk, dbeta, dg) for K = V = 128 on the Blackwell tensor cores, as two kernels of
// one CTA per (chunk, head) each, sized so that two CTAs share an SM (<= 113 KB of shared memory, 256 TMEM
// columns, 256 threads): while one CTA waits on a TMA load or on the TMEM round trip between two dependent
// products, the other one computes.
//
//   sg_grads_q  (query side)   dP = scale (dO Vn^T) D        dQ = scale (cin Gamma)(dO S^T) + dP K
//                              dG partial = rowsum(E) - colsum(E) + <q, dQ_inter>,  E = dP (Q K^T)
//                              dP (16-bit) and the dG partial go to the backward scratch for the second kernel
//   sg_grads_k  (key side)     dAg = tril(dVn W^T)   dT0 = dAg D beta_j   dA0 = -strict(T0^T dT0 T0^T) same
//                              dK = dP^T Q + (dA0 beta_i) K + (dA0 beta_i)^T K
//                                   - (cin Gamma)(dW S^T) + (tail Gamma_r)(Vn dS+^T)
//                              dbeta, and dg = reverse cumulative sum of dG (+ keep gamma <S, dS+>)
//
// Every product is a tcgen05.mma (M = 64 tokens) on 128-byte-swizzled 16-bit tiles that TMA lands in shared
// memory; the residuals S^T, Vn^T, W^T and the state gradients dS+^T, dVn^T are stored transposed ([V][K],
// [V][64]) by the forward and reverse state passes, and a transposed operand only changes the descriptor view.
// The key-side kernel streams S^T and dS+^T in two 64-column halves over buffers whose first contents (q, dP,
// W^T, dVn^T) are dead by then. Accumulators are read back in the m16n8 fragment layout: warp w owns rows
// 16 (w % 4) .. +15 (its TMEM lane quadrant) and the (w / 4)-th half of the columns.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {

namespace {

using umma::swz_tile;

constexpr int KD = 128, VD = 128;
constexpr int NTHREADS = 256;

struct GradParams {
  const ChunkMeta* meta;
  const float* gates;
  const unsigned char* runs;
  void *dq, *dk;
  float *dq_acc, *dk_acc;
  float *dg, *dbeta;
  unsigned char* dp;  // [slot][64 x 64] 16-bit in the swizzled tile layout (8 KB per slot)
  float* dga;         // [slot][64] dG partial of the query-side kernel
  int H, Hk;
  float scale;
  int nitems;  // chunk slots x heads
  int* status;  // device status word: set non-zero when a bounded wait gave up
};

struct GradMaps {
  CUtensorMap q, k, v, d_o, dv, h, dh, vn, dvn, w, t0;
};

// zero rows [first, 64) of a [64 x COLS] swizzled tile (tokens past the end of a partial chunk)
template <typename T, int COLS>
__device__ __forceinline__ void zero_tail_rows(unsigned char* tile, int first, int tid) {
  T* dst = reinterpret_cast<T*>(tile);
  constexpr int VPR = COLS / 8;
  for (int idx = tid; idx < (64 - first) * VPR; idx += NTHREADS) {
    const int r = first + idx / VPR, c = (idx % VPR) * 8;
    *reinterpret_cast<uint4*>(dst + swz_tile(64, r, c)) = make_uint4(0, 0, 0, 0);
  }
}

template <typename T, int NT>
__device__ __forceinline__ void store_acc_swz(unsigned char* tile, int r0, int c0, const float (&acc)[NT][4], int lane) {
  T* dst = reinterpret_cast<T*>(tile);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = c0 + nt * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(dst + swz_tile(64, r0 + g, col)) = pack2<T>(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<uint32_t*>(dst + swz_tile(64, r0 + g + 8, col)) = pack2<T>(acc[nt][2], acc[nt][3]);
  }
}

// Reductions never use shared-memory float atomics (a compare-and-swap loop that serialises under contention):
// row quantities are accumulated per thread in registers and reduced over the quad once, column sums are reduced
// over the warp's 16 rows with shuffles and stored to a slot that only this warp writes.
template <int NT>
__device__ __forceinline__ void row_sums_acc(const float (&x)[NT][4], float& a, float& b) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    a += x[nt][0] + x[nt][1];
    b += x[nt][2] + x[nt][3];
  }
}

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// out[c0 + 8 nt + 2 t + {0, 1}] = sum over this warp's 16 rows of x (out is this warp's own slot)
template <int NT>
__device__ __forceinline__ void col_sums_store(const float (&x)[NT][4], float* out, int c0, int lane) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float a = x[nt][0] + x[nt][2], b = x[nt][1] + x[nt][3];
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, off);
      b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    if (lane < 4) *reinterpret_cast<float2*>(out + c0 + nt * 8 + 2 * lane) = make_float2(a, b);
  }
}

// this thread's part of sum_c x[i][c] * tile[i][c] for its rows g and g + 8 ([64 x 128] swizzled 16-bit tile)
template <typename T, int NT>
__device__ __forceinline__ void row_dots_part(const float (&x)[NT][4], const unsigned char* tile, int r0, int c0, int lane,
                                              float& d0, float& d1) {
  const T* src = reinterpret_cast<const T*>(tile);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = c0 + nt * 8 + 2 * t;
    const float2 a = unpack2<T>(*reinterpret_cast<const uint32_t*>(src + swz_tile(64, r0 + g, col)));
    const float2 b = unpack2<T>(*reinterpret_cast<const uint32_t*>(src + swz_tile(64, r0 + g + 8, col)));
    d0 += x[nt][0] * a.x + x[nt][1] * a.y;
    d1 += x[nt][2] * b.x + x[nt][3] * b.y;
  }
}

// writes this thread's fragment of a [64 x 128] gradient tile (rows i0, i0 + 8; columns c0 + 8 nt + 2t, +1)
template <typename T, int NT>
__device__ __forceinline__ void store_key_grad(const float (&x)[NT][4], float* acc_out, void* out, long tok0, int i0, int len,
                                               int c0, int t, int H, int h, int Hk, int hk) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = c0 + nt * 8 + 2 * t;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      if (i0 + 8 * hh >= len) continue;
      const long tok = tok0 + i0 + 8 * hh;
      if (acc_out) {
        *reinterpret_cast<float2*>(acc_out + (tok * H + h) * KD + col) = make_float2(x[nt][2 * hh], x[nt][2 * hh + 1]);
      } else {
        *reinterpret_cast<uint32_t*>(static_cast<T*>(out) + (tok * Hk + hk) * KD + col) = pack2<T>(x[nt][2 * hh], x[nt][2 * hh + 1]);
      }
    }
  }
}

__device__ __forceinline__ void cta_sync_tc() {
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
}

// ---------------------------------------------------------------------------------------------------------------
// Query side. Shared memory: dO [64][V], Vn^T [V][64] (or V [64][V] without the delta rule), S^T [V][K], q, k
// [64][K], dP [64][64]. TMEM columns: [0,64) dO Vn^T, then [0,128) dP K; [128,256) dO S^T.
// The gate gradient of the in-chunk scores needs no score matrix: with E = dP (Q K^T), rowsum_i(E) = q_i . (dP K)_i
// and colsum_j(E) = k_j . (dP^T Q)_j, so this kernel contributes q_i . dq_i and the key side subtracts k_j . (dP^T Q)_j.
struct SmemQ {
  static constexpr int kDo = 0;
  static constexpr int kVn = kDo + 64 * VD * 2;
  static constexpr int kS = kVn + 64 * VD * 2;
  static constexpr int kQ = kS + KD * VD * 2;
  static constexpr int kK = kQ + 64 * KD * 2;
  static constexpr int kXa = kK + 64 * KD * 2;
  static constexpr int kVecStride = 2 * 256 + 64;        // per item buffer: G, gam [64] f32; runs[64] u8
  static constexpr int kVec = kXa + 8192;                // two item buffers, then rowG [2][64] f32
  static constexpr int kBars = kVec + 2 * kVecStride + 2 * 256;  // 4 mbarriers, tmem slot
  static constexpr int kBytes = kBars + 4 * 8 + 8 + 1024;
  static_assert(kBars % 8 == 0, "mbarrier alignment");
  static_assert(2 * (kBytes + 1024) <= 233472, "two CTAs per SM");
};

// Persistent: CTA b walks units b, b + gridDim.x, ... (a unit is one (chunk, head) with tokens). The next unit's
// dO, Vn^T, S^T are requested as soon as this unit's products have consumed them, its q, k after the last read of
// this unit's, its gate vectors into the other of two small buffers, so only the first unit of a CTA sees a cold load.
template <typename T, bool DELTA>
__global__ void __launch_bounds__(NTHREADS, 2)
sg_grads_q_tc_kernel(const __grid_constant__ GradMaps maps, GradParams p) {
  using L = SmemQ;
  constexpr int FMT = umma::Fmt<T>::value;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), cq = warp >> 2;
  const int cc0 = 32 * cq, kc0 = 64 * cq;
  const int i0 = r0 + g, i1 = r0 + g + 8;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* doS = base + L::kDo;
  unsigned char* vnS = base + L::kVn;
  unsigned char* SS = base + L::kS;
  unsigned char* qS = base + L::kQ;
  unsigned char* kS = base + L::kK;
  unsigned char* Xa = base + L::kXa;
  float* rowG = reinterpret_cast<float*>(base + L::kVec + 2 * L::kVecStride);  // [2][64]: q . dq over each column half
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::kBars);
  enum { LX = 0, LY, M1, M2 };  // loads of dO | Vn | S and of q | k; MMA batches (M1 completes twice per unit)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  const uint32_t aDo = umma::smem_addr(doS), aVn = umma::smem_addr(vnS), aS = umma::smem_addr(SS), aK = umma::smem_addr(kS),
                 aXa = umma::smem_addr(Xa);

  auto next_live = [&](int it) {
    while (it < p.nitems && p.meta[it / p.H].len == 0) it += gridDim.x;
    return it;
  };
  auto load_x = [&](int item) {  // tid 0
    const int c = item / p.H, h = item - c * p.H;
    const int tok0 = p.meta[c].tok0;
    tma::expect_tx(bars + LX, 2 * 64 * VD * 2 + KD * VD * 2);
    tma::load_tile<64, VD>(doS, &maps.d_o, 0, h, tok0, bars + LX);
    if (DELTA) tma::load_tile<VD, 64>(vnS, &maps.vn, 0, 0, item * VD, bars + LX);
    else tma::load_tile<64, VD>(vnS, &maps.v, 0, h, tok0, bars + LX);
    tma::load_tile<VD, KD>(SS, &maps.h, 0, 0, item * VD, bars + LX);
  };
  auto load_y = [&](int item) {  // tid 0
    const int c = item / p.H, h = item - c * p.H;
    const int hk = h / (p.H / p.Hk);
    const int tok0 = p.meta[c].tok0;
    tma::expect_tx(bars + LY, 2 * 64 * KD * 2);
    tma::load_tile<64, KD>(kS, &maps.k, 0, hk, tok0, bars + LY);
    tma::load_tile<64, KD>(qS, &maps.q, 0, hk, tok0, bars + LY);
  };
  auto load_vec = [&](int item, int buf) {  // tid < 64
    float* Gs = reinterpret_cast<float*>(base + L::kVec + buf * L::kVecStride);
    unsigned char* runs = reinterpret_cast<unsigned char*>(Gs + 128);
    Gs[tid] = p.gates[(long)item * 128 + tid];
    runs[tid] = p.runs[(long)(item / p.H) * 64 + tid];
  };

  int item = next_live(blockIdx.x);
  if (tid == 0) {
    for (int i = 0; i < 4; ++i) umma::mbar_init(bars + i, 1);
    umma::mbar_init_fence();
    if (item < p.nitems) {
      load_x(item);
      load_y(item);
    }
  }
  if (warp == 1) umma::tmem_alloc(tmem_slot, 256);
  if (tid < 64 && item < p.nitems) load_vec(item, 0);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * (warp & 3)) << 16);  // this warp's lane quadrant
  constexpr uint32_t cP1 = 0, cT1 = 0, cQ = 128;
  bool ok = true, x_inflight = false, y_inflight = false;

  for (int it = 0; item < p.nitems; ++it) {
    const int c = item / p.H, h = item - c * p.H;
    const int hk = h / (p.H / p.Hk);
    const ChunkMeta m = p.meta[c];
    const int nxt = next_live(item + gridDim.x);
    const uint32_t ph = it & 1;
    float* Gs = reinterpret_cast<float*>(base + L::kVec + (it & 1) * L::kVecStride);
    float* gam = Gs + 64;
    unsigned char* runs = reinterpret_cast<unsigned char*>(Gs + 128);
    if (tid < 64) gam[tid] = row_scalars(Gs, runs, m.flags, tid).gam;
    ok = ok && umma::mbar_wait(bars + LX, ph);
    x_inflight = false;
    if (m.len < 64) zero_tail_rows<T, VD>(doS, m.len, tid);
    cta_sync_tc();
    // ---- batch 1: P1 = dO Vn^T, accQ = dO S^T ----------------------------------------------------------------------
    if (tid == 0 && ok) {
      if (DELTA) umma::gemm<64, 64, VD / 16, false, true, FMT>(tmem + cP1, aDo, 64, aVn, VD, false);
      else umma::gemm<64, 64, VD / 16, false, false, FMT>(tmem + cP1, aDo, 64, aVn, 64, false);
      umma::commit(bars + M1);
      umma::gemm<64, KD, VD / 16, false, true, FMT>(tmem + cQ, aDo, 64, aS, VD, false);
      umma::commit(bars + M2);
    }
    __syncwarp();
    {  // epilogue 1: dP = scale (dO Vn^T) D
      ok = ok && umma::mbar_wait(bars + M1, 0);
      umma::fence_after_sync();
      if (ok) {
        const float G0 = Gs[i0], G1 = Gs[i1];
        const int run0 = runs[i0], run1 = runs[i1];
        float accP[4][4];
        umma::ld_16x256b<4>(accP, tl + cP1 + cc0);
        umma::wait_ld();
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = cc0 + nt * 8 + 2 * t + (e & 1);
            const float d = (e >> 1) ? decay_ij(Gs, runs, i1, j, G1, run1) : decay_ij(Gs, runs, i0, j, G0, run0);
            accP[nt][e] *= p.scale * d;
          }
        }
        store_acc_swz<T, 4>(Xa, r0, cc0, accP, lane);
      }
    }
    ok = ok && umma::mbar_wait(bars + LY, ph);  // q, k (rows past a partial chunk only ever meet zeros of dP / dq)
    y_inflight = false;
    cta_sync_tc();
    // ---- batch 2: T1 = dP K (over the 64 x 64 tile, which every warp has read) -------------------------------------
    if (tid == 0 && ok) {
      umma::gemm<64, KD, 4, false, true, FMT>(tmem + cT1, aXa, 64, aK, 64, false);
      umma::commit(bars + M1);
    }
    __syncwarp();
    if (ok) {  // dP goes to the scratch in its tile layout: the key-side kernel lands it with one bulk copy
      const uint4* src = reinterpret_cast<const uint4*>(Xa);
      uint4* dst = reinterpret_cast<uint4*>(p.dp + (size_t)item * 8192);
      dst[tid] = src[tid];
      dst[tid + NTHREADS] = src[tid + NTHREADS];
    }
    {  // epilogue 2: dq = scale (cin Gamma)(dO S^T) + dP K ; dG partial = q . dq
      float accQ[8][4], accT[8][4];
      ok = ok && umma::mbar_wait(bars + M2, ph);
      umma::fence_after_sync();
      if (nxt < p.nitems && ok) {  // dO, Vn, S are consumed: the next unit's may land
        if (tid == 0) load_x(nxt);
        x_inflight = true;
        if (tid < 64) load_vec(nxt, (it & 1) ^ 1);
      }
      __syncwarp();
      if (ok) {
        umma::ld_16x256b<8>(accQ, tl + cQ + kc0);
        umma::wait_ld();
        const float s0 = p.scale * gam[i0], s1 = p.scale * gam[i1];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          accQ[nt][0] *= s0;
          accQ[nt][1] *= s0;
          accQ[nt][2] *= s1;
          accQ[nt][3] *= s1;
        }
      }
      ok = ok && umma::mbar_wait(bars + M1, 1);
      umma::fence_after_sync();
      if (ok) {
        umma::ld_16x256b<8>(accT, tl + cT1 + kc0);
        umma::wait_ld();
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) accQ[nt][e] += accT[nt][e];
        }
        float d0 = 0.f, d1 = 0.f;
        row_dots_part<T, 8>(accQ, qS, r0, kc0, lane, d0, d1);
        d0 = quad_sum(d0);
        d1 = quad_sum(d1);
        if (t == 0) {
          rowG[cq * 64 + i0] = d0;
          rowG[cq * 64 + i1] = d1;
        }
        store_key_grad<T, 8>(accQ, p.dq_acc, p.dq, m.tok0, i0, m.len, kc0, t, p.H, h, p.Hk, hk);
      }
    }
    umma::fence_before_sync();
    ok = __syncthreads_and(ok);  // q, k, the accumulators and rowG are final for this unit
    umma::fence_after_sync();
    if (!ok) break;
    if (nxt < p.nitems) {
      if (tid == 0) load_y(nxt);
      y_inflight = true;
    }
    if (tid < 64) p.dga[(size_t)item * 64 + tid] = rowG[tid] + rowG[64 + tid];
    item = nxt;
  }
  if (!ok) {  // let requested copies land before the shared memory goes away (bounded waits)
    if (x_inflight) umma::mbar_wait(bars + LX, 0), umma::mbar_wait(bars + LX, 1);
    if (y_inflight) umma::mbar_wait(bars + LY, 0), umma::mbar_wait(bars + LY, 1);
    if (tid == 0) atomicExch(p.status, 1);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, 256);
}

// ---------------------------------------------------------------------------------------------------------------
// Key side. Shared memory: k, q [64][K]; W^T, dVn^T [V][64]; T0, Xb, dP [64][64]; a 16 KB tile for dS+^T halves.
// Second phase over the dead tiles: S^T half -> q, dW [64][V] -> W^T, Vn^T -> dVn^T. Without the delta rule only
// k, q, dP, V and the state halves are used. TMEM columns: [0,128) dK, [128,192) and [192,256) 64 x 64 tiles.
struct SmemK {
  static constexpr int kK = 0;
  static constexpr int kQ = kK + 64 * KD * 2;
  static constexpr int kW = kQ + 64 * KD * 2;
  static constexpr int kDvn = kW + 64 * VD * 2;
  static constexpr int kT0 = kDvn + 64 * VD * 2;
  static constexpr int kXb = kT0 + 8192;
  static constexpr int kDp = kXb + 8192;
  static constexpr int kEx = kDp + 8192;
  static constexpr int kVecStride = 4 * 256 + 64;  // per unit buffer: G beta gam gamr [64] f32; runs[64] u8
  static constexpr int kVec = kEx + 64 * VD * 2;   // two unit buffers, then the shared reduction slots
  // rowG rowB [2][64]; colF colB [4][64]; dG[64]; tot[8] sdot[8]
  static constexpr int kBars = kVec + 2 * kVecStride + 13 * 256 + 64;  // 8 mbarriers, tmem slot
  static constexpr int kBytes = kBars + 8 * 8 + 16 + 1024;
  static_assert(kBars % 8 == 0, "mbarrier alignment");
  static_assert(2 * (kBytes + 1024) <= 233472, "two CTAs per SM");
};

// Persistent like the query side: while the last epilogue of a unit runs, the next unit's q, dP, W^T, dVn^T, T0 and
// first dS+^T half land in the tiles the unit no longer needs; its k follows after the unit's last read of k.
template <typename T, bool DELTA>
__global__ void __launch_bounds__(NTHREADS, 2)
sg_grads_k_tc_kernel(const __grid_constant__ GradMaps maps, GradParams p) {
  using L = SmemK;
  constexpr int FMT = umma::Fmt<T>::value;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), cq = warp >> 2;
  const int cc0 = 32 * cq;
  const int i0 = r0 + g, i1 = r0 + g + 8;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* kS = base + L::kK;
  unsigned char* qS = base + L::kQ;      // later a 64-column half of S^T
  unsigned char* wS = base + L::kW;      // W^T, later dW
  unsigned char* dvnS = base + L::kDvn;  // dVn^T, later Vn^T (V itself without the delta rule)
  unsigned char* t0S = base + L::kT0;
  unsigned char* Xb = base + L::kXb;     // dT0, later dA0 beta_i
  unsigned char* dpS = base + L::kDp;    // dP, later M1
  unsigned char* exS = base + L::kEx;    // a 64-column half of dS+^T
  float* rowG = reinterpret_cast<float*>(base + L::kVec + 2 * L::kVecStride);  // [2][64] row-wise dG terms per column half
  float* rowB = rowG + 128;  // [2][64] row-wise dbeta terms
  float* colF = rowB + 128;  // [4][64] column sums of F over each row quadrant
  float* colB = colF + 256;  // [4][64] column sums of dAg T0 D
  float* dGv = colB + 256;   // [64]
  float* tot = dGv + 64;     // [8] per warp: sum over rows of k . (tail Gamma_r)(Vn dS+^T)
  float* sdot = tot + 8;     // [8] per warp: <S, dS+>
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::kBars);
  enum { L0 = 0, L1, L2, M0, M1, M2, M3, M4 };  // M4 completes twice per unit, L1 takes two arrivals per unit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  const uint32_t aK = umma::smem_addr(kS), aQ = umma::smem_addr(qS), aW = umma::smem_addr(wS), aDvn = umma::smem_addr(dvnS),
                 aT0 = umma::smem_addr(t0S), aXb = umma::smem_addr(Xb), aDp = umma::smem_addr(dpS),
                 aEx = umma::smem_addr(exS);

  // Units are walked from the last one down: the query-side kernel, which runs just before and hands over dP, walks
  // them upwards, so the tiles both kernels read (q, k, S^T, Vn^T and the dP hand-off) of the units it touched last
  // are still in L2 when this kernel starts with them. A negative index ends the walk.
  auto next_live = [&](int it) {
    while (it >= 0 && p.meta[it / p.H].len == 0) it -= gridDim.x;
    return it;
  };
  // tid 0: everything of a unit's first phase except k (whose tile the previous unit reads until its end)
  auto load_first = [&](int item) {
    const int c = item / p.H, h = item - c * p.H;
    const int hk = h / (p.H / p.Hk);
    const int tok0 = p.meta[c].tok0;
    tma::expect_tx(bars + L0, 2 * 64 * KD * 2 + 8192 + (DELTA ? 2 * 64 * VD * 2 + 8192 : 64 * VD * 2));
    if (DELTA) {
      tma::load_tile<VD, 64>(wS, &maps.w, 0, 0, item * VD, bars + L0);
      tma::load_tile<VD, 64>(dvnS, &maps.dvn, 0, 0, item * VD, bars + L0);
      tma::load_tile<64, 64>(t0S, &maps.t0, 0, 0, item * 64, bars + L0);
    } else {
      tma::load_tile<64, VD>(dvnS, &maps.v, 0, h, tok0, bars + L0);
    }
    tma::load_tile<64, KD>(qS, &maps.q, 0, hk, tok0, bars + L0);
    tma::load_bulk(dpS, p.dp + (size_t)item * 8192, 8192, bars + L0);
    tma::expect_tx(bars + L1, VD * 64 * 2);  // first half of dS+^T
    tma::load_3d(exS, &maps.dh, 0, 0, item * VD, bars + L1);
  };
  auto load_k = [&](int item) {  // tid 0; its bytes are part of what load_first announced
    const int c = item / p.H, h = item - c * p.H;
    tma::load_tile<64, KD>(kS, &maps.k, 0, h / (p.H / p.Hk), p.meta[c].tok0, bars + L0);
  };
  auto load_vec = [&](int item, int buf) {  // tid < 64
    float* Gs = reinterpret_cast<float*>(base + L::kVec + buf * L::kVecStride);
    unsigned char* runs = reinterpret_cast<unsigned char*>(Gs + 256);
    Gs[tid] = p.gates[(long)item * 128 + tid];
    Gs[64 + tid] = p.gates[(long)item * 128 + 64 + tid];
    runs[tid] = p.runs[(long)(item / p.H) * 64 + tid];
  };

  int item = next_live(p.nitems - 1 - (int)blockIdx.x);
  if (tid == 0) {
    for (int i = 0; i < 8; ++i) umma::mbar_init(bars + i, i == L1 ? 2 : 1);
    umma::mbar_init_fence();
    if (item >= 0) {
      load_first(item);
      load_k(item);
    }
  }
  if (warp == 1) umma::tmem_alloc(tmem_slot, 256);
  if (tid < 64 && item >= 0) load_vec(item, 0);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
  constexpr uint32_t cK = 0, cP1 = 128, cP2 = 192;
  bool ok = true, first_inflight = false, k_inflight = false;

  for (int it = 0; item >= 0; ++it) {
    const int c = item / p.H, h = item - c * p.H;
    const int hk = h / (p.H / p.Hk);
    const ChunkMeta m = p.meta[c];
    const int nxt = next_live(item - (int)gridDim.x);
    const uint32_t ph = it & 1;
    float* Gs = reinterpret_cast<float*>(base + L::kVec + (it & 1) * L::kVecStride);
    float* betas = Gs + 64;
    float* gam = betas + 64;
    float* gamr = gam + 64;
    unsigned char* runs = reinterpret_cast<unsigned char*>(Gs + 256);
    const float dga = tid < 64 ? p.dga[(size_t)item * 64 + tid] : 0.f;  // needed at the very end of the unit
    if (tid < 64) {
      const RowScalars rs = row_scalars(Gs, runs, m.flags, tid);
      gam[tid] = rs.gam;
      gamr[tid] = rs.gamr;
    }
    ok = ok && umma::mbar_wait(bars + L0, ph);
    first_inflight = k_inflight = false;
    if (m.len < 64) {
      zero_tail_rows<T, KD>(kS, m.len, tid);
      zero_tail_rows<T, KD>(qS, m.len, tid);
      if (!DELTA) zero_tail_rows<T, VD>(dvnS, m.len, tid);
    }
    cta_sync_tc();
    const float G0 = Gs[i0], G1 = Gs[i1];
    const int run0 = runs[i0], run1 = runs[i1];
    float rG0 = 0.f, rG1 = 0.f;  // this thread's part of the row-wise dG terms of rows i0, i1
    float rB0 = 0.f, rB1 = 0.f;  // likewise for dbeta
    float tot_part = 0.f, sdot_part = 0.f;

    // ---- batch 1: P1 = dVn W^T ; P2 = K K^T ; accK = dP^T Q --------------------------------------------------------
    if (tid == 0 && ok) {
      if (DELTA) {
        umma::gemm<64, 64, VD / 16, true, true, FMT>(tmem + cP1, aDvn, VD, aW, VD, false);
        umma::commit(bars + M0);
        umma::gemm<64, 64, KD / 16, false, false, FMT>(tmem + cP2, aK, 64, aK, 64, false);
      }
      umma::gemm<64, KD, 4, true, true, FMT>(tmem + cK, aDp, 64, aQ, 64, false);
      umma::commit(bars + M4);  // (M4 is reused by the second state half: its first phase ends here)
    }
    __syncwarp();
    // subtracts k_j . (dP^T Q)_j, the column sums of dP (Q K^T), from the dG rows; the accumulator must be read
    // before the dA0 terms are added to it
    auto key_score_dots = [&]() {
      float accK[8][4];
      umma::ld_16x256b<8>(accK, tl + cK + 64 * cq);
      umma::wait_ld();
      float d0 = 0.f, d1 = 0.f;
      row_dots_part<T, 8>(accK, kS, r0, 64 * cq, lane, d0, d1);
      rG0 -= d0;
      rG1 -= d1;
    };
    if (DELTA) {
      ok = ok && umma::mbar_wait(bars + M0, ph);
      umma::fence_after_sync();
      if (ok) {  // dAg = tril(dVn W^T); F = dAg Ag; dT0 = dAg D beta_j
        float accA[4][4], accF[4][4], accB[4][4];
        umma::ld_16x256b<4>(accA, tl + cP1 + cc0);
        umma::wait_ld();
        const T* t0t = reinterpret_cast<const T*>(t0S);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const int j = cc0 + nt * 8 + 2 * t;
          const float2 ta = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i0, j)));
          const float2 tb = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i1, j)));
          const float tt[4] = {ta.x, ta.y, tb.x, tb.y};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int jj = j + (e & 1);
            const float d = (e >> 1) ? decay_ij(Gs, runs, i1, jj, G1, run1) : decay_ij(Gs, runs, i0, jj, G0, run0);
            const float bj = betas[jj];
            const float dag = accA[nt][e];
            accB[nt][e] = dag * tt[e] * d;
            accF[nt][e] = accB[nt][e] * bj;
            accA[nt][e] = dag * d * bj;
          }
        }
        store_acc_swz<T, 4>(Xb, r0, cc0, accA, lane);
        row_sums_acc<4>(accF, rG0, rG1);
        col_sums_store<4>(accF, colF + (warp & 3) * 64, cc0, lane);
        col_sums_store<4>(accB, colB + (warp & 3) * 64, cc0, lane);
      }
      cta_sync_tc();
      // ---- batch 2: M1 = dT0 T0^T ----------------------------------------------------------------------------------
      if (tid == 0 && ok) {
        umma::gemm<64, 64, 4, false, false, FMT>(tmem + cP1, aXb, 64, aT0, 64, false);
        umma::commit(bars + M1);
      }
      __syncwarp();
      ok = ok && umma::mbar_wait(bars + M4, 0);  // dP^T Q: long done; q, dP, W^T, dVn^T are consumed
      umma::fence_after_sync();
      if (tid == 0 && ok) {  // fetch the second-phase tiles over them
        tma::expect_tx(bars + L1, VD * 64 * 2 + 2 * 64 * VD * 2);
        tma::load_3d(qS, &maps.h, 0, 0, item * VD, bars + L1);
        tma::load_tile<64, VD>(wS, &maps.dv, 0, h, m.tok0, bars + L1);
        tma::load_tile<VD, 64>(dvnS, &maps.vn, 0, 0, item * VD, bars + L1);
      }
      __syncwarp();
      ok = ok && umma::mbar_wait(bars + M1, ph);
      umma::fence_after_sync();
      if (ok) {
        float accM[4][4];
        umma::ld_16x256b<4>(accM, tl + cP1 + cc0);
        umma::wait_ld();
        store_acc_swz<T, 4>(dpS, r0, cc0, accM, lane);  // dP is consumed: M1 takes its tile
      }
      cta_sync_tc();
      // ---- batch 3: P1 = T0^T M1 -----------------------------------------------------------------------------------
      if (tid == 0 && ok) {
        umma::gemm<64, 64, 4, true, true, FMT>(tmem + cP1, aT0, 64, aDp, 64, false);
        umma::commit(bars + M2);
      }
      __syncwarp();
      if (ok) key_score_dots();  // while the product runs
      ok = ok && umma::mbar_wait(bars + M2, ph);
      umma::fence_after_sync();
      if (ok) {  // dA0 = -strict(P1) same; dbeta_i += sum_j dA0_ij (k_i . k_j); Xb = dA0 beta_i
        float accA0[4][4], accKK[4][4];
        umma::ld_16x256b<4>(accA0, tl + cP1 + cc0);
        umma::ld_16x256b<4>(accKK, tl + cP2 + cc0);
        umma::wait_ld();
        const float b0 = betas[i0], b1 = betas[i1];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = (e >> 1) ? i1 : i0, j = cc0 + nt * 8 + 2 * t + (e & 1);
            const float a = (j < i && runs[j] == ((e >> 1) ? run1 : run0)) ? -accA0[nt][e] : 0.f;
            accKK[nt][e] *= a;
            accA0[nt][e] = a * ((e >> 1) ? b1 : b0);
          }
        }
        store_acc_swz<T, 4>(Xb, r0, cc0, accA0, lane);
        row_sums_acc<4>(accKK, rB0, rB1);
      }
    } else {
      ok = ok && umma::mbar_wait(bars + M4, 0);
      umma::fence_after_sync();
      if (tid == 0 && ok) {  // q and dP are consumed: fetch the first half of S^T over q
        tma::expect_tx(bars + L1, VD * 64 * 2);
        tma::load_3d(qS, &maps.h, 0, 0, item * VD, bars + L1);
      }
      __syncwarp();
      if (ok) key_score_dots();
    }
    ok = ok && umma::mbar_wait(bars + L1, ph);
    if (DELTA && m.len < 64) zero_tail_rows<T, VD>(wS, m.len, tid);  // dW rows past the end were never written
    cta_sync_tc();
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
      // ---- state terms over key columns [64 hh, 64 hh + 64): P1 = dW S^T, P2 = Vn dS+^T (first pass: also the dA0 terms)
      if (tid == 0 && ok) {
        if (DELTA) {
          umma::gemm<64, 64, VD / 16, false, true, FMT>(tmem + cP1, aW, 64, aQ, VD, false);
          umma::gemm<64, 64, VD / 16, true, true, FMT>(tmem + cP2, aDvn, VD, aEx, VD, false);
          if (hh == 0) {
            umma::gemm<64, KD, 4, false, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
            umma::gemm<64, KD, 4, true, true, FMT>(tmem + cK, aXb, 64, aK, 64, true);
          }
        } else {
          umma::gemm<64, 64, VD / 16, false, true, FMT>(tmem + cP2, aDvn, 64, aEx, VD, false);
        }
        umma::commit(bars + (hh == 0 ? M3 : M4));
      }
      __syncwarp();
      {  // keep gamma <S, dS+> over this half while the products run (both tiles share one layout)
        const uint4* a = reinterpret_cast<const uint4*>(qS);
        const uint4* b = reinterpret_cast<const uint4*>(exS);
#pragma unroll
        for (int k4 = 0; k4 < VD * 64 * 2 / 16 / NTHREADS; ++k4) {
          const uint4 x = a[tid + k4 * NTHREADS], y = b[tid + k4 * NTHREADS];
          const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 u = unpack2<T>(xs[e]), v = unpack2<T>(ys[e]);
            sdot_part += u.x * v.x + u.y * v.y;
          }
        }
      }
      __syncthreads();  // every thread is past its reads of the two half tiles
      ok = ok && umma::mbar_wait(bars + (hh == 0 ? M3 : M4), hh == 0 ? ph : 1u);
      umma::fence_after_sync();
      if (hh == 0) {
        if (tid == 0 && ok) {  // the products are done with the half tiles too: fetch the second halves
          tma::expect_tx(bars + L2, 2 * VD * 64 * 2);
          tma::load_3d(qS, &maps.h, 64, 0, item * VD, bars + L2);
          tma::load_3d(exS, &maps.dh, 64, 0, item * VD, bars + L2);
        }
      } else if (nxt >= 0 && ok) {  // every product of this unit is done: the next unit's tiles may land
        if (tid == 0) load_first(nxt);
        first_inflight = true;
        if (tid < 64) load_vec(nxt, (it & 1) ^ 1);
      }
      __syncwarp();
      if (ok) {  // dk columns and the state terms of dG
        const int kc = 64 * hh + cc0;
        float accK[4][4], accT[4][4];
        umma::ld_16x256b<4>(accK, tl + cK + kc);
        if (DELTA) {
          umma::ld_16x256b<4>(accT, tl + cP1 + cc0);
          umma::wait_ld();
          const float gam0 = gam[i0], gam1 = gam[i1];
#pragma unroll
          for (int nt = 0; nt < 4; ++nt) {
            accT[nt][0] *= gam0;
            accT[nt][1] *= gam0;
            accT[nt][2] *= gam1;
            accT[nt][3] *= gam1;
#pragma unroll
            for (int e = 0; e < 4; ++e) accK[nt][e] -= accT[nt][e];
          }
          float d0 = 0.f, d1 = 0.f;
          row_dots_part<T, 4>(accT, kS, r0, kc, lane, d0, d1);
          rG0 -= d0;
          rG1 -= d1;
        }
        umma::ld_16x256b<4>(accT, tl + cP2 + cc0);
        umma::wait_ld();
        const float gamr0 = gamr[i0], gamr1 = gamr[i1];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          accT[nt][0] *= gamr0;
          accT[nt][1] *= gamr0;
          accT[nt][2] *= gamr1;
          accT[nt][3] *= gamr1;
#pragma unroll
          for (int e = 0; e < 4; ++e) accK[nt][e] += accT[nt][e];
        }
        float d0 = 0.f, d1 = 0.f;
        row_dots_part<T, 4>(accT, kS, r0, kc, lane, d0, d1);
        rG0 -= d0;
        rG1 -= d1;
        tot_part += d0 + d1;
        store_key_grad<T, 4>(accK, p.dk_acc, p.dk, m.tok0, i0, m.len, kc, t, p.H, h, p.Hk, hk);
      }
      if (hh == 0) {
        ok = ok && umma::mbar_wait(bars + L2, ph);
        umma::fence_before_sync();
        __syncthreads();  // every warp has read the two 64 x 64 accumulators of the first half
        umma::fence_after_sync();
      }
    }
    // ---- fold the per-thread and per-warp partial sums --------------------------------------------------------------
    rG0 = quad_sum(rG0);
    rG1 = quad_sum(rG1);
    rB0 = quad_sum(rB0);
    rB1 = quad_sum(rB1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      tot_part += __shfl_xor_sync(0xffffffffu, tot_part, off);
      sdot_part += __shfl_xor_sync(0xffffffffu, sdot_part, off);
    }
    if (t == 0) {
      rowG[cq * 64 + i0] = rG0;
      rowG[cq * 64 + i1] = rG1;
      rowB[cq * 64 + i0] = rB0;
      rowB[cq * 64 + i1] = rB1;
    }
    if (lane == 0) {
      tot[warp] = tot_part;
      sdot[warp] = sdot_part;
    }
    umma::fence_before_sync();
    ok = __syncthreads_and(ok);  // k and the accumulators are final for this unit
    umma::fence_after_sync();
    if (!ok) break;
    if (nxt >= 0) {
      if (tid == 0) load_k(nxt);
      k_inflight = true;
    }
    if (tid < 64) {
      float dG = dga + rowG[tid] + rowG[64 + tid];
      if (DELTA) dG -= colF[tid] + colF[64 + tid] + colF[128 + tid] + colF[192 + tid];
      if (tid == 63) {
#pragma unroll
        for (int w = 0; w < 8; ++w) dG += tot[w];
      }
      dGv[tid] = dG;
    }
    __syncthreads();
    if (tid < 64) {  // dg = reverse cumulative sum of dG over the chunk
      float acc = 0.f;
      for (int j = 63; j >= tid; --j) acc += dGv[j];
      float sd = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) sd += sdot[w];
      acc += keep_gamma(Gs, runs, m.flags) * sd;
      if (tid < m.len) {
        if (p.dg) p.dg[((long)m.tok0 + tid) * p.H + h] = acc;
        if (DELTA) {
          p.dbeta[((long)m.tok0 + tid) * p.H + h] =
              rowB[tid] + rowB[64 + tid] + colB[tid] + colB[64 + tid] + colB[128 + tid] + colB[192 + tid];
        }
      }
    }
    item = nxt;
  }
  if (!ok) {  // let requested copies land before the shared memory goes away (bounded waits)
    if (first_inflight || k_inflight) {
      if (!k_inflight && tid == 0) load_k(next_live(item - (int)gridDim.x));  // complete the byte count of the phase
      umma::mbar_wait(bars + L0, 0), umma::mbar_wait(bars + L0, 1);
    }
    if (tid == 0) atomicExch(p.status, 1);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 1) umma::tmem_dealloc(tmem, 256);
}

template <typename T, bool DELTA>
int launch_pair(const GradMaps& maps, const GradParams& gp, int blocks, cudaStream_t s) {
  int dev = 0, sms = 0;
  JLA_CUDA_OK(cudaGetDevice(&dev));
  JLA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  auto* kq = sg_grads_q_tc_kernel<T, DELTA>;
  auto* kk = sg_grads_k_tc_kernel<T, DELTA>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemQ::kBytes));
  JLA_CUDA_OK(cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemK::kBytes));
  {
    ProfScope ps(kProfSgGradsQ, s);
    kq<<<blocks < 2 * sms ? blocks : 2 * sms, NTHREADS, SmemQ::kBytes, s>>>(maps, gp);
  }
  JLA_LAUNCH_OK();
  {
    ProfScope ps(kProfSgGradsK, s);
    kk<<<blocks < 2 * sms ? blocks : 2 * sms, NTHREADS, SmemK::kBytes, s>>>(maps, gp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

// Chunk gradients after the reverse state pass has written dS+^T, dVn^T and dv (= dW). `direct`: dq and dk go
// straight to the output tensors (no head groups to sum, no L2-norm backward), else to the fp32 accumulators.
int launch_chunk_grads_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, bool direct, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (p.K != KD || p.V != VD) return JLA_ERR_UNSUPPORTED;
  const uint64_t tokens = (uint64_t)p.B * p.T, slots = (uint64_t)pl.nc * p.H;
  GradMaps maps;
  bool ok = tma::encode_3d(&maps.q, c.q_eff, p.K, p.Hk, tokens, 64) && tma::encode_3d(&maps.k, c.k_eff, p.K, p.Hk, tokens, 64) &&
            tma::encode_3d(&maps.v, p.v, p.V, p.H, tokens, 64) && tma::encode_3d(&maps.d_o, io.d_o, p.V, p.H, tokens, 64) &&
            tma::encode_3d(&maps.dv, io.dv, p.V, p.H, tokens, 64) &&
            tma::encode_3d(&maps.h, c.res + pl.h, p.K, 1, slots * p.V, p.V) &&
            tma::encode_3d(&maps.dh, scratch + pl.dh, p.K, 1, slots * p.V, p.V);
  if (ok && pl.delta) {
    ok = tma::encode_3d(&maps.vn, c.res + pl.vn, 64, 1, slots * p.V, p.V) &&
         tma::encode_3d(&maps.dvn, scratch + pl.dvn, 64, 1, slots * p.V, p.V) &&
         tma::encode_3d(&maps.w, c.res + pl.w, 64, 1, slots * p.V, p.V) &&
         tma::encode_3d(&maps.t0, c.res + pl.t0, 64, 1, slots * 64, 64);
  } else if (ok) {
    maps.vn = maps.v;
    maps.dvn = maps.v;
    maps.w = maps.v;
    maps.t0 = maps.v;
  }
  if (!ok) return JLA_ERR_CUDA;
  GradParams gp{};
  gp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  gp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  gp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  gp.dq = io.dq;
  gp.dk = io.dk;
  gp.dq_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dq_acc);
  gp.dk_acc = direct ? nullptr : reinterpret_cast<float*>(scratch + pl.dk_acc);
  gp.dg = io.dg;
  gp.dbeta = io.dbeta;
  gp.dp = reinterpret_cast<unsigned char*>(scratch + pl.dp);
  gp.dga = reinterpret_cast<float*>(scratch + pl.dga);
  gp.H = p.H;
  gp.Hk = p.Hk;
  gp.scale = p.scale;
  gp.nitems = pl.nc * p.H;
  gp.status = tc_status_ptr();
  if (!gp.status) return JLA_ERR_CUDA;
  const int blocks = pl.nc * p.H;
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_pair<__nv_bfloat16, true>(maps, gp, blocks, s) : launch_pair<__nv_bfloat16, false>(maps, gp, blocks, s);
  }
  return pl.delta ? launch_pair<__half, true>(maps, gp, blocks, s) : launch_pair<__half, false>(maps, gp, blocks, s);
}

}  // namespace jla
