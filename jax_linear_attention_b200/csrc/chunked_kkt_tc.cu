// T0 = (I + strict_lower(beta_i k_i.k_j, same document))^-1 and its gated form Ag = T0 D beta_j for K = 128 on the
// Blackwell tensor cores (the UT transform of the delta rule; reference: kkt_fwd,
// src/jla/ops/mosaic_gpu/gated_delta_rule_kernels.py:351-453 -- K K^T on the tensor cores, 16 x 16 diagonal blocks
// by fp32 substitution, 16 -> 32 -> 64 merges as tensor-core products in the operand dtype, :323-333).
//
// One CTA of four warps per (chunk, head) unit, persistent over units, several CTAs per SM (about 31 KB of shared
// memory and 64 TMEM columns each) so that one unit's chain of dependent products overlaps the others'. Per unit:
//
//   A   = beta_i (K K^T)_ij for j < i in one document        tcgen05.mma, M = N = 64, eight k-steps; TMA-landed k tile
//   D   = blockdiag of the four inverted 16 x 16 diagonal blocks of I + A    fp32 forward substitution, 64 threads
//   X32 = D - D (L1 D)      L1 = blocks (1,0) and (3,2) of A   the exact inverse of the two 32 x 32 diagonal blocks,
//   X64 = X32 - X32 (L2 X32)   L2 = block rows 32-63, cols 0-31     because (D L1)^2 = 0 and (X32 L2)^2 = 0
//
// i.e. four 64 x 64 x 64 products per unit with 16-bit operands and fp32 accumulation in TMEM, each followed by a
// register epilogue (accumulator fragments of rows 16 w .. 16 w + 15 for warp w). The operand tiles live in
// 128-byte-swizzled shared memory; a product reads its left factor K-major and its right factor MN-major, so no
// transposed copy is ever made. The k tile's space is reused for D / X32 and L1 once K K^T is done.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {
namespace {

using umma::swz_tile;

constexpr int KD = 128;
constexpr int kDiagLd = 17;  // fp32 diagonal blocks [4][16][17]

struct KktTcParams {
  const ChunkMeta* meta;
  const float* gates;
  const unsigned char* runs;
  void* t0;
  void* ag;
  int H, Hk;
  int nitems;
  int* status;
};

struct SmemKkt {
  static constexpr int kK = 0;             // k tile [64 x 128] (two column blocks); later D / X32 (first 8 KB) and L1 / T1
  static constexpr int kL2 = 64 * KD * 2;  // L2 / T2 tile [64 x 64]
  static constexpr int kDiag = kL2 + 8192;
  static constexpr int kVec = kDiag + 4 * 16 * kDiagLd * 4;  // beta[64], G[64] f32; runs[64] u8
  static constexpr int kBars = kVec + 2 * 256 + 64;
  static constexpr int kBytes = kBars + 2 * 8 + 16 + 1024;
  static_assert(kBars % 8 == 0, "mbarrier alignment");
};

template <typename T>
__device__ __forceinline__ void store_frag_swz(unsigned char* tile, int r0, const float (&acc)[8][4], int lane) {
  T* dst = reinterpret_cast<T*>(tile);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const int col = nt * 8 + 2 * t;
    *reinterpret_cast<uint32_t*>(dst + swz_tile(64, r0 + g, col)) = pack2<T>(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<uint32_t*>(dst + swz_tile(64, r0 + g + 8, col)) = pack2<T>(acc[nt][2], acc[nt][3]);
  }
}

template <typename T>
__global__ void __launch_bounds__(128, 5) kkt_inv_tc_kernel(const __grid_constant__ CUtensorMap kmap, KktTcParams p) {
  using L = SmemKkt;
  constexpr int FMT = umma::Fmt<T>::value;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * warp, i0 = r0 + g, i1 = r0 + g + 8;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* kS = base + L::kK;
  unsigned char* dS = base + L::kK;          // D, then X32 (over the first column block of the consumed k tile)
  unsigned char* l1S = base + L::kK + 8192;  // L1, then T1 = L1 D (over the second column block)
  unsigned char* l2S = base + L::kL2;        // L2, then T2 = L2 X32; finally the row-major copy of Ag for the stores
  float* diag = reinterpret_cast<float*>(base + L::kDiag);
  float* betas = reinterpret_cast<float*>(base + L::kVec);
  float* Gs = betas + 64;
  unsigned char* runs = reinterpret_cast<unsigned char*>(Gs + 64);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + L::kBars);  // [0] TMA load, [1] MMA completion
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  const uint32_t aK = umma::smem_addr(kS), aD = umma::smem_addr(dS), aL1 = umma::smem_addr(l1S), aL2 = umma::smem_addr(l2S);

  if (tid == 0) {
    umma::mbar_init(bars + 0, 1);
    umma::mbar_init(bars + 1, 1);
    umma::mbar_init_fence();
  }
  if (warp == 0) umma::tmem_alloc(tmem_slot, 64);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * warp) << 16);  // this warp's lane quadrant (rows 16 w .. of an M = 64 product)

  auto next_live = [&](int it) {
    while (it < p.nitems && p.meta[it / p.H].len == 0) it += gridDim.x;
    return it;
  };
  bool ok = true;
  uint32_t lph = 0, mph = 0;  // phases of the two barriers
  auto sync_tc = [&]() {      // generic-proxy writes of every thread -> visible to the next product
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
  };
  auto product = [&](uint32_t a_tile, uint32_t b_tile) {  // acc = a (K-major) x b (MN-major), 64 x 64 x 64; all threads wait
    if (tid == 0 && ok) {
      umma::gemm<64, 64, 4, false, true, FMT>(tmem, a_tile, 64, b_tile, 64, false);
      umma::commit(bars + 1);
    }
    __syncwarp();
    ok = ok && umma::mbar_wait(bars + 1, mph);
    mph ^= 1;
    umma::fence_after_sync();
  };

  for (int item = next_live(blockIdx.x); item < p.nitems; item = next_live(item + gridDim.x)) {
    const int c = item / p.H, h = item - c * p.H;
    const int hk = h / (p.H / p.Hk);
    const ChunkMeta m = p.meta[c];
    if (tid == 0) {
      tma::expect_tx(bars + 0, 64 * KD * 2);
      tma::load_tile<64, KD>(kS, &kmap, 0, hk, m.tok0, bars + 0);
    }
    if (tid < 64) {
      betas[tid] = p.gates[(long)item * 128 + 64 + tid];
      Gs[tid] = p.gates[(long)item * 128 + tid];
      runs[tid] = p.runs[(long)c * 64 + tid];
    }
    ok = ok && umma::mbar_wait(bars + 0, lph);
    lph ^= 1;
    if (m.len < 64) {  // rows past the end of a partial chunk hold other rows' keys: they must act as zero keys
      T* kt = reinterpret_cast<T*>(kS);
      for (int idx = tid; idx < (64 - m.len) * (KD / 8); idx += 128) {
        const int r = m.len + idx / (KD / 8), c8 = (idx % (KD / 8)) * 8;
        *reinterpret_cast<uint4*>(kt + swz_tile(64, r, c8)) = make_uint4(0, 0, 0, 0);
      }
    }
    sync_tc();
    // ---- K K^T
    if (tid == 0 && ok) {
      umma::gemm<64, 64, KD / 16, false, false, FMT>(tmem, aK, 64, aK, 64, false);
      umma::commit(bars + 1);
    }
    __syncwarp();
    ok = ok && umma::mbar_wait(bars + 1, mph);
    mph ^= 1;
    umma::fence_after_sync();
    float acc[8][4];
    umma::ld_16x256b<8>(acc, tl);
    umma::wait_ld();
    // ---- A = beta_i (k_i . k_j) below the diagonal inside one document; split into the diagonal blocks (fp32), L1, L2
    {
      const float b0 = betas[i0], b1 = betas[i1];
      const int run0 = runs[i0], run1 = runs[i1];
      // (every thread holds its K K^T fragment in registers and the product is complete: once all warps are past the
      // barrier below the k tile may be overwritten by D, L1)
      __syncthreads();
      T* l1t = reinterpret_cast<T*>(l1S);
      T* l2t = reinterpret_cast<T*>(l2S);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float a[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (e >> 1) ? i1 : i0, j = nt * 8 + 2 * t + (e & 1);
          a[e] = (j < i && runs[j] == ((e >> 1) ? run1 : run0)) ? ((e >> 1) ? b1 : b0) * acc[nt][e] : 0.f;
          if ((i >> 4) == (j >> 4)) diag[((i >> 4) * 16 + (i & 15)) * kDiagLd + (j & 15)] = a[e];
        }
        const int col = nt * 8 + 2 * t, bj = nt >> 1;  // both columns of the pair lie in block column bj
        const int bi = warp;                            // rows i0 and i1 lie in block row `warp`
        const bool in1 = (bj + 1 == bi) && (bi & 1);    // blocks (1,0) and (3,2)
        const bool in2 = bi >= 2 && bj < 2;             // rows 32-63, columns 0-31
        *reinterpret_cast<uint32_t*>(l1t + swz_tile(64, i0, col)) = in1 ? pack2<T>(a[0], a[1]) : 0u;
        *reinterpret_cast<uint32_t*>(l1t + swz_tile(64, i1, col)) = in1 ? pack2<T>(a[2], a[3]) : 0u;
        *reinterpret_cast<uint32_t*>(l2t + swz_tile(64, i0, col)) = in2 ? pack2<T>(a[0], a[1]) : 0u;
        *reinterpret_cast<uint32_t*>(l2t + swz_tile(64, i1, col)) = in2 ? pack2<T>(a[2], a[3]) : 0u;
      }
      for (int idx = tid; idx < 512; idx += 128) reinterpret_cast<uint4*>(dS)[idx] = make_uint4(0, 0, 0, 0);  // D starts as zero
    }
    __syncthreads();
    // ---- the four 16 x 16 diagonal blocks of (I + A)^-1 by forward substitution, one column per thread
    if (tid < 64) {
      const int b = tid >> 4, col = tid & 15;
      const float* Ab = diag + b * 16 * kDiagLd;
      T* dt = reinterpret_cast<T*>(dS);
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float s = (i == col) ? 1.f : 0.f;
#pragma unroll
        for (int mm = 0; mm < i; ++mm) s -= Ab[i * kDiagLd + mm] * x[mm];
        x[i] = s;
        dt[swz_tile(64, 16 * b + i, 16 * b + col)] = from_f32<T>(s);
      }
    }
    sync_tc();
    // ---- 16 -> 32: X32 = D - D (L1 D)
    product(aL1, aD);  // T1 = L1 D
    umma::ld_16x256b<8>(acc, tl);
    umma::wait_ld();
    umma::fence_before_sync();
    __syncthreads();  // every warp has read the accumulator and the product has consumed L1
    store_frag_swz<T>(l1S, r0, acc, lane);
    sync_tc();
    product(aD, aL1);  // U1 = D T1
    umma::ld_16x256b<8>(acc, tl);
    umma::wait_ld();
    {
      const T* dt = reinterpret_cast<const T*>(dS);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        const float2 da = unpack2<T>(*reinterpret_cast<const uint32_t*>(dt + swz_tile(64, i0, col)));
        const float2 db = unpack2<T>(*reinterpret_cast<const uint32_t*>(dt + swz_tile(64, i1, col)));
        acc[nt][0] = da.x - acc[nt][0];
        acc[nt][1] = da.y - acc[nt][1];
        acc[nt][2] = db.x - acc[nt][2];
        acc[nt][3] = db.y - acc[nt][3];
      }
    }
    umma::fence_before_sync();
    __syncthreads();  // the product has consumed D, every thread has read its part of it
    store_frag_swz<T>(dS, r0, acc, lane);  // X32 in place of D
    sync_tc();
    // ---- 32 -> 64: X64 = X32 - X32 (L2 X32)
    product(aL2, aD);  // T2 = L2 X32
    umma::ld_16x256b<8>(acc, tl);
    umma::wait_ld();
    umma::fence_before_sync();
    __syncthreads();
    store_frag_swz<T>(l2S, r0, acc, lane);
    sync_tc();
    product(aD, aL2);  // U2 = X32 T2
    float (&x64)[8][4] = acc;
    umma::ld_16x256b<8>(x64, tl);
    umma::wait_ld();
    {
      const T* dt = reinterpret_cast<const T*>(dS);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        const float2 da = unpack2<T>(*reinterpret_cast<const uint32_t*>(dt + swz_tile(64, i0, col)));
        const float2 db = unpack2<T>(*reinterpret_cast<const uint32_t*>(dt + swz_tile(64, i1, col)));
        x64[nt][0] = da.x - x64[nt][0];
        x64[nt][1] = da.y - x64[nt][1];
        x64[nt][2] = db.x - x64[nt][2];
        x64[nt][3] = db.y - x64[nt][3];
      }
    }
    // ---- T0 and Ag = T0 exp(G_i - G_j) beta_j (same document, j <= i) through shared memory so that the global stores
    // are full 16-byte vectors of a row-major tile: T0 over the (consumed) L1 tile, Ag over the L2 tile
    umma::fence_before_sync();
    __syncthreads();  // the last product has consumed X32 and T2
    {
      const float G0 = Gs[i0], G1 = Gs[i1];
      const int run0 = runs[i0], run1 = runs[i1];
      T* t0t = reinterpret_cast<T*>(l1S);  // (swizzled: conflict-free; the copy below undoes the chunk permutation)
      T* agt = reinterpret_cast<T*>(l2S);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float a[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (e >> 1) ? i1 : i0, j = nt * 8 + 2 * t + (e & 1);
          const bool on = j <= i && runs[j] == ((e >> 1) ? run1 : run0);
          a[e] = on ? x64[nt][e] * __expf(((e >> 1) ? G1 : G0) - Gs[j]) * betas[j] : 0.f;
        }
        const int col = nt * 8 + 2 * t;
        *reinterpret_cast<uint32_t*>(t0t + swz_tile(64, i0, col)) = pack2<T>(x64[nt][0], x64[nt][1]);
        *reinterpret_cast<uint32_t*>(t0t + swz_tile(64, i1, col)) = pack2<T>(x64[nt][2], x64[nt][3]);
        *reinterpret_cast<uint32_t*>(agt + swz_tile(64, i0, col)) = pack2<T>(a[0], a[1]);
        *reinterpret_cast<uint32_t*>(agt + swz_tile(64, i1, col)) = pack2<T>(a[2], a[3]);
      }
    }
    __syncthreads();
    {
      uint4* o0 = reinterpret_cast<uint4*>(static_cast<T*>(p.t0) + (size_t)item * 4096);
      uint4* o1 = reinterpret_cast<uint4*>(static_cast<T*>(p.ag) + (size_t)item * 4096);
      const uint4* s0 = reinterpret_cast<const uint4*>(l1S);
      const uint4* s1 = reinterpret_cast<const uint4*>(l2S);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = tid + 128 * i, r = idx >> 3, ch = idx & 7;
        o0[idx] = s0[r * 8 + (ch ^ (r & 7))];
        o1[idx] = s1[r * 8 + (ch ^ (r & 7))];
      }
    }
    ok = __syncthreads_and(ok);  // the tiles may be reused; a wait that gave up ends the CTA's work
    if (!ok) break;
  }
  if (!ok && tid == 0) atomicExch(p.status, 4);
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 64);
}

template <typename T>
int launch_one(const CUtensorMap& kmap, const KktTcParams& kp, cudaStream_t s) {
  int dev = 0, sms = 0;
  JLA_CUDA_OK(cudaGetDevice(&dev));
  JLA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  auto* kern = kkt_inv_tc_kernel<T>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemKkt::kBytes));
  const int per_sm = 5;  // registers allow five CTAs per SM (31 KB of shared memory and 64 TMEM columns each)
  const int blocks = kp.nitems < per_sm * sms ? kp.nitems : per_sm * sms;
  {
    ProfScope ps(kProfKktInv, s);
    kern<<<blocks, 128, SmemKkt::kBytes, s>>>(kmap, kp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

// T0 and Ag of every (chunk, head) for the scalar-gate delta-rule kinds with K = 128 (after the chunk table and the
// gate vectors have been built); same outputs as kkt_inv_kernel of chunked_prep.cu.
int launch_kkt_tc(const ChunkedCtx& c, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (p.K != KD) return JLA_ERR_UNSUPPORTED;
  CUtensorMap kmap;
  if (!tma::encode_3d(&kmap, c.k_eff, p.K, p.Hk, (uint64_t)p.B * p.T, 64)) return JLA_ERR_CUDA;
  KktTcParams kp{};
  kp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  kp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  kp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  kp.t0 = c.res + pl.t0;
  kp.ag = c.res + pl.ag;
  kp.H = p.H;
  kp.Hk = p.Hk;
  kp.nitems = pl.nc * p.H;
  kp.status = tc_status_ptr();
  if (!kp.status) return JLA_ERR_CUDA;
  return p.dtype == JLA_DTYPE_BF16 ? launch_one<__nv_bfloat16>(kmap, kp, s) : launch_one<__half>(kmap, kp, s);
}

}  // namespace jla
