// Forward of the scalar-gate family for K = V = 128 on the Blackwell tensor cores, one persistent CTA per
// (row, head) walking the row's chunks. Everything on the serial chain lives in TMEM and registers:
//
//   * the state is kept TRANSPOSED, S^T [V lanes x K columns] fp32, as the accumulator of the update product;
//     a bf16/f16 copy of it (packed pairs) sits next to it and is the A operand (from TMEM) of S^T K^T and S^T Q^T;
//   * W^T = V^T - (cin Gamma)_j (S^T K^T), Vn^T = W^T Ag^T and (tail Gamma_r Vn)^T are produced by four warps whose
//     thread index IS the value row v, written back to TMEM as packed 16-bit A operands; no shared-memory round
//     trip and no CTA-wide barrier sits between two dependent products;
//   * per chunk the chain is  S^T K^T -> W^T -> W^T Ag^T -> Vn^T -> S^T += (Gamma_r Vn)^T K  (three M = 128 products),
//     while a second group of four warps builds P = (Q K^T) D and Ag = T0 D beta (64 x 64 tiles, into swizzled shared
//     memory) one chunk ahead and writes the outputs O^T = scale[(cin Gamma)_i (S^T Q^T) + Vn^T P^T];
//   * one thread issues all tcgen05.mma, one thread issues the TMA loads (q, k, v, T0 tiles, gate vectors) into a
//     3-stage ring; mbarriers (bounded waits, shared abort flag) connect the roles.
//
// Same math and roundings as sg_fwd_kernel (chunked_fwd.cu). The residuals it saves are transposed
// (h^T [V][K], Vn^T [V][64] per chunk and head) because a thread owns a value row.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {
namespace {

using umma::swz_tile;

constexpr int K = 128, V = 128;
constexpr int NS = 3;  // stages of the input ring

struct FwdTcMaps {
  CUtensorMap q, k, v, t0;
};

struct FwdTcParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;
  const unsigned char* runs;
  const float* h0;
  void* o;
  float* final_state;
  void *hT_out, *vnT_out;  // residuals (nullptr when not saving)
  int H, Hk;
  float scale;
  int* status;
};

struct Smem {
  static constexpr int kStage = 64 * K * 2 * 2 + 64 * V * 2 + 8192;  // q, k, v, T0
  static constexpr int kTiles = NS * kStage;
  static constexpr int kPb = kTiles;            // P tiles [2][64x64]
  static constexpr int kAgb = kPb + 2 * 8192;   // Ag tiles [2][64x64]
  static constexpr int kGates = kAgb + 2 * 8192;         // per stage: G[64], beta[64] f32 (512 B) + runs (64 B) + meta (16 B)
  static constexpr int kGateStride = 640;
  static constexpr int kScal = kGates + NS * kGateStride;  // per stage and warp: gam[64], gamr[64] (state group); gam[64] (score group)
  static constexpr int kBars = kScal + NS * 3072;
  static constexpr int kNumBars = 2 * NS + 16;
  static constexpr int kBytes = kBars + kNumBars * 8 + 64 + 1024;
};

enum {  // mbarrier indices after the 2 * NS full / empty barriers
  B_PDONE = 2 * NS, B_PFREE, B_PA0, B_PA1, B_ST, B_M1, B_W, B_M2, B_VN, B_M3, B_ODONE, B_OFREE
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(bar)) : "memory");
}

// Bounded wait that also gives up as soon as another role has raised the abort flag.
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t addr = umma::smem_addr(bar);
  for (uint32_t spin = 0; spin < umma::kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void bulk_copy(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   umma::smem_addr(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(umma::smem_addr(bar))
               : "memory");
}

template <typename T>
__device__ __forceinline__ void ld_row32(float (&v)[32], uint32_t taddr) {
  umma::ld_32x32b_x32(v, taddr);
  umma::wait_ld();
}

template <typename T, bool DELTA>
__global__ void __launch_bounds__(384, 1) sg_fwd_tc_kernel(const __grid_constant__ FwdTcMaps maps, FwdTcParams p) {
  constexpr int FMT = umma::Fmt<T>::value;
  const int row = blockIdx.x / p.H, h = blockIdx.x - row * p.H;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int2 rc = p.row_chunks[row];
  const int n = rc.y;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  auto st_q = [&](int s) { return base + s * Smem::kStage; };
  auto st_k = [&](int s) { return st_q(s) + 64 * K * 2; };
  auto st_v = [&](int s) { return st_k(s) + 64 * K * 2; };
  auto st_t0 = [&](int s) { return st_v(s) + 64 * V * 2; };
  auto st_G = [&](int s) { return reinterpret_cast<float*>(base + Smem::kGates + s * Smem::kGateStride); };
  auto st_runs = [&](int s) { return reinterpret_cast<unsigned char*>(st_G(s) + 128); };
  auto st_meta = [&](int s) { return reinterpret_cast<volatile int*>(st_runs(s) + 64); };
  auto st_gam = [&](int s) { return reinterpret_cast<float*>(base + Smem::kScal + s * 3072); };
  unsigned char* Pb = base + Smem::kPb;
  unsigned char* Agb = base + Smem::kAgb;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      umma::mbar_init(bars + s, 1);                  // full: the producer's expect_tx arrival (+ bytes)
      umma::mbar_init(bars + NS + s, 1 + 4 + 4);     // empty: MMA commit + the warps of both groups
    }
    umma::mbar_init(bars + B_PDONE, 1);
    umma::mbar_init(bars + B_PFREE, 4);
    umma::mbar_init(bars + B_PA0, 4);
    umma::mbar_init(bars + B_PA1, 4);
    umma::mbar_init(bars + B_ST, 4);
    umma::mbar_init(bars + B_M1, 1);
    umma::mbar_init(bars + B_W, 4);
    umma::mbar_init(bars + B_M2, 1);
    umma::mbar_init(bars + B_VN, 4);
    umma::mbar_init(bars + B_M3, 1);
    umma::mbar_init(bars + B_ODONE, 1);
    umma::mbar_init(bars + B_OFREE, 4);
    umma::mbar_init_fence();
    *abort_flag = 0;
  }
  if (warp == 2) umma::tmem_alloc(tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cS = 0, cSb = 128, cA1 = 192, cWb = 256, cVg = 288, cO1 = 320, cO2 = 384, cP = 448;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it % NS, c = rc.x + it;
        if (!wait(bars + NS + s, ((it / NS) & 1) ^ 1, abort_flag)) break;
        const ChunkMeta m = p.meta[c];
        volatile int* ms = st_meta(s);
        ms[0] = m.tok0;
        ms[1] = m.len;
        ms[2] = m.flags;
        const uint32_t bytes = 64 * K * 2 * 2 + 64 * V * 2 + (DELTA ? 8192 : 0) + 512 + 64;
        tma::expect_tx(bars + s, bytes);
        tma::load_tile<64, K>(st_k(s), &maps.k, 0, hk, m.tok0, bars + s);
        tma::load_tile<64, K>(st_q(s), &maps.q, 0, hk, m.tok0, bars + s);
        tma::load_tile<64, V>(st_v(s), &maps.v, 0, h, m.tok0, bars + s);
        if (DELTA) tma::load_tile<64, 64>(st_t0(s), &maps.t0, 0, 0, (c * p.H + h) * 64, bars + s);
        bulk_copy(st_G(s), p.gates + ((long)c * p.H + h) * 128, 512, bars + s);
        bulk_copy(st_runs(s), p.runs + (long)c * 64, 64, bars + s);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it % NS;
        const uint32_t ph = it & 1;
        const uint32_t aq = umma::smem_addr(st_q(s)), ak = umma::smem_addr(st_k(s));
        if (!wait(bars + s, (it / NS) & 1, abort_flag)) break;
        if (!wait(bars + B_PFREE, ph ^ 1, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP, aq, 64, ak, 64, false);  // Q K^T
        umma::commit(bars + B_PDONE);
        if (!wait(bars + B_ST, ph, abort_flag)) break;
        if (!wait(bars + B_OFREE, ph ^ 1, abort_flag)) break;
        umma::fence_after_sync();
        if (DELTA) umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cA1, tmem + cSb, ak, 64, false);  // S^T K^T
        umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cO1, tmem + cSb, aq, 64, false);             // S^T Q^T
        umma::commit(bars + B_M1);
        if (!wait(bars + B_PA0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
        if (DELTA) {
          if (!wait(bars + B_W, ph, abort_flag)) break;
          umma::fence_after_sync();
          umma::gemm_ts<128, 64, 4, false, FMT>(tmem + cA1, tmem + cWb, umma::smem_addr(Agb + (it & 1) * 8192), 64,
                                                false);  // W^T Ag^T
          umma::commit(bars + B_M2);
        }
        if (!wait(bars + B_VN, ph, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cVg, ak, 64, true);  // S^T += (Gamma_r Vn)^T K
        umma::commit(bars + B_M3);
        umma::gemm_ts<128, 64, 4, false, FMT>(tmem + cO2, tmem + cWb, umma::smem_addr(Pb + (it & 1) * 8192), 64,
                                              false);  // Vn^T P^T
        umma::commit(bars + B_ODONE);
        umma::commit(bars + NS + s);
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------------------- state group (thread = row v)
    const int q4 = warp - 4, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int s = it % NS, c = rc.x + it;
      const uint32_t ph = it & 1;
      ok = wait(bars + s, (it / NS) & 1, abort_flag);
      if (!ok) break;
      const float* Gs = st_G(s);
      const unsigned char* runs = st_runs(s);
      const int len = st_meta(s)[1], flags = st_meta(s)[2];
      float* gam = st_gam(s) + q4 * 128;  // this warp's own copy: no cross-warp barrier on the serial chain
      float* gamr = gam + 64;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = lane + 32 * jj;
        const RowScalars rs = row_scalars(Gs, runs, flags, j);
        gam[j] = rs.gam;
        gamr[j] = (j < len) ? rs.gamr : 0.f;  // tokens past a partial chunk must not write the state
      }
      __syncwarp();
      const float kg = keep_gamma(Gs, runs, flags);
      // ---- the state entering this chunk: 16-bit copy for the products, decayed fp32 copy for the update
      if (it > 0) {
        ok = wait(bars + B_M3, ph ^ 1, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
      }
      T* hT = p.hT_out ? static_cast<T*>(p.hT_out) + (((long)c * p.H + h) * V + v) * K : nullptr;
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        float x[32];
        if (it == 0) {
          const float* h0 = p.h0 ? p.h0 + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = h0 ? h0[(long)(blk * 32 + i) * V + v] : 0.f;
        } else {
          ld_row32<T>(x, tl + cS + blk * 32);
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack2<T>(x[2 * i], x[2 * i + 1]);
        umma::st_32x32b_x16(tl + cSb + blk * 16, pk);
        if (hT) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<uint4*>(hT + blk * 32 + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= kg;
        umma::st_32x32b_x32(tl + cS + blk * 32, x);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_ST);

      const T* vs = reinterpret_cast<const T*>(st_v(s));
      if (DELTA) {
        // ---- W^T = V^T - (cin Gamma)_j (S^T K^T)
        ok = wait(bars + B_M1, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          float x[32];
          ld_row32<T>(x, tl + cA1 + blk * 32);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = blk * 32 + 2 * i;
            const float w0 = to_f32(vs[swz_tile(64, j, v)]) - gam[j] * x[2 * i];
            const float w1 = to_f32(vs[swz_tile(64, j + 1, v)]) - gam[j + 1] * x[2 * i + 1];
            pk[i] = pack2<T>(w0, w1);
          }
          umma::st_32x32b_x16(tl + cWb + blk * 16, pk);
        }
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_W);
        // ---- Vn^T = W^T Ag^T
        ok = wait(bars + B_M2, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        T* vnT = p.vnT_out ? static_cast<T*>(p.vnT_out) + (((long)c * p.H + h) * V + v) * 64 : nullptr;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          float x[32];
          ld_row32<T>(x, tl + cA1 + blk * 32);
          uint32_t pk[16], pg[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = blk * 32 + 2 * i;
            pk[i] = pack2<T>(x[2 * i], x[2 * i + 1]);
            pg[i] = pack2<T>(x[2 * i] * gamr[j], x[2 * i + 1] * gamr[j + 1]);
          }
          umma::st_32x32b_x16(tl + cWb + blk * 16, pk);
          umma::st_32x32b_x16(tl + cVg + blk * 16, pg);
          if (vnT) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              *reinterpret_cast<uint4*>(vnT + blk * 32 + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
          }
        }
      } else {
        // ---- Vn = V: the value rows themselves, and their Gamma_r-scaled copy
        if (it > 0) {  // the previous chunk's Vn^T P^T must have consumed the operand columns
          ok = wait(bars + B_ODONE, ph ^ 1, abort_flag);
          if (!ok) break;
          umma::fence_after_sync();
        }
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          uint32_t pk[16], pg[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = blk * 32 + 2 * i;
            const float a = to_f32(vs[swz_tile(64, j, v)]), b = to_f32(vs[swz_tile(64, j + 1, v)]);
            pk[i] = pack2<T>(a, b);
            pg[i] = pack2<T>(a * gamr[j], b * gamr[j + 1]);
          }
          umma::st_32x32b_x16(tl + cWb + blk * 16, pk);
          umma::st_32x32b_x16(tl + cVg + blk * 16, pg);
        }
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bars + B_VN);
        mbar_arrive(bars + NS + s);  // done with this stage's v and gate vectors
      }
    }
    // ---- final state
    if (ok && n > 0) ok = wait(bars + B_M3, (n - 1) & 1, abort_flag);
    umma::fence_after_sync();
    if (ok && p.final_state) {
      float* f = p.final_state + ((long)row * p.H + h) * K * V;
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        float x[32];
        if (n == 0) {
          const float* h0 = p.h0 ? p.h0 + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = h0 ? h0[(long)(blk * 32 + i) * V + v] : 0.f;
        } else {
          ld_row32<T>(x, tl + cS + blk * 32);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) f[(long)(blk * 32 + i) * V + v] = x[i];
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------- score group: P, Ag one chunk ahead; outputs
    const int q4 = warp - 8, g = lane >> 2, t = lane & 3;
    const int r0 = 16 * q4, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    auto build = [&](int it) {  // P = (Q K^T) D and Ag = T0 D beta_j of chunk `it`, rows r0 .. r0 + 15
      const int s = it % NS, buf = it & 1;
      if (!wait(bars + s, (it / NS) & 1, abort_flag)) return false;
      const float* Gs = st_G(s);
      const float* betas = Gs + 64;
      const unsigned char* runs = st_runs(s);
      if (!wait(bars + B_PDONE, it & 1, abort_flag)) return false;
      umma::fence_after_sync();
      float acc[8][4];
      umma::ld_16x256b<8>(acc, tl + cP);
      umma::wait_ld();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_PFREE);
      const int i0 = r0 + g, i1 = r0 + g + 8;
      const float G0 = Gs[i0], G1 = Gs[i1];
      const int run0 = runs[i0], run1 = runs[i1];
      T* pt = reinterpret_cast<T*>(Pb + buf * 8192);
      T* at = reinterpret_cast<T*>(Agb + buf * 8192);
      const T* t0t = reinterpret_cast<const T*>(st_t0(s));
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int j = nt * 8 + 2 * t;
        const float d00 = decay_ij(Gs, runs, i0, j, G0, run0), d01 = decay_ij(Gs, runs, i0, j + 1, G0, run0);
        const float d10 = decay_ij(Gs, runs, i1, j, G1, run1), d11 = decay_ij(Gs, runs, i1, j + 1, G1, run1);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i0, j)) = pack2<T>(acc[nt][0] * d00, acc[nt][1] * d01);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i1, j)) = pack2<T>(acc[nt][2] * d10, acc[nt][3] * d11);
        if (DELTA) {
          const float2 ta = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i0, j)));
          const float2 tb = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0t + swz_tile(64, i1, j)));
          const float b0 = betas[j], b1 = betas[j + 1];
          *reinterpret_cast<uint32_t*>(at + swz_tile(64, i0, j)) = pack2<T>(ta.x * d00 * b0, ta.y * d01 * b1);
          *reinterpret_cast<uint32_t*>(at + swz_tile(64, i1, j)) = pack2<T>(tb.x * d10 * b0, tb.y * d11 * b1);
        }
      }
      umma::fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_PA0 + buf);
      return true;
    };
    if (n > 0) ok = build(0);
    for (int it = 0; it < n && ok; ++it) {
      const int s = it % NS;
      if (it + 1 < n) {
        ok = build(it + 1);
        if (!ok) break;
      }
      // ---- O^T = scale [(cin Gamma)_i (S^T Q^T) + Vn^T P^T], thread = value row v
      ok = wait(bars + B_ODONE, it & 1, abort_flag);
      if (!ok) break;
      umma::fence_after_sync();
      const float* Gs = st_G(s);
      const unsigned char* runs = st_runs(s);
      const int tok0 = st_meta(s)[0], len = st_meta(s)[1], flags = st_meta(s)[2];
      T* o = static_cast<T*>(p.o) + ((long)tok0 * p.H + h) * V + v;
      float* gamP = st_gam(s) + 512 + q4 * 64;
      gamP[lane] = row_scalars(Gs, runs, flags, lane).gam;
      gamP[lane + 32] = row_scalars(Gs, runs, flags, lane + 32).gam;
      __syncwarp();
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        float a[32], b[32];
        umma::ld_32x32b_x32(a, tl + cO1 + blk * 32);
        umma::ld_32x32b_x32(b, tl + cO2 + blk * 32);
        umma::wait_ld();
        if (blk == 1) {
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + B_OFREE);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int tok = blk * 32 + i;
          if (tok < len) o[(long)tok * p.H * V] = from_f32<T>(p.scale * (gamP[tok] * a[i] + b[i]));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + NS + s);  // done with this stage's T0 and gate vectors
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicExch(p.status, 2);
}

template <typename T, bool DELTA>
int launch_one(const FwdTcMaps& maps, const FwdTcParams& fp, int blocks, cudaStream_t s) {
  auto* kern = sg_fwd_tc_kernel<T, DELTA>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kBytes));
  {
    ProfScope ps(kProfSgFwd, s);
    kern<<<blocks, 384, Smem::kBytes, s>>>(maps, fp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

int* tc_status_ptr();  // chunked_bwd_tc.cu

// Same contract as launch_sg_fwd (chunked_fwd.cu) for K = V = 128; the residuals h and Vn are written transposed.
int launch_sg_fwd_tc(const ChunkedCtx& c, const jla_fwd_io& io, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.rows == 0) return JLA_OK;
  const uint64_t tokens = (uint64_t)p.B * p.T, slots = (uint64_t)pl.nc * p.H;
  FwdTcMaps maps;
  bool ok = tma::encode_3d(&maps.q, c.q_eff, p.K, p.Hk, tokens, 64) && tma::encode_3d(&maps.k, c.k_eff, p.K, p.Hk, tokens, 64) &&
            tma::encode_3d(&maps.v, p.v, p.V, p.H, tokens, 64);
  if (ok && pl.delta) ok = tma::encode_3d(&maps.t0, c.res + pl.t0, 64, 1, slots * 64, 64);
  if (ok && !pl.delta) maps.t0 = maps.v;
  if (!ok) return JLA_ERR_CUDA;
  FwdTcParams fp{};
  fp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  fp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  fp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  fp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  fp.h0 = p.h0;
  fp.o = io.o;
  fp.final_state = io.final_state;
  fp.hT_out = pl.save ? c.res + pl.h : nullptr;
  fp.vnT_out = pl.save && pl.delta ? c.res + pl.vn : nullptr;
  fp.H = p.H;
  fp.Hk = p.Hk;
  fp.scale = p.scale;
  fp.status = tc_status_ptr();
  if (!fp.status) return JLA_ERR_CUDA;
  const int blocks = pl.rows * p.H;
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_one<__nv_bfloat16, true>(maps, fp, blocks, s) : launch_one<__nv_bfloat16, false>(maps, fp, blocks, s);
  }
  return pl.delta ? launch_one<__half, true>(maps, fp, blocks, s) : launch_one<__half, false>(maps, fp, blocks, s);
}

}  // namespace jla
