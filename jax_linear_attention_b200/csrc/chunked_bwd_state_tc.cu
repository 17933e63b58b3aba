// Reverse state pass of the backward for K = V = 128 on the Blackwell tensor cores: the mirror image of
// sg_fwd_tc_kernel (chunked_fwd_tc.cu). One persistent CTA per (row, head) walks the row's chunks from last to
// first with dS^T [V lanes x K columns] fp32 in TMEM:
//
//   dVn^T = dO^T (scale P) + (tail Gamma_r)_j (dS+^T K^T)      two accumulators, combined by the state group
//   dW^T  = dVn^T Ag                    (= dV^T)                A operand dVn^T from TMEM
//   dS^T  = keep gamma dS+^T + (scale cin Gamma dO)^T-rows Q - (cin Gamma dW)^T-rows K
//                                                               A operands from TMEM, Q and K read MN-major
//
// Roles: one TMA thread (q, k, dO, Ag tiles + gate vectors, 3-stage ring), one MMA thread, eight "state" warps
// (thread = value row v; warp pairs split the 64 token columns) and eight "score" warps that build scale (Q K^T) D
// one chunk ahead. Residuals for the chunk-gradient kernel are written transposed: dh^T [V][K], dVn^T [V][64].
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {
namespace {

using umma::swz_tile;

constexpr int K = 128, V = 128;
constexpr int kBarBase = 6;  // full / empty barriers of the ring (at most 3 stages) come first

// VG (per-channel gates, KDA): gate-folded tiles per chunk slot as in the forward (chunked_kda_prep.cu):
// q -> cin q exp(G), k -> cin k exp(G), k2 -> tail k exp(G_63 - G), p -> the masked score tile, ag -> T beta_j; the
// gate vector of the stage carries exp(G_63) per key channel.
struct BwdTcMaps {
  CUtensorMap q, k, d_o, ag, k2, p;
};

struct BwdTcParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;
  const unsigned char* runs;
  const float* d_final;
  void* dv;
  float* dh0;
  void *dhT_out, *dvnT_out;
  int H, Hk;
  float scale;
  int* status;
};

template <bool VG>
struct SmemT {
  static constexpr int NS = VG ? 2 : 3;
  static constexpr int kStage = 64 * K * 2 * 2 + 64 * V * 2 + 8192 + (VG ? 64 * K * 2 + 8192 : 0);  // q, k, dO, Ag (+ k2, P)
  static constexpr int kPb = NS * kStage;                // scale P tiles [2][64x64]
  static constexpr int kGates = kPb + (VG ? 0 : 2 * 8192);
  static constexpr int kGateStride = 640;
  static constexpr int kScal = kGates + NS * kGateStride;  // per stage and state warp: gam[64], gamr[64]
  static constexpr int kBars = kScal + NS * 4096;
  static constexpr int kNumBars = kBarBase + 12;
  static constexpr int kBytes = kBars + kNumBars * 8 + 64 + 1024;
};

enum { B_PDONE = kBarBase, B_PFREE, B_PA0, B_PA1, B_ST, B_MA, B_DV, B_MB, B_DW, B_MC };

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_addr(bar)) : "memory");
}

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

__device__ __forceinline__ void ld_row32(float (&v)[32], uint32_t taddr) {
  umma::ld_32x32b_x32(v, taddr);
  umma::wait_ld();
}

template <typename T, bool DELTA, bool VG>
__global__ void __launch_bounds__(640, 1) sg_bwd_state_tc_kernel(const __grid_constant__ BwdTcMaps maps, BwdTcParams p) {
  static_assert(DELTA || !VG, "per-channel gates come with the delta rule");
  using Smem = SmemT<VG>;
  constexpr int NS = Smem::NS;
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
  auto st_do = [&](int s) { return st_k(s) + 64 * K * 2; };
  auto st_ag = [&](int s) { return st_do(s) + 64 * V * 2; };
  auto st_k2 = [&](int s) { return st_ag(s) + 8192; };       // VG only
  auto st_p = [&](int s) { return st_k2(s) + 64 * K * 2; };  // VG only
  auto st_G = [&](int s) { return reinterpret_cast<float*>(base + Smem::kGates + s * Smem::kGateStride); };
  auto st_runs = [&](int s) { return reinterpret_cast<unsigned char*>(st_G(s) + 128); };
  auto st_meta = [&](int s) { return reinterpret_cast<volatile int*>(st_runs(s) + 64); };
  auto st_gam = [&](int s) { return reinterpret_cast<float*>(base + Smem::kScal + s * 4096); };
  unsigned char* Pb = base + Smem::kPb;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      umma::mbar_init(bars + s, 1);
      umma::mbar_init(bars + NS + s, 1 + 8 + 8);
    }
    umma::mbar_init(bars + B_PDONE, 1);
    umma::mbar_init(bars + B_PFREE, 8);
    umma::mbar_init(bars + B_PA0, 8);
    umma::mbar_init(bars + B_PA1, 8);
    umma::mbar_init(bars + B_ST, 8);
    umma::mbar_init(bars + B_MA, 1);
    umma::mbar_init(bars + B_DV, 8);
    umma::mbar_init(bars + B_MB, 1);
    umma::mbar_init(bars + B_DW, 8);
    umma::mbar_init(bars + B_MC, 1);
    umma::mbar_init_fence();
    *abort_flag = 0;
  }
  if (warp == 2) umma::tmem_alloc(tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // dS^T fp32 | dS^T 16-bit | acc1 = dS+^T K^T, later dW^T | acc2 = dO^T (scale P) | dVn^T 16-bit |
  // -(cin Gamma) dW^T 16-bit | scale (cin Gamma) dO^T 16-bit | Q K^T
  constexpr uint32_t cS = 0, cSb = 128, cA1 = 192, cA2 = 256, cDVb = 320, cDWb = 352, cDOb = 384, cP = 416;

  if (warp == 0) {
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it % NS, c = rc.x + (n - 1 - it);
        if (!wait(bars + NS + s, ((it / NS) & 1) ^ 1, abort_flag)) break;
        const ChunkMeta m = p.meta[c];
        volatile int* ms = st_meta(s);
        ms[0] = m.tok0;
        ms[1] = m.len;
        ms[2] = m.flags;
        const uint32_t bytes = 64 * K * 2 * 2 + 64 * V * 2 + (DELTA ? 8192 : 0) + (VG ? 64 * K * 2 + 8192 : 0) + 512 + 64;
        tma::expect_tx(bars + s, bytes);
        const int slot_row = (c * p.H + h) * 64;
        if (VG) {
          tma::load_tile<64, K>(st_k(s), &maps.k, 0, 0, slot_row, bars + s);
          tma::load_tile<64, K>(st_q(s), &maps.q, 0, 0, slot_row, bars + s);
          tma::load_tile<64, K>(st_k2(s), &maps.k2, 0, 0, slot_row, bars + s);
          tma::load_tile<64, 64>(st_p(s), &maps.p, 0, 0, slot_row, bars + s);
        } else {
          tma::load_tile<64, K>(st_k(s), &maps.k, 0, hk, m.tok0, bars + s);
          tma::load_tile<64, K>(st_q(s), &maps.q, 0, hk, m.tok0, bars + s);
        }
        tma::load_tile<64, V>(st_do(s), &maps.d_o, 0, h, m.tok0, bars + s);
        if (DELTA) tma::load_tile<64, 64>(st_ag(s), &maps.ag, 0, 0, slot_row, bars + s);
        bulk_copy(st_G(s), p.gates + ((long)c * p.H + h) * 128, 512, bars + s);
        bulk_copy(st_runs(s), p.runs + (long)c * 64, 64, bars + s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      auto issue_p = [&](int it) {
        const int s = it % NS;
        if (!wait(bars + s, (it / NS) & 1, abort_flag)) return false;
        if (!wait(bars + B_PFREE, (it & 1) ^ 1, abort_flag)) return false;
        umma::fence_after_sync();
        umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP, umma::smem_addr(st_q(s)), 64, umma::smem_addr(st_k(s)), 64,
                                                      false);
        umma::commit(bars + B_PDONE);
        return true;
      };
      bool okm = n > 0 && !VG ? issue_p(0) : true;
      for (int it = 0; it < n && okm; ++it) {
        const int s = it % NS;
        const uint32_t ph = it & 1;
        const uint32_t aq = umma::smem_addr(st_q(s)), ak = umma::smem_addr(st_k(s)), ado = umma::smem_addr(st_do(s));
        if (!wait(bars + B_ST, ph, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cA1, tmem + cSb, VG ? umma::smem_addr(st_k2(s)) : ak, 64,
                                                   false);  // dS+^T K^T
        if (!VG && !wait(bars + B_PA0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
        // dO^T (scale P): A = dO tile read MN-major (M = value index), B = P tile read MN-major (rows i)
        umma::gemm<128, 64, 4, true, true, FMT>(tmem + cA2, ado, 64,
                                                VG ? umma::smem_addr(st_p(s)) : umma::smem_addr(Pb + (it & 1) * 8192), 64, false);
        umma::commit(bars + B_MA);
        if (!VG && it + 1 < n && !issue_p(it + 1)) break;
        if (DELTA) {
          if (!wait(bars + B_DV, ph, abort_flag)) break;
          umma::fence_after_sync();
          umma::gemm_ts<128, 64, 4, true, FMT>(tmem + cA1, tmem + cDVb, umma::smem_addr(st_ag(s)), 64, false);  // dVn^T Ag
          umma::commit(bars + B_MB);
        }
        if (!wait(bars + B_DW, ph, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cDOb, aq, 64, true);                // += (s cg dO)^T Q
        if (DELTA) umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cDWb, ak, 64, true);     // += (-cg dW)^T K
        umma::commit(bars + B_MC);
        umma::commit(bars + NS + s);
      }
    }
  } else if (warp >= 4 && warp < 12) {
    const int q4 = warp & 3, half = (warp - 4) >> 2, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int s = it % NS, c = rc.x + (n - 1 - it);
      const uint32_t ph = it & 1;
      ok = wait(bars + s, (it / NS) & 1, abort_flag);
      if (!ok) break;
      const float* Gs = st_G(s);
      const unsigned char* runs = st_runs(s);
      const int tok0 = st_meta(s)[0], len = st_meta(s)[1], flags = st_meta(s)[2];
      float* gam = st_gam(s) + (warp - 4) * 128;
      float* gamr = gam + 64;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = lane + 32 * jj;
        if (VG) {  // masks and decays are folded into the operands
          gam[j] = 1.f;
          gamr[j] = 1.f;
        } else {
          const RowScalars rs = row_scalars(Gs, runs, flags, j);
          gam[j] = rs.gam;
          gamr[j] = rs.gamr;
        }
      }
      __syncwarp();
      const float kg = VG ? 0.f : keep_gamma(Gs, runs, flags);
      const float pscale = VG ? p.scale : 1.f;  // VG: the score tile comes unscaled
      const int j0 = 32 * half;
      // ---- dS+ of this chunk: 16-bit copy, residual, decayed fp32 copy
      if (it > 0) {
        ok = wait(bars + B_MC, ph ^ 1, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
      }
      uint32_t hpk[32];
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
        const int blk = 2 * half + b2;
        float x[32];
        if (it == 0) {
          const float* df = p.d_final ? p.d_final + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = df ? df[(long)(blk * 32 + i) * V + v] : 0.f;
        } else {
          ld_row32(x, tl + cS + blk * 32);
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk[i] = pack2<T>(x[2 * i], x[2 * i + 1]);
          hpk[b2 * 16 + i] = pk[i];
        }
        umma::st_32x32b_x16(tl + cSb + blk * 16, pk);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= VG ? Gs[blk * 32 + i] : kg;  // VG: exp(G_63) of key channel blk * 32 + i
        umma::st_32x32b_x32(tl + cS + blk * 32, x);
      }
      // ---- scale (cin Gamma)_i dO^T as a 16-bit A operand (tokens i of this warp's half)
      const T* dos = reinterpret_cast<const T*>(st_do(s));
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = j0 + 2 * i;
          const float a = (j < len) ? to_f32(dos[swz_tile(64, j, v)]) * p.scale * gam[j] : 0.f;
          const float b = (j + 1 < len) ? to_f32(dos[swz_tile(64, j + 1, v)]) * p.scale * gam[j + 1] : 0.f;
          pk[i] = pack2<T>(a, b);
        }
        umma::st_32x32b_x16(tl + cDOb + 16 * half, pk);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_ST);
      {
        T* dhT = static_cast<T*>(p.dhT_out) + (((long)c * p.H + h) * V + v) * K + 64 * half;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          *reinterpret_cast<uint4*>(dhT + i * 8) = make_uint4(hpk[4 * i], hpk[4 * i + 1], hpk[4 * i + 2], hpk[4 * i + 3]);
        }
      }
      // ---- dVn^T = dO^T (scale P) + (tail Gamma_r)_j (dS+^T K^T)
      ok = wait(bars + B_MA, ph, abort_flag);
      if (!ok) break;
      umma::fence_after_sync();
      uint32_t dvn[16];
      {
        float x[32], y[32];
        umma::ld_32x32b_x32(x, tl + cA1 + j0);
        umma::ld_32x32b_x32(y, tl + cA2 + j0);
        umma::wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = j0 + 2 * i;
          // columns of tokens past a partial chunk are forced to zero (their inputs are other rows' data)
          dvn[i] = pack2<T>(j < len ? pscale * y[2 * i] + gamr[j] * x[2 * i] : 0.f,
                            j + 1 < len ? pscale * y[2 * i + 1] + gamr[j + 1] * x[2 * i + 1] : 0.f);
        }
      }
      T* stg = reinterpret_cast<T*>(st_do(s)) + (warp - 4) * 32 * 32;  // [32 tokens][32 values]: dv staging (dO is dead)
      if (DELTA) {
        umma::st_32x32b_x16(tl + cDVb + 16 * half, dvn);
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DV);
        {
          T* dvnT = static_cast<T*>(p.dvnT_out) + (((long)c * p.H + h) * V + v) * 64 + j0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<uint4*>(dvnT + i * 8) = make_uint4(dvn[4 * i], dvn[4 * i + 1], dvn[4 * i + 2], dvn[4 * i + 3]);
          }
        }
        // ---- dW^T = dVn^T Ag ; -(cin Gamma)_j dW^T as the next A operand; dv
        ok = wait(bars + B_MB, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        float x[32];
        ld_row32(x, tl + cA1 + j0);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = j0 + 2 * i;
          pk[i] = pack2<T>(-gam[j] * x[2 * i], -gam[j + 1] * x[2 * i + 1]);
        }
        umma::st_32x32b_x16(tl + cDWb + 16 * half, pk);
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DW);
#pragma unroll
        for (int i = 0; i < 32; ++i) stg[i * 32 + lane] = from_f32<T>(x[i]);
      } else {
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DW);  // dW = dVn: nothing more for the state update
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 f = unpack2<T>(dvn[i]);
          stg[(2 * i) * 32 + lane] = from_f32<T>(f.x);
          stg[(2 * i + 1) * 32 + lane] = from_f32<T>(f.y);
        }
      }
      __syncwarp();
      T* dv = static_cast<T*>(p.dv) + ((long)(tok0 + j0) * p.H + h) * V + 32 * q4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = lane + 32 * i, tok = idx >> 2, part = idx & 3;
        if (j0 + tok < len) {
          *reinterpret_cast<uint4*>(dv + (long)tok * p.H * V + part * 8) = *reinterpret_cast<const uint4*>(stg + tok * 32 + part * 8);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + NS + s);
    }
    // ---- gradient of the initial state
    if (ok && n > 0) ok = wait(bars + B_MC, (n - 1) & 1, abort_flag);
    umma::fence_after_sync();
    if (ok && p.dh0) {
      float* f = p.dh0 + ((long)row * p.H + h) * K * V;
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
        const int blk = 2 * half + b2;
        float x[32];
        if (n == 0) {
          const float* df = p.d_final ? p.d_final + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = df ? df[(long)(blk * 32 + i) * V + v] : 0.f;
        } else {
          ld_row32(x, tl + cS + blk * 32);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) f[(long)(blk * 32 + i) * V + v] = x[i];
      }
    }
  } else if (warp >= 12) {
    // ---- score group: scale (Q K^T) D one chunk ahead, stored [i][j] (read MN-major by the dO^T P product)
    const int q4 = warp & 3, half = (warp - 12) >> 2, g = lane >> 2, t = lane & 3;
    const int r0 = 16 * q4;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int s = it % NS, buf = it & 1;
      ok = wait(bars + s, (it / NS) & 1, abort_flag);
      if (!ok) break;
      if (VG) {  // the score tile arrives with the stage: nothing to build
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + NS + s);
        continue;
      }
      const float* Gs = st_G(s);
      const unsigned char* runs = st_runs(s);
      ok = wait(bars + B_PDONE, it & 1, abort_flag);
      if (!ok) break;
      umma::fence_after_sync();
      float acc[4][4];
      umma::ld_16x256b<4>(acc, tl + cP + 32 * half);
      umma::wait_ld();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_PFREE);
      const int i0 = r0 + g, i1 = r0 + g + 8;
      const float G0 = Gs[i0], G1 = Gs[i1];
      const int run0 = runs[i0], run1 = runs[i1];
      const int len = st_meta(s)[1];
      // rows of tokens past a partial chunk hold other rows' q and dO: their scores must not reach dVn
      const float s0 = i0 < len ? p.scale : 0.f, s1 = i1 < len ? p.scale : 0.f;
      T* pt = reinterpret_cast<T*>(Pb + buf * 8192);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int j = 32 * half + nt * 8 + 2 * t;
        const float d00 = s0 * decay_ij(Gs, runs, i0, j, G0, run0), d01 = s0 * decay_ij(Gs, runs, i0, j + 1, G0, run0);
        const float d10 = s1 * decay_ij(Gs, runs, i1, j, G1, run1), d11 = s1 * decay_ij(Gs, runs, i1, j + 1, G1, run1);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i0, j)) = pack2<T>(acc[nt][0] * d00, acc[nt][1] * d01);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i1, j)) = pack2<T>(acc[nt][2] * d10, acc[nt][3] * d11);
      }
      umma::fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bars + B_PA0 + buf);
        mbar_arrive(bars + NS + s);
      }
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicExch(p.status, 3);
}

template <typename T, bool DELTA, bool VG = false>
int launch_one(const BwdTcMaps& maps, const BwdTcParams& bp, int blocks, cudaStream_t s) {
  auto* kern = sg_bwd_state_tc_kernel<T, DELTA, VG>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemT<VG>::kBytes));
  {
    ProfScope ps(VG ? kProfKdaBwdState : kProfSgBwdState, s);
    kern<<<blocks, 640, SmemT<VG>::kBytes, s>>>(maps, bp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

// The reverse state pass of launch_sg_bwd for K = V = 128; dh and dVn are written transposed.
int launch_sg_bwd_state_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.rows == 0) return JLA_OK;
  const uint64_t tokens = (uint64_t)p.B * p.T, slots = (uint64_t)pl.nc * p.H;
  const bool vg = p.kind == JLA_KIND_KDA;
  BwdTcMaps maps;
  bool ok = tma::encode_3d(&maps.d_o, io.d_o, p.V, p.H, tokens, 64);
  if (vg) {
    ok = ok && tma::encode_3d(&maps.q, c.res + pl.kda_q, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.k, c.res + pl.kda_kr, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.k2, c.res + pl.kda_kw, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.p, c.res + pl.kda_p, 64, 1, slots * 64, 64);
  } else {
    ok = ok && tma::encode_3d(&maps.q, c.q_eff, p.K, p.Hk, tokens, 64) && tma::encode_3d(&maps.k, c.k_eff, p.K, p.Hk, tokens, 64);
  }
  if (ok && pl.delta) ok = tma::encode_3d(&maps.ag, c.res + pl.ag, 64, 1, slots * 64, 64);
  if (ok && !pl.delta) maps.ag = maps.d_o;
  if (!ok) return JLA_ERR_CUDA;
  if (!vg) maps.k2 = maps.p = maps.d_o;  // unused
  BwdTcParams bp{};
  bp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  bp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  bp.gates = reinterpret_cast<const float*>(c.res + (vg ? pl.kda_d : pl.gates));
  bp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  bp.d_final = io.d_final;
  bp.dv = io.dv;
  bp.dh0 = io.dh0;
  bp.dhT_out = scratch + pl.dh;
  bp.dvnT_out = scratch + pl.dvn;
  bp.H = p.H;
  bp.Hk = p.Hk;
  bp.scale = p.scale;
  bp.status = tc_status_ptr();
  if (!bp.status) return JLA_ERR_CUDA;
  const int blocks = pl.rows * p.H;
  if (vg) return launch_one<__nv_bfloat16, true, true>(maps, bp, blocks, s);
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_one<__nv_bfloat16, true>(maps, bp, blocks, s) : launch_one<__nv_bfloat16, false>(maps, bp, blocks, s);
  }
  return pl.delta ? launch_one<__half, true>(maps, bp, blocks, s) : launch_one<__half, false>(maps, bp, blocks, s);
}

}  // namespace jla
