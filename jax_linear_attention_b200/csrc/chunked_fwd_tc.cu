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
constexpr int kBarBase = 6;  // full / empty barriers of the ring (at most 3 stages) come first

// Build with -DJLA_TRACE to record, for the first CTA, the global timer at the hand-offs of the serial chain
// (16 slots per chunk: 0-8 by the first state warp, 9-14 by the MMA issuer); jla_debug_fwd_trace() copies them out.
#ifdef JLA_TRACE
__device__ unsigned long long g_fwd_trace[64 * 16];
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define JLA_MARK(it, slot)                                                                     \
  do {                                                                                         \
    if (blockIdx.x == 0 && (it) < 64) g_fwd_trace[(it) * 16 + (slot)] = global_timer();         \
  } while (0)
#else
#define JLA_MARK(it, slot) \
  do {                     \
  } while (0)
#endif

// VG (per-channel gates, KDA): the tiles come gate-folded from kda_prep_kernel, one set per chunk slot:
// q -> cin q exp(G), k -> cin k exp(G) (recall), k2 -> tail k exp(G_63 - G) (write), p -> the masked score tile,
// ag -> T beta_j, and the G/beta vector of the stage carries the decay exp(G_63) of the K state columns instead.
struct FwdTcMaps {
  CUtensorMap q, k, v, ag, k2, p;
};

struct FwdTcParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;  // VG: the per-slot decay vectors [K]
  const unsigned char* runs;
  const float* h0;
  void* o;
  float* final_state;
  void *hT_out, *vnT_out, *wT_out;  // residuals (nullptr when not saving)
  int H, Hk;
  float scale;
  int* status;
  int state_only;  // final state (and residuals) only: no scores, no outputs
};

template <bool VG>
struct SmemT {
  static constexpr int NS = VG ? 2 : 3;  // stages of the input ring
  // q, k, v, T0 (Ag); VG adds the write-side keys and the score tile
  static constexpr int kStage = 64 * K * 2 * 2 + 64 * V * 2 + 8192 + (VG ? 64 * K * 2 + 8192 : 0);
  static constexpr int kTiles = NS * kStage;
  static constexpr int kPb = kTiles;            // P tiles [2][64x64]
  static constexpr int kAgb = kPb + (VG ? 0 : 2 * 8192);   // Ag tiles [2][64x64]
  static constexpr int kGates = kAgb + (VG ? 0 : 2 * 8192);  // per stage: G[64], beta[64] f32 (512 B) + runs (64 B) + meta (16 B)
  static constexpr int kGateStride = 640;
  static constexpr int kScal = kGates + NS * kGateStride;  // per stage and warp: gam[64], gamr[64] (state group); gam[64] (score group)
  static constexpr int kBars = kScal + NS * 4096;
  static constexpr int kNumBars = kBarBase + 16;
  static constexpr int kBytes = kBars + kNumBars * 8 + 64 + 1024;
};

enum {  // mbarrier indices after the full / empty barriers
  B_PDONE = kBarBase, B_PFREE, B_PA0, B_PA1, B_ST, B_M1, B_W, B_M2, B_VN, B_M3, B_ODONE, B_OFREE0, B_OFREE1
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

template <typename T, bool DELTA, bool VG>
__global__ void __launch_bounds__(640, 1) sg_fwd_tc_kernel(const __grid_constant__ FwdTcMaps maps, FwdTcParams p) {
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
  auto st_v = [&](int s) { return st_k(s) + 64 * K * 2; };
  auto st_t0 = [&](int s) { return st_v(s) + 64 * V * 2; };
  auto st_k2 = [&](int s) { return st_t0(s) + 8192; };      // VG only
  auto st_p = [&](int s) { return st_k2(s) + 64 * K * 2; };  // VG only
  auto st_G = [&](int s) { return reinterpret_cast<float*>(base + Smem::kGates + s * Smem::kGateStride); };
  auto st_runs = [&](int s) { return reinterpret_cast<unsigned char*>(st_G(s) + 128); };
  auto st_meta = [&](int s) { return reinterpret_cast<volatile int*>(st_runs(s) + 64); };
  auto st_gam = [&](int s) { return reinterpret_cast<float*>(base + Smem::kScal + s * 4096); };
  unsigned char* Pb = base + Smem::kPb;
  unsigned char* Agb = base + Smem::kAgb;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      umma::mbar_init(bars + s, 1);                  // full: the producer's expect_tx arrival (+ bytes)
      umma::mbar_init(bars + NS + s, 1 + 8 + 8);     // empty: MMA commit + the warps of both groups
    }
    umma::mbar_init(bars + B_PDONE, 1);
    umma::mbar_init(bars + B_PFREE, 8);
    umma::mbar_init(bars + B_PA0, 8);
    umma::mbar_init(bars + B_PA1, 8);
    umma::mbar_init(bars + B_ST, 8);
    umma::mbar_init(bars + B_M1, 1);
    umma::mbar_init(bars + B_W, 8);
    umma::mbar_init(bars + B_M2, 1);
    umma::mbar_init(bars + B_VN, 8);
    umma::mbar_init(bars + B_M3, 1);
    umma::mbar_init(bars + B_ODONE, 1);
    umma::mbar_init(bars + B_OFREE0, 8);
    umma::mbar_init(bars + B_OFREE1, 8);
    umma::mbar_init_fence();
    *abort_flag = 0;
  }
  if (warp == 2) umma::tmem_alloc(tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cS = 0, cSb = 128, cA1 = 192, cWb = 256, cVg = 288, cO = 320 /* two 64-column buffers */, cP = 448;

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
        tma::load_tile<64, V>(st_v(s), &maps.v, 0, h, m.tok0, bars + s);
        if (DELTA) tma::load_tile<64, 64>(st_t0(s), &maps.ag, 0, 0, slot_row, bars + s);
        bulk_copy(st_G(s), p.gates + ((long)c * p.H + h) * 128, 512, bars + s);
        bulk_copy(st_runs(s), p.runs + (long)c * 64, 64, bars + s);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      auto issue_p = [&](int it) {  // Q K^T of chunk `it` (its inputs are prefetched): runs one chunk ahead of the chain
        const int s = it % NS;
        if (!wait(bars + s, (it / NS) & 1, abort_flag)) return false;
        if (!wait(bars + B_PFREE, (it & 1) ^ 1, abort_flag)) return false;
        umma::fence_after_sync();
        umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP, umma::smem_addr(st_q(s)), 64, umma::smem_addr(st_k(s)), 64,
                                                      false);
        umma::commit(bars + B_PDONE);
        return true;
      };
      bool okm = n > 0 && !p.state_only && !VG ? issue_p(0) : true;
      for (int it = 0; it < n && okm; ++it) {
        const int s = it % NS;
        const uint32_t ph = it & 1;
        const uint32_t aq = umma::smem_addr(st_q(s)), ak = umma::smem_addr(st_k(s));
        if (!wait(bars + B_ST, ph, abort_flag)) break;
        umma::fence_after_sync();
        JLA_MARK(it, 9);
        if (DELTA) {
          umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cA1, tmem + cSb, ak, 64, false);  // S^T K^T
          umma::commit(bars + B_M1);
        }
        JLA_MARK(it, 10);
        const uint32_t co = cO + (it & 1) * 64;
        if (!p.state_only) {
          if (!VG) {
            if (it + 1 < n && !issue_p(it + 1)) break;
            // q has been scaled by (cin Gamma)_i in place by the score group (part of "PA ready")
            if (!wait(bars + B_PA0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
          }
          if (!wait(bars + B_OFREE0 + (it & 1), ((it >> 1) & 1) ^ 1, abort_flag)) break;
          umma::fence_after_sync();
          umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + co, tmem + cSb, aq, 64, false);  // S^T ((cin Gamma) Q)^T
        }
        if (DELTA) {
          if (!wait(bars + B_W, ph, abort_flag)) break;
          umma::fence_after_sync();
          JLA_MARK(it, 11);
          umma::gemm_ts<128, 64, 4, false, FMT>(tmem + cA1, tmem + cWb, umma::smem_addr(st_t0(s)), 64, false);  // W^T Ag^T
          umma::commit(bars + B_M2);
          JLA_MARK(it, 12);
        }
        if (!wait(bars + B_VN, ph, abort_flag)) break;
        umma::fence_after_sync();
        JLA_MARK(it, 13);
        umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cVg, VG ? umma::smem_addr(st_k2(s)) : ak, 64,
                                              true);  // S^T += (Gamma_r Vn)^T K
        umma::commit(bars + B_M3);
        JLA_MARK(it, 14);
        if (!p.state_only) {
          const uint32_t ap = VG ? umma::smem_addr(st_p(s)) : umma::smem_addr(Pb + (it & 1) * 8192);
          umma::gemm_ts<128, 64, 4, false, FMT>(tmem + co, tmem + cWb, ap, 64, true);  // += Vn^T P^T
        }
        umma::commit(bars + B_ODONE);
        umma::commit(bars + NS + s);
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------- state group: thread = value row v, warp pair = column halves
    const int q4 = warp & 3, half = (warp - 4) >> 2, v = 32 * q4 + lane;
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
      float* gam = st_gam(s) + (warp - 4) * 128;  // this warp's own copy: no cross-warp barrier on the serial chain
      float* gamr = gam + 64;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = lane + 32 * jj;
        if (VG) {  // the masks and decays are folded into the operands
          gam[j] = 1.f;
          gamr[j] = 1.f;
        } else {
          const RowScalars rs = row_scalars(Gs, runs, flags, j);
          gam[j] = rs.gam;
          gamr[j] = (j < len) ? rs.gamr : 0.f;  // tokens past a partial chunk must not write the state
        }
      }
      __syncwarp();
      const float kg = VG ? 0.f : keep_gamma(Gs, runs, flags);
      // ---- the state entering this chunk: 16-bit copy for the products, decayed fp32 copy for the update
      if (it > 0) {
        ok = wait(bars + B_M3, ph ^ 1, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
      }
      if (tid == 128) JLA_MARK(it, 0);
      uint32_t hpk[32];  // the 16-bit copy of this half row, stored as a residual once the chain is released
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
        const int blk = 2 * half + b2;
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
        for (int i = 0; i < 16; ++i) {
          pk[i] = pack2<T>(x[2 * i], x[2 * i + 1]);
          hpk[b2 * 16 + i] = pk[i];
        }
        umma::st_32x32b_x16(tl + cSb + blk * 16, pk);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= VG ? Gs[blk * 32 + i] : kg;  // VG: exp(G_63) of key channel blk * 32 + i
        umma::st_32x32b_x32(tl + cS + blk * 32, x);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_ST);
      if (tid == 128) JLA_MARK(it, 1);
      if (p.hT_out) {
        T* hT = static_cast<T*>(p.hT_out) + (((long)c * p.H + h) * V + v) * K + 64 * half;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          *reinterpret_cast<uint4*>(hT + i * 8) = make_uint4(hpk[4 * i], hpk[4 * i + 1], hpk[4 * i + 2], hpk[4 * i + 3]);
        }
      }

      if (tid == 128) JLA_MARK(it, 2);
      const T* vs = reinterpret_cast<const T*>(st_v(s));
      const int j0 = 32 * half;  // this warp's 32 tokens (columns of the [V x 64] accumulators)
      if (DELTA) {
        // ---- W^T = V^T - (cin Gamma)_j (S^T K^T)
        ok = wait(bars + B_M1, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        if (tid == 128) JLA_MARK(it, 3);
        {
          float x[32];
          ld_row32<T>(x, tl + cA1 + j0);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = j0 + 2 * i;
            const float w0 = to_f32(vs[swz_tile(64, j, v)]) - gam[j] * x[2 * i];
            const float w1 = to_f32(vs[swz_tile(64, j + 1, v)]) - gam[j + 1] * x[2 * i + 1];
            pk[i] = pack2<T>(w0, w1);
          }
          umma::st_32x32b_x16(tl + cWb + 16 * half, pk);
          umma::wait_st();
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + B_W);
          if (tid == 128) JLA_MARK(it, 4);
          if (p.wT_out) {  // residual for the key-side gradient kernel (dAg = dVn W^T)
            T* wT = static_cast<T*>(p.wT_out) + (((long)c * p.H + h) * V + v) * 64 + j0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              *reinterpret_cast<uint4*>(wT + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
          }
        }
        // ---- Vn^T = W^T Ag^T
        if (tid == 128) JLA_MARK(it, 5);
        ok = wait(bars + B_M2, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        if (tid == 128) JLA_MARK(it, 6);
        {
          float x[32];
          ld_row32<T>(x, tl + cA1 + j0);
          uint32_t pk[16], pg[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = j0 + 2 * i;
            pk[i] = pack2<T>(x[2 * i], x[2 * i + 1]);
            pg[i] = pack2<T>(x[2 * i] * gamr[j], x[2 * i + 1] * gamr[j + 1]);
          }
          umma::st_32x32b_x16(tl + cWb + 16 * half, pk);
          umma::st_32x32b_x16(tl + cVg + 16 * half, pg);
          umma::wait_st();
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bars + B_VN);
            mbar_arrive(bars + NS + s);  // done with this stage's v and gate vectors
          }
          if (tid == 128) JLA_MARK(it, 7);
          if (p.vnT_out) {
            T* vnT = static_cast<T*>(p.vnT_out) + (((long)c * p.H + h) * V + v) * 64 + j0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              *reinterpret_cast<uint4*>(vnT + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            }
          }
          if (tid == 128) JLA_MARK(it, 8);
        }
      } else {
        // ---- Vn = V: the value rows themselves, and their Gamma_r-scaled copy
        if (it > 0) {  // the previous chunk's Vn^T P^T must have consumed the operand columns
          ok = wait(bars + B_ODONE, ph ^ 1, abort_flag);
          if (!ok) break;
          umma::fence_after_sync();
        }
        uint32_t pk[16], pg[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = j0 + 2 * i;
          const float a = to_f32(vs[swz_tile(64, j, v)]), b = to_f32(vs[swz_tile(64, j + 1, v)]);
          pk[i] = pack2<T>(a, b);
          pg[i] = pack2<T>(a * gamr[j], b * gamr[j + 1]);
        }
        umma::st_32x32b_x16(tl + cWb + 16 * half, pk);
        umma::st_32x32b_x16(tl + cVg + 16 * half, pg);
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bars + B_VN);
          mbar_arrive(bars + NS + s);
        }
      }
    }
    // ---- final state
    if (ok && n > 0) ok = wait(bars + B_M3, (n - 1) & 1, abort_flag);
    umma::fence_after_sync();
    if (ok && p.final_state) {
      float* f = p.final_state + ((long)row * p.H + h) * K * V;
#pragma unroll
      for (int b2 = 0; b2 < 2; ++b2) {
        const int blk = 2 * half + b2;
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
  } else if (warp >= 12) {
    // ---------------------------------- score group: P and the scaled q one chunk ahead; outputs. Warp pairs split
    // the 64 columns (tokens j for P, tokens i for the outputs) in halves.
    const int q4 = warp & 3, half = (warp - 12) >> 2, g = lane >> 2, t = lane & 3;
    const int r0 = 16 * q4, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    auto build = [&](int it) {  // P = (Q K^T) D of chunk `it`: rows r0 .. r0 + 15, columns 32 half .. + 31
      const int s = it % NS, buf = it & 1;
      if (!wait(bars + s, (it / NS) & 1, abort_flag)) return false;
      const float* Gs = st_G(s);
      const unsigned char* runs = st_runs(s);
      if (!wait(bars + B_PDONE, it & 1, abort_flag)) return false;
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
      T* pt = reinterpret_cast<T*>(Pb + buf * 8192);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int j = 32 * half + nt * 8 + 2 * t;
        const float d00 = decay_ij(Gs, runs, i0, j, G0, run0), d01 = decay_ij(Gs, runs, i0, j + 1, G0, run0);
        const float d10 = decay_ij(Gs, runs, i1, j, G1, run1), d11 = decay_ij(Gs, runs, i1, j + 1, G1, run1);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i0, j)) = pack2<T>(acc[nt][0] * d00, acc[nt][1] * d01);
        *reinterpret_cast<uint32_t*>(pt + swz_tile(64, i1, j)) = pack2<T>(acc[nt][2] * d10, acc[nt][3] * d11);
      }
      {  // q <- (cin Gamma)_i q in place (Q K^T has been read): the S^T Q^T product then needs no column scaling
        const int flags = st_meta(s)[2];
        const int tg = (warp - 12) * 32 + lane, i = tg >> 2, quarter = tg & 3;
        const float cgi = row_scalars(Gs, runs, flags, i).gam;
        T* qt = reinterpret_cast<T*>(st_q(s));
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4* ptr = reinterpret_cast<uint4*>(qt + swz_tile(64, i, quarter * 32 + ch * 8));
          uint4 x = *ptr;
          uint32_t* w = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack2<T>(w[e]);
            w[e] = pack2<T>(f.x * cgi, f.y * cgi);
          }
          *ptr = x;
        }
      }
      umma::fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_PA0 + buf);
      return true;
    };
    if (p.state_only) {  // nothing to build or to write: only release the stages
      for (int it = 0; it < n && ok; ++it) {
        const int s = it % NS;
        ok = wait(bars + s, (it / NS) & 1, abort_flag);
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(bars + NS + s);
      }
    }
    const int n_out = p.state_only ? 0 : n;
    if (n_out > 0 && !VG) ok = build(0);
    for (int it = 0; it < n_out && ok; ++it) {
      const int s = it % NS;
      if (it + 1 < n_out && !VG) {
        ok = build(it + 1);
        if (!ok) break;
      }
      // ---- O^T = scale [S^T ((cin Gamma) Q)^T + Vn^T P^T], thread = value row v, 32 tokens per warp
      ok = wait(bars + B_ODONE, it & 1, abort_flag);
      if (!ok) break;
      umma::fence_after_sync();
      const int tok0 = st_meta(s)[0], len = st_meta(s)[1];
      // Free the accumulator, then transpose through this warp's slice of the (dead) q tile so that the global
      // stores are 16-byte vectors along the value axis.
      T* stg = reinterpret_cast<T*>(st_q(s)) + (warp - 12) * 32 * 32;  // [32 tokens][32 value columns]
      {
        float a[32];
        umma::ld_32x32b_x32(a, tl + cO + (it & 1) * 64 + 32 * half);
        umma::wait_ld();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_OFREE0 + (it & 1));
#pragma unroll
        for (int i = 0; i < 32; ++i) stg[i * 32 + lane] = from_f32<T>(p.scale * a[i]);
      }
      __syncwarp();
      T* o = static_cast<T*>(p.o) + ((long)(tok0 + 32 * half) * p.H + h) * V + 32 * q4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = lane + 32 * i, tok = idx >> 2, part = idx & 3;
        if (32 * half + tok < len) {
          *reinterpret_cast<uint4*>(o + (long)tok * p.H * V + part * 8) = *reinterpret_cast<const uint4*>(stg + tok * 32 + part * 8);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + NS + s);  // done with this stage's gate vectors and the q tile
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicExch(p.status, 2);
}

template <typename T, bool DELTA, bool VG = false>
int launch_one(const FwdTcMaps& maps, const FwdTcParams& fp, int blocks, cudaStream_t s) {
  auto* kern = sg_fwd_tc_kernel<T, DELTA, VG>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemT<VG>::kBytes));
  {
    ProfScope ps(VG ? kProfKdaFwd : kProfSgFwd, s);
    kern<<<blocks, 640, SmemT<VG>::kBytes, s>>>(maps, fp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

// Same contract as launch_sg_fwd (chunked_fwd.cu) for K = V = 128; the residuals h and Vn are written transposed.
int launch_sg_fwd_tc(const ChunkedCtx& c, const jla_fwd_io& io, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.rows == 0) return JLA_OK;
  const uint64_t tokens = (uint64_t)p.B * p.T, slots = (uint64_t)pl.nc * p.H;
  const bool vg = p.kind == JLA_KIND_KDA;
  FwdTcMaps maps;
  bool ok = tma::encode_3d(&maps.v, p.v, p.V, p.H, tokens, 64);
  if (vg) {  // gate-folded operands, one [64 x K] tile per chunk slot
    ok = ok && tma::encode_3d(&maps.q, c.res + pl.kda_q, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.k, c.res + pl.kda_kr, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.k2, c.res + pl.kda_kw, p.K, 1, slots * 64, 64) &&
         tma::encode_3d(&maps.p, c.res + pl.kda_p, 64, 1, slots * 64, 64);
  } else {
    ok = ok && tma::encode_3d(&maps.q, c.q_eff, p.K, p.Hk, tokens, 64) && tma::encode_3d(&maps.k, c.k_eff, p.K, p.Hk, tokens, 64);
  }
  if (ok && pl.delta) ok = tma::encode_3d(&maps.ag, c.res + pl.ag, 64, 1, slots * 64, 64);
  if (ok && !pl.delta) maps.ag = maps.v;
  if (!ok) return JLA_ERR_CUDA;
  if (!vg) maps.k2 = maps.p = maps.v;  // unused
  FwdTcParams fp{};
  fp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  fp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  fp.gates = reinterpret_cast<const float*>(c.res + (vg ? pl.kda_d : pl.gates));
  fp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  fp.h0 = p.h0;
  fp.o = io.o;
  fp.final_state = io.final_state;
  fp.hT_out = pl.save ? c.res + pl.h : nullptr;
  fp.vnT_out = pl.save && pl.delta ? c.res + pl.vn : nullptr;
  fp.wT_out = pl.save && pl.delta ? c.res + pl.w : nullptr;
  fp.H = p.H;
  fp.Hk = p.Hk;
  fp.scale = p.scale;
  fp.status = tc_status_ptr();
  fp.state_only = (p.flags & JLA_FLAG_STATE_ONLY) != 0;
  if (!fp.status) return JLA_ERR_CUDA;
  const int blocks = pl.rows * p.H;
  if (vg) {
    if (p.dtype != JLA_DTYPE_BF16) {
      set_error("chunked KDA: bf16 tensors only");
      return JLA_ERR_UNSUPPORTED;
    }
    return launch_one<__nv_bfloat16, true, true>(maps, fp, blocks, s);
  }
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_one<__nv_bfloat16, true>(maps, fp, blocks, s) : launch_one<__nv_bfloat16, false>(maps, fp, blocks, s);
  }
  return pl.delta ? launch_one<__half, true>(maps, fp, blocks, s) : launch_one<__half, false>(maps, fp, blocks, s);
}

}  // namespace jla

#ifdef JLA_TRACE
extern "C" int jla_debug_fwd_trace(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, jla::g_fwd_trace, sizeof(unsigned long long) * 64 * 16) == cudaSuccess ? 0 : -4;
}
#endif
