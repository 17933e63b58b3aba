// Reverse state pass of the backward for K = V = 128 on the Blackwell tensor cores: the mirror image of
// sg_fwd_tc_kernel (chunked_fwd_tc.cu). One persistent CTA per (row, head) walks the row's chunks from last to
// first with dS^T [V lanes x K columns] fp32 in TMEM:
//
//   dVn^T = dO^T (scale P) + (tail Gamma_r)_j (dS+^T K^T)      two accumulators, combined by the state group
//   dW^T  = dVn^T Ag                    (= dV^T)                A operand dVn^T from TMEM
//   dS^T  = keep gamma dS+^T + (scale cin Gamma dO)^T-rows Q - (cin Gamma dW)^T-rows K
//                                                               A operands from TMEM, Q and K read MN-major
//
// Roles: one TMA thread (ring A: q, k and gate vectors, three slots because the scores are built a chunk ahead; ring
// B: dO and the Ag tile, two slots), one MMA thread, eight "state" warps (thread = value row v; warp pairs split the
// 64 token columns) and eight "score" warps that work one chunk ahead, off the serial chain: scale (Q K^T) D, the
// scaled 16-bit copy (scale cin Gamma dO)^T as a TMEM operand, and the per-token scalars. The MMA thread issues the
// chain's products the moment their operands are ready and the others (next chunk's scores, the dO^T Q part of the
// state update) in the gap in which the chain waits for an epilogue.
// As in the forward, nothing leaves the chunk loop through ordinary global stores (they slow down the issue of every
// tcgen05.mma of the CTA): the residuals dh^T [V][K], dVn^T [V][64] and the output dv are written into swizzled
// shared-memory tiles and stored by TMA from two otherwise idle threads.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {
namespace {

using umma::swz_tile;

constexpr int K = 128, V = 128;
constexpr int kThreads = 640;

// VG (per-channel gates, KDA): gate-folded tiles per chunk slot as in the forward (chunked_kda_prep.cu):
// q -> cin q exp(G), k -> cin k exp(G), k2 -> tail k exp(G_63 - G), p -> the masked score tile, ag -> T beta_j; the
// gate vector of the stage carries exp(G_63) per key channel.
struct BwdTcMaps {
  CUtensorMap q, k, d_o, ag, k2, p;   // loads
  CUtensorMap dv, dh_res, dvn_res;    // stores
};

struct BwdTcParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;
  const unsigned char* runs;
  const float* d_final;
  void* dv;
  float* dh0;
  int H, Hk;
  float scale;
  int* status;
};

template <bool VG>
struct SmemT {
  static constexpr int NA = VG ? 2 : 3;
  static constexpr int NB = 2;
  static constexpr int kSlotA = 2 * 64 * K * 2;                                           // q, k
  static constexpr int kSlotB = 64 * V * 2 + 8192 + (VG ? 64 * K * 2 + 8192 : 0);         // dO, Ag (+ k2, P)
  static constexpr int kRingB = NA * kSlotA;
  static constexpr int kPb = kRingB + NB * kSlotB;           // scale P tiles [2][64 x 64] (not VG)
  static constexpr int kStgH = kPb + (VG ? 0 : 2 * 8192);    // dh^T staging, two [V x 64] column blocks
  static constexpr int kStgDvn = kStgH + V * K * 2;          // dVn^T staging [V x 64]
  static constexpr int kGates = kStgDvn + V * 64 * 2;
  static constexpr int kGateStride = 640;
  static constexpr int kScal = kGates + NA * kGateStride;    // per A slot: gam[64], gamr[64], keep gamma
  static constexpr int kScalStride = 1024;
  static constexpr int kBars = kScal + NA * kScalStride;
  static constexpr int kNumBars = 40;
  static constexpr int kBytes = kBars + kNumBars * 8 + 64 + 1024;
  static_assert(kBytes <= 232448, "shared memory of one CTA");
};

enum {
  B_FULLA = 0, B_EMPTYA = 3, B_FULLB = 6, B_EMPTYB = 8,
  B_PDONE = 10, B_PFREE, B_PA0, B_PA1, B_ST, B_MA, B_DV, B_MB, B_DW, B_MC,
  B_HS_FULL, B_HS_FREE, B_DVN_FULL, B_DVN_FREE, B_DVO_FULL0, B_DVO_FULL1, B_DOB0, B_DOB1, B_DOBFREE0, B_DOBFREE1, B_GAM /* 3 */
};

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

// 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 64] swizzled column block
__device__ __forceinline__ uint4* swz_chunk(unsigned char* block, int row, int chunk) {
  return reinterpret_cast<uint4*>(block + row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <typename T, bool DELTA, bool VG>
__global__ void __launch_bounds__(kThreads, 1) sg_bwd_state_tc_kernel(const __grid_constant__ BwdTcMaps maps, BwdTcParams p) {
  static_assert(DELTA || !VG, "per-channel gates come with the delta rule");
  using Smem = SmemT<VG>;
  constexpr int NA = Smem::NA, NB = Smem::NB;
  constexpr int FMT = umma::Fmt<T>::value;
  const int row = blockIdx.x / p.H, h = blockIdx.x - row * p.H;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int2 rc = p.row_chunks[row];
  const int n = rc.y;

  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  auto st_q = [&](int sa) { return base + sa * Smem::kSlotA; };
  auto st_k = [&](int sa) { return st_q(sa) + 64 * K * 2; };
  auto st_do = [&](int sb) { return base + Smem::kRingB + sb * Smem::kSlotB; };
  auto st_ag = [&](int sb) { return st_do(sb) + 64 * V * 2; };
  auto st_k2 = [&](int sb) { return st_ag(sb) + 8192; };       // VG only
  auto st_p = [&](int sb) { return st_k2(sb) + 64 * K * 2; };  // VG only
  auto st_G = [&](int sa) { return reinterpret_cast<float*>(base + Smem::kGates + sa * Smem::kGateStride); };
  auto st_runs = [&](int sa) { return reinterpret_cast<unsigned char*>(st_G(sa) + 128); };
  auto st_meta = [&](int sa) { return reinterpret_cast<volatile int*>(st_runs(sa) + 64); };
  auto st_gam = [&](int sa) { return reinterpret_cast<float*>(base + Smem::kScal + sa * Smem::kScalStride); };
  unsigned char* Pb = base + Smem::kPb;
  unsigned char* stgH = base + Smem::kStgH;
  unsigned char* stgDvn = base + Smem::kStgDvn;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < 3; ++s) {
      umma::mbar_init(bars + B_FULLA + s, 1);
      umma::mbar_init(bars + B_EMPTYA + s, 1 + 8);  // MMA commit + the state warps
      umma::mbar_init(bars + B_GAM + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      umma::mbar_init(bars + B_FULLB + s, 1);
      umma::mbar_init(bars + B_EMPTYB + s, 1 + 1);  // MMA commit + the dv store thread
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
    umma::mbar_init(bars + B_HS_FULL, 8);
    umma::mbar_init(bars + B_HS_FREE, 1);
    umma::mbar_init(bars + B_DVN_FULL, 8);
    umma::mbar_init(bars + B_DVN_FREE, 1);
    umma::mbar_init(bars + B_DVO_FULL0, 8);
    umma::mbar_init(bars + B_DVO_FULL1, 8);
    umma::mbar_init(bars + B_DOB0, 8);
    umma::mbar_init(bars + B_DOB1, 8);
    umma::mbar_init(bars + B_DOBFREE0, 1);
    umma::mbar_init(bars + B_DOBFREE1, 1);
    umma::mbar_init_fence();
    *abort_flag = 0;
  }
  if (warp == 2) umma::tmem_alloc(tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // dS^T fp32 | dS^T 16-bit | acc1 = dS+^T K^T, later dW^T | acc2 = dO^T (scale P) | dVn^T 16-bit |
  // -(cin Gamma) dW^T 16-bit | scale (cin Gamma) dO^T 16-bit, two buffers (written a chunk ahead) | Q K^T
  constexpr uint32_t cS = 0, cSb = 128, cA1 = 192, cA2 = 256, cDVb = 320, cDWb = 352, cDOb0 = 384, cP = 448;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int sa = it % NA, sb = it % NB, c = rc.x + (n - 1 - it);
        if (!wait(bars + B_EMPTYA + sa, ((it / NA) & 1) ^ 1, abort_flag)) break;
        const ChunkMeta m = p.meta[c];
        volatile int* ms = st_meta(sa);
        ms[0] = m.tok0;
        ms[1] = m.len;
        ms[2] = m.flags;
        const int slot_row = (c * p.H + h) * 64;
        tma::expect_tx(bars + B_FULLA + sa, 2 * 64 * K * 2 + 512 + 64);
        if (VG) {
          tma::load_tile<64, K>(st_k(sa), &maps.k, 0, 0, slot_row, bars + B_FULLA + sa);
          tma::load_tile<64, K>(st_q(sa), &maps.q, 0, 0, slot_row, bars + B_FULLA + sa);
        } else {
          tma::load_tile<64, K>(st_k(sa), &maps.k, 0, hk, m.tok0, bars + B_FULLA + sa);
          tma::load_tile<64, K>(st_q(sa), &maps.q, 0, hk, m.tok0, bars + B_FULLA + sa);
        }
        bulk_copy(st_G(sa), p.gates + ((long)c * p.H + h) * 128, 512, bars + B_FULLA + sa);
        bulk_copy(st_runs(sa), p.runs + (long)c * 64, 64, bars + B_FULLA + sa);
        if (!wait(bars + B_EMPTYB + sb, ((it / NB) & 1) ^ 1, abort_flag)) break;
        tma::expect_tx(bars + B_FULLB + sb, 64 * V * 2 + (DELTA ? 8192 : 0) + (VG ? 64 * K * 2 + 8192 : 0));
        tma::load_tile<64, V>(st_do(sb), &maps.d_o, 0, h, m.tok0, bars + B_FULLB + sb);
        if (DELTA) tma::load_tile<64, 64>(st_ag(sb), &maps.ag, 0, 0, slot_row, bars + B_FULLB + sb);
        if (VG) {
          tma::load_tile<64, K>(st_k2(sb), &maps.k2, 0, 0, slot_row, bars + B_FULLB + sb);
          tma::load_tile<64, 64>(st_p(sb), &maps.p, 0, 0, slot_row, bars + B_FULLB + sb);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      auto issue_p = [&](int it) {
        const int sa = it % NA;
        if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) return false;
        if (!wait(bars + B_PFREE, (it & 1) ^ 1, abort_flag)) return false;
        umma::fence_after_sync();
        umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP, umma::smem_addr(st_q(sa)), 64, umma::smem_addr(st_k(sa)), 64,
                                                      false);
        umma::commit(bars + B_PDONE);
        return true;
      };
      bool okm = n > 0 && !VG ? issue_p(0) : true;
      for (int it = 0; it < n && okm; ++it) {
        const int sa = it % NA, sb = it % NB;
        const uint32_t ph = it & 1;
        const uint32_t aq = umma::smem_addr(st_q(sa)), ak = umma::smem_addr(st_k(sa)), ado = umma::smem_addr(st_do(sb));
        if (!wait(bars + B_ST, ph, abort_flag)) break;
        if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) break;
        if (!wait(bars + B_FULLB + sb, (it / NB) & 1, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cA1, tmem + cSb, VG ? umma::smem_addr(st_k2(sb)) : ak, 64,
                                                   false);  // dS+^T K^T
        if (!VG && !wait(bars + B_PA0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
        // dO^T (scale P): A = dO tile read MN-major (M = value index), B = P tile read MN-major (rows i)
        umma::gemm<128, 64, 4, true, true, FMT>(tmem + cA2, ado, 64,
                                                VG ? umma::smem_addr(st_p(sb)) : umma::smem_addr(Pb + (it & 1) * 8192), 64, false);
        umma::commit(bars + B_MA);
        // Off the chain, while the state group combines the two accumulators: the dO part of the state update (its
        // 16-bit operand was written a chunk ahead by the score group) and the next chunk's scores.
        if (!wait(bars + B_DOB0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
        umma::fence_after_sync();
        umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cDOb0 + 32 * ph, aq, 64, true);  // += (s cg dO)^T Q
        umma::commit(bars + B_DOBFREE0 + (it & 1));  // the operand buffer may be rewritten once this product is done
        if (!VG && it + 1 < n && !issue_p(it + 1)) break;
        if (DELTA) {
          if (!wait(bars + B_DV, ph, abort_flag)) break;
          umma::fence_after_sync();
          umma::gemm_ts<128, 64, 4, true, FMT>(tmem + cA1, tmem + cDVb, umma::smem_addr(st_ag(sb)), 64, false);  // dVn^T Ag
          umma::commit(bars + B_MB);
          umma::commit(bars + B_EMPTYB + sb);  // dO, Ag (and with VG k2, P) are consumed when these products are done
        } else {
          umma::commit(bars + B_EMPTYB + sb);
        }
        if (!wait(bars + B_DW, ph, abort_flag)) break;
        umma::fence_after_sync();
        if (DELTA) umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cDWb, ak, 64, true);     // += (-cg dW)^T K
        umma::commit(bars + B_MC);
        umma::commit(bars + B_EMPTYA + sa);
      }
    }
  } else if (warp == 2) {
    // --------------------------------------------------------- residual stores: dh^T, dVn^T as TMA tensor stores
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n && ok; ++it) {
        const int row0 = ((rc.x + (n - 1 - it)) * p.H + h) * V;
        ok = wait(bars + B_HS_FULL, it & 1, abort_flag);
        if (!ok) break;
        tma::store_3d(&maps.dh_res, stgH, 0, 0, row0);
        tma::store_3d(&maps.dh_res, stgH + V * 128, 64, 0, row0);
        tma::store_commit();
        tma::store_wait_read<0>();
        mbar_arrive(bars + B_HS_FREE);
        if (DELTA) {
          ok = wait(bars + B_DVN_FULL, it & 1, abort_flag);
          if (!ok) break;
          tma::store_3d(&maps.dvn_res, stgDvn, 0, 0, row0);
          tma::store_commit();
          tma::store_wait_read<0>();
          mbar_arrive(bars + B_DVN_FREE);
        }
      }
      tma::store_wait<0>();
    }
  } else if (warp == 3) {
    // ------------------------------------------------ dv: the staged tile of a full chunk as TMA tensor stores
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n && ok; ++it) {
        const int sb = it % NB;
        ok = wait(bars + B_DVO_FULL0 + (it & 1), (it >> 1) & 1, abort_flag);
        if (!ok) break;
        const ChunkMeta m = p.meta[rc.x + (n - 1 - it)];
        if (m.len == 64) {  // a partial chunk was written by the state warps themselves (rows past its end belong to others)
          tma::store_3d(&maps.dv, st_do(sb), 0, h, m.tok0);
          tma::store_3d(&maps.dv, st_do(sb) + 64 * 128, 64, h, m.tok0);
          tma::store_commit();
          tma::store_wait_read<0>();
        }
        mbar_arrive(bars + B_EMPTYB + sb);
      }
      tma::store_wait<0>();
    }
  } else if (warp >= 4 && warp < 12) {
    const int q4 = warp & 3, half = (warp - 4) >> 2, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int sa = it % NA, sb = it % NB;
      const uint32_t ph = it & 1;
      // the chunk's tiles have landed (and, without VG, its per-token scalars are written)
      ok = wait(bars + (VG ? B_FULLA : B_GAM) + sa, (it / NA) & 1, abort_flag);
      if (!ok) break;
      const float* Gs = st_G(sa);
      const int tok0 = st_meta(sa)[0], len = st_meta(sa)[1];
      const float* gam = st_gam(sa);
      const float* gamr = gam + 64;
      const float kg = VG ? 0.f : gam[128];
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
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_ST);
      {  // this half row of dS+^T into the staging tile (column block `half`, row v)
        if (it > 0) {
          ok = wait(bars + B_HS_FREE, ph ^ 1, abort_flag);
          if (!ok) break;
        }
        unsigned char* blk = stgH + half * (V * 128);
#pragma unroll
        for (int i = 0; i < 8; ++i) *swz_chunk(blk, v, i) = make_uint4(hpk[4 * i], hpk[4 * i + 1], hpk[4 * i + 2], hpk[4 * i + 3]);
        umma::fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_HS_FULL);
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
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 gr = VG ? make_float4(1.f, 1.f, 1.f, 1.f) : *reinterpret_cast<const float4*>(gamr + j0 + 4 * i4);
          const int j = j0 + 4 * i4;
          // columns of tokens past a partial chunk are forced to zero (their inputs are other rows' data)
          const float a0 = j < len ? pscale * y[4 * i4] + gr.x * x[4 * i4] : 0.f;
          const float a1 = j + 1 < len ? pscale * y[4 * i4 + 1] + gr.y * x[4 * i4 + 1] : 0.f;
          const float a2 = j + 2 < len ? pscale * y[4 * i4 + 2] + gr.z * x[4 * i4 + 2] : 0.f;
          const float a3 = j + 3 < len ? pscale * y[4 * i4 + 3] + gr.w * x[4 * i4 + 3] : 0.f;
          dvn[2 * i4] = pack2<T>(a0, a1);
          dvn[2 * i4 + 1] = pack2<T>(a2, a3);
        }
      }
      // the dead dO tile of this chunk takes dv as a [64 tokens x V] swizzled tile (thread = value column v)
      T* stg = reinterpret_cast<T*>(st_do(sb));
      if (DELTA) {
        umma::st_32x32b_x16(tl + cDVb + 16 * half, dvn);
        {  // (the shared-memory stores run while the TMEM store completes)
          if (it > 0) {
            ok = wait(bars + B_DVN_FREE, ph ^ 1, abort_flag);
            if (!ok) break;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) *swz_chunk(stgDvn, v, 4 * half + i) = make_uint4(dvn[4 * i], dvn[4 * i + 1], dvn[4 * i + 2], dvn[4 * i + 3]);
        }
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DV);
        umma::fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DVN_FULL);
        // ---- dW^T = dVn^T Ag ; -(cin Gamma)_j dW^T as the next A operand; dv
        ok = wait(bars + B_MB, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        float x[32];
        ld_row32(x, tl + cA1 + j0);
        uint32_t pk[16];
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4) {
          const float4 gm = VG ? make_float4(1.f, 1.f, 1.f, 1.f) : *reinterpret_cast<const float4*>(gam + j0 + 4 * i4);
          pk[2 * i4] = pack2<T>(-gm.x * x[4 * i4], -gm.y * x[4 * i4 + 1]);
          pk[2 * i4 + 1] = pack2<T>(-gm.z * x[4 * i4 + 2], -gm.w * x[4 * i4 + 3]);
        }
        umma::st_32x32b_x16(tl + cDWb + 16 * half, pk);
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bars + B_DW);
          mbar_arrive(bars + B_EMPTYA + sa);  // done with this chunk's gate vectors
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) stg[swz_tile(64, j0 + i, v)] = from_f32<T>(x[i]);
      } else {
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bars + B_DW);  // dW = dVn: nothing more for the state update
          mbar_arrive(bars + B_EMPTYA + sa);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 f = unpack2<T>(dvn[i]);
          stg[swz_tile(64, j0 + 2 * i, v)] = from_f32<T>(f.x);
          stg[swz_tile(64, j0 + 2 * i + 1, v)] = from_f32<T>(f.y);
        }
      }
      if (len < 64) {  // partial chunk: this warp writes its own 32 tokens x 32 value columns, up to the chunk's end
        __syncwarp();
        T* dv = static_cast<T*>(p.dv) + ((long)(tok0 + j0) * p.H + h) * V + 32 * q4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = lane + 32 * i, tok = idx >> 2, part = idx & 3;
          if (j0 + tok < len) {
            *reinterpret_cast<uint4*>(dv + (long)tok * p.H * V + part * 8) =
                *reinterpret_cast<const uint4*>(stg + swz_tile(64, j0 + tok, 32 * q4 + part * 8));
          }
        }
      }
      umma::fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_DVO_FULL0 + (it & 1));
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
    // ---- score group, one chunk ahead of the chain: the per-token scalars (first warp), the scaled 16-bit copy
    // (scale cin Gamma dO)^T as a TMEM operand (thread = value row v, 32 tokens per warp), and scale (Q K^T) D stored
    // [i][j] (read MN-major by the dO^T P product)
    const int q4 = warp & 3, half = (warp - 12) >> 2, g = lane >> 2, t = lane & 3;
    const int r0 = 16 * q4, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    auto prepare = [&](int it) {
      const int sa = it % NA, sb = it % NB, buf = it & 1;
      if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) return false;
      const float* Gs = st_G(sa);
      const unsigned char* runs = st_runs(sa);
      const int len = st_meta(sa)[1], flags = st_meta(sa)[2];
      float* gam = st_gam(sa);
      if (!VG && warp == 12) {  // per-token scalars, once for the CTA
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = lane + 32 * jj;
          const RowScalars rs = row_scalars(Gs, runs, flags, j);
          gam[j] = rs.gam;
          gam[64 + j] = rs.gamr;
        }
        if (lane == 0) gam[128] = keep_gamma(Gs, runs, flags);
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_GAM + sa);
      }
      // ---- scale (cin Gamma)_i dO^T, tokens 32 half .. + 31 of value row v
      if (!wait(bars + B_FULLB + sb, (it / NB) & 1, abort_flag)) return false;
      if (it >= 2) {  // the product that read this buffer two chunks ago is done (one barrier per buffer: a wait on a
        // barrier that completes every chunk could be two phases late and would then mistake the parity)
        if (!wait(bars + B_DOBFREE0 + buf, ((it >> 1) & 1) ^ 1, abort_flag)) return false;
        umma::fence_after_sync();
      }
      {
        if (!VG && !wait(bars + B_GAM + sa, (it / NA) & 1, abort_flag)) return false;  // the first warp's scalars
        const T* dos = reinterpret_cast<const T*>(st_do(sb));
        const int j0 = 32 * half;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int j = j0 + 2 * i;
          const float2 cg = VG ? make_float2(1.f, 1.f) : *reinterpret_cast<const float2*>(gam + j);
          const float a = (j < len) ? to_f32(dos[swz_tile(64, j, v)]) * p.scale * cg.x : 0.f;
          const float b = (j + 1 < len) ? to_f32(dos[swz_tile(64, j + 1, v)]) * p.scale * cg.y : 0.f;
          pk[i] = pack2<T>(a, b);
        }
        umma::st_32x32b_x16(tl + cDOb0 + 32 * buf + 16 * half, pk);
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_DOB0 + buf);
      }
      if (VG) return true;  // the score tile arrives with the stage: nothing to build
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
      if (lane == 0) mbar_arrive(bars + B_PA0 + buf);
      return true;
    };
    for (int it = 0; it < n && ok; ++it) ok = prepare(it);
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
    kern<<<blocks, kThreads, SmemT<VG>::kBytes, s>>>(maps, bp);
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
  bool ok = tma::encode_3d(&maps.d_o, io.d_o, p.V, p.H, tokens, 64) && tma::encode_3d(&maps.dv, io.dv, p.V, p.H, tokens, 64) &&
            tma::encode_3d(&maps.dh_res, scratch + pl.dh, p.K, 1, slots * p.V, p.V);
  if (ok && pl.delta) ok = tma::encode_3d(&maps.dvn_res, scratch + pl.dvn, 64, 1, slots * p.V, p.V);
  if (ok && !pl.delta) maps.dvn_res = maps.d_o;
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
  bp.H = p.H;
  bp.Hk = p.Hk;
  bp.scale = p.scale;
  bp.status = tc_status_ptr();
  if (!bp.status) return JLA_ERR_CUDA;
  const int blocks = pl.rows * p.H;
  if (vg) {
    return p.dtype == JLA_DTYPE_BF16 ? launch_one<__nv_bfloat16, true, true>(maps, bp, blocks, s)
                                     : launch_one<__half, true, true>(maps, bp, blocks, s);
  }
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_one<__nv_bfloat16, true>(maps, bp, blocks, s) : launch_one<__nv_bfloat16, false>(maps, bp, blocks, s);
  }
  return pl.delta ? launch_one<__half, true>(maps, bp, blocks, s) : launch_one<__half, false>(maps, bp, blocks, s);
}

}  // namespace jla
