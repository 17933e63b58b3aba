// Forward of the scalar-gate family for K = V = 128 on the Blackwell tensor cores, one persistent CTA per
// (row, head) walking the row's chunks. Everything on the serial chain lives in TMEM and registers:
//
//   * the state is kept TRANSPOSED, S^T [V lanes x K columns] fp32, as the accumulator of the update product;
//     a bf16/f16 copy of it (packed pairs) sits next to it and is the A operand (from TMEM) of S^T K^T and S^T Q^T;
//   * W^T = V^T - (cin Gamma)_j (S^T K^T), Vn^T = W^T Ag^T and (tail Gamma_r Vn)^T are produced by four warps whose
//     thread index IS the value row v, written back to TMEM as packed 16-bit A operands; no shared-memory round
//     trip and no CTA-wide barrier sits between two dependent products;
//   * per chunk the chain is  S^T K^T -> W^T -> W^T Ag^T -> Vn^T -> S^T += (Gamma_r Vn)^T K  (three M = 128 products),
//     while a second group of four warps builds P = (Q K^T) D (64 x 64 tiles, into swizzled shared memory) for the
//     next chunk and writes the outputs O^T = scale[(cin Gamma)_i (S^T Q^T) + Vn^T P^T]; the one thread that issues
//     every product (40 - 100 ns of its time per tcgen05.mma) issues the chain's products the moment their operands
//     are ready and everything else in the gaps in which the chain waits for an epilogue (the next chunk's scores
//     behind the first chain product, the two output products behind the state update);
//   * one thread issues all tcgen05.mma, one thread issues the TMA loads into two rings -- q, k and the gate
//     vectors in three slots (they are read one chunk ahead by the score product), v and the Ag tile in two --
//     and mbarriers (bounded waits, shared abort flag) connect the roles;
//   * NOTHING is stored to global memory with ordinary store instructions inside the chunk loop. While warps of the
//     CTA issue st.global (above all the 16-byte stores of a residual row per thread, 32 different sectors per
//     instruction) every tcgen05.mma of the issuing thread takes about 125 ns to issue instead of about 40: measured
//     with the global timer, the products of the chain were issued exactly as slowly as the stores next to them took.
//     The residuals h^T, W^T, Vn^T and the outputs are therefore written into 128-byte-swizzled shared-memory tiles
//     (conflict-free 16-byte / 2-byte accesses) and leave the SM as TMA tensor stores issued by two otherwise idle
//     threads; the tiles are handed back through mbarriers once the copy has read them.
//
// Same math and roundings as sg_fwd_kernel (chunked_fwd.cu). The residuals it saves are transposed
// (h^T [V][K], Vn^T, W^T [V][64] per chunk and head) because a thread owns a value row.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace jla {
namespace {

using umma::swz_tile;

constexpr int K = 128, V = 128;
constexpr int kThreads = 640;  // 20 warps: loads, products, two store threads, 8 state + 8 score warps

// Build with -DJLA_TRACE to record, for the first CTA, the global timer at the hand-offs of the serial chain
// (32 slots per chunk: 0, 1, 3, 4, 6, 7 by the first state warp, 20 and up by the first score warp, the others by the MMA issuer); jla_debug_fwd_trace() copies them out.
#ifdef JLA_TRACE
__device__ unsigned long long g_fwd_trace[64 * 32];
__device__ unsigned long long g_fwd_cta[4096 * 4];
__device__ unsigned long long g_fwd_warps[64 * 16 * 6];  // first CTA: per chunk and compute warp, six event times  // per CTA: kernel entry, first chunk start, last chunk end, exit
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
#define JLA_MARK(it, slot)                                                                     \
  do {                                                                                         \
    if (blockIdx.x == 0 && (it) < 64) g_fwd_trace[(it) * 32 + (slot)] = global_timer();         \
  } while (0)
#define JLA_WMARK(it, w, ev)                                                                                   \
  do {                                                                                                         \
    if (blockIdx.x == 0 && (it) < 64 && lane == 0) g_fwd_warps[((it) * 16 + (w)) * 6 + (ev)] = global_timer(); \
  } while (0)
#else
#define JLA_MARK(it, slot) \
  do {                     \
  } while (0)
#define JLA_WMARK(it, w, ev) \
  do {                       \
  } while (0)
#endif

// VG (per-channel gates, KDA): the tiles come gate-folded from kda_prep_kernel, one set per chunk slot:
// q -> cin q exp(G), k -> cin k exp(G) (recall), k2 -> tail k exp(G_63 - G) (write), p -> the masked score tile,
// ag -> T beta_j, and the G/beta vector of the stage carries the decay exp(G_63) of the K state columns instead.
struct FwdTcMaps {
  CUtensorMap q, k, v, ag, k2, p;     // loads
  CUtensorMap o, h_res, w_res, vn_res;  // stores: outputs [tokens][H][V]; residuals [slot * V][K] and [slot * V][64]
};

struct FwdTcParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;  // VG: the per-slot decay vectors [K]
  const unsigned char* runs;
  const float* h0;
  void* o;
  float* final_state;
  int save;  // write the residuals h^T, Vn^T, W^T (through the tensor maps)
  int H, Hk;
  float scale;
  int* status;
  int state_only;  // final state (and residuals) only: no scores, no outputs
};

// Shared memory. Ring A (NA slots): q, k [64 x K] and the gate vectors of a chunk; ring B (2 slots): v [64 x V], the Ag
// tile and, with VG, the write-side keys and the score tile. Staging tiles for the residual stores: h^T [V x K] and one
// [V x 64] tile that W^T and Vn^T use in turn. The outputs are staged in the chunk's dead q tile.
template <bool VG>
struct SmemT {
  static constexpr int NA = VG ? 2 : 3;  // the score product of chunk it + 1 is built during chunk it (not with VG)
  static constexpr int NB = 2;
  static constexpr int kSlotA = 2 * 64 * K * 2;
  static constexpr int kSlotB = 64 * V * 2 + 8192 + (VG ? 64 * K * 2 + 8192 : 0);
  static constexpr int kRingB = NA * kSlotA;
  static constexpr int kPb = kRingB + NB * kSlotB;          // P tiles [2][64 x 64] (not VG)
  static constexpr int kStgH = kPb + (VG ? 0 : 2 * 8192);   // h^T staging, two [V x 64] column blocks
  static constexpr int kStgWV = kStgH + V * K * 2;          // W^T / Vn^T staging [V x 64]
  static constexpr int kGates = kStgWV + V * 64 * 2;        // per A slot: G[64], beta[64] f32 (512 B) + runs (64 B) + meta (16 B)
  static constexpr int kGateStride = 640;
  static constexpr int kScal = kGates + NA * kGateStride;   // per A slot: gam[64], gamr[64], keep gamma (one warp writes them)
  static constexpr int kScalStride = 1024;
  static constexpr int kBars = kScal + NA * kScalStride;
  static constexpr int kNumBars = 40;
  static constexpr int kBytes = kBars + kNumBars * 8 + 64 + 1024;
  static_assert(kBytes <= 232448, "shared memory of one CTA");
};

enum {  // mbarrier indices
  B_FULLA = 0, B_EMPTYA = 3, B_FULLB = 6, B_EMPTYB = 8,
  B_PDONE = 10, B_PFREE, B_PA0, B_PA1, B_ST, B_M1, B_W, B_M2, B_VN, B_M3, B_ODONE, B_OFREE, B_SPARE,
  B_HS_FULL, B_HS_FREE, B_WV_FULL, B_WV_FREE, B_O_FULL0, B_O_FULL1, B_GAM /* 3 */
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

// 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 64] swizzled column block
__device__ __forceinline__ uint4* swz_chunk(unsigned char* block, int row, int chunk) {
  return reinterpret_cast<uint4*>(block + row * 128 + ((chunk ^ (row & 7)) << 4));
}

template <typename T, bool DELTA, bool VG>
__global__ void __launch_bounds__(kThreads, 1) sg_fwd_tc_kernel(const __grid_constant__ FwdTcMaps maps, FwdTcParams p) {
  static_assert(DELTA || !VG, "per-channel gates come with the delta rule");
  using Smem = SmemT<VG>;
  constexpr int NA = Smem::NA, NB = Smem::NB;
  constexpr int FMT = umma::Fmt<T>::value;
  const int row = blockIdx.x / p.H, h = blockIdx.x - row * p.H;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int2 rc = p.row_chunks[row];
  const int n = rc.y;
  const bool save = p.save != 0;

#ifdef JLA_TRACE
  if (tid == 128 && blockIdx.x < 4096) g_fwd_cta[blockIdx.x * 4] = global_timer();
#endif
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  auto st_q = [&](int sa) { return base + sa * Smem::kSlotA; };
  auto st_k = [&](int sa) { return st_q(sa) + 64 * K * 2; };
  auto st_v = [&](int sb) { return base + Smem::kRingB + sb * Smem::kSlotB; };
  auto st_t0 = [&](int sb) { return st_v(sb) + 64 * V * 2; };
  auto st_k2 = [&](int sb) { return st_t0(sb) + 8192; };      // VG only
  auto st_p = [&](int sb) { return st_k2(sb) + 64 * K * 2; };  // VG only
  auto st_G = [&](int sa) { return reinterpret_cast<float*>(base + Smem::kGates + sa * Smem::kGateStride); };
  auto st_runs = [&](int sa) { return reinterpret_cast<unsigned char*>(st_G(sa) + 128); };
  auto st_meta = [&](int sa) { return reinterpret_cast<volatile int*>(st_runs(sa) + 64); };
  auto st_gam = [&](int sa) { return reinterpret_cast<float*>(base + Smem::kScal + sa * Smem::kScalStride); };
  unsigned char* Pb = base + Smem::kPb;
  unsigned char* stgH = base + Smem::kStgH;
  unsigned char* stgWV = base + Smem::kStgWV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + Smem::kBars);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Smem::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (tid == 0) {
    for (int s = 0; s < 3; ++s) {
      umma::mbar_init(bars + B_FULLA + s, 1);        // the producer's expect_tx arrival (+ bytes)
      umma::mbar_init(bars + B_EMPTYA + s, 1 + 8 + 1);  // MMA commit + the state warps + the output store thread
    }
    for (int s = 0; s < 2; ++s) {
      umma::mbar_init(bars + B_FULLB + s, 1);
      umma::mbar_init(bars + B_EMPTYB + s, 8 + (DELTA ? 1 : 0));  // the state warps (+ MMA commit)
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
    umma::mbar_init(bars + B_OFREE, 8);
    umma::mbar_init(bars + B_HS_FULL, 8);
    umma::mbar_init(bars + B_HS_FREE, 1);
    umma::mbar_init(bars + B_WV_FULL, 8);
    umma::mbar_init(bars + B_WV_FREE, 1);
    umma::mbar_init(bars + B_O_FULL0, 8);
    umma::mbar_init(bars + B_O_FULL1, 8);
    for (int s = 0; s < 3; ++s) umma::mbar_init(bars + B_GAM + s, 1);
    umma::mbar_init_fence();
    *abort_flag = 0;
  }
  if (warp == 2) umma::tmem_alloc(tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  // TMEM columns: S^T fp32 | its 16-bit copy, two buffers (chunk parity: the output product of a chunk still reads
  // one while the next chunk's copy is written) | chain accumulator | Vn^T / W^T 16-bit | (Gamma_r Vn)^T 16-bit |
  // output accumulator | score accumulator
  constexpr uint32_t cS = 0, cSb0 = 128, cA1 = 256, cWb = 320, cVg = 352, cO = 384, cP = 448;

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int sa = it % NA, sb = it % NB, c = rc.x + it;
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
        tma::load_tile<64, V>(st_v(sb), &maps.v, 0, h, m.tok0, bars + B_FULLB + sb);
        if (DELTA) tma::load_tile<64, 64>(st_t0(sb), &maps.ag, 0, 0, slot_row, bars + B_FULLB + sb);
        if (VG) {
          tma::load_tile<64, K>(st_k2(sb), &maps.k2, 0, 0, slot_row, bars + B_FULLB + sb);
          tma::load_tile<64, 64>(st_p(sb), &maps.p, 0, 0, slot_row, bars + B_FULLB + sb);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      auto issue_p = [&](int it) {  // Q K^T of chunk `it` (its inputs are prefetched): runs one chunk ahead of the chain
        const int sa = it % NA;
        if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) return false;
        if (!wait(bars + B_PFREE, (it & 1) ^ 1, abort_flag)) return false;
        umma::fence_after_sync();
        JLA_MARK(it - 1, 15);
        umma::gemm<64, 64, K / 16, false, false, FMT>(tmem + cP, umma::smem_addr(st_q(sa)), 64, umma::smem_addr(st_k(sa)), 64,
                                                      false);
        umma::commit(bars + B_PDONE);
        return true;
      };
      bool okm = n > 0 && !p.state_only && !VG ? issue_p(0) : true;
      for (int it = 0; it < n && okm; ++it) {
        const int sa = it % NA, sb = it % NB;
        const uint32_t ph = it & 1;
        const uint32_t aq = umma::smem_addr(st_q(sa)), ak = umma::smem_addr(st_k(sa));
        const uint32_t cSb = cSb0 + 64 * ph;
        if (!wait(bars + B_ST, ph, abort_flag)) break;
        if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) break;  // (long complete; makes the tiles visible to this thread)
        umma::fence_after_sync();
        JLA_MARK(it, 9);
        if (DELTA) {
          umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cA1, tmem + cSb, ak, 64, false);  // S^T K^T
          umma::commit(bars + B_M1);
        }
        JLA_MARK(it, 10);
        // Products that are not on the chain are issued while the chain waits for an epilogue anyway: the next chunk's
        // scores here (the state group is busy with W), this chunk's two output products after the state update (the
        // state group is busy with the new state).
        if (!p.state_only && !VG && it + 1 < n) {
          if (!issue_p(it + 1)) break;
          JLA_MARK(it, 2);
        }
        if (DELTA) {
          if (!wait(bars + B_W, ph, abort_flag)) break;
          if (!wait(bars + B_FULLB + sb, (it / NB) & 1, abort_flag)) break;
          umma::fence_after_sync();
          JLA_MARK(it, 11);
          umma::gemm_ts<128, 64, 4, false, FMT>(tmem + cA1, tmem + cWb, umma::smem_addr(st_t0(sb)), 64, false);  // W^T Ag^T
          umma::commit(bars + B_M2);
          if (!VG) umma::commit(bars + B_EMPTYB + sb);  // the Ag tile is consumed when these products are done
          JLA_MARK(it, 12);
        }
        if (!wait(bars + B_VN, ph, abort_flag)) break;
        umma::fence_after_sync();
        JLA_MARK(it, 13);
        umma::gemm_ts<128, 128, 4, true, FMT>(tmem + cS, tmem + cVg, VG ? umma::smem_addr(st_k2(sb)) : ak, 64,
                                              true);  // S^T += (Gamma_r Vn)^T K
        umma::commit(bars + B_M3);
        JLA_MARK(it, 14);
        if (!p.state_only) {
          // q has been scaled by (cin Gamma)_i in place by the score group (part of "PA ready"); the previous chunk's
          // outputs have left the accumulator
          if (!VG && !wait(bars + B_PA0 + (it & 1), (it >> 1) & 1, abort_flag)) break;
          if (!wait(bars + B_OFREE, ph ^ 1, abort_flag)) break;
          umma::fence_after_sync();
          JLA_MARK(it, 5);
          umma::gemm_ts<128, 64, K / 16, false, FMT>(tmem + cO, tmem + cSb, aq, 64, false);  // S^T ((cin Gamma) Q)^T
          const uint32_t ap = VG ? umma::smem_addr(st_p(sb)) : umma::smem_addr(Pb + (it & 1) * 8192);
          umma::gemm_ts<128, 64, 4, false, FMT>(tmem + cO, tmem + cWb, ap, 64, true);  // += Vn^T P^T
          JLA_MARK(it, 8);
        }
        umma::commit(bars + B_ODONE);
        if (VG) umma::commit(bars + B_EMPTYB + sb);  // write-side keys and the score tile are consumed
        umma::commit(bars + B_EMPTYA + sa);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------- residual stores: h^T, W^T, Vn^T as TMA tensor stores
    if (lane == 0 && save) {
      bool ok = true;
      for (int it = 0; it < n && ok; ++it) {
        const int row0 = ((rc.x + it) * p.H + h) * V;  // first row of this (chunk, head) in the [slot * V][.] residuals
        ok = wait(bars + B_HS_FULL, it & 1, abort_flag);
        if (!ok) break;
        tma::store_3d(&maps.h_res, stgH, 0, 0, row0);
        tma::store_3d(&maps.h_res, stgH + V * 128, 64, 0, row0);
        tma::store_commit();
        tma::store_wait_read<0>();
        mbar_arrive(bars + B_HS_FREE);
        if (DELTA) {
          ok = wait(bars + B_WV_FULL, 0, abort_flag);
          if (!ok) break;
          tma::store_3d(&maps.w_res, stgWV, 0, 0, row0);
          tma::store_commit();
          tma::store_wait_read<0>();
          mbar_arrive(bars + B_WV_FREE);
          ok = wait(bars + B_WV_FULL, 1, abort_flag);
          if (!ok) break;
          tma::store_3d(&maps.vn_res, stgWV, 0, 0, row0);
          tma::store_commit();
          tma::store_wait_read<0>();
          mbar_arrive(bars + B_WV_FREE);
        }
      }
      tma::store_wait<0>();
    }
  } else if (warp == 3) {
    // ------------------------------------------- output stores: the staged O tile of a full chunk as TMA tensor stores
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n && ok; ++it) {
        const int sa = it % NA;
        if (p.state_only) {  // nothing is staged: only hand the slot back once it has been filled
          ok = wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag);
          if (ok) mbar_arrive(bars + B_EMPTYA + sa);
          continue;
        }
        // (two barriers in turn: the score warps may be up to two chunks ahead of this thread)
        ok = wait(bars + B_O_FULL0 + (it & 1), (it >> 1) & 1, abort_flag);
        if (!ok) break;
        const ChunkMeta m = p.meta[rc.x + it];
        if (m.len == 64) {  // a partial chunk was written by the score warps themselves (rows past its end belong to others)
          tma::store_3d(&maps.o, st_q(sa), 0, h, m.tok0);
          tma::store_3d(&maps.o, st_q(sa) + 64 * 128, 64, h, m.tok0);
          tma::store_commit();
          tma::store_wait_read<0>();
        }
        mbar_arrive(bars + B_EMPTYA + sa);
      }
      tma::store_wait<0>();
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------- state group: thread = value row v, warp pair = column halves
    const int q4 = warp & 3, half = (warp - 4) >> 2, v = 32 * q4 + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * q4) << 16);
    bool ok = true;
    for (int it = 0; it < n && ok; ++it) {
      const int sa = it % NA, sb = it % NB;
      const uint32_t ph = it & 1;
      // the chunk's tiles have landed (and, without VG, its per-token scalars are written)
      ok = wait(bars + (VG ? B_FULLA : B_GAM) + sa, (it / NA) & 1, abort_flag);
      if (!ok) break;
      if (tid == 128 && it > 0) JLA_MARK(it - 1, 18);
      const float* Gs = st_G(sa);
      const float* gam = st_gam(sa);  // (cin Gamma)_j, (tail Gamma_r)_j (zero past a partial chunk), keep gamma
      const float* gamr = gam + 64;
      const float kg = VG ? 0.f : gam[128];
      if (tid == 128 && it > 0) JLA_MARK(it - 1, 17);
      // ---- the state entering this chunk: 16-bit copy for the products, decayed fp32 copy for the update
      if (it > 0) {
        ok = wait(bars + B_M3, ph ^ 1, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
      }
      if (tid == 128) JLA_MARK(it, 0);
      JLA_WMARK(it, warp - 4, 0);
#ifdef JLA_TRACE
      if (tid == 128 && it == 0 && blockIdx.x < 4096) g_fwd_cta[blockIdx.x * 4 + 1] = global_timer();
#endif
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
        umma::st_32x32b_x16(tl + cSb0 + 64 * ph + blk * 16, pk);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] *= VG ? Gs[blk * 32 + i] : kg;  // VG: exp(G_63) of key channel blk * 32 + i
        umma::st_32x32b_x32(tl + cS + blk * 32, x);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_ST);
      if (tid == 128) JLA_MARK(it, 1);
      JLA_WMARK(it, warp - 4, 1);
      if (save) {  // this half row of h^T into the staging tile (column block `half`, row v)
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

      ok = wait(bars + B_FULLB + sb, (it / NB) & 1, abort_flag);
      if (!ok) break;
      const T* vs = reinterpret_cast<const T*>(st_v(sb));
      const int j0 = 32 * half;  // this warp's 32 tokens (columns of the [V x 64] accumulators)
      if (DELTA) {
        // ---- W^T = V^T - (cin Gamma)_j (S^T K^T)
        ok = wait(bars + B_M1, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        if (tid == 128) JLA_MARK(it, 3);
        JLA_WMARK(it, warp - 4, 2);
        {
          float x[32];
          ld_row32<T>(x, tl + cA1 + j0);
          uint32_t pk[16];
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 gm = VG ? make_float4(1.f, 1.f, 1.f, 1.f) : *reinterpret_cast<const float4*>(gam + j0 + 4 * i4);
            const int j = j0 + 4 * i4;
            const float w0 = to_f32(vs[swz_tile(64, j, v)]) - gm.x * x[4 * i4];
            const float w1 = to_f32(vs[swz_tile(64, j + 1, v)]) - gm.y * x[4 * i4 + 1];
            const float w2 = to_f32(vs[swz_tile(64, j + 2, v)]) - gm.z * x[4 * i4 + 2];
            const float w3 = to_f32(vs[swz_tile(64, j + 3, v)]) - gm.w * x[4 * i4 + 3];
            pk[2 * i4] = pack2<T>(w0, w1);
            pk[2 * i4 + 1] = pack2<T>(w2, w3);
          }
          umma::st_32x32b_x16(tl + cWb + 16 * half, pk);
          if (save) {  // residual for the key-side gradient kernel (dAg = dVn W^T): row v, tokens j0 .. j0 + 31; the
            if (it > 0) {  // shared-memory stores run while the TMEM store completes
              ok = wait(bars + B_WV_FREE, 1, abort_flag);  // the previous chunk's Vn^T has left the tile
              if (!ok) break;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) *swz_chunk(stgWV, v, 4 * half + i) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
          umma::wait_st();
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bars + B_W);
            mbar_arrive(bars + B_EMPTYB + sb);  // done with this chunk's v
          }
          if (tid == 128) JLA_MARK(it, 4);
          JLA_WMARK(it, warp - 4, 3);
          if (save) {
            umma::fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + B_WV_FULL);
          }
        }
        // ---- Vn^T = W^T Ag^T
        ok = wait(bars + B_M2, ph, abort_flag);
        if (!ok) break;
        umma::fence_after_sync();
        if (tid == 128) JLA_MARK(it, 6);
        JLA_WMARK(it, warp - 4, 4);
        {
          float x[32];
          ld_row32<T>(x, tl + cA1 + j0);
          uint32_t pk[16], pg[16];
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 gr = VG ? make_float4(1.f, 1.f, 1.f, 1.f) : *reinterpret_cast<const float4*>(gamr + j0 + 4 * i4);
            pk[2 * i4] = pack2<T>(x[4 * i4], x[4 * i4 + 1]);
            pk[2 * i4 + 1] = pack2<T>(x[4 * i4 + 2], x[4 * i4 + 3]);
            pg[2 * i4] = pack2<T>(x[4 * i4] * gr.x, x[4 * i4 + 1] * gr.y);
            pg[2 * i4 + 1] = pack2<T>(x[4 * i4 + 2] * gr.z, x[4 * i4 + 3] * gr.w);
          }
          umma::st_32x32b_x16(tl + cWb + 16 * half, pk);
          umma::st_32x32b_x16(tl + cVg + 16 * half, pg);
          umma::wait_st();
          umma::fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bars + B_VN);
            mbar_arrive(bars + B_EMPTYA + sa);  // done with this chunk's gate vectors
          }
          if (tid == 128) JLA_MARK(it, 7);
          JLA_WMARK(it, warp - 4, 5);
          if (save) {  // only after the chain has been handed on: the tile may still be on its way out with W^T
            ok = wait(bars + B_WV_FREE, 0, abort_flag);
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 4; ++i) *swz_chunk(stgWV, v, 4 * half + i) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
            umma::fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + B_WV_FULL);
          }
          if (tid == 128) JLA_MARK(it, 16);
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
          mbar_arrive(bars + B_EMPTYB + sb);
          mbar_arrive(bars + B_EMPTYA + sa);
        }
      }
    }
    // ---- final state
    if (ok && n > 0) ok = wait(bars + B_M3, (n - 1) & 1, abort_flag);
    umma::fence_after_sync();
#ifdef JLA_TRACE
    if (tid == 128 && blockIdx.x < 4096) g_fwd_cta[blockIdx.x * 4 + 2] = global_timer();
#endif
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
    // Per-token scalars of chunk `it`, written once by the first score warp as soon as the chunk's gate vectors have
    // landed (about a chunk ahead of their use): the state group then starts a chunk without arithmetic of its own.
    auto scalars = [&](int it) {
      const int sa = it % NA;
      float* gam = st_gam(sa);
      const float* Gs = st_G(sa);
      const unsigned char* runs = st_runs(sa);
      const int len = st_meta(sa)[1], flags = st_meta(sa)[2];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = lane + 32 * jj;
        const RowScalars rs = row_scalars(Gs, runs, flags, j);
        gam[j] = rs.gam;
        gam[64 + j] = (j < len) ? rs.gamr : 0.f;  // tokens past a partial chunk must not write the state
      }
      if (lane == 0) gam[128] = keep_gamma(Gs, runs, flags);
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_GAM + sa);  // (release: the stores above are visible to whoever acquires the phase)
    };
    auto build = [&](int it) {  // P = (Q K^T) D of chunk `it`: rows r0 .. r0 + 15, columns 32 half .. + 31
      const int sa = it % NA, buf = it & 1;
      if (!wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag)) return false;
      if (warp == 12) scalars(it);
      const float* Gs = st_G(sa);
      const unsigned char* runs = st_runs(sa);
      if (tid == 384) JLA_MARK(it, 20);
      JLA_WMARK(it, warp - 4, 0);
      if (!wait(bars + B_PDONE, it & 1, abort_flag)) return false;
      umma::fence_after_sync();
      if (tid == 384) JLA_MARK(it, 21);
      JLA_WMARK(it, warp - 4, 1);
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
        const int flags = st_meta(sa)[2];
        const int tg = (warp - 12) * 32 + lane, i = tg >> 2, quarter = tg & 3;
        const float cgi = row_scalars(Gs, runs, flags, i).gam;
        T* qt = reinterpret_cast<T*>(st_q(sa));
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
      if (tid == 384) JLA_MARK(it, 22);
      JLA_WMARK(it, warp - 4, 2);
      return true;
    };
    const int n_out = p.state_only ? 0 : n;
    if (p.state_only && !VG && warp == 12) {  // no scores to build: only the scalars
      for (int it = 0; it < n && ok; ++it) {
        ok = wait(bars + B_FULLA + it % NA, (it / NA) & 1, abort_flag);
        if (ok) scalars(it);
      }
    }
    if (n_out > 0 && !VG) ok = build(0);
    for (int it = 0; it < n_out && ok; ++it) {
      const int sa = it % NA;
      if (it + 1 < n_out && !VG) {  // its product is issued right after this chunk's first chain product
        ok = build(it + 1);
        if (!ok) break;
      }
      if (VG) {  // (without VG, build(it) has waited for this slot already)
        ok = wait(bars + B_FULLA + sa, (it / NA) & 1, abort_flag);
        if (!ok) break;
      }
      // ---- O^T = scale [S^T ((cin Gamma) Q)^T + Vn^T P^T], thread = value row v, 32 tokens per warp
      if (tid == 384) JLA_MARK(it, 23);
      ok = wait(bars + B_ODONE, it & 1, abort_flag);
      if (!ok) break;
      umma::fence_after_sync();
      if (tid == 384) JLA_MARK(it, 24);
      JLA_WMARK(it, warp - 4, 3);
      const int tok0 = st_meta(sa)[0], len = st_meta(sa)[1];
      // Free the accumulator, then transpose through the chunk's dead q tile ([64 tokens x V], swizzled): a full chunk
      // leaves from there as two TMA tensor stores issued by the output store thread.
      T* stg = reinterpret_cast<T*>(st_q(sa));
      {
        float a[32];
        umma::ld_32x32b_x32(a, tl + cO + 32 * half);
        umma::wait_ld();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_OFREE);
#pragma unroll
        for (int i = 0; i < 32; ++i) stg[swz_tile(64, 32 * half + i, v)] = from_f32<T>(p.scale * a[i]);
      }
      if (len < 64) {  // partial chunk: this warp writes its own 32 tokens x 32 value columns, up to the chunk's end
        __syncwarp();
        T* o = static_cast<T*>(p.o) + ((long)(tok0 + 32 * half) * p.H + h) * V + 32 * q4;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = lane + 32 * i, tok = idx >> 2, part = idx & 3;
          if (32 * half + tok < len) {
            *reinterpret_cast<uint4*>(o + (long)tok * p.H * V + part * 8) =
                *reinterpret_cast<const uint4*>(stg + swz_tile(64, 32 * half + tok, 32 * q4 + part * 8));
          }
        }
      }
      umma::fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + B_O_FULL0 + (it & 1));
      if (tid == 384) JLA_MARK(it, 25);
      JLA_WMARK(it, warp - 4, 4);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 2) umma::tmem_dealloc(tmem, 512);
#ifdef JLA_TRACE
  if (tid == 128 && blockIdx.x < 4096) g_fwd_cta[blockIdx.x * 4 + 3] = global_timer();
#endif
  if (tid == 0 && *abort_flag) atomicExch(p.status, 2);
}

template <typename T, bool DELTA, bool VG = false>
int launch_one(const FwdTcMaps& maps, const FwdTcParams& fp, int blocks, cudaStream_t s) {
  auto* kern = sg_fwd_tc_kernel<T, DELTA, VG>;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemT<VG>::kBytes));
  {
    ProfScope ps(VG ? kProfKdaFwd : kProfSgFwd, s);
    kern<<<blocks, kThreads, SmemT<VG>::kBytes, s>>>(maps, fp);
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
  bool ok = tma::encode_3d(&maps.v, p.v, p.V, p.H, tokens, 64) && tma::encode_3d(&maps.o, io.o, p.V, p.H, tokens, 64);
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
  if (ok && pl.save) {
    ok = tma::encode_3d(&maps.h_res, c.res + pl.h, p.K, 1, slots * p.V, p.V);
    if (ok && pl.delta) {
      ok = tma::encode_3d(&maps.w_res, c.res + pl.w, 64, 1, slots * p.V, p.V) &&
           tma::encode_3d(&maps.vn_res, c.res + pl.vn, 64, 1, slots * p.V, p.V);
    }
  }
  if (!ok) return JLA_ERR_CUDA;
  if (!vg) maps.k2 = maps.p = maps.v;  // unused
  if (!pl.save) maps.h_res = maps.v;
  if (!pl.save || !pl.delta) maps.w_res = maps.vn_res = maps.v;
  FwdTcParams fp{};
  fp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  fp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  fp.gates = reinterpret_cast<const float*>(c.res + (vg ? pl.kda_d : pl.gates));
  fp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  fp.h0 = p.h0;
  fp.o = io.o;
  fp.final_state = io.final_state;
  fp.save = pl.save ? 1 : 0;
  fp.H = p.H;
  fp.Hk = p.Hk;
  fp.scale = p.scale;
  fp.status = tc_status_ptr();
  fp.state_only = (p.flags & JLA_FLAG_STATE_ONLY) != 0;
  if (!fp.status) return JLA_ERR_CUDA;
  const int blocks = pl.rows * p.H;
  if (vg) {
    return p.dtype == JLA_DTYPE_BF16 ? launch_one<__nv_bfloat16, true, true>(maps, fp, blocks, s)
                                     : launch_one<__half, true, true>(maps, fp, blocks, s);
  }
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_one<__nv_bfloat16, true>(maps, fp, blocks, s) : launch_one<__nv_bfloat16, false>(maps, fp, blocks, s);
  }
  return pl.delta ? launch_one<__half, true>(maps, fp, blocks, s) : launch_one<__half, false>(maps, fp, blocks, s);
}

}  // namespace jla

#ifdef JLA_TRACE
extern "C" int jla_debug_fwd_warps(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, jla::g_fwd_warps, sizeof(unsigned long long) * 64 * 16 * 6) == cudaSuccess ? 0 : -4;
}
extern "C" int jla_debug_fwd_cta(unsigned long long* out, int n) {
  return cudaMemcpyFromSymbol(out, jla::g_fwd_cta, sizeof(unsigned long long) * 4 * n) == cudaSuccess ? 0 : -4;
}
extern "C" int jla_debug_fwd_trace(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, jla::g_fwd_trace, sizeof(unsigned long long) * 64 * 32) == cudaSuccess ? 0 : -4;
}
#endif
