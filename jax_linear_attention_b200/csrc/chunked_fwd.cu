// Forward of the scalar-gate family (simple GLA / DeltaNet / Gated DeltaNet), chunk-64, one CTA per
// (row, head) walking the row's chunks with the fp32 state in registers.
//
// Per chunk (see chunked.cuh for the math): W = V - (cin Gamma)(K S); Vn = Ag W; P = (Q K^T) D;
// O = scale[(cin Gamma)(Q S) + P Vn]; S+ = keep gamma S + K^T (tail Gamma_r Vn). All products are
// mma.sync m16n8k16 with 16-bit operands staged in shared memory and fp32 accumulation; the state is rounded
// to the operand dtype only as an MMA operand (the carried copy stays fp32), like the reference's kernels
// (src/jla/ops/mosaic_gpu/scalar_gate_fused.py:436-458). q/k/v/T0 tiles of the next chunk are prefetched with
// cp.async while the current chunk computes.
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"

namespace jla {
namespace {

struct FwdParams {
  const ChunkMeta* meta;
  const int2* row_chunks;
  const float* gates;
  const unsigned char* runs;
  const void *q, *k, *v, *t0;
  const float* h0;
  const float* qk_tab;  // Q K^T per (chunk, key head) in fragment order (qk_table_kernel), or nullptr
  void* o;
  float* final_state;
  void *h_out, *vn_out;  // residuals (nullptr when not saving)
  int H, Hk;
  float scale;
};

template <typename T, int K, int V, bool DELTA>
struct FwdSmem {
  static constexpr int LDK = K + 8, LDV = V + 8, LDC = 72;
  static constexpr int kStageElems = 2 * 64 * LDK + 64 * LDV + (DELTA ? 64 * LDC : 0);
  static constexpr int kStageBytes = kStageElems * 2 + 512 + 64;  // + gates (128 f32) + runs (64 u8)
  // Without the delta rule only the 16-bit state copy lives outside the stages: the output is staged in the chunk's
  // dead q tile and the Gamma_r factor of the state update is applied to the key fragments in registers. Where the
  // output is wider than the q tile (K = 64, V = 128) it gets a tile of its own behind the state copy.
  static constexpr bool kOwnOutTile = !DELTA && V > K;
  static constexpr int kBytes =
      2 * kStageBytes + (K * LDV + (DELTA ? 3 * 64 * LDV + 64 * LDC : 0) + (kOwnOutTile ? 64 * LDV : 0)) * 2;
};

// (Without the delta rule and with V = 64 -- the Mamba-2 shape, 4 x 128 chains at B = 8, H = 64 -- two CTAs share an SM:
// 108 KB of shared memory and at most 128 registers each. The pass is bound by the latency of its dependent products
// and barriers, so the second chain runs in the first one's gaps.)
template <typename T, int K, int V, bool DELTA>
__global__ void __launch_bounds__(256, (!DELTA && V == 64) ? 2 : 1) sg_fwd_kernel(FwdParams p) {
  using L = FwdSmem<T, K, V, DELTA>;
  constexpr int LDK = L::LDK, LDV = L::LDV, LDC = L::LDC;
  constexpr int WR = K / 16, WC = 8 / WR;   // warps over state rows / columns
  constexpr int SNT = V / 8 / WC;           // state n-tiles per warp
  constexpr int ONT = V / 16;               // n-tiles per warp of a [64 x V] product (16 rows x V/2 columns)
  const int row = blockIdx.x / p.H, h = blockIdx.x - row * p.H;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int r0 = 16 * (warp & 3), c0 = (V / 2) * (warp >> 2);
  const int sr0 = 16 * (warp % WR), sc0 = (V / WC) * (warp / WR);
  const int2 rc = p.row_chunks[row];

  extern __shared__ __align__(16) unsigned char smem_raw[];
  auto stage_q = [&](int s) { return reinterpret_cast<T*>(smem_raw + s * L::kStageBytes); };
  auto stage_k = [&](int s) { return stage_q(s) + 64 * LDK; };
  auto stage_v = [&](int s) { return stage_k(s) + 64 * LDK; };
  auto stage_t0 = [&](int s) { return stage_v(s) + 64 * LDV; };
  auto stage_g = [&](int s) { return reinterpret_cast<float*>(smem_raw + s * L::kStageBytes + L::kStageElems * 2); };
  auto stage_runs = [&](int s) { return reinterpret_cast<unsigned char*>(stage_g(s) + 128); };
  T* Sb = reinterpret_cast<T*>(smem_raw + 2 * L::kStageBytes);
  T* Wb = Sb + K * LDV;
  T* Vnb = Wb + 64 * LDV;
  T* VnS = Vnb + 64 * LDV;
  T* Agb = VnS + 64 * LDV;

  auto issue_load = [&](int ci, int s) {
    const int c = rc.x + ci;
    const ChunkMeta m = p.meta[c];
    const T* q = static_cast<const T*>(p.q) + ((long)m.tok0 * p.Hk + hk) * K;
    const T* k = static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * K;
    const T* v = static_cast<const T*>(p.v) + ((long)m.tok0 * p.H + h) * V;
    load_tile_async<T, 64, K>(stage_q(s), LDK, q, (long)p.Hk * K, m.len, tid, 256);
    load_tile_async<T, 64, K>(stage_k(s), LDK, k, (long)p.Hk * K, m.len, tid, 256);
    load_tile_async<T, 64, V>(stage_v(s), LDV, v, (long)p.H * V, m.len, tid, 256);
    if (DELTA) {
      load_tile_async<T, 64, 64>(stage_t0(s), LDC, static_cast<const T*>(p.t0) + ((long)c * p.H + h) * 4096, 64, 64,
                                 tid, 256);
    }
    if (tid < 32) cp_async16(stage_g(s) + tid * 4, p.gates + ((long)c * p.H + h) * 128 + tid * 4);
    if (tid >= 32 && tid < 36) cp_async16(stage_runs(s) + (tid - 32) * 16, p.runs + (long)c * 64 + (tid - 32) * 16);
    cp_async_commit();
  };

  // state: rows sr0 + g (+8), columns sc0 + 8 nt + 2t (+1)
  float accS[SNT][4];
  {
    const float* h0 = p.h0 ? p.h0 + ((long)row * p.H + h) * K * V : nullptr;
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float2 x = make_float2(0.f, 0.f);
        if (h0) x = *reinterpret_cast<const float2*>(h0 + (long)(sr0 + g + 8 * hh) * V + sc0 + nt * 8 + 2 * t);
        accS[nt][2 * hh] = x.x;
        accS[nt][2 * hh + 1] = x.y;
      }
    }
    store_acc<T, SNT>(Sb, LDV, sr0, sc0, accS, lane);
  }
  if (rc.y > 0) issue_load(0, 0);

  for (int ci = 0; ci < rc.y; ++ci) {
    const int s = ci & 1;
    const int c = rc.x + ci;
    cp_async_wait<0>();
    __syncthreads();  // S0: stage s landed, Sb holds the entering state, previous chunk fully consumed
    if (ci + 1 < rc.y) issue_load(ci + 1, s ^ 1);
    const ChunkMeta m = p.meta[c];
    const T* qS = stage_q(s);
    const T* kS = stage_k(s);
    const T* vS = stage_v(s);
    const float* Gs = stage_g(s);
    const float* betas = Gs + 64;
    const unsigned char* runs = stage_runs(s);
    const RowScalars rs0 = row_scalars(Gs, runs, m.flags, r0 + g);
    const RowScalars rs1 = row_scalars(Gs, runs, m.flags, r0 + g + 8);

    if (p.h_out) {
      store_tile<T, V>(static_cast<T*>(p.h_out) + ((long)c * p.H + h) * K * V, V, Sb, LDV, K, tid, 256);
    }
    if (DELTA) {
      // Ag = T0 * D * beta_j (row tid / 4, 16 columns per thread)
      const T* t0S = stage_t0(s);
      const int i = tid >> 2, j0 = (tid & 3) * 16;
      const float Gi = Gs[i];
      const int runi = runs[i];
#pragma unroll
      for (int jj = 0; jj < 16; jj += 2) {
        const int j = j0 + jj;
        const float2 tv = unpack2<T>(*reinterpret_cast<const uint32_t*>(t0S + i * LDC + j));
        const float a0 = tv.x * decay_ij(Gs, runs, i, j, Gi, runi) * betas[j];
        const float a1 = tv.y * decay_ij(Gs, runs, i, j + 1, Gi, runi) * betas[j + 1];
        *reinterpret_cast<uint32_t*>(Agb + i * LDC + j) = pack2<T>(a0, a1);
      }
      // W = V - (cin Gamma) (K S)
      float acc[ONT][4];
      zero_acc(acc);
      warp_gemm<T, ONT, K / 16, A_ROW, B_KN>(acc, kS + r0 * LDK, LDK, Sb + c0, LDV, lane);
#pragma unroll
      for (int nt = 0; nt < ONT; ++nt) {
        const int col = c0 + nt * 8 + 2 * t;
        const float2 v0 = unpack2<T>(*reinterpret_cast<const uint32_t*>(vS + (r0 + g) * LDV + col));
        const float2 v1 = unpack2<T>(*reinterpret_cast<const uint32_t*>(vS + (r0 + g + 8) * LDV + col));
        acc[nt][0] = v0.x - rs0.gam * acc[nt][0];
        acc[nt][1] = v0.y - rs0.gam * acc[nt][1];
        acc[nt][2] = v1.x - rs1.gam * acc[nt][2];
        acc[nt][3] = v1.y - rs1.gam * acc[nt][3];
      }
      store_acc<T, ONT>(Wb, LDV, r0, c0, acc, lane);
      __syncthreads();  // S2: Wb, Agb complete
      zero_acc(acc);
      warp_gemm<T, ONT, 4, A_ROW, B_KN>(acc, Agb + r0 * LDC, LDC, Wb + c0, LDV, lane);
      store_acc<T, ONT>(Vnb, LDV, r0, c0, acc, lane);
      store_acc<T, ONT>(VnS, LDV, r0, c0, acc, lane, rs0.gamr, rs1.gamr);
    } else if (tid < 64) {
      // Vn = V. The state update needs tail Gamma_r per token: kept in the (unused) beta half of the gate vectors
      // and applied to the key fragments (ordered before its readers by S3 / S4)
      stage_g(s)[64 + tid] = row_scalars(Gs, runs, m.flags, tid).gamr;
    }

    // P = (Q K^T) D for this warp's 16 rows and all 64 columns, kept as A fragments
    uint32_t pfrag[4][4];
    {
      float accP[8][4];
      if (p.qk_tab) {  // the product is shared by the value heads of the key head: this warp's fragments from the table
        const float4* src = reinterpret_cast<const float4*>(p.qk_tab + ((long)c * p.Hk + hk) * kQkTabFloats) +
                            (warp & 3) * 8 * 32 + lane;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const float4 x = __ldg(src + nt * 32);
          accP[nt][0] = x.x, accP[nt][1] = x.y, accP[nt][2] = x.z, accP[nt][3] = x.w;
        }
      } else {
        zero_acc(accP);
        warp_gemm<T, 8, K / 16, A_ROW, B_NK>(accP, qS + r0 * LDK, LDK, kS, LDK, lane);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int j = nt * 8 + 2 * t;
        accP[nt][0] *= decay_ij(Gs, runs, r0 + g, j, rs0.G, rs0.run);
        accP[nt][1] *= decay_ij(Gs, runs, r0 + g, j + 1, rs0.G, rs0.run);
        accP[nt][2] *= decay_ij(Gs, runs, r0 + g + 8, j, rs1.G, rs1.run);
        accP[nt][3] *= decay_ij(Gs, runs, r0 + g + 8, j + 1, rs1.G, rs1.run);
      }
      acc_to_afrag<T, 4>(pfrag, accP);
    }
    float accO[ONT][4];
    zero_acc(accO);
    warp_gemm<T, ONT, K / 16, A_ROW, B_KN>(accO, qS + r0 * LDK, LDK, Sb + c0, LDV, lane);
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt) {
      accO[nt][0] *= rs0.gam;
      accO[nt][1] *= rs0.gam;
      accO[nt][2] *= rs1.gam;
      accO[nt][3] *= rs1.gam;
    }
    __syncthreads();  // S3: Vnb / VnS complete
    const T* vn = DELTA ? Vnb : vS;
    warp_gemm_ra<T, ONT, 4, B_KN>(accO, pfrag, vn + c0, LDV, lane);
    // O staged in Wb; without the delta rule in the q tile, which every warp finished reading before S3
    T* oS = (DELTA || L::kOwnOutTile) ? Wb : stage_q(s);  // (Wb: the first tile behind the state copy)
    constexpr int LDO = (DELTA || L::kOwnOutTile) ? LDV : LDK;
    store_acc<T, ONT>(oS, LDO, r0, c0, accO, lane, p.scale, p.scale);
    __syncthreads();  // S4: every warp is done with Sb and the staging tile holds O
    store_tile<T, V>(static_cast<T*>(p.o) + ((long)m.tok0 * p.H + h) * V, (long)p.H * V, oS, LDO, m.len, tid, 256);
    if (DELTA && p.vn_out) {
      store_tile<T, V>(static_cast<T*>(p.vn_out) + ((long)c * p.H + h) * 64 * V, V, Vnb, LDV, 64, tid, 256);
    }
    // S+ = keep gamma S + K^T (tail Gamma_r Vn)
    const float kg = keep_gamma(Gs, runs, m.flags);
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
      accS[nt][0] *= kg;
      accS[nt][1] *= kg;
      accS[nt][2] *= kg;
      accS[nt][3] *= kg;
    }
    if (DELTA) {
      warp_gemm<T, SNT, 4, A_COL, B_KN>(accS, kS + sr0, LDK, VnS + sc0, LDV, lane);
    } else {
      warp_gemm_scaled_a<T, SNT, 4, B_KN>(accS, kS + sr0, LDK, betas, vS + sc0, LDV, lane);
    }
    store_acc<T, SNT>(Sb, LDV, sr0, sc0, accS, lane);
  }

  if (p.final_state) {
    float* f = p.final_state + ((long)row * p.H + h) * K * V;
#pragma unroll
    for (int nt = 0; nt < SNT; ++nt) {
      *reinterpret_cast<float2*>(f + (long)(sr0 + g) * V + sc0 + nt * 8 + 2 * t) = make_float2(accS[nt][0], accS[nt][1]);
      *reinterpret_cast<float2*>(f + (long)(sr0 + g + 8) * V + sc0 + nt * 8 + 2 * t) =
          make_float2(accS[nt][2], accS[nt][3]);
    }
  }
}

template <typename T, int K, int V, bool DELTA>
int launch_one(const FwdParams& fp, int blocks, cudaStream_t s) {
  auto* kern = sg_fwd_kernel<T, K, V, DELTA>;
  constexpr int smem = FwdSmem<T, K, V, DELTA>::kBytes;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  {
    ProfScope ps(kProfSgFwd, s);
    kern<<<blocks, 256, smem, s>>>(fp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <typename T, bool DELTA>
int launch_kv(const FwdParams& fp, int K, int V, int blocks, cudaStream_t s) {
  if (K == 128 && V == 128) return launch_one<T, 128, 128, DELTA>(fp, blocks, s);
  if (K == 128 && V == 64) return launch_one<T, 128, 64, DELTA>(fp, blocks, s);
  if (K == 64 && V == 128) return launch_one<T, 64, 128, DELTA>(fp, blocks, s);
  return launch_one<T, 64, 64, DELTA>(fp, blocks, s);
}

}  // namespace

int launch_sg_fwd(const ChunkedCtx& c, const jla_fwd_io& io, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.rows == 0) return JLA_OK;
  FwdParams fp{};
  fp.meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  fp.row_chunks = reinterpret_cast<const int2*>(c.res + pl.row_chunks);
  fp.gates = reinterpret_cast<const float*>(c.res + pl.gates);
  fp.runs = reinterpret_cast<const unsigned char*>(c.res + pl.runs);
  fp.q = c.q_eff;
  fp.k = c.k_eff;
  fp.v = p.v;
  fp.t0 = c.res + pl.t0;
  fp.h0 = p.h0;
  fp.qk_tab = shares_scores(p) ? reinterpret_cast<const float*>(c.res + pl.qk_tab) : nullptr;
  fp.o = io.o;
  fp.final_state = io.final_state;
  fp.h_out = pl.save ? c.res + pl.h : nullptr;
  fp.vn_out = pl.save && pl.delta ? c.res + pl.vn : nullptr;
  fp.H = p.H;
  fp.Hk = p.Hk;
  fp.scale = p.scale;
  const int blocks = pl.rows * p.H;
  if (p.dtype == JLA_DTYPE_BF16) {
    return pl.delta ? launch_kv<__nv_bfloat16, true>(fp, p.K, p.V, blocks, s)
                    : launch_kv<__nv_bfloat16, false>(fp, p.K, p.V, blocks, s);
  }
  return pl.delta ? launch_kv<__half, true>(fp, p.K, p.V, blocks, s) : launch_kv<__half, false>(fp, p.K, p.V, blocks, s);
}

}  // namespace jla
