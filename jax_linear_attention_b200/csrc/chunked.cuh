// Shared definitions of the chunk-64 tensor-core kernels (JLA_PATH_CHUNKED): the chunk table, the layout of
// the residual and scratch buffers, and the per-token decay / document scalars every kernel derives.
//
// Chunk math (per head and chunk, S = state entering the chunk), gate-free formulation as in the reference's
// kernels (src/jla/ops/mosaic_gpu/gated_delta_rule_kernels.py:351-370, scalar_gate_fused.py:427-504):
//   A0 = strict_lower(beta_i k_i.k_j) * same      T0 = (I + A0)^-1        Ag = T0 * D * beta_j
//   D_ij = exp(G_i - G_j) * same (i >= j)         W = V - (cin Gamma) * (K S)        Vn = Ag W
//   O = scale [(cin Gamma) * (Q S) + ((Q K^T) * D) Vn]      S+ = keep gamma S + ((tail Gamma_r) * K)^T Vn
// Chunks never straddle rows: every row (batch element or cu_seqlens sequence) is cut into its own chunks, the
// last one possibly partial (missing tokens behave as zero padding: k = 0, g = 0, beta = 0).
#pragma once

#include "common.cuh"

namespace jla {

struct ChunkMeta {
  int tok0;   // first token (flat index over B*T)
  int len;    // valid tokens, 1..64; 0 = unused slot
  int row;
  int flags;  // bit 0: the chunk's first token starts a new document (the entering state is not seen)
};

// Byte offsets inside the residual buffer (forward -> backward) and the backward scratch.
struct Plan {
  int rows, nc;       // rows; chunk slots (upper bound on the number of chunks)
  bool delta, l2norm, save;
  size_t meta, row_chunks, gates, runs, t0, ag, qn, kn, h, vn, w, residual_bytes;  // residual buffer
  size_t kda_q, kda_kr, kda_kw, kda_p, kda_d;  // KDA: gate-folded operands per chunk slot (see chunked_kda_prep.cu)
  size_t qk_tab;  // grouped simple GLA on the mma.sync kernels: Q K^T and K Q^T per (chunk, key head), see qk_table_kernel
  size_t kda_dag, kda_dqs, kda_dks, kda_dku, kda_dd;  // KDA backward scratch (see chunked_kda_bwd.cu)
  size_t fwd_scratch_bytes;                                                 // same layout without h, vn
  size_t dh, dvn, dq_acc, dk_acc, dp, dga, bwd_scratch_bytes;               // backward scratch
};

// The tcgen05 kernels cover K = V = 128 and keep the residuals h, Vn and W transposed ([V][K], [V][64]); other head
// sizes, or JLA_B200_LEGACY=1 (A/B comparison), use the mma.sync kernels with row-major residuals.
bool use_tc_kernels(const jla_problem& p);  // chunked_api.cu
// JLA_B200_KDA_SCAN_BWD=1: the KDA backward runs the fp32 token scan instead of the chunked kernels (A/B comparison).
bool kda_scan_backward();  // chunked_api.cu

inline int elem_size(int dtype) { return dtype == JLA_DTYPE_F32 ? 4 : 2; }

// Per-channel gates (KDA): a chunk's in-chunk scores run on the tensor cores, factored through the mid point of each
// channel's decay, while no channel decays by more than exp(-bound) over the chunk; the factors then reach
// exp(+-bound / 2) times an element of q or k and must stay inside the 16-bit type's range (bf16 shares fp32's
// exponent; f16 ends at 65504, so its factors stop at exp(6) = 403). Chunks beyond the bound take the exact fp32 loop.
template <typename T>
__host__ __device__ constexpr float kda_bounded_log() { return 60.f; }
template <>
__host__ __device__ constexpr float kda_bounded_log<__half>() { return 12.f; }

// Without the delta rule the in-chunk scores Q K^T do not depend on the value head: when several value heads share a
// key head (Mamba-2: all of them) the mma.sync kernels take the two 64 x 64 products Q K^T and K Q^T from a table
// that a small kernel fills once per (chunk, key head), in the accumulator-fragment order of the warps that use
// them (fp32, so the decayed scores round exactly as when every head computes the product itself).
constexpr int kQkTabFloats = 2 * 64 * 64;  // per (chunk, key head): Q K^T then K Q^T
inline bool shares_scores(const jla_problem& p) {
  return p.kind == JLA_KIND_SIMPLE_GLA && !use_tc_kernels(p) && p.Hk > 0 && p.H / p.Hk >= 2;
}

inline Plan make_plan(const jla_problem& p) {
  Plan pl{};
  const bool varlen = p.num_seqs > 0;
  pl.rows = varlen ? p.num_seqs : p.B;
  const int per_row = (p.T + kChunk - 1) / kChunk;
  pl.nc = varlen ? per_row + p.num_seqs : p.B * per_row;
  pl.delta = p.kind != JLA_KIND_SIMPLE_GLA;
  pl.l2norm = (p.flags & JLA_FLAG_QK_L2NORM) != 0;
  const bool kda = p.kind == JLA_KIND_KDA;
  // with the token-scan backward (kda_scan_backward()) the KDA forward keeps no residuals
  pl.save = (p.flags & JLA_FLAG_SAVE_RESIDUALS) != 0 && !(kda && kda_scan_backward());
  const size_t es = elem_size(p.dtype);
  const size_t tokens = (size_t)p.B * p.T;
  Carver c(nullptr);
  auto off = [&](size_t bytes) {
    c.off = align_up(c.off);
    const size_t o = c.off;
    c.off += bytes;
    return o;
  };
  pl.meta = off((size_t)pl.nc * sizeof(ChunkMeta));
  pl.row_chunks = off((size_t)(pl.rows + 1) * 2 * sizeof(int));
  pl.gates = off((size_t)pl.nc * p.H * 128 * sizeof(float));  // per (chunk, head): G[64] then beta[64]
  pl.runs = off((size_t)pl.nc * 64);
  pl.t0 = off(pl.delta ? (size_t)pl.nc * p.H * 64 * 64 * es : 0);
  pl.ag = off(pl.delta ? (size_t)pl.nc * p.H * 64 * 64 * es : 0);  // Ag = T0 * D * beta_j (gated), for the forward
  pl.qn = off(pl.l2norm ? tokens * p.Hk * p.K * es : 0);
  pl.kn = off(pl.l2norm ? tokens * p.Hk * p.K * es : 0);
  const size_t slot_tile = kda ? (size_t)pl.nc * p.H * 64 * p.K * es : 0;
  pl.kda_q = off(slot_tile);
  pl.kda_kr = off(slot_tile);
  pl.kda_kw = off(slot_tile);
  pl.kda_p = off(kda ? (size_t)pl.nc * p.H * 64 * 64 * es : 0);
  pl.kda_d = off(kda ? (size_t)pl.nc * p.H * p.K * sizeof(float) : 0);
  pl.qk_tab = off(shares_scores(p) ? (size_t)pl.nc * p.Hk * kQkTabFloats * sizeof(float) : 0);
  pl.fwd_scratch_bytes = align_up(c.off);
  pl.h = off((size_t)pl.nc * p.H * p.K * p.V * es);
  pl.vn = off(pl.delta ? (size_t)pl.nc * p.H * 64 * p.V * es : 0);
  const bool tc = use_tc_kernels(p);
  pl.w = off(pl.delta && tc ? (size_t)pl.nc * p.H * 64 * p.V * es : 0);  // W^T, for the key-side gradient kernel
  pl.residual_bytes = align_up(c.off);
  Carver b(nullptr);
  auto boff = [&](size_t bytes) {
    b.off = align_up(b.off);
    const size_t o = b.off;
    b.off += bytes;
    return o;
  };
  const bool direct = p.H == p.Hk && !pl.l2norm;  // dq, dk written straight in the tensor dtype
  pl.dh = boff((size_t)pl.nc * p.H * p.K * p.V * es);
  pl.dvn = boff(pl.delta ? (size_t)pl.nc * p.H * 64 * p.V * es : 0);
  pl.dq_acc = boff(direct ? 0 : tokens * p.H * p.K * sizeof(float));
  pl.dk_acc = boff(direct ? 0 : tokens * p.H * p.K * sizeof(float));
  pl.dp = boff(tc ? (size_t)pl.nc * p.H * 64 * 64 * es : 0);       // dP tiles, query-side -> key-side gradient kernel
  pl.dga = boff(tc ? (size_t)pl.nc * p.H * 64 * sizeof(float) : 0);  // dG partial sums, likewise
  const size_t slot_f32 = kda ? (size_t)pl.nc * p.H * 64 * p.K * sizeof(float) : 0;
  pl.kda_dag = boff(kda ? (size_t)pl.nc * p.H * 64 * 64 * es : 0);  // dAg tiles
  pl.kda_dqs = boff(slot_f32);                                      // gradients of the folded state-side operands
  pl.kda_dks = boff(slot_f32);
  pl.kda_dku = boff(slot_f32);
  pl.kda_dd = boff(kda ? (size_t)pl.nc * p.H * p.K * sizeof(float) : 0);  // gradient of the state decay vector
  pl.bwd_scratch_bytes = align_up(b.off);
  return pl;
}

// Per-token scalars of one chunk, derived from the staged G[64] (chunk-local cumulative log decay) and run ids.
struct RowScalars {
  float G, gam, gamr;  // exp(G) if the token sees the entering state else 0; exp(G_last - G) if it reaches S+ else 0
  int run;
};

__device__ __forceinline__ RowScalars row_scalars(const float* Gs, const unsigned char* runs, int flags, int i) {
  RowScalars r;
  r.G = Gs[i];
  r.run = runs[i];
  const bool cin = r.run == 0 && !(flags & 1);
  const bool tail = r.run == runs[63];
  r.gam = cin ? __expf(r.G) : 0.f;
  r.gamr = tail ? __expf(Gs[63] - r.G) : 0.f;
  return r;
}

__device__ __forceinline__ float keep_gamma(const float* Gs, const unsigned char* runs, int flags) {
  return (runs[63] == 0 && !(flags & 1)) ? __expf(Gs[63]) : 0.f;
}

// D_ij for i >= j in the same run, else 0.
__device__ __forceinline__ float decay_ij(const float* Gs, const unsigned char* runs, int i, int j, float Gi, int runi) {
  return (j <= i && runs[j] == runi) ? __expf(Gi - Gs[j]) : 0.f;
}

// ---- launchers (chunked_*.cu) -----------------------------------------------------------------------------
struct ChunkedCtx {
  jla_problem p;
  Plan plan;
  char* res;            // residual-layout buffer (residuals when saving, else the forward scratch)
  const void* q_eff;    // q, k after the optional L2 norm
  const void* k_eff;
};

int launch_prep(const ChunkedCtx& c, cudaStream_t s);                           // tables, G/beta/runs, T0, l2norm
int launch_kkt_tc(const ChunkedCtx& c, cudaStream_t s);                         // T0, Ag for K = 128 (tcgen05)
int launch_kda_prep(const ChunkedCtx& c, cudaStream_t s);                       // KDA: gate-folded operands, P, Ag
int launch_kda_grads(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s);  // after the reverse pass
int launch_sg_fwd(const ChunkedCtx& c, const jla_fwd_io& io, cudaStream_t s);
int launch_sg_bwd(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s);
int l2norm_fwd(const void* x, void* y, int dtype, long rows, int K, cudaStream_t stream);
int launch_sg_fwd_tc(const ChunkedCtx& c, const jla_fwd_io& io, cudaStream_t s);
int launch_sg_bwd_state_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, cudaStream_t s);
int launch_chunk_grads_tc(const ChunkedCtx& c, const jla_bwd_io& io, char* scratch, bool direct, cudaStream_t s);
int* tc_status_ptr();  // status.cu: the current device's status word (set non-zero when a bounded wait gave up)

}  // namespace jla
