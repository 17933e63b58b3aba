// Prologue kernels of the chunked path: the chunk table, the per-chunk gate cumsum / document runs, and the
// gate-free triangular inverse T0 = (I + strict_lower(beta_i k_i.k_j))^-1 (K K^T on tensor cores, the inverse by
// blocked fp32 elimination).
#include "chunked.cuh"
#include "profile.cuh"
#include "mma.cuh"
#include "tri_inverse.cuh"

namespace jla {
namespace {

// One block. Dense rows: chunk id = row * per_row + i. Packed sequences: every sequence gets ceil(len / 64)
// consecutive slots; unused slots get len = 0.
__global__ void build_tables_kernel(Rows rows, int nc, ChunkMeta* meta, int2* row_chunks) {
  const int nrows = rows.count();
  const int tid = threadIdx.x, nt = blockDim.x;
  if (rows.cu == nullptr) {
    const int per = (rows.T + kChunk - 1) / kChunk;
    for (int r = tid; r <= nrows; r += nt) row_chunks[r] = make_int2(r * per, r < nrows ? per : 0);
    for (int c = tid; c < nc; c += nt) {
      const int r = c / max(per, 1), i = c - r * per;
      ChunkMeta m;
      m.tok0 = r * rows.T + i * kChunk;
      m.len = min(kChunk, rows.T - i * kChunk);
      m.row = r;
      m.flags = 0;
      meta[c] = m;
    }
    return;
  }
  // cu_seqlens is device data nobody has looked at: a table that is not monotonic, leaves [0, T] or would need more
  // slots than the buffers hold must not send any later kernel to an out-of-range token. Such a row is treated as
  // empty (its tokens are skipped); a well-formed table takes none of these branches.
  auto row_range = [&](int r, int& tok0, int& len) { rows.range(r, tok0, len); };  // clamps to [0, B * T]
  __shared__ int total;
  if (tid == 0) {
    int acc = 0;
    for (int r = 0; r < nrows; ++r) {
      int tok0, len;
      row_range(r, tok0, len);
      int cnt = (len + kChunk - 1) / kChunk;
      if (acc + cnt > nc) cnt = nc - acc;  // never more slots than the buffers were sized for
      row_chunks[r] = make_int2(acc, cnt);
      acc += cnt;
    }
    row_chunks[nrows] = make_int2(acc, 0);
    total = acc;
  }
  __syncthreads();
  for (int r = tid; r < nrows; r += nt) {
    const int2 rc = row_chunks[r];
    int tok0, len;
    row_range(r, tok0, len);
    for (int i = 0; i < rc.y; ++i) {
      ChunkMeta m;
      m.tok0 = tok0 + i * kChunk;
      m.len = min(kChunk, len - i * kChunk);
      m.row = r;
      m.flags = 0;
      meta[rc.x + i] = m;
    }
  }
  for (int c = total + tid; c < nc; c += nt) meta[c] = ChunkMeta{0, 0, 0, 0};
}

// Gate vectors of every (chunk, head): G = chunk-local cumulative sum of g, beta head-major; plus, once per chunk,
// the run ids of its tokens and flag bit 0. One warp per (chunk, head): a lane owns two tokens, the cumulative sum is
// a warp scan. Blocks of eight warps cover eight heads of one chunk; the block of the first head group also writes
// the chunk's run ids and, for dense rows (`dense_tables`), the chunk table itself, so that the one-block table kernel
// only runs for packed sequences.
__global__ void __launch_bounds__(256) prep_gates_kernel(Rows rows, int H, int nc, int dense_tables, const float* __restrict__ g,
                                                         const float* __restrict__ beta, ChunkMeta* meta, int2* row_chunks,
                                                         float* __restrict__ gates, unsigned char* __restrict__ runs) {
  const int c = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ChunkMeta m;
  if (dense_tables) {
    const int per = (rows.T + kChunk - 1) / kChunk;
    const int r = c / max(per, 1), i = c - r * per;
    m.tok0 = r * rows.T + i * kChunk;
    m.len = min(kChunk, rows.T - i * kChunk);
    m.row = r;
    m.flags = 0;
    if (blockIdx.y == 0 && threadIdx.x == 0 && c == 0) {
      for (int rr = 0; rr <= rows.B; ++rr) row_chunks[rr] = make_int2(rr * per, rr < rows.B ? per : 0);
    }
  } else {
    m = meta[c];
  }
  if (blockIdx.y == 0 && warp == 7) {  // run ids and the "starts a document" flag, once per chunk (also for len == 0)
    int row_tok0 = 0, row_len = 0;
    if (m.len > 0) rows.range(m.row, row_tok0, row_len);
    const int t0 = 2 * lane, t1 = 2 * lane + 1;
    const int s0 = (m.len > 0 && t0 > 0 && t0 < m.len && rows.resets(m.tok0 + t0, row_tok0)) ? 1 : 0;
    const int s1 = (m.len > 0 && t1 < m.len && rows.resets(m.tok0 + t1, row_tok0)) ? 1 : 0;
    int incl = s0 + s1;  // inclusive scan of the number of document starts up to this lane's second token
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += x;
    }
    runs[(long)c * 64 + t0] = (unsigned char)(incl - s1);
    runs[(long)c * 64 + t1] = (unsigned char)incl;
    if (lane == 0) {
      m.flags = (m.len > 0 && rows.resets(m.tok0, row_tok0)) ? 1 : 0;
      if (dense_tables || m.flags) meta[c] = m;
    }
  }
  const int h = blockIdx.y * 8 + warp;
  if (h >= H || m.len == 0) return;
  const int t0 = 2 * lane, t1 = 2 * lane + 1;
  const float g0 = (g && t0 < m.len) ? g[(long)(m.tok0 + t0) * H + h] : 0.f;
  const float g1 = (g && t1 < m.len) ? g[(long)(m.tok0 + t1) * H + h] : 0.f;
  const float b0 = (beta && t0 < m.len) ? beta[(long)(m.tok0 + t0) * H + h] : 0.f;
  const float b1 = (beta && t1 < m.len) ? beta[(long)(m.tok0 + t1) * H + h] : 0.f;
  float incl = g0 + g1;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float x = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += x;
  }
  float* out = gates + ((long)c * H + h) * 128;
  *reinterpret_cast<float2*>(out + t0) = make_float2(incl - g1, incl);
  *reinterpret_cast<float2*>(out + 64 + t0) = make_float2(b0, b1);
}

struct KktParams {
  const ChunkMeta* meta;
  const void* k;
  const float* gates;
  const unsigned char* runs;
  void* t0;
  void* ag;
  int H, Hk;
};

// T0 for one (chunk, head). 4 warps: K K^T with mma.sync (each warp 16 rows x 64 columns), then the inverse of
// the unit lower-triangular 64 x 64 matrix in fp32: the four 16 x 16 diagonal blocks by forward substitution
// (one column per thread), then X21 = -X22 L21 X11 at block sizes 16 and 32. The block products are bound by
// shared-memory loads, so every thread computes a strip of four adjacent columns (one 16-byte load per operand row)
// and, at block size 32, of two rows. The fp32 inverse X takes over the key tile once K K^T is in registers.
template <typename T, int K>
__global__ void __launch_bounds__(128) kkt_inv_kernel(KktParams p) {
  constexpr int LDK = K + 8, LDA = kTriLda, LDM = kTriLdm;
  constexpr int kFirst = 64 * LDK * (int)sizeof(T) > 64 * LDA * 4 ? 64 * LDK * (int)sizeof(T) : 64 * LDA * 4;
  const int c = blockIdx.x / p.H, h = blockIdx.x - c * p.H;
  const ChunkMeta m = p.meta[c];
  if (m.len == 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* ks = reinterpret_cast<T*>(smem_raw);
  float* X = reinterpret_cast<float*>(smem_raw);  // [64][LDA], after the key tile is consumed
  float* A = reinterpret_cast<float*>(smem_raw + kFirst);
  float* M = A + 64 * LDA;        // [32][LDM]
  float* betas = M + 32 * LDM;    // [64]
  float* Gs = betas + 64;         // [64]
  int* run = reinterpret_cast<int*>(Gs + 64);

  load_tile_async<T, 64, K>(ks, LDK, static_cast<const T*>(p.k) + ((long)m.tok0 * p.Hk + hk) * K, (long)p.Hk * K,
                            m.len, tid, 128);
  cp_async_commit();
  if (tid < 64) {
    betas[tid] = p.gates[((long)c * p.H + h) * 128 + 64 + tid];
    Gs[tid] = p.gates[((long)c * p.H + h) * 128 + tid];
    run[tid] = p.runs[(long)c * 64 + tid];
  }
  cp_async_wait<0>();
  __syncthreads();

  {
    float acc[8][4];
    zero_acc(acc);
    warp_gemm<T, 8, K / 16, A_ROW, B_NK>(acc, ks + warp * 16 * LDK, LDK, ks, LDK, lane);
    __syncthreads();  // every warp has read the key tile: X may take its place
    for (int idx = tid; idx < 64 * LDA / 4; idx += 128) reinterpret_cast<float4*>(X)[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int i = warp * 16 + g + 8 * hh, j = nt * 8 + 2 * t;
        const float bi = betas[i];
        const int ri = run[i];
        float2 v;
        v.x = (j < i && ri == run[j]) ? bi * acc[nt][2 * hh] : 0.f;
        v.y = (j + 1 < i && ri == run[j + 1]) ? bi * acc[nt][2 * hh + 1] : 0.f;
        *reinterpret_cast<float2*>(A + i * LDA + j) = v;
      }
    }
  }
  __syncthreads();

  invert_unit_lower_64(A, X, M, tid);

  T* out = static_cast<T*>(p.t0) + ((long)c * p.H + h) * 64 * 64;
  for (int idx = tid; idx < 64 * 8; idx += 128) {
    const int r = idx >> 3, c8 = (idx & 7) * 8;
    uint4 v;
    v.x = pack2<T>(X[r * LDA + c8 + 0], X[r * LDA + c8 + 1]);
    v.y = pack2<T>(X[r * LDA + c8 + 2], X[r * LDA + c8 + 3]);
    v.z = pack2<T>(X[r * LDA + c8 + 4], X[r * LDA + c8 + 5]);
    v.w = pack2<T>(X[r * LDA + c8 + 6], X[r * LDA + c8 + 7]);
    *reinterpret_cast<uint4*>(out + r * 64 + c8) = v;
  }
  // the gated form Ag_ij = T0_ij exp(G_i - G_j) beta_j (same run, j <= i) that the forward multiplies with
  T* outg = static_cast<T*>(p.ag) + ((long)c * p.H + h) * 64 * 64;
  for (int idx = tid; idx < 64 * 8; idx += 128) {
    const int r = idx >> 3, c8 = (idx & 7) * 8;
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int j = c8 + e;
      a[e] = (j <= r && run[j] == run[r]) ? X[r * LDA + j] * __expf(Gs[r] - Gs[j]) * betas[j] : 0.f;
    }
    uint4 v;
    v.x = pack2<T>(a[0], a[1]);
    v.y = pack2<T>(a[2], a[3]);
    v.z = pack2<T>(a[4], a[5]);
    v.w = pack2<T>(a[6], a[7]);
    *reinterpret_cast<uint4*>(outg + r * 64 + c8) = v;
  }
}

template <typename T, int K>
int launch_kkt(const KktParams& kp, int blocks, cudaStream_t s) {
  const size_t first = 64 * (K + 8) * sizeof(T) > 64 * 68 * sizeof(float) ? 64 * (K + 8) * sizeof(T) : 64 * 68 * sizeof(float);
  const size_t smem = first + (64 * 68 + 32 * 36 + 128) * sizeof(float) + 64 * sizeof(int);
  auto* kern = kkt_inv_kernel<T, K>;
  if (smem > 48 * 1024) JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  {
    ProfScope ps(kProfKktInv, s);
    kern<<<blocks, 128, smem, s>>>(kp);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

// Q K^T and K Q^T of one (chunk, key head) in fp32, stored in the accumulator-fragment order of warp_gemm: for the row
// block rb = warp (16 rows), fragment register i (0 .. 31 = n-tile * 4 + e) of lane l sits at ((rb * 8 + i / 4) * 32 + l)
// * 4 + i % 4, so that a warp of the state-pass kernels reads its whole 16 x 64 block with eight coalesced 16-byte
// loads per lane. The products are the same instruction sequence the kernels would otherwise run per value head.
template <typename T, int K>
__global__ void __launch_bounds__(128) qk_table_kernel(const ChunkMeta* meta, const void* q, const void* k, float* tab, int Hk) {
  constexpr int LDK = K + 8;
  const int c = blockIdx.x / Hk, hk = blockIdx.x - c * Hk;
  const ChunkMeta m = meta[c];
  if (m.len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* qS = reinterpret_cast<T*>(smem_raw);
  T* kS = qS + 64 * LDK;
  load_tile_async<T, 64, K>(qS, LDK, static_cast<const T*>(q) + ((long)m.tok0 * Hk + hk) * K, (long)Hk * K, m.len, tid, 128);
  load_tile_async<T, 64, K>(kS, LDK, static_cast<const T*>(k) + ((long)m.tok0 * Hk + hk) * K, (long)Hk * K, m.len, tid, 128);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  float* out = tab + (long)blockIdx.x * kQkTabFloats;
#pragma unroll
  for (int variant = 0; variant < 2; ++variant) {
    float acc[8][4];
    zero_acc(acc);
    warp_gemm<T, 8, K / 16, A_ROW, B_NK>(acc, (variant ? kS : qS) + 16 * warp * LDK, LDK, variant ? qS : kS, LDK, lane);
    float4* dst = reinterpret_cast<float4*>(out + variant * 4096) + warp * 8 * 32 + lane;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) dst[nt * 32] = make_float4(acc[nt][0], acc[nt][1], acc[nt][2], acc[nt][3]);
  }
}

template <typename T>
int launch_qk_table(const ChunkedCtx& c, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  const ChunkMeta* meta = reinterpret_cast<const ChunkMeta*>(c.res + pl.meta);
  float* tab = reinterpret_cast<float*>(c.res + pl.qk_tab);
  const int blocks = pl.nc * p.Hk;
  if (p.K == 128) {
    const int smem = 2 * 64 * (128 + 8) * sizeof(T);
    JLA_CUDA_OK(cudaFuncSetAttribute(qk_table_kernel<T, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    qk_table_kernel<T, 128><<<blocks, 128, smem, s>>>(meta, c.q_eff, c.k_eff, tab, p.Hk);
  } else {
    const int smem = 2 * 64 * (64 + 8) * sizeof(T);
    qk_table_kernel<T, 64><<<blocks, 128, smem, s>>>(meta, c.q_eff, c.k_eff, tab, p.Hk);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}

}  // namespace

int launch_prep(const ChunkedCtx& c, cudaStream_t s) {
  const jla_problem& p = c.p;
  const Plan& pl = c.plan;
  if (pl.nc == 0 || pl.rows == 0) return JLA_OK;
  const Rows rows = make_rows(p);
  ChunkMeta* meta = reinterpret_cast<ChunkMeta*>(c.res + pl.meta);
  int2* row_chunks = reinterpret_cast<int2*>(c.res + pl.row_chunks);
  float* gates = reinterpret_cast<float*>(c.res + pl.gates);
  unsigned char* runs = reinterpret_cast<unsigned char*>(c.res + pl.runs);
  const bool dense = p.cu_seqlens == nullptr;
  if (!dense) {
    ProfScope ps(kProfTables, s);
    build_tables_kernel<<<1, 256, 0, s>>>(rows, pl.nc, meta, row_chunks);
  }
  JLA_LAUNCH_OK();
  {
    ProfScope ps(kProfGates, s);
    // KDA gates are per channel: its own prologue folds them into the operands; here G stays zero
    prep_gates_kernel<<<dim3(pl.nc, (p.H + 7) / 8), 256, 0, s>>>(rows, p.H, pl.nc, dense ? 1 : 0,
                                                                 p.kind == JLA_KIND_KDA ? nullptr : p.g, p.beta, meta, row_chunks,
                                                                 gates, runs);
  }
  JLA_LAUNCH_OK();
  if (pl.l2norm) {
    const long nrows = (long)p.B * p.T * p.Hk;
    int rc = l2norm_fwd(p.q, c.res + pl.qn, p.dtype, nrows, p.K, s);
    if (rc != JLA_OK) return rc;
    rc = l2norm_fwd(p.k, c.res + pl.kn, p.dtype, nrows, p.K, s);
    if (rc != JLA_OK) return rc;
  }
  if (shares_scores(p)) {  // grouped simple GLA on the mma.sync kernels: the in-chunk scores once per key head
    const int rc = p.dtype == JLA_DTYPE_BF16 ? launch_qk_table<__nv_bfloat16>(c, s) : launch_qk_table<__half>(c, s);
    if (rc != JLA_OK) return rc;
  }
  if (!pl.delta) return JLA_OK;
  if (p.kind == JLA_KIND_KDA) return launch_kda_prep(c, s);
  if (use_tc_kernels(p)) return launch_kkt_tc(c, s);  // K = V = 128: the inverse on the Blackwell tensor cores
  KktParams kp{meta, c.k_eff, gates, runs, c.res + pl.t0, c.res + pl.ag, p.H, p.Hk};
  const int blocks = pl.nc * p.H;
  if (p.dtype == JLA_DTYPE_BF16) {
    return p.K == 64 ? launch_kkt<__nv_bfloat16, 64>(kp, blocks, s) : launch_kkt<__nv_bfloat16, 128>(kp, blocks, s);
  }
  return p.K == 64 ? launch_kkt<__half, 64>(kp, blocks, s) : launch_kkt<__half, 128>(kp, blocks, s);
}

}  // namespace jla
