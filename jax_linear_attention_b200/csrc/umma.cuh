// Blackwell (sm_100a) tensor-core primitives: tcgen05.mma with shared-memory operand descriptors, TMEM
// allocation and loads, mbarrier completion with bounded waits, and the 128-byte-swizzled tile layout the
// operands live in.
//
// Operand tiles are 16-bit, [ROWS x 64] "column blocks": 128 bytes per row, rows grouped by 8 into 1024-byte
// swizzle atoms (Swizzle<3,4,3>: the 16-byte chunk index of a row is XORed with row % 8). A wider tile is
// several column blocks one after the other. Every tile base is 1024-byte aligned.
//
// The same bytes serve two operand views of tcgen05.mma.kind::f16:
//   K-major  : contraction along the 64 contiguous elements, M/N along the rows
//              (descriptor: SBO = 1024 between 8-row groups; one k-step of 16 elements = +32 bytes)
//   MN-major : M/N along the 64 contiguous elements, contraction along the rows
//              (descriptor: SBO = 1024 between 8-row K groups, LBO = bytes between column blocks;
//               one k-step of 16 rows = +2048 bytes)
//
// Accumulators: an M = 64 product puts row r in TMEM lane (r % 16) + 32 * (r / 16), so warp w of a 4-warp
// group owns rows 16w .. 16w+15, and tcgen05.ld.16x256b hands them out in the m16n8 accumulator fragment
// layout (thread g = lane / 4, t = lane % 4 holds rows g and g + 8, columns 8 nt + 2t, +1). An M = 128
// product puts row r in lane r (tcgen05.ld.32x32b: thread = row).
#pragma once

#include "common.cuh"

namespace jla {
namespace umma {

constexpr uint32_t kSpinLimit = 1u << 22;  // bounded waits: a lost arrival returns an error instead of hanging

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// element offset of (row, col) inside a [ROWS x 64] swizzled column block
__device__ __forceinline__ int swz(int row, int col) {
  return row * 64 + ((((col >> 3) ^ (row & 7)) << 3) | (col & 7));
}
// element offset inside a tile of several column blocks of `rows` rows each
__device__ __forceinline__ int swz_tile(int rows, int row, int col) { return (col >> 6) * rows * 64 + swz(row, col & 63); }

// ---- descriptors -----------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, A and B both bf16 (fmt 1) or both f16 (fmt 0).
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int fmt, int a_mn_major, int b_mn_major) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <typename T> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr int value = 1; };
template <> struct Fmt<__half> { static constexpr int value = 0; };

// ---- TMEM ------------------------------------------------------------------------------------------------
// One full warp allocates `cols` (power of two >= 32) columns and publishes the base address in *slot (smem).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// generic-proxy writes to shared memory become visible to the tensor core / TMA (async proxy)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- mbarrier --------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// Returns false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// ---- MMA -------------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// Same with the A operand in TMEM: rows = lanes, 16-bit elements packed two per 32-bit column (element k of a row in
// column k / 2, even k in the low half), as tcgen05.st writes them. One k-step of 16 = 8 columns.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// Arrive on `bar` once all MMAs issued so far by this thread have completed (implies fence::before_thread_sync).
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar))
               : "memory");
}

// A product over KSTEPS k-steps of 16 with both operands in swizzled shared memory.
//   a_tile / b_tile : 1024-byte aligned tile bases (byte addresses in the shared window)
//   *_MN            : operand view (see the file header); *_rows: rows of one column block of that tile
// K-major operands may span several column blocks along the contraction (4 k-steps per block).
// The two base descriptors are built once; every further k-step only adds a compile-time constant to the
// address field (the single issuing thread is on the critical path, so its instruction count matters).
template <int M, int N, int KSTEPS, bool A_MN, bool B_MN, int FMT>
__device__ __forceinline__ void gemm(uint32_t d_tmem, uint32_t a_tile, int a_rows, uint32_t b_tile, int b_rows,
                                     bool accumulate) {
  constexpr uint32_t idesc = instr_desc(M, N, FMT, A_MN, B_MN);
  const uint64_t a0 = smem_desc(a_tile, A_MN ? a_rows * 128 : 16, 1024);
  const uint64_t b0 = smem_desc(b_tile, B_MN ? b_rows * 128 : 16, 1024);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint32_t a_off = A_MN ? ks * 2048 : (ks >> 2) * a_rows * 128 + (ks & 3) * 32;
    const uint32_t b_off = B_MN ? ks * 2048 : (ks >> 2) * b_rows * 128 + (ks & 3) * 32;
    mma(d_tmem, a0 + (a_off >> 4), b0 + (b_off >> 4), idesc, accumulate || ks > 0);
  }
}

// D[tmem] (+)= A[tmem, M x 16*KSTEPS packed 16-bit] * B[smem]. A is always "K-major" (its rows are the lanes).
template <int M, int N, int KSTEPS, bool B_MN, int FMT>
__device__ __forceinline__ void gemm_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_tile, int b_rows, bool accumulate) {
  constexpr uint32_t idesc = instr_desc(M, N, FMT, 0, B_MN);
  const uint64_t b0 = smem_desc(b_tile, B_MN ? b_rows * 128 : 16, 1024);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const uint32_t b_off = B_MN ? ks * 2048 : (ks >> 2) * b_rows * 128 + (ks & 3) * 32;
    mma_ts(d_tmem, a_tmem + ks * 8, b0 + (b_off >> 4), idesc, accumulate || ks > 0);
  }
}

// ---- TMEM loads / stores -----------------------------------------------------------------------------------
// 16 lanes x (8 * NT) columns -> acc[NT][4] in the m16n8 fragment layout. taddr = lane base (32 * warp) | column.
template <int NT>
__device__ __forceinline__ void ld_16x256b(float (&acc)[NT][4], uint32_t taddr) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    uint32_t r0, r1, r2, r3;
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(taddr + nt * 8));
    acc[nt][0] = __uint_as_float(r0);
    acc[nt][1] = __uint_as_float(r1);
    acc[nt][2] = __uint_as_float(r2);
    acc[nt][3] = __uint_as_float(r3);
  }
}
// 32 lanes x 32 columns: thread = lane (row), v[c] = column c.
__device__ __forceinline__ void ld_32x32b_x32(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, "
      "[%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void st_32x32b_x32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::
          "r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
      "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
      "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
      "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
      "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// 32 lanes x 16 columns (thread = lane): used for packed 16-bit operand rows (32 elements).
__device__ __forceinline__ void st_32x32b_x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

}  // namespace umma
}  // namespace jla
