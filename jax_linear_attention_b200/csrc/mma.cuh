// Warp-level tensor-core building blocks (mma.sync m16n8k16, ldmatrix, cp.async) for the chunk-64 kernels.
//
// Shared-memory operands are 16-bit tiles with a row stride `ld` (elements) that is a multiple of 8 and
// chosen so that ldmatrix row addresses fall on distinct banks (ld = cols + 8).
//
// Fragment layouts (PTX ISA, mma.m16n8k16): with g = lane / 4, t = lane % 4
//   A (16x16): a[0] = (g, 2t..2t+1)   a[1] = (g+8, 2t..)   a[2] = (g, 2t+8..)   a[3] = (g+8, 2t+8..)
//   B (16x8) : b[0] = (k = 2t..2t+1, n = g)   b[1] = (k = 2t+8.., n = g)
//   C (16x8) : c[0..1] = (g, 2t..2t+1)   c[2..3] = (g+8, 2t..2t+1)
#pragma once

#include "common.cuh"

namespace jla {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t x);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t x) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&x));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t x) {
  return __half22float2(*reinterpret_cast<__half2*>(&x));
}

// Operand storage modes.
//   A_ROW : A[m][k] stored row-major, k contiguous           (pointer at row m0, k = 0)
//   A_COL : A[m][k] stored as X[k][m], m contiguous          (pointer at X[0][m0])
//   B_NK  : B[k][n] stored as Y[n][k], k contiguous          (pointer at Y[n0][0])
//   B_KN  : B[k][n] stored as Z[k][n], n contiguous          (pointer at Z[0][n0])
enum { A_ROW = 0, A_COL = 1 };
enum { B_NK = 0, B_KN = 1 };

template <typename T, int AMODE>
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const T* base, int ld, int k0, int lane) {
  if (AMODE == A_ROW) {
    ldsm_x4(a, base + (lane & 15) * ld + k0 + ((lane >> 4) << 3));
  } else {
    // matrices: (m 0-7, k 0-7), (m 8-15, k 0-7), (m 0-7, k 8-15), (m 8-15, k 8-15), each read transposed
    ldsm_x4_t(a, base + (k0 + (lane & 7) + ((lane >> 4) << 3)) * ld + (((lane >> 3) & 1) << 3));
  }
}

// Loads the B fragments of two adjacent n-tiles (n0 .. n0+15) for one k-step: b[0..1] tile 0, b[2..3] tile 1.
template <typename T, int BMODE>
__device__ __forceinline__ void load_b2(uint32_t (&b)[4], const T* base, int ld, int n0, int k0, int lane) {
  if (BMODE == B_NK) {
    ldsm_x4(b, base + (n0 + (lane & 7) + ((lane >> 4) << 3)) * ld + k0 + (((lane >> 3) & 1) << 3));
  } else {
    ldsm_x4_t(b, base + (k0 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ld + n0 + ((lane >> 4) << 3));
  }
}

// acc[NT][4] (16 rows x 8*NT cols, NT even) += A(16 x 16*KSTEPS) * B(16*KSTEPS x 8*NT), operands in smem.
template <typename T, int NT, int KSTEPS, int AMODE, int BMODE>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT][4], const T* a_base, int lda, const T* b_base, int ldb,
                                          int lane) {
  static_assert(NT % 2 == 0, "n-tiles come in pairs");
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t a[4];
    load_a<T, AMODE>(a, a_base, lda, ks * 16, lane);
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      load_b2<T, BMODE>(b, b_base, ldb, np * 16, ks * 16, lane);
      mma16816<T>(acc[2 * np], a, b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// acc += (A diag(w))(16 x 16*KSTEPS) * B with A stored A_COL (X[k][m]) and one fp32 weight per k index: the weights
// are applied to the 16-bit A fragments in registers (one rounding, as if X's rows had been scaled in memory).
template <typename T, int NT, int KSTEPS, int BMODE>
__device__ __forceinline__ void warp_gemm_scaled_a(float (&acc)[NT][4], const T* a_base, int lda, const float* w,
                                                   const T* b_base, int ldb, int lane) {
  static_assert(NT % 2 == 0, "n-tiles come in pairs");
  const int t2 = (lane & 3) * 2;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t a[4];
    load_a<T, A_COL>(a, a_base, lda, ks * 16, lane);
    // a[0], a[1]: k = 16 ks + 2t, +1 (rows g, g + 8); a[2], a[3]: k = 16 ks + 8 + 2t, +1
    const float2 w0 = *reinterpret_cast<const float2*>(w + ks * 16 + t2);
    const float2 w1 = *reinterpret_cast<const float2*>(w + ks * 16 + 8 + t2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack2<T>(a[i]);
      const float2 ww = i < 2 ? w0 : w1;
      a[i] = pack2<T>(x.x * ww.x, x.y * ww.y);
    }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      load_b2<T, BMODE>(b, b_base, ldb, np * 16, ks * 16, lane);
      mma16816<T>(acc[2 * np], a, b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// Same with the A fragments already in registers: afrag[ks] is the 16x16 A block of k-step ks.
template <typename T, int NT, int KSTEPS, int BMODE>
__device__ __forceinline__ void warp_gemm_ra(float (&acc)[NT][4], const uint32_t (&afrag)[KSTEPS][4], const T* b_base,
                                             int ldb, int lane) {
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      load_b2<T, BMODE>(b, b_base, ldb, np * 16, ks * 16, lane);
      mma16816<T>(acc[2 * np], afrag[ks], b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], afrag[ks], b[2], b[3]);
    }
  }
}

// A 16 x 16*KSTEPS accumulator block (NT = 2*KSTEPS n-tiles) re-used as the A operand of the next product.
template <typename T, int KSTEPS>
__device__ __forceinline__ void acc_to_afrag(uint32_t (&afrag)[KSTEPS][4], const float (&acc)[2 * KSTEPS][4]) {
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    afrag[ks][0] = pack2<T>(acc[2 * ks][0], acc[2 * ks][1]);
    afrag[ks][1] = pack2<T>(acc[2 * ks][2], acc[2 * ks][3]);
    afrag[ks][2] = pack2<T>(acc[2 * ks + 1][0], acc[2 * ks + 1][1]);
    afrag[ks][3] = pack2<T>(acc[2 * ks + 1][2], acc[2 * ks + 1][3]);
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
}

// Store a 16 x 8*NT accumulator block as 16-bit values: row r0 + g (+8), columns c0 + 8*nt + 2t.
template <typename T, int NT>
__device__ __forceinline__ void store_acc(T* dst, int ld, int r0, int c0, const float (&acc)[NT][4], int lane,
                                          float s_lo = 1.f, float s_hi = 1.f) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<uint32_t*>(dst + (r0 + g) * ld + c0 + nt * 8 + 2 * t) =
        pack2<T>(acc[nt][0] * s_lo, acc[nt][1] * s_lo);
    *reinterpret_cast<uint32_t*>(dst + (r0 + g + 8) * ld + c0 + nt * 8 + 2 * t) =
        pack2<T>(acc[nt][2] * s_hi, acc[nt][3] * s_hi);
  }
}

// ---- cp.async -----------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Copy a [rows_valid x COLS] 16-bit tile (global row stride `gstride` elements) into smem rows of stride `ld`;
// rows rows_valid..ROWS-1 are zero-filled. All `nthreads` threads of the CTA call it.
template <typename T, int ROWS, int COLS>
__device__ __forceinline__ void load_tile_async(T* dst, int ld, const T* src, long gstride, int rows_valid, int tid,
                                                int nthreads) {
  constexpr int VPR = COLS / 8;  // 16-byte vectors per row
  for (int idx = tid; idx < ROWS * VPR; idx += nthreads) {
    const int r = idx / VPR, c = (idx - r * VPR) * 8;
    if (r < rows_valid) {
      cp_async16(dst + r * ld + c, src + r * gstride + c);
    } else {
      *reinterpret_cast<uint4*>(dst + r * ld + c) = make_uint4(0, 0, 0, 0);
    }
  }
}

// Copy a [rows_valid x COLS] 16-bit tile from smem to global with 16-byte stores.
template <typename T, int COLS>
__device__ __forceinline__ void store_tile(T* dst, long gstride, const T* src, int ld, int rows_valid, int tid,
                                           int nthreads) {
  constexpr int VPR = COLS / 8;
  for (int idx = tid; idx < rows_valid * VPR; idx += nthreads) {
    const int r = idx / VPR, c = (idx - r * VPR) * 8;
    *reinterpret_cast<uint4*>(dst + r * gstride + c) = *reinterpret_cast<const uint4*>(src + r * ld + c);
  }
}

}  // namespace jla
