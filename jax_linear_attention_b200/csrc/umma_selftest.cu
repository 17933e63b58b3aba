// Self-test of the tcgen05 primitive layer (umma.cuh): one CTA computes C = A * B for the operand views the
// kernels use (K-major and MN-major, M = 64 and 128) so that descriptor, swizzle and TMEM-load conventions are
// checked against a plain matmul by tests/test_gpu_umma.py.
#include "umma.cuh"

namespace jla {
namespace {

template <int M, int N, int KD, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ a,
                                                            const __nv_bfloat16* __restrict__ b, float* __restrict__ c,
                                                            int* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __nv_bfloat16* sa = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sb = sa + M * KD;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int A_ROWS = A_MN ? KD : M, B_ROWS = B_MN ? KD : N;

  // a: K-major view expects A[M][KD]; MN-major view expects A^T[KD][M]. Likewise b: B^T[N][KD] or B[KD][N].
  for (int idx = tid; idx < M * KD; idx += 128) {
    const int r = A_MN ? idx / M : idx / KD, col = A_MN ? idx % M : idx % KD;
    sa[umma::swz_tile(A_ROWS, r, col)] = a[idx];
  }
  for (int idx = tid; idx < N * KD; idx += 128) {
    const int r = B_MN ? idx / N : idx / KD, col = B_MN ? idx % N : idx % KD;
    sb[umma::swz_tile(B_ROWS, r, col)] = b[idx];
  }
  if (tid == 0) {
    umma::mbar_init(&bar, 1);
    umma::mbar_init_fence();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, N < 32 ? 32 : N);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    umma::gemm<M, N, KD / 16, A_MN, B_MN, 1>(tmem, umma::smem_addr(sa), A_ROWS, umma::smem_addr(sb), B_ROWS, false);
    umma::commit(&bar);
  }
  const bool ok = umma::mbar_wait(&bar, 0);
  umma::fence_after_sync();
  if (!ok) {
    if (tid == 0) atomicExch(status, 1);
  } else if (M == 64) {
    float acc[N / 8][4];
    umma::ld_16x256b<N / 8>(acc, tmem + ((uint32_t)(32 * warp) << 16));
    umma::wait_ld();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < N / 8; ++nt) {
      c[(16 * warp + g) * N + nt * 8 + 2 * t] = acc[nt][0];
      c[(16 * warp + g) * N + nt * 8 + 2 * t + 1] = acc[nt][1];
      c[(16 * warp + g + 8) * N + nt * 8 + 2 * t] = acc[nt][2];
      c[(16 * warp + g + 8) * N + nt * 8 + 2 * t + 1] = acc[nt][3];
    }
  } else {
#pragma unroll
    for (int cb = 0; cb < N / 32; ++cb) {
      float v[32];
      umma::ld_32x32b_x32(v, tmem + ((uint32_t)(32 * warp) << 16) + cb * 32);
      umma::wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) c[(32 * warp + lane) * N + cb * 32 + i] = v[i];
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, N < 32 ? 32 : N);
}

// A from TMEM: thread = row of A[128][KD]; the row is rounded to bf16 pairs and stored with tcgen05.st.
template <int N, int KD, bool B_MN>
__global__ void __launch_bounds__(128) umma_selftest_ts_kernel(const __nv_bfloat16* __restrict__ a,
                                                               const __nv_bfloat16* __restrict__ b,
                                                               float* __restrict__ c, int* status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __nv_bfloat16* sb = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int B_ROWS = B_MN ? KD : N;
  for (int idx = tid; idx < N * KD; idx += 128) {
    const int r = B_MN ? idx / N : idx / KD, col = B_MN ? idx % N : idx % KD;
    sb[umma::swz_tile(B_ROWS, r, col)] = b[idx];
  }
  if (tid == 0) {
    umma::mbar_init(&bar, 1);
    umma::mbar_init_fence();
  }
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 256);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tl = tmem + ((uint32_t)(32 * warp) << 16);
  constexpr uint32_t cA = 128;  // A operand columns [128, 128 + KD / 2)
#pragma unroll
  for (int blk = 0; blk < KD / 32; ++blk) {
    uint32_t v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_bfloat162 pr = __halves2bfloat162(a[tid * KD + blk * 32 + 2 * i], a[tid * KD + blk * 32 + 2 * i + 1]);
      v[i] = *reinterpret_cast<const uint32_t*>(&pr);
    }
    umma::st_32x32b_x16(tl + cA + blk * 16, v);
  }
  umma::wait_st();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (tid == 0) {
    umma::gemm_ts<128, N, KD / 16, B_MN, 1>(tmem, tmem + cA, umma::smem_addr(sb), B_ROWS, false);
    umma::commit(&bar);
  }
  const bool ok = umma::mbar_wait(&bar, 0);
  umma::fence_after_sync();
  if (!ok) {
    if (tid == 0) atomicExch(status, 1);
  } else {
#pragma unroll
    for (int cb = 0; cb < N / 32; ++cb) {
      float v[32];
      umma::ld_32x32b_x32(v, tl + cb * 32);
      umma::wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) c[tid * N + cb * 32 + i] = v[i];
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 256);
}

template <int N, int KD, bool B_MN>
int run_ts(const void* a, const void* b, float* c, int* status, cudaStream_t s) {
  auto* kern = umma_selftest_ts_kernel<N, KD, B_MN>;
  const int smem = N * KD * 2 + 1024;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<1, 128, smem, s>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), c, status);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <int M, int N, int KD, bool A_MN, bool B_MN>
int run(const void* a, const void* b, float* c, int* status, cudaStream_t s) {
  auto* kern = umma_selftest_kernel<M, N, KD, A_MN, B_MN>;
  const int smem = (M + N) * KD * 2 + 1024;
  JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<1, 128, smem, s>>>(static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), c, status);
  JLA_LAUNCH_OK();
  return JLA_OK;
}

template <int M, int N, int KD>
int run_modes(int a_mn, int b_mn, const void* a, const void* b, float* c, int* status, cudaStream_t s) {
  if (!a_mn && !b_mn) return run<M, N, KD, false, false>(a, b, c, status, s);
  if (!a_mn && b_mn) return run<M, N, KD, false, true>(a, b, c, status, s);
  if (a_mn && !b_mn) return run<M, N, KD, true, false>(a, b, c, status, s);
  return run<M, N, KD, true, true>(a, b, c, status, s);
}

}  // namespace
}  // namespace jla

extern "C" int jla_selftest_umma(int m, int n, int kd, int a_mn_major, int b_mn_major, const void* a, const void* b,
                                 float* c, int* status, jla_stream_t stream) {
  using namespace jla;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a_mn_major == 2) {  // A operand from TMEM (a = A[128][kd])
    if (m == 128 && n == 64 && kd == 128) return b_mn_major ? run_ts<64, 128, true>(a, b, c, status, s) : run_ts<64, 128, false>(a, b, c, status, s);
    if (m == 128 && n == 128 && kd == 64) return b_mn_major ? run_ts<128, 64, true>(a, b, c, status, s) : run_ts<128, 64, false>(a, b, c, status, s);
    if (m == 128 && n == 64 && kd == 64) return b_mn_major ? run_ts<64, 64, true>(a, b, c, status, s) : run_ts<64, 64, false>(a, b, c, status, s);
    set_error("TMEM-A selftest shape (%d, %d, %d) is not instantiated", m, n, kd);
    return JLA_ERR_UNSUPPORTED;
  }
  if (m == 64 && n == 128 && kd == 128) return run_modes<64, 128, 128>(a_mn_major, b_mn_major, a, b, c, status, s);
  if (m == 64 && n == 64 && kd == 64) return run_modes<64, 64, 64>(a_mn_major, b_mn_major, a, b, c, status, s);
  if (m == 64 && n == 64 && kd == 128) return run_modes<64, 64, 128>(a_mn_major, b_mn_major, a, b, c, status, s);
  if (m == 128 && n == 128 && kd == 64) return run_modes<128, 128, 64>(a_mn_major, b_mn_major, a, b, c, status, s);
  set_error("selftest shape (%d, %d, %d) is not instantiated", m, n, kd);
  return JLA_ERR_UNSUPPORTED;
}
