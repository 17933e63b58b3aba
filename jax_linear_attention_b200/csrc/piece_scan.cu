// Scan over the pieces of a sequence that has been cut into independently processed pieces joined by affine maps
// (reference: gdr_piece_scan / gdr_piece_scan_bwd, src/jla/ops/mosaic_gpu/scalar_gate_scan.py:49-140).
//
// A piece p maps the state entering it affinely: S_out[p] = M[p] S_in[p] + E[p] with M[p] [K x K] and E[p] [K x V]
// per head, both fp32 (M is the piece's response to an identity state, E its final state from a zero state). Where a
// piece continues the document of the piece before it (cont[p] != 0), S_in[p] = S_out[p - 1]; otherwise the piece
// starts from zero and its map is never read (a document start inside a piece makes M exactly zero as well).
//
//   forward   for p = p_lo .. p_hi - 1:   S_out[p] = E[p] + M[p] S_out[p - 1]        if cont[p]   (p = 0: `boundary`)
//   backward  for p = p_hi - 1 .. p_lo:   dS_out[p] = boundary (p = P - 1) | dS_in[p + 1] (cont[p + 1]) | untouched
//                                         dS_in[p] += M[p]^T dS_out[p]                 if cont[p]
//
// All arithmetic is fp32 on the CUDA cores (the maps multiply a carried state thousands of tokens long; the kernels
// that produce them already rounded their operands to 16 bits once). One CTA per (head, 32 value columns) walks the
// pieces in order with its slice of the running state in shared memory; a map is streamed through shared memory in
// [K x 32] panels. Nothing is allocated; everything runs on the caller's stream.
#include "common.cuh"

namespace jla {
namespace {

constexpr int kVS = 32;       // value columns per CTA
constexpr int kThreads = 256;

template <int K>
__global__ void __launch_bounds__(kThreads) piece_scan_fwd_kernel(int P, int H, int V, const float* __restrict__ maps,
                                                                   const int* __restrict__ cont,
                                                                   const float* __restrict__ boundary, float* states,
                                                                   int p_lo, int p_hi) {
  const int h = blockIdx.x, v0 = blockIdx.y * kVS;
  const int tid = threadIdx.x, r = tid >> 1, c0 = (tid & 1) * 16;
  extern __shared__ float smem[];
  float* prev = smem;               // [K][kVS] the state leaving the previous piece
  float* panel = smem + K * kVS;    // [K][33] a [K x 32] panel of the map
  const bool active = r < K;  // (K = 64: the upper half of the CTA only helps with the copies)
  bool have_prev = false;
  for (int p = p_lo; p < p_hi; ++p) {
    float* out = states + (((size_t)p * H + h) * K) * V + v0;
    if (!cont[p]) {  // starts from zero: E[p] is already the answer; the next piece reads it from global memory
      have_prev = false;
      continue;
    }
    if (!have_prev) {  // bring the entering state into shared memory
      const float* src = p > 0 ? states + (((size_t)(p - 1) * H + h) * K) * V + v0
                               : (boundary ? boundary + ((size_t)h * K) * V + v0 : nullptr);
      for (int idx = tid; idx < K * kVS / 4; idx += kThreads) {
        const int row = idx / (kVS / 4), c4 = (idx % (kVS / 4)) * 4;
        reinterpret_cast<float4*>(prev)[idx] = src ? *reinterpret_cast<const float4*>(src + (size_t)row * V + c4)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    float acc[16];
    if (active) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 e = *reinterpret_cast<const float4*>(out + (size_t)r * V + c0 + 4 * i);
        acc[4 * i] = e.x, acc[4 * i + 1] = e.y, acc[4 * i + 2] = e.z, acc[4 * i + 3] = e.w;
      }
    }
    const float* M = maps + (((size_t)p * H + h) * K) * K;
    for (int j0 = 0; j0 < K; j0 += 32) {
      __syncthreads();  // prev is complete / the previous panel has been consumed
      for (int idx = tid; idx < K * 32; idx += kThreads) {
        const int row = idx >> 5, jj = idx & 31;
        panel[row * 33 + jj] = M[(size_t)row * K + j0 + jj];
      }
      __syncthreads();
      if (active) {
#pragma unroll 4
        for (int jj = 0; jj < 32; ++jj) {
          const float m = panel[r * 33 + jj];
          const float4* s = reinterpret_cast<const float4*>(prev + (j0 + jj) * kVS + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 x = s[i];
            acc[4 * i] += m * x.x, acc[4 * i + 1] += m * x.y, acc[4 * i + 2] += m * x.z, acc[4 * i + 3] += m * x.w;
          }
        }
      }
    }
    __syncthreads();  // every thread has read prev: it becomes this piece's output
    if (active) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 o = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        *reinterpret_cast<float4*>(out + (size_t)r * V + c0 + 4 * i) = o;
        *reinterpret_cast<float4*>(prev + r * kVS + c0 + 4 * i) = o;
      }
    }
    have_prev = true;
  }
}

template <int K>
__global__ void __launch_bounds__(kThreads) piece_scan_bwd_kernel(int P, int H, int V, const float* __restrict__ maps,
                                                                   const int* __restrict__ cont,
                                                                   const float* __restrict__ boundary, float* ds_in,
                                                                   float* ds_out, int p_lo, int p_hi) {
  const int h = blockIdx.x, v0 = blockIdx.y * kVS;
  const int tid = threadIdx.x, r = tid >> 1, c0 = (tid & 1) * 16;
  extern __shared__ float smem[];
  float* x = smem;                // [K][kVS] dS_out of the current piece
  float* panel = smem + K * kVS;  // [32][K] a [32 x K] panel of the map (rows kk)
  const bool active = r < K;
  for (int p = p_hi - 1; p >= p_lo; --p) {
    const float* src;
    if (p == P - 1) src = boundary ? boundary + ((size_t)h * K) * V + v0 : nullptr;
    else if (cont[p + 1]) src = ds_in + (((size_t)(p + 1) * H + h) * K) * V + v0;
    else continue;  // nothing flows back into this piece's end: dS_out[p] stays as the caller left it (zero)
    float* dso = ds_out + (((size_t)p * H + h) * K) * V + v0;
    __syncthreads();  // the previous piece's products have consumed x
    for (int idx = tid; idx < K * kVS / 4; idx += kThreads) {
      const int row = idx / (kVS / 4), c4 = (idx % (kVS / 4)) * 4;
      const float4 val = src ? *reinterpret_cast<const float4*>(src + (size_t)row * V + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(x)[idx] = val;
      *reinterpret_cast<float4*>(dso + (size_t)row * V + c4) = val;
    }
    if (!cont[p]) continue;  // the piece starts from zero: nothing reaches dS_in through the map
    float* dsi = ds_in + (((size_t)p * H + h) * K) * V + v0;
    float acc[16];
    if (active) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 e = *reinterpret_cast<const float4*>(dsi + (size_t)r * V + c0 + 4 * i);
        acc[4 * i] = e.x, acc[4 * i + 1] = e.y, acc[4 * i + 2] = e.z, acc[4 * i + 3] = e.w;
      }
    }
    const float* M = maps + (((size_t)p * H + h) * K) * K;
    for (int k0 = 0; k0 < K; k0 += 32) {  // dS_in[j][:] += sum_kk M[kk][j] x[kk][:]
      __syncthreads();
      for (int idx = tid; idx < 32 * K; idx += kThreads) {
        const int kk = idx / K, j = idx % K;
        panel[kk * K + j] = M[(size_t)(k0 + kk) * K + j];
      }
      __syncthreads();
      if (active) {
#pragma unroll 4
        for (int kk = 0; kk < 32; ++kk) {
          const float m = panel[kk * K + r];
          const float4* s = reinterpret_cast<const float4*>(x + (k0 + kk) * kVS + c0);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 xv = s[i];
            acc[4 * i] += m * xv.x, acc[4 * i + 1] += m * xv.y, acc[4 * i + 2] += m * xv.z, acc[4 * i + 3] += m * xv.w;
          }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        *reinterpret_cast<float4*>(dsi + (size_t)r * V + c0 + 4 * i) =
            make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      }
    }
    // (the next iteration's first barrier orders these global writes before any thread of this CTA reads them: a CTA
    // only ever reads the value columns it wrote itself)
  }
}

}  // namespace
}  // namespace jla

using namespace jla;

extern "C" int jla_piece_scan(int backward, int P, int H, int K, int V, const float* maps, const int32_t* cont,
                              const float* boundary, float* states, float* ds_out, int p_lo, int p_hi,
                              jla_stream_t stream) {
  if (P < 0 || H <= 0 || p_lo < 0 || p_hi > P || !cont || !states || (backward && !ds_out)) {
    set_error("piece scan: bad argument");
    return JLA_ERR_BAD_ARGUMENT;
  }
  if ((K != 64 && K != 128) || V % kVS != 0 || V <= 0) {
    set_error("piece scan: K must be 64 or 128 and V a multiple of %d; got K = %d, V = %d", kVS, K, V);
    return JLA_ERR_UNSUPPORTED;
  }
  if (p_lo >= p_hi) return JLA_OK;
  if (!maps) {
    set_error("piece scan: null maps");
    return JLA_ERR_BAD_ARGUMENT;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(H, V / kVS);
  const size_t smem = (size_t)(K * kVS + (backward ? 32 * K : K * 33)) * sizeof(float);
  if (backward) {
    auto* kern = K == 128 ? piece_scan_bwd_kernel<128> : piece_scan_bwd_kernel<64>;
    JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, s>>>(P, H, V, maps, cont, boundary, states, ds_out, p_lo, p_hi);
  } else {
    auto* kern = K == 128 ? piece_scan_fwd_kernel<128> : piece_scan_fwd_kernel<64>;
    JLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kThreads, smem, s>>>(P, H, V, maps, cont, boundary, states, p_lo, p_hi);
  }
  JLA_LAUNCH_OK();
  return JLA_OK;
}
