// Inverse of a unit lower-triangular 64 x 64 matrix I + A in fp32 by blocked elimination, shared by the
// triangular-solve prologues of the scalar-gate and the per-channel-gate (KDA) kernels. Threads 0..127 work; a CTA
// with more threads passes all of them through (the others only take part in the barriers).
//   A [64][LDA] : the strictly lower part (everything else zero)
//   X [64][LDA] : zero-filled by the caller; receives the inverse (unit diagonal included)
//   M [32][LDM] : scratch
// The four 16 x 16 diagonal blocks are inverted by forward substitution (one column per thread), then
// X21 = -X22 L21 X11 at block sizes 16 and 32. The block products are bound by shared-memory loads, so every thread
// computes a strip of four adjacent columns (one 16-byte load per operand row) and, at block size 32, of two rows.
// The caller synchronises the CTA before the call (A and the zeroed X complete); the function ends with a barrier.
#pragma once

#include "common.cuh"

namespace jla {

constexpr int kTriLda = 68, kTriLdm = 36;

namespace tri {

// diagonal 16 x 16 blocks: column `col` of the inverse of block `b` (threads 0..63)
__device__ __forceinline__ void diag_blocks(const float* A, float* X, int tid) {
  constexpr int LDA = kTriLda;
  const int b = tid >> 4, col = tid & 15;
  float x[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float s = (i == col) ? 1.f : 0.f;
#pragma unroll
    for (int mm = 0; mm < i; ++mm) s -= A[(16 * b + i) * LDA + 16 * b + mm] * x[mm];
    x[i] = s;
    X[(16 * b + i) * LDA + 16 * b + col] = s;
  }
}

// level 1: two problems (blocks 0-1 and 2-3), 16 x 16 each; thread = one row, four columns. M = L21 X11.
__device__ __forceinline__ void level1_a(const float* A, const float* X, float* M, int tid) {
  constexpr int LDA = kTriLda, LDM = kTriLdm;
  const int pr = tid >> 6, i = (tid >> 2) & 15, j4 = (tid & 3) * 4;
  const int r0 = 32 * pr + 16, c0 = 32 * pr;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int mm = 0; mm < 16; ++mm) {
    const float a = A[(r0 + i) * LDA + c0 + mm];
    const float4 x = *reinterpret_cast<const float4*>(X + (c0 + mm) * LDA + c0 + j4);
    s[0] += a * x.x;
    s[1] += a * x.y;
    s[2] += a * x.z;
    s[3] += a * x.w;
  }
  *reinterpret_cast<float4*>(M + (pr * 16 + i) * LDM + j4) = make_float4(s[0], s[1], s[2], s[3]);
}

// X21 = -X22 M
__device__ __forceinline__ void level1_b(float* X, const float* M, int tid) {
  constexpr int LDA = kTriLda, LDM = kTriLdm;
  const int pr = tid >> 6, i = (tid >> 2) & 15, j4 = (tid & 3) * 4;
  const int r0 = 32 * pr + 16, c0 = 32 * pr;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int mm = 0; mm < 16; ++mm) {
    const float a = X[(r0 + i) * LDA + r0 + mm];
    const float4 x = *reinterpret_cast<const float4*>(M + (pr * 16 + mm) * LDM + j4);
    s[0] += a * x.x;
    s[1] += a * x.y;
    s[2] += a * x.z;
    s[3] += a * x.w;
  }
  *reinterpret_cast<float4*>(X + (r0 + i) * LDA + c0 + j4) = make_float4(-s[0], -s[1], -s[2], -s[3]);
}

// level 2: rows 32-63, columns 0-31; thread = rows i and i + 16, four columns. M = L21 X11.
__device__ __forceinline__ void level2_a(const float* A, const float* X, float* M, int tid) {
  constexpr int LDA = kTriLda, LDM = kTriLdm;
  const int i = tid >> 3, j4 = (tid & 7) * 4;
  float s[2][4] = {};
#pragma unroll 8
  for (int mm = 0; mm < 32; ++mm) {
    const float a0 = A[(32 + i) * LDA + mm], a1 = A[(48 + i) * LDA + mm];
    const float4 x = *reinterpret_cast<const float4*>(X + mm * LDA + j4);
    s[0][0] += a0 * x.x;
    s[0][1] += a0 * x.y;
    s[0][2] += a0 * x.z;
    s[0][3] += a0 * x.w;
    s[1][0] += a1 * x.x;
    s[1][1] += a1 * x.y;
    s[1][2] += a1 * x.z;
    s[1][3] += a1 * x.w;
  }
  *reinterpret_cast<float4*>(M + i * LDM + j4) = make_float4(s[0][0], s[0][1], s[0][2], s[0][3]);
  *reinterpret_cast<float4*>(M + (16 + i) * LDM + j4) = make_float4(s[1][0], s[1][1], s[1][2], s[1][3]);
}

// X21 = -X22 M
__device__ __forceinline__ void level2_b(float* X, const float* M, int tid) {
  constexpr int LDA = kTriLda, LDM = kTriLdm;
  const int i = tid >> 3, j4 = (tid & 7) * 4;
  float s[2][4] = {};
#pragma unroll 8
  for (int mm = 0; mm < 32; ++mm) {
    const float a0 = X[(32 + i) * LDA + 32 + mm], a1 = X[(48 + i) * LDA + 32 + mm];
    const float4 x = *reinterpret_cast<const float4*>(M + mm * LDM + j4);
    s[0][0] += a0 * x.x;
    s[0][1] += a0 * x.y;
    s[0][2] += a0 * x.z;
    s[0][3] += a0 * x.w;
    s[1][0] += a1 * x.x;
    s[1][1] += a1 * x.y;
    s[1][2] += a1 * x.z;
    s[1][3] += a1 * x.w;
  }
  *reinterpret_cast<float4*>(X + (32 + i) * LDA + j4) = make_float4(-s[0][0], -s[0][1], -s[0][2], -s[0][3]);
  *reinterpret_cast<float4*>(X + (48 + i) * LDA + j4) = make_float4(-s[1][0], -s[1][1], -s[1][2], -s[1][3]);
}

}  // namespace tri

__device__ __forceinline__ void invert_unit_lower_64(const float* A, float* X, float* M, int tid) {
  const bool active = tid < 128;
  if (tid < 64) tri::diag_blocks(A, X, tid);
  __syncthreads();
  if (active) tri::level1_a(A, X, M, tid);
  __syncthreads();
  if (active) tri::level1_b(X, M, tid);
  __syncthreads();
  if (active) tri::level2_a(A, X, M, tid);  // (the level-1 contents of M were consumed before the barrier above)
  __syncthreads();
  if (active) tri::level2_b(X, M, tid);
  __syncthreads();
}

}  // namespace jla
