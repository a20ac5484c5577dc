// The matrix product of the true 32-bit path: out[M, N] = x[M, K] . w[N, K]^T
// with 32-bit inputs, FMA on the CUDA cores and no tensor-core instruction, so
// nothing is rounded to a shorter type on the way (the reference's oracle is its
// CPU backend, a 32-bit dot product per output: src/backend/cpu.rs:107-136).
//
// Each output element is one running sum over k = 0 .. K-1 in ascending order,
// held by one thread; it depends neither on M nor on where the element lies in
// its tile.  A row's result is therefore the same bits whether it is computed
// alone, inside a prompt or inside a batch.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define TM 64
#define TN 64
#define TK 16

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ w, int ldw,
                float* __restrict__ out, int ldo, int M, int N, int K) {
  __shared__ float xs[TK][TM + 4];
  __shared__ float ws[TK][TN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int ty = tid / 16, tx = tid % 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += TK) {
    // 64 rows x 16 k of each operand: 1024 values, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int r = idx / TK, c = idx % TK;
      const int k = k0 + c;
      xs[c][r] = (m0 + r < M && k < K) ? x[(size_t)(m0 + r) * ldx + k] : 0.f;
      ws[c][r] = (n0 + r < N && k < K) ? w[(size_t)(n0 + r) * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < TK; ++c) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[c][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[c][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * ldo + n] = acc[i][j];
    }
  }
}

RL_API int rl_gemm_f32(const float* x, int ldx, const float* w, int ldw, float* out, int ldo, int M, int N, int K,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemm_f32: M=%d N=%d K=%d", M, N, K);
  if (ldx < K || ldw < K || ldo < N) RL_REFUSE(2, "gemm_f32: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  const int gy = (M + TM - 1) / TM;
  if (gy > 65535) RL_REFUSE(3, "gemm_f32: %d rows exceed %d", M, 65535 * TM);
  dim3 grid((N + TN - 1) / TN, gy);
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, ldx, w, ldw, out, ldo, M, N, K);
  RL_LAUNCH_RESULT();
}
