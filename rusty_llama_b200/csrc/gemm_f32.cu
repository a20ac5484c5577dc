// The matrix product of the true 32-bit path: out[M, N] = x[M, K] . w[N, K]^T
// with 32-bit inputs, FMA on the CUDA cores and no tensor-core instruction, so
// nothing is rounded to a shorter type on the way (the reference's oracle is its
// CPU backend, a 32-bit dot product per output: src/backend/cpu.rs:107-136).
//
// Each output element is one running sum over k = 0 .. K-1 in ascending order,
// held by one thread; it depends neither on M nor on where the element lies in
// its tile.  A row's result is therefore the same bits whether it is computed
// alone, inside a prompt or inside a batch.
//
// The same kernel with bfloat16 operands (widened on load, the same 32-bit sums, the result rounded
// once, optionally through silu(gate) * up of neighbouring columns) takes the bfloat16 products whose
// k is no multiple of 8: the streaming and tensor-core kernels move rows in 16-byte pieces and refuse
// those.  It is slow and only there so that every size a configuration allows runs.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define TM 64
#define TN 64
#define TK 16

// SWIGLU: w's rows alternate gate and up; out[M, N/2] = silu(gate) * up from the 32-bit sums.
template <typename TA, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(256)
gemm_fma_kernel(const TA* __restrict__ x, int ldx, const TA* __restrict__ w, int ldw,
                TO* __restrict__ out, int ldo, int M, int N, int K) {
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
      xs[c][r] = (m0 + r < M && k < K) ? to_f32(x[(size_t)(m0 + r) * ldx + k]) : 0.f;
      ws[c][r] = (n0 + r < N && k < K) ? to_f32(w[(size_t)(n0 + r) * ldw + k]) : 0.f;
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
    if (SWIGLU) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;  // even: the gate's row; n + 1: the up's
        if (n + 1 < N) out[(size_t)m * ldo + n / 2] = from_f32<TO>(acc[i][j] * (1.0f / (1.0f + expf(-acc[i][j]))) * acc[i][j + 1]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n < N) out[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
      }
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
  gemm_fma_kernel<float, float, false><<<grid, 256, 0, stream>>>(x, ldx, w, ldw, out, ldo, M, N, K);
  RL_LAUNCH_RESULT();
}

// bfloat16 operands of any k and any alignment; out_dtype bfloat16 or float32.
RL_API int rl_gemm_bf16_any(const bf16* x, int ldx, const bf16* w, int ldw, void* out, int out_dtype, int ldo, int M,
                            int N, int K, int swiglu, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemm_bf16_any: M=%d N=%d K=%d", M, N, K);
  if (swiglu && (N & 1)) RL_REFUSE(4, "gemm_bf16_any: %d rows of gate and up are not pairs", N);
  if (ldx < K || ldw < K || ldo < (swiglu ? N / 2 : N)) RL_REFUSE(2, "gemm_bf16_any: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  const int gy = (M + TM - 1) / TM;
  if (gy > 65535) RL_REFUSE(3, "gemm_bf16_any: %d rows exceed %d", M, 65535 * TM);
  dim3 grid((N + TN - 1) / TN, gy);
#define RL_ANY(TO, SW) gemm_fma_kernel<bf16, TO, SW><<<grid, 256, 0, stream>>>(x, ldx, w, ldw, (TO*)out, ldo, M, N, K)
  if (out_dtype == RL_BF16 && swiglu) RL_ANY(bf16, true);
  else if (out_dtype == RL_BF16) RL_ANY(bf16, false);
  else if (out_dtype == RL_F32 && swiglu) RL_ANY(float, true);
  else if (out_dtype == RL_F32) RL_ANY(float, false);
  else RL_REFUSE(5, "gemm_bf16_any: unknown output dtype %d", out_dtype);
#undef RL_ANY
  RL_LAUNCH_RESULT();
}
