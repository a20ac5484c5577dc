// Matrix products of the decode step in bfloat16: out[M, N] = x[M, K] . w[N, K]^T
// for a handful of rows (M <= 64), where every weight is read from HBM exactly
// once and the arithmetic is free.  Counterpart of the reference's warp-per-row
// GEMV family (src/backend/cuda.rs:354-442), with tensor cores instead of dp4a.
//
// A block owns 16 output features; its 8 warps take the 32-wide k blocks in
// turn, so the block streams 512 contiguous bytes of each of its 16 weight rows
// per round.  Inside a warp the weights are the A operand of
// mma.sync.m16n8k16 (16 features x 16 k) and the activations the B operand
// (16 k x 8 batch rows), accumulated in 32-bit.  A lane loads 16 contiguous
// bytes of a weight row and uses them as its k elements of two consecutive
// MMAs; the activations are loaded with the same rule, so both operands agree
// on which k sits where and the sum over k is unchanged.  The eight partial
// sums of a block are added in warp order through shared memory: no atomics,
// no scratch, the same bits every run.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define WARPS 8

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const bf16* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <typename TO>
__device__ __forceinline__ void store_out(TO* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// SWIGLU: the weight rows alternate gate and up (row 2i is gate i, row 2i+1 is up i) and the
// kernel writes h[m, i] = silu(gate) * up, N / 2 values per row, from the 32-bit sums.
template <int NT, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(WARPS * 32)
gemv_bf16_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ w, int ldw, TO* __restrict__ out,
                 int ldo, int M, int N, int K) {
  __shared__ float red[WARPS][NT * 128];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * 16;
  // blockIdx.y: which slice of k this block sums (k_splits > 1: out receives one partial result
  // per slice, [slice][M][ldo], that the consumer adds up)
  const int k_blocks_total = (K + 31) / 32;
  const int per_split = (k_blocks_total + gridDim.y - 1) / gridDim.y;
  const int kb_begin = blockIdx.y * per_split;
  const int kb_end = min(k_blocks_total, kb_begin + per_split);
  out += (size_t)blockIdx.y * M * ldo;
  const bool row0_ok = n0 + g < N, row1_ok = n0 + g + 8 < N;
  const bf16* w0 = w + (size_t)(row0_ok ? n0 + g : 0) * ldw;
  const bf16* w1 = w + (size_t)(row1_ok ? n0 + g + 8 : 0) * ldw;

  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  // U k blocks of weights are requested before the first is used, so that each lane keeps
  // 2 * U 16-byte loads in flight (measured: 8 is slower than 4, the registers cost more
  // resident warps than the deeper queue gains).
  constexpr int U = 4;
  uint4 a0[U], a1[U];
  auto request = [&](int kb) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + u * WARPS) * 32 + 8 * t4;
      const bool k_ok = k + 8 <= K && kb + u * WARPS < kb_end;
      a0[u] = (k_ok && row0_ok) ? ld_stream(w0 + k) : zero;
      a1[u] = (k_ok && row1_ok) ? ld_stream(w1 + k) : zero;
    }
  };
  request(kb_begin + warp);
  for (int kb = kb_begin + warp; kb < kb_end; kb += WARPS * U) {
    if (kb != kb_begin + warp) request(kb);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (kb + u * WARPS) * 32 + 8 * t4;
      const bool k_ok = k + 8 <= K && kb + u * WARPS < kb_end;
      uint4 b[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int m = nt * 8 + g;
        b[nt] = (k_ok && m < M) ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k)) : zero;
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_bf16(acc[nt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, b[nt].x, b[nt].y);
        mma_bf16(acc[nt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, b[nt].z, b[nt].w);
      }
    }
  }

#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][nt * 128 + lane * 4 + c] = acc[nt][c];
  __syncthreads();
  if (SWIGLU) {
    // 8 (gate, up) pairs of features x NT * 8 batch rows
    for (int e = tid; e < NT * 64; e += WARPS * 32) {
      const int pr = e & 7, m = e >> 3;
      const int nt = m >> 3, t = (m & 7) >> 1, c_lo = m & 1;
      const int ng = 2 * pr, nu = 2 * pr + 1;  // feature index inside the block's 16
      const int ig = nt * 128 + ((ng & 7) * 4 + t) * 4 + (ng >> 3) * 2 + c_lo;
      const int iu = nt * 128 + ((nu & 7) * 4 + t) * 4 + (nu >> 3) * 2 + c_lo;
      float gsum = 0.f, usum = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; ++wq) {
        gsum += red[wq][ig];
        usum += red[wq][iu];
      }
      const int col = (n0 >> 1) + pr;
      if (col < (N >> 1) && m < M) store_out<TO>(out + (size_t)m * ldo + col, gsum * (1.0f / (1.0f + expf(-gsum))) * usum);
    }
  } else {
    for (int e = tid; e < NT * 128; e += WARPS * 32) {
      float sum = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; ++wq) sum += red[wq][e];
      const int nt = e >> 7, l = (e & 127) >> 2, c = e & 3;
      const int n = n0 + (l >> 2) + 8 * (c >> 1);
      const int m = nt * 8 + 2 * (l & 3) + (c & 1);
      if (n < N && m < M) store_out<TO>(out + (size_t)m * ldo + n, sum);
    }
  }
}

template <int NT>
static int launch_gemv(const bf16* x, int ldx, const bf16* w, int ldw, void* out, int out_dtype, int ldo, int M,
                       int N, int K, int swiglu, int k_splits, cudaStream_t stream) {
  const dim3 blocks((N + 15) / 16, k_splits);
  if (swiglu && out_dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(gemv_bf16_kernel<NT, float, true>, blocks, WARPS * 32, 0, stream, x, ldx, w, ldw, (float*)out, ldo, M, N, K));
  else if (swiglu)
    RL_LAUNCH_CHECK(rl_launch<false>(gemv_bf16_kernel<NT, bf16, true>, blocks, WARPS * 32, 0, stream, x, ldx, w, ldw, (bf16*)out, ldo, M, N, K));
  else if (out_dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(gemv_bf16_kernel<NT, float, false>, blocks, WARPS * 32, 0, stream, x, ldx, w, ldw, (float*)out, ldo, M, N, K));
  else
    RL_LAUNCH_CHECK(rl_launch<false>(gemv_bf16_kernel<NT, bf16, false>, blocks, WARPS * 32, 0, stream, x, ldx, w, ldw, (bf16*)out, ldo, M, N, K));
  return 0;
}

RL_API int rl_gemv_bf16_max_rows() { return 64; }

// swiglu != 0: w holds N rows alternating gate and up, out gets N / 2 columns (see the kernel).
// k_splits > 1: the k range is cut into that many slices, each summed by blocks of its own; out is then
// [k_splits][M][ldo] float32 partial results (more blocks in flight for matrices with few rows).
RL_API int rl_gemv_bf16(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M,
                        int N, int K, int swiglu, int k_splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemv_bf16: M=%d N=%d K=%d", M, N, K);
  if (M > 64) RL_REFUSE(2, "gemv_bf16: %d rows, this kernel takes at most 64", M);
  if (K % 8 || ldx % 8 || ldw % 8) RL_REFUSE(3, "gemv_bf16: K=%d, ldx=%d, ldw=%d must be multiples of 8 (16-byte loads)", K, ldx, ldw);
  if (swiglu && (N & 1)) RL_REFUSE(6, "gemv_bf16: %d gate/up rows are not pairs", N);
  if (k_splits < 1 || k_splits > 64) RL_REFUSE(7, "gemv_bf16: %d k slices", k_splits);
  if (k_splits > 1 && (swiglu || out_dtype != RL_F32)) RL_REFUSE(8, "gemv_bf16: partial sums over k slices are float32 and cannot go through the activation");
  if (ldx < K || ldw < K || ldo < (swiglu ? N / 2 : N)) RL_REFUSE(4, "gemv_bf16: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) RL_REFUSE(5, "gemv_bf16: unknown output dtype %d", out_dtype);
  const bf16* xx = (const bf16*)x;
  const bf16* ww = (const bf16*)w;
  if (M <= 8) return launch_gemv<1>(xx, ldx, ww, ldw, out, out_dtype, ldo, M, N, K, swiglu, k_splits, stream);
  if (M <= 16) return launch_gemv<2>(xx, ldx, ww, ldw, out, out_dtype, ldo, M, N, K, swiglu, k_splits, stream);
  if (M <= 32) return launch_gemv<4>(xx, ldx, ww, ldw, out, out_dtype, ldo, M, N, K, swiglu, k_splits, stream);
  return launch_gemv<8>(xx, ldx, ww, ldw, out, out_dtype, ldo, M, N, K, swiglu, k_splits, stream);
}
