// Row-wise kernels around the residual stream: embedding rows, the fused
// residual sum + RMSNorm, and the gated activation of the feed-forward.
//
// The residual stream is kept in 32-bit in both precisions.  What a mixer or a
// feed-forward returns (in the activation type, possibly as several partial
// sums of a split matrix product) is added to it in 32-bit inside the norm
// kernel, which then writes the normalised row in the activation type: one
// pass over the row instead of the reference's separate `add_kernel` and
// `rmsnorm_kernel` (src/backend/cuda.rs:90-116).
#include <type_traits>

#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

// ---------------------------------------------------------------- embedding
// out[t, :] = table[tokens[t], :] widened to 32-bit, no scale (src/model.rs:1237-1242).
template <typename TW, bool VEC>
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                    float* __restrict__ out, int d) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const TW* row = table + (size_t)tokens[t] * d;
  float* o = out + (size_t)t * d;
  if (VEC) {  // d is a multiple of 4: every thread moves four values per round, all loads in flight at once
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float v[4];
      load4_g<TW>(row + i, v);
      store4<float>(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32(row[i]);
  }
}

static int row_threads(int d) {
  int t = ((d / 4 + 31) / 32) * 32;
  return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

RL_API int rl_embed_gather(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens,
                           int d, cudaStream_t stream) {
  if (n_tokens <= 0 || d <= 0) RL_REFUSE(1, "embed_gather: n_tokens=%d d=%d", n_tokens, d);
  const int th = row_threads(d);
  if (table_dtype == RL_BF16 && d % 4 == 0)
    RL_LAUNCH_CHECK(rl_launch(embed_gather_kernel<bf16, true>, n_tokens, th, 0, stream, tokens, (const bf16*)table, out, d));
  else if (table_dtype == RL_BF16)
    RL_LAUNCH_CHECK(rl_launch<false>(embed_gather_kernel<bf16, false>, n_tokens, 256, 0, stream, tokens, (const bf16*)table, out, d));
  else if (table_dtype == RL_F32 && d % 4 == 0)
    RL_LAUNCH_CHECK(rl_launch(embed_gather_kernel<float, true>, n_tokens, th, 0, stream, tokens, (const float*)table, out, d));
  else if (table_dtype == RL_F32)
    RL_LAUNCH_CHECK(rl_launch<false>(embed_gather_kernel<float, false>, n_tokens, 256, 0, stream, tokens, (const float*)table, out, d));
  else
    RL_REFUSE(2, "embed_gather: unknown table dtype %d", table_dtype);
  return 0;
}

// ---------------------------------------------------------------- residual sum + RMSNorm
// For output row r (stream row t = rows ? rows[r] : r):
//   v = x[t] + delta[0][t] + delta[1][t] + ...        (32-bit, in this order)
//   if write_x: x[t] = v
//   if w: out[r] = v * (1 / sqrt(sum(v^2)/d + eps)) * w   (src/backend/cpu.rs:96-105)
// The row is held in shared memory between the two passes.
// With VEC (d a multiple of 4) a thread handles four neighbouring values per round and the block
// is sized so that a row of up to 4096 values takes one round: all loads are in flight together,
// which is what the few rows of a decode step need.
// TD is the type of the parts that are added: the activation type, or float32 for the partial sums
// of a product that was split over k.
template <typename TA, typename TW, typename TD, bool VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_parts,
                                   long long part_stride, const TW* __restrict__ w, TA* __restrict__ out,
                                   const int* __restrict__ rows, int d, float eps, int write_x) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * d;
  float ss = 0.f;
  if (VEC && d <= (int)blockDim.x * 4) {
    // One round (what the launcher arranges up to 4096 values): the row stays in registers, the parts are asked for
    // four at a time and added in their order, and the norm weight is asked for BEFORE the block adds up its squares,
    // so that no trip to L2 stands between the sum and the stores (the kernel is a chain of such trips and little else).
    const int i = threadIdx.x * 4;
    const bool mine = i < d;
    float v[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
    if (mine) {
      load4_g<float>(xr + i, v);
      if (w != nullptr) load4_g<TW>(w + i, wv);
      const TD* dp = delta + (size_t)t * d + i;
      int p = 0;
      for (; p + 4 <= n_parts; p += 4) {
        float dv[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) load4_g<TD>(dp + (size_t)(p + u) * part_stride, dv[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] += dv[u][e];
      }
      for (; p < n_parts; ++p) {
        float dv[4];
        load4_g<TD>(dp + (size_t)p * part_stride, dv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += dv[e];
      }
      if (write_x) store4<float>(xr + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
    }
    if (w == nullptr) return;
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)d + eps);
    if (mine) {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = v[e] * inv * wv[e];
      store4<TA>(out + (size_t)r * d + i, v);
    }
    return;
  }
  if (VEC) {
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float v[4];
      load4_g<float>(xr + i, v);
      for (int p = 0; p < n_parts; ++p) {
        float dv[4];
        load4_g<TD>(delta + (size_t)p * part_stride + (size_t)t * d + i, dv);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += dv[e];
      }
      store4<float>(row + i, v);
      if (write_x) store4<float>(xr + i, v);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float v = xr[i];
      for (int p = 0; p < n_parts; ++p) v += to_f32(delta[(size_t)p * part_stride + (size_t)t * d + i]);
      row[i] = v;
      if (write_x) xr[i] = v;
      ss += v * v;
    }
  }
  if (w == nullptr) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)d + eps);
  TA* o = out + (size_t)r * d;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float v[4], wv[4];
      load4<float>(row + i, v);
      load4_g<TW>(w + i, wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = v[e] * inv * wv[e];
      store4<TA>(o + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_f32<TA>(row[i] * inv * to_f32(w[i]));
  }
}

// The same for the many rows of a prompt step (bfloat16 runs): a quarter of the threads per row,
// each keeping up to CHUNKS pieces of four values in registers between the two passes, so that
// eight blocks share an SM and no shared-memory row is needed.  The sum of squares is added in
// another order than above, so 32-bit runs, whose bits must not depend on how many rows a step
// has, never come here.
template <typename TA, typename TW, typename TD, int CHUNKS>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_parts, long long part_stride,
                        const TW* __restrict__ w, TA* __restrict__ out, const int* __restrict__ rows, int d, float eps,
                        int write_x) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * d;
  float v[CHUNKS][4];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (threadIdx.x + c * 256) * 4;
    if (i < d) load4_g<float>(xr + i, v[c]);
    else v[c][0] = v[c][1] = v[c][2] = v[c][3] = 0.f;
  }
  // the norm weight is asked for here, long before it is used (see add_rmsnorm_kernel)
  float wv[CHUNKS][4];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (threadIdx.x + c * 256) * 4;
    if (w != nullptr && i < d) load4_g<TW>(w + i, wv[c]);
    else wv[c][0] = wv[c][1] = wv[c][2] = wv[c][3] = 0.f;
  }
  // the parts two at a time (all their loads in flight together), added in their order
  int p = 0;
  for (; p + 2 <= n_parts; p += 2) {
    float dv[2][CHUNKS][4];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int i = (threadIdx.x + c * 256) * 4;
        if (i < d) load4_g<TD>(delta + (size_t)(p + u) * part_stride + (size_t)t * d + i, dv[u][c]);
        else dv[u][c][0] = dv[u][c][1] = dv[u][c][2] = dv[u][c][3] = 0.f;
      }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c][e] += dv[u][c][e];
  }
  for (; p < n_parts; ++p) {
    float dv[CHUNKS][4];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int i = (threadIdx.x + c * 256) * 4;
      if (i < d) load4_g<TD>(delta + (size_t)p * part_stride + (size_t)t * d + i, dv[c]);
      else dv[c][0] = dv[c][1] = dv[c][2] = dv[c][3] = 0.f;
    }
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
      for (int e = 0; e < 4; ++e) v[c][e] += dv[c][e];
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (threadIdx.x + c * 256) * 4;
    if (write_x && i < d) store4<float>(xr + i, v[c]);
#pragma unroll
    for (int e = 0; e < 4; ++e) ss += v[c][e] * v[c][e];
  }
  if (w == nullptr) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / (float)d + eps);
  TA* o = out + (size_t)r * d;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int i = (threadIdx.x + c * 256) * 4;
    if (i < d) {
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = v[c][e] * inv * wv[c][e];
      store4<TA>(o + i, y);
    }
  }
}

#define ROWS_KERNEL_MIN_ROWS 64
#define ROWS_KERNEL_CHUNKS 4

template <typename TA, typename TW, typename TD>
static int launch_add_rmsnorm(float* x, const void* delta, int n_parts, long long part_stride, const void* w,
                              void* out, const int* rows, int n_rows, int d, float eps, int write_x,
                              cudaStream_t stream) {
  const bool vec = d % 4 == 0;
  if (vec && !std::is_same<TA, float>::value && n_rows >= ROWS_KERNEL_MIN_ROWS && d <= 256 * 4 * ROWS_KERNEL_CHUNKS) {
    RL_LAUNCH_CHECK(rl_launch(add_rmsnorm_rows_kernel<TA, TW, TD, ROWS_KERNEL_CHUNKS>, n_rows, 256, 0, stream, x,
                              (const TD*)delta, n_parts, part_stride, (const TW*)w, (TA*)out, rows, d, eps, write_x));
    return 0;
  }
  const size_t smem = (size_t)d * sizeof(float);
  auto kern = vec ? add_rmsnorm_kernel<TA, TW, TD, true> : add_rmsnorm_kernel<TA, TW, TD, false>;
  if (smem > 48 * 1024) {
    if (smem > 200 * 1024) RL_REFUSE(3, "add_rmsnorm: a row of %d values does not fit shared memory", d);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(4, "add_rmsnorm: cannot get %zu bytes of shared memory", smem);
  }
  if (vec)
    RL_LAUNCH_CHECK(rl_launch(kern, n_rows, row_threads(d), smem, stream, x, (const TD*)delta, n_parts, part_stride,
                              (const TW*)w, (TA*)out, rows, d, eps, write_x));
  else  // the element-by-element variant uses ordinary loads: plain stream order for it
    RL_LAUNCH_CHECK(rl_launch<false>(kern, n_rows, 256, smem, stream, x, (const TD*)delta, n_parts, part_stride,
                                     (const TW*)w, (TA*)out, rows, d, eps, write_x));
  return 0;
}

RL_API int rl_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_parts, long long part_stride,
                          const void* w, int w_dtype, void* out, int act_dtype, const int* rows, int n_rows, int d,
                          float eps, int write_x, cudaStream_t stream) {
  if (n_rows <= 0 || d <= 0 || n_parts < 0) RL_REFUSE(1, "add_rmsnorm: n_rows=%d d=%d n_parts=%d", n_rows, d, n_parts);
  if (n_parts > 0 && delta == nullptr) RL_REFUSE(2, "add_rmsnorm: %d parts but no delta", n_parts);
  if (w != nullptr && out == nullptr) RL_REFUSE(2, "add_rmsnorm: a weight but no output");
  if (n_parts == 0) delta_dtype = act_dtype;
  if (delta_dtype != act_dtype && delta_dtype != RL_F32) RL_REFUSE(6, "add_rmsnorm: parts of dtype %d in a run of dtype %d", delta_dtype, act_dtype);
#define RL_NORM(TA, TW, TD) \
  return launch_add_rmsnorm<TA, TW, TD>(x, delta, n_parts, part_stride, w, out, rows, n_rows, d, eps, write_x, stream)
  if (act_dtype == RL_BF16 && w_dtype == RL_BF16 && delta_dtype == RL_BF16) RL_NORM(bf16, bf16, bf16);
  if (act_dtype == RL_BF16 && w_dtype == RL_BF16 && delta_dtype == RL_F32) RL_NORM(bf16, bf16, float);
  if (act_dtype == RL_BF16 && w_dtype == RL_F32 && delta_dtype == RL_BF16) RL_NORM(bf16, float, bf16);
  if (act_dtype == RL_BF16 && w_dtype == RL_F32 && delta_dtype == RL_F32) RL_NORM(bf16, float, float);
  if (act_dtype == RL_F32 && w_dtype == RL_F32) RL_NORM(float, float, float);
  if (act_dtype == RL_F32 && w_dtype == RL_BF16) RL_NORM(float, bf16, float);
#undef RL_NORM
  RL_REFUSE(5, "add_rmsnorm: unknown dtypes act=%d w=%d", act_dtype, w_dtype);
}

// ---------------------------------------------------------------- per-sequence records
// A sequence's fixed-size record lives on the device, one row of four integers per slot of the cache:
// [0] positions held, [1] tokens decoded so far, [2] the most it may decode, [3] flags.  The reference keeps the
// same as a device-side position (src/backend/cuda.rs:523-526, :1385-1387) and host-side slot fields
// (src/server.rs:286-296).  A decode step takes its positions from here, so that a captured graph replays
// without the host telling it where each sequence stands.
#define SEQ_FIELDS 4

// Row i of the batch belongs to slot slot_ids[i]: its new token stands at position len, the sequence holds len + 1
// afterwards; the record moves on by one position and one decoded token.
__global__ void seq_begin_decode_kernel(int* __restrict__ state, const int* __restrict__ slot_ids, int n_seqs,
                                        int* __restrict__ tok_pos, int* __restrict__ seq_pos0, int* __restrict__ seq_len) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seqs) return;
  int* rec = state + (size_t)slot_ids[i] * SEQ_FIELDS;
  const int len = rec[0];
  tok_pos[i] = len;
  seq_pos0[i] = len;
  seq_len[i] = len + 1;
  rec[0] = len + 1;
  rec[1] += 1;
}

// After a step whose positions the host gave: the records of its sequences hold seq_len[i] positions.
__global__ void seq_set_len_kernel(int* __restrict__ state, const int* __restrict__ slot_ids, const int* __restrict__ seq_len, int n_seqs) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_seqs) state[(size_t)slot_ids[i] * SEQ_FIELDS] = seq_len[i];
}

RL_API int rl_seq_begin_decode(int* state, const int* slot_ids, int n_seqs, int* tok_pos, int* seq_pos0, int* seq_len, cudaStream_t stream) {
  if (n_seqs <= 0) RL_REFUSE(1, "seq_begin_decode: %d sequences", n_seqs);
  RL_LAUNCH_CHECK(rl_launch(seq_begin_decode_kernel, (n_seqs + 127) / 128, 128, 0, stream, state, slot_ids, n_seqs, tok_pos, seq_pos0, seq_len));
  return 0;
}

RL_API int rl_seq_set_len(int* state, const int* slot_ids, const int* seq_len, int n_seqs, cudaStream_t stream) {
  if (n_seqs <= 0) RL_REFUSE(1, "seq_set_len: %d sequences", n_seqs);
  seq_set_len_kernel<<<(n_seqs + 127) / 128, 128, 0, stream>>>(state, slot_ids, seq_len, n_seqs);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- gated activation
// h[t, i] = silu(g) * u with g = gu[t, i], u = gu[t, ff + i], silu(z) = z / (1 + exp(-z))
// in 32-bit (src/math.rs:25-27, src/backend/cuda.rs:94-97).
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ h, int ff, long long total) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; idx < total; idx += step) {
    const long long t = idx / ff;
    const int i = (int)(idx - t * ff);
    const float g = to_f32(gu[t * 2 * ff + i]);
    const float u = to_f32(gu[t * 2 * ff + ff + i]);
    h[idx] = from_f32<TA>(g * (1.0f / (1.0f + expf(-g))) * u);
  }
}

// The same, four values per thread and one row per blockIdx.y (ff a multiple of 4): a prompt step
// moves hundreds of megabytes through this kernel, so loads are wide and there is no division.
template <typename TA>
__global__ void swiglu_vec_kernel(const TA* __restrict__ gu, TA* __restrict__ h, int ff) {
  const TA* row = gu + (size_t)blockIdx.y * 2 * ff;
  TA* out = h + (size_t)blockIdx.y * ff;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < ff; i += gridDim.x * blockDim.x * 4) {
    float g[4], u[4], o[4];
    load4<TA>(row + i, g);
    load4<TA>(row + ff + i, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = g[e] * (1.0f / (1.0f + expf(-g[e]))) * u[e];
    store4<TA>(out + i, o);
  }
}

RL_API int rl_swiglu(const void* gate_up, void* h, int act_dtype, int n_tokens, int ff, cudaStream_t stream) {
  if (n_tokens <= 0 || ff <= 0) RL_REFUSE(1, "swiglu: n_tokens=%d ff=%d", n_tokens, ff);
  if (ff % 4 == 0 && n_tokens <= 65535) {
    const int bx = (ff / 4 + 255) / 256;
    dim3 grid(bx > 16 ? 16 : bx, n_tokens);
    if (act_dtype == RL_BF16)
      swiglu_vec_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)h, ff);
    else if (act_dtype == RL_F32)
      swiglu_vec_kernel<float><<<grid, 256, 0, stream>>>((const float*)gate_up, (float*)h, ff);
    else
      RL_REFUSE(2, "swiglu: unknown dtype %d", act_dtype);
    RL_LAUNCH_RESULT();
  }
  const long long total = (long long)n_tokens * ff;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (act_dtype == RL_BF16)
    swiglu_kernel<bf16><<<(int)blocks, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)h, ff, total);
  else if (act_dtype == RL_F32)
    swiglu_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)gate_up, (float*)h, ff, total);
  else
    RL_REFUSE(2, "swiglu: unknown dtype %d", act_dtype);
  RL_LAUNCH_RESULT();
}
