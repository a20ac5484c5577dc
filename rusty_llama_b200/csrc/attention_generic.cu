// Causal grouped-query attention over the paged cache, the plain way: one warp
// per (token, query head), keys taken 32 at a time in position order with an
// online softmax (src/backend/cpu.rs:363-433, src/backend/cuda.rs:157-232).
//
// It is the attention of the 32-bit path, for prompts and for decoding alike:
// the keys of a query are always cut into the same groups of 32, counted from
// the first key the query may see, so the bits of the result do not depend on
// how the sequence was cut into steps or on what else is in the batch.  It also
// serves any head size up to 256 in both element types.
//
// Cache layout of one layer: pages[page][kv_head][slot_in_page][hd]; the page of
// position p of batch sequence s is block_table[s][p / page_size].
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define MAX_DIMS_PER_LANE 8  // head sizes up to 256

template <typename T>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages,
                                    const T* __restrict__ v_pages, const int* __restrict__ block_table,
                                    int table_width, const int* __restrict__ tok_seq,
                                    const int* __restrict__ tok_pos, T* __restrict__ out, int out_stride, int H,
                                    int K, int hd, int page_size, int window, float scale) {
  extern __shared__ float q_s[];  // hd floats
  const int lane = threadIdx.x;
  const int t = blockIdx.x, h = blockIdx.y;
  const int kh = h / (H / K);
  const int pos = tok_pos[t];
  const int* table = block_table + (size_t)tok_seq[t] * table_width;
  const T* qh = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = lane; i < hd; i += 32) q_s[i] = to_f32(qh[i]);
  __syncwarp();

  // keep when pos - key < window (src/backend/cpu.rs:404-409)
  const int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  float m = -INFINITY, l = 0.f;
  float acc[MAX_DIMS_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] = 0.f;

  for (int base = first; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float s = -INFINITY;
    if (valid) {
      const int page = table[key / page_size];
      const T* kr = k_pages + (((size_t)page * K + kh) * page_size + key % page_size) * hd;
      float dot = 0.f;
      for (int i = 0; i < hd; ++i) dot += q_s[i] * to_f32(kr[i]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));  // finite: the group holds at least key `base`
    const float alpha = expf(m - m_new);        // 0 for the first group, where m is -inf
    const float p = valid ? expf(s - m_new) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] *= alpha;
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = table[kj / page_size];
      const T* vr = v_pages + (((size_t)page * K + kh) * page_size + kj % page_size) * hd;
#pragma unroll
      for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
        const int dim = lane + 32 * i;
        if (dim < hd) acc[i] += pj * to_f32(vr[dim]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
    const int dim = lane + 32 * i;
    if (dim < hd) o[dim] = from_f32<T>(acc[i] * inv);
  }
}

RL_API int rl_attn_generic(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages,
                           const int* block_table, int table_width, const int* tok_seq, const int* tok_pos,
                           void* out, int out_stride, int n_tokens, int H, int K, int hd, int page_size,
                           int window, float scale, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || K <= 0 || hd <= 0 || page_size <= 0)
    RL_REFUSE(1, "attn_generic: T=%d H=%d K=%d hd=%d page=%d", n_tokens, H, K, hd, page_size);
  if (H % K) RL_REFUSE(2, "attn_generic: %d query heads are not a multiple of %d kv heads", H, K);
  if (hd > 32 * MAX_DIMS_PER_LANE) RL_REFUSE(3, "attn_generic: head size %d exceeds %d", hd, 32 * MAX_DIMS_PER_LANE);
  if (H > 65535) RL_REFUSE(4, "attn_generic: %d heads exceed 65535", H);
  if (window < 0) RL_REFUSE(5, "attn_generic: negative window");
  dim3 grid(n_tokens, H);
  const size_t smem = (size_t)hd * sizeof(float);
  if (dtype == RL_BF16)
    attn_generic_kernel<bf16><<<grid, 32, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)k_pages,
                                                          (const bf16*)v_pages, block_table, table_width, tok_seq,
                                                          tok_pos, (bf16*)out, out_stride, H, K, hd, page_size,
                                                          window, scale);
  else if (dtype == RL_F32)
    attn_generic_kernel<float><<<grid, 32, smem, stream>>>((const float*)q, q_stride, (const float*)k_pages,
                                                           (const float*)v_pages, block_table, table_width,
                                                           tok_seq, tok_pos, (float*)out, out_stride, H, K, hd,
                                                           page_size, window, scale);
  else
    RL_REFUSE(6, "attn_generic: unknown dtype %d", dtype);
  RL_LAUNCH_RESULT();
}
