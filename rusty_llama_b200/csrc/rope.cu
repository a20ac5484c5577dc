// Rotary position encoding fused with the write of keys and values into the
// paged cache: one kernel where the reference runs a projection into the cache
// span, `rope_kernel` and `kv_append` (src/backend/cuda.rs:119-149, :1511-1512).
//
// Input: the fused projection qkv[T, row_stride] holding, per token, H query
// heads, then K key heads, then K value heads, each of `hd` values.
//   - q is rotated in place;
//   - k is rotated and stored, v is stored, at (page, slot in page) of the
//     token's position in its sequence's page table.
// Angle of pair j at position p: (float)p * inv_freq[j], one 32-bit multiply,
// then sincosf (src/backend/cpu.rs:337-352).  Pairs are neighbours (2j, 2j+1)
// when `interleaved`, else halves (j, j + rot/2); dimensions from `rot` on pass
// through unrotated (partial rotary, src/backend/cpu.rs:319-341).
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                     int table_width, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const float* __restrict__ inv_freq, int H, int K, int hd, int rot,
                                     int interleaved, int page_size, int write_kv) {
  extern __shared__ float trig[];  // cos[rot/2], sin[rot/2]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float a = (float)pos * inv_freq[j];
    float s, c;
    sincosf(a, &s, &c);
    cs[j] = c;
    sn[j] = s;
  }
  __syncthreads();

  T* row = qkv + (size_t)t * row_stride;
  // query heads, in place
  const int q_pairs = H * half;
  for (int idx = threadIdx.x; idx < q_pairs; idx += blockDim.x) {
    const int h = idx / half, j = idx - h * half;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    T* head = row + (size_t)h * hd;
    const float x0 = to_f32(head[i0]), x1 = to_f32(head[i1]);
    head[i0] = from_f32<T>(x0 * cs[j] - x1 * sn[j]);
    head[i1] = from_f32<T>(x0 * sn[j] + x1 * cs[j]);
  }
  if (!write_kv) return;

  const int seq = tok_seq[t];
  const int page = block_table[(size_t)seq * table_width + pos / page_size];
  const int in_page = pos % page_size;
  const T* krow = row + (size_t)H * hd;
  const T* vrow = krow + (size_t)K * hd;
  // key heads: rotated pairs, then the unrotated tail
  const int k_pairs = K * half;
  for (int idx = threadIdx.x; idx < k_pairs; idx += blockDim.x) {
    const int h = idx / half, j = idx - h * half;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    const T* head = krow + (size_t)h * hd;
    T* dst = k_pages + (((size_t)page * K + h) * page_size + in_page) * hd;
    const float x0 = to_f32(head[i0]), x1 = to_f32(head[i1]);
    dst[i0] = from_f32<T>(x0 * cs[j] - x1 * sn[j]);
    dst[i1] = from_f32<T>(x0 * sn[j] + x1 * cs[j]);
  }
  const int tail = hd - rot;
  for (int idx = threadIdx.x; idx < K * tail; idx += blockDim.x) {
    const int h = idx / tail, i = rot + (idx - h * tail);
    k_pages[(((size_t)page * K + h) * page_size + in_page) * hd + i] = krow[(size_t)h * hd + i];
  }
  for (int idx = threadIdx.x; idx < K * hd; idx += blockDim.x) {
    const int h = idx / hd, i = idx - h * hd;
    v_pages[(((size_t)page * K + h) * page_size + in_page) * hd + i] = vrow[idx];
  }
}

// The same work four values at a time: a thread takes one group of four neighbouring values of a
// query head, a key head (with its cache write) or a value head, so a token's row is done in one
// or two rounds with every load in flight at once; a decode step has few tokens and would
// otherwise wait for one load after the other.  Needs head size, rotary size / 2 (or rotary size
// when interleaved) and the row stride to be multiples of 4.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
                                         const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                         int table_width, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         const float* __restrict__ inv_freq, int H, int K, int hd, int rot,
                                         int interleaved, int page_size, int write_kv) {
  extern __shared__ float trig[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float a = (float)pos * inv_freq[j];
    float s, c;
    sincosf(a, &s, &c);
    cs[j] = c;
    sn[j] = s;
  }
  __syncthreads();

  T* row = qkv + (size_t)t * row_stride;
  size_t page_base = 0;
  if (write_kv) {
    const int page = block_table[(size_t)tok_seq[t] * table_width + pos / page_size];
    page_base = ((size_t)page * K * page_size + pos % page_size) * hd;  // + h * page_size * hd per head
  }
  // groups per head: rotated part (pairs) and unrotated tail
  const int rot_groups = interleaved ? rot / 4 : half / 4;  // each covers 2 (interleaved) or 4 pairs
  const int tail_groups = (hd - rot) / 4;
  const int per_head = rot_groups + tail_groups;
  const int n_q = H * rot_groups;  // the tail of q stays as it is
  const int n_k = write_kv ? K * per_head : 0;
  const int n_v = write_kv ? K * (hd / 4) : 0;
  for (int item = threadIdx.x; item < n_q + n_k + n_v; item += blockDim.x) {
    if (item < n_q + n_k) {
      const bool is_q = item < n_q;
      const int idx = is_q ? item : item - n_q;
      const int groups = is_q ? rot_groups : per_head;
      const int h = idx / groups, gq = idx - h * groups;
      T* head = row + (size_t)(is_q ? h : H + h) * hd;
      T* dst = is_q ? head : k_pages + page_base + (size_t)h * page_size * hd;
      if (gq >= rot_groups) {  // unrotated tail of a key head
        const int i = rot + 4 * (gq - rot_groups);
        float v[4];
        load4_g<T>(head + i, v);
        store4<T>(dst + i, v);
      } else if (interleaved) {
        const int i = 4 * gq, j = 2 * gq;
        float v[4], o[4];
        load4_g<T>(head + i, v);
        o[0] = v[0] * cs[j] - v[1] * sn[j];
        o[1] = v[0] * sn[j] + v[1] * cs[j];
        o[2] = v[2] * cs[j + 1] - v[3] * sn[j + 1];
        o[3] = v[2] * sn[j + 1] + v[3] * cs[j + 1];
        store4<T>(dst + i, o);
      } else {
        const int j = 4 * gq;
        float a[4], b[4], oa[4], ob[4];
        load4_g<T>(head + j, a);
        load4_g<T>(head + j + half, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          oa[e] = a[e] * cs[j + e] - b[e] * sn[j + e];
          ob[e] = a[e] * sn[j + e] + b[e] * cs[j + e];
        }
        store4<T>(dst + j, oa);
        store4<T>(dst + j + half, ob);
      }
    } else {
      const int idx = item - n_q - n_k;
      const int h = idx / (hd / 4), i = 4 * (idx - h * (hd / 4));
      float v[4];
      load4_g<T>(row + (size_t)(H + K + h) * hd + i, v);
      store4<T>(v_pages + page_base + (size_t)h * page_size * hd + i, v);
    }
  }
}

// The same eight bfloat16 at a time (16-byte loads and stores), for the many tokens of a prompt step, where the
// kernel is a pass over 12 KB a token and its memory instructions are what it costs: 2048 tokens of 32 + 8 + 8
// heads of 128 took 16.4 us with 8-byte pieces.  Needs head size, rotary size / 2 (or rotary size when interleaved)
// and the row stride to be multiples of 8, and 16-byte aligned rows and pages.
__device__ __forceinline__ void load8_g_bf16(const bf16* p, float* f) {
  const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}
__device__ __forceinline__ void store8_bf16(bf16* p, const float* f) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&a);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
__global__ void rope_kv_write_vec8_kernel(bf16* __restrict__ qkv, int row_stride, const int* __restrict__ tok_pos,
                                          const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                                          int table_width, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                          const float* __restrict__ inv_freq, int H, int K, int hd, int rot,
                                          int interleaved, int page_size, int write_kv) {
  extern __shared__ float trig[];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = rot >> 1;
  float* cs = trig;
  float* sn = trig + half;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    const float a = (float)pos * inv_freq[j];
    float s, c;
    sincosf(a, &s, &c);
    cs[j] = c;
    sn[j] = s;
  }
  __syncthreads();

  bf16* row = qkv + (size_t)t * row_stride;
  size_t page_base = 0;
  if (write_kv) {
    const int page = block_table[(size_t)tok_seq[t] * table_width + pos / page_size];
    page_base = ((size_t)page * K * page_size + pos % page_size) * hd;  // + h * page_size * hd per head
  }
  // groups per head: rotated part (each covers 4 neighbouring pairs when interleaved, else 8 pairs) and unrotated tail
  const int rot_groups = interleaved ? rot / 8 : half / 8;
  const int tail_groups = (hd - rot) / 8;
  const int per_head = rot_groups + tail_groups;
  const int n_q = H * rot_groups;  // the tail of q stays as it is
  const int n_k = write_kv ? K * per_head : 0;
  const int n_v = write_kv ? K * (hd / 8) : 0;
  for (int item = threadIdx.x; item < n_q + n_k + n_v; item += blockDim.x) {
    if (item < n_q + n_k) {
      const bool is_q = item < n_q;
      const int idx = is_q ? item : item - n_q;
      const int groups = is_q ? rot_groups : per_head;
      const int h = idx / groups, gq = idx - h * groups;
      bf16* head = row + (size_t)(is_q ? h : H + h) * hd;
      bf16* dst = is_q ? head : k_pages + page_base + (size_t)h * page_size * hd;
      if (gq >= rot_groups) {  // unrotated tail of a key head
        const int i = rot + 8 * (gq - rot_groups);
        *reinterpret_cast<uint4*>(dst + i) = __ldcg(reinterpret_cast<const uint4*>(head + i));
      } else if (interleaved) {
        const int i = 8 * gq, j = 4 * gq;
        float v[8], o[8];
        load8_g_bf16(head + i, v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[2 * e] = v[2 * e] * cs[j + e] - v[2 * e + 1] * sn[j + e];
          o[2 * e + 1] = v[2 * e] * sn[j + e] + v[2 * e + 1] * cs[j + e];
        }
        store8_bf16(dst + i, o);
      } else {
        const int j = 8 * gq;
        float a[8], b[8], oa[8], ob[8];
        load8_g_bf16(head + j, a);
        load8_g_bf16(head + j + half, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          oa[e] = a[e] * cs[j + e] - b[e] * sn[j + e];
          ob[e] = a[e] * sn[j + e] + b[e] * cs[j + e];
        }
        store8_bf16(dst + j, oa);
        store8_bf16(dst + j + half, ob);
      }
    } else {
      const int idx = item - n_q - n_k;
      const int h = idx / (hd / 8), i = 8 * (idx - h * (hd / 8));
      *reinterpret_cast<uint4*>(v_pages + page_base + (size_t)h * page_size * hd + i) =
          __ldcg(reinterpret_cast<const uint4*>(row + (size_t)(H + K + h) * hd + i));
    }
  }
}

RL_API int rl_rope_kv_write(void* qkv, int dtype, int row_stride, const int* tok_pos, const int* tok_seq,
                            const int* block_table, int table_width, void* k_pages, void* v_pages,
                            const float* inv_freq, int n_tokens, int H, int K, int hd, int rot, int interleaved,
                            int page_size, int write_kv, cudaStream_t stream) {
  if (n_tokens <= 0 || H <= 0 || K < 0 || hd <= 0) RL_REFUSE(1, "rope_kv_write: T=%d H=%d K=%d hd=%d", n_tokens, H, K, hd);
  if (rot < 0 || rot > hd || (rot & 1)) RL_REFUSE(2, "rope_kv_write: rotary size %d does not fit a head of %d", rot, hd);
  if (row_stride < (H + (write_kv ? 2 * K : 0)) * hd) RL_REFUSE(3, "rope_kv_write: row stride %d too small", row_stride);
  if (write_kv && (page_size <= 0 || !block_table || !k_pages || !v_pages || table_width <= 0))
    RL_REFUSE(4, "rope_kv_write: a cache write needs pages and a page table");
  if (rot > 0 && inv_freq == nullptr) RL_REFUSE(5, "rope_kv_write: no frequency table");
  const size_t smem = (size_t)rot * sizeof(float);
  if (smem > 48 * 1024) RL_REFUSE(6, "rope_kv_write: rotary size %d too large", rot);
  const bool vec = hd % 4 == 0 && row_stride % 4 == 0 && (interleaved ? rot % 4 == 0 : rot % 8 == 0);
  int threads = 128;
  if (vec) {
    const int items = H * (rot / 8 + 1) + (write_kv ? K * (hd / 4) * 2 : 0);
    threads = ((items + 31) / 32) * 32;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  }
  const bool vec8 = dtype == RL_BF16 && n_tokens >= 64 && hd % 8 == 0 && row_stride % 8 == 0 && (interleaved ? rot % 8 == 0 : rot % 16 == 0) &&
                    (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
  if (vec8) {
    const int items = H * (rot / 16 + 1) + (write_kv ? K * (hd / 8) * 2 : 0);
    int th = ((items + 31) / 32) * 32;
    th = th < 64 ? 64 : (th > 512 ? 512 : th);
    RL_LAUNCH_CHECK(rl_launch<true>(rope_kv_write_vec8_kernel, n_tokens, th, smem, stream, (bf16*)qkv, row_stride, tok_pos, tok_seq, block_table,
                                    table_width, (bf16*)k_pages, (bf16*)v_pages, inv_freq, H, K, hd, rot, interleaved, page_size, write_kv));
    return 0;
  }
  // only the four-at-a-time kernel (L2 loads) may start before its predecessor has finished
#define RL_ROPE(KERNEL, T, EARLY)                                                                                      \
  RL_LAUNCH_CHECK(rl_launch<EARLY>(KERNEL<T>, n_tokens, threads, smem, stream, (T*)qkv, row_stride, tok_pos, tok_seq,   \
                                   block_table, table_width, (T*)k_pages, (T*)v_pages, inv_freq, H, K, hd, rot,       \
                                   interleaved, page_size, write_kv))
  if (dtype == RL_BF16 && vec) RL_ROPE(rope_kv_write_vec_kernel, bf16, true);
  else if (dtype == RL_BF16) RL_ROPE(rope_kv_write_kernel, bf16, false);
  else if (dtype == RL_F32 && vec) RL_ROPE(rope_kv_write_vec_kernel, float, true);
  else if (dtype == RL_F32) RL_ROPE(rope_kv_write_kernel, float, false);
  else RL_REFUSE(7, "rope_kv_write: unknown dtype %d", dtype);
#undef RL_ROPE
  return 0;
}
