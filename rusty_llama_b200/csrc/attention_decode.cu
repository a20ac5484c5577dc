// Decode attention over the paged cache: one new token per sequence, keys and
// values streamed from HBM once per (sequence, kv head) for all query heads of
// the group, the key range cut into splits so that a small batch still fills
// the GPU (flash-decoding).  The reference runs its one prefill kernel with a
// single row here (src/backend/cuda.rs:1189-1192), one block per query head,
// which reads every key `group size` times.
//
// Kernel 1 (grid: splits x (kv heads * head groups of GT) x sequences): for its
// pages, tile = one page of 64 keys, K and V tiles copied to shared memory with
// cp.async (two stages), scores and the online softmax in 32-bit, partial
// (max, sum, unnormalised output) written to scratch.
// Kernel 2 (grid: query heads x sequences): merges the splits in split order.
//
// Scratch layout: part_o[seq][head][split][hd] floats, part_ml[seq][head][split][2].
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define GT 4          // query heads per block
#define TILE 64       // keys per tile = page size
#define THREADS 128

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);  // elements per 16 bytes
};

template <typename T>
__device__ __forceinline__ void load_vec_f32(const T* p, float* f);
template <>
__device__ __forceinline__ void load_vec_f32<bf16>(const bf16* p, float* f) {
  bf16x8_to_f32(*reinterpret_cast<const uint4*>(p), f);
}
template <>
__device__ __forceinline__ void load_vec_f32<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}

// Copy one page tile [TILE][hd] (contiguous in global memory) into rows of
// `stride` elements in shared memory.
template <typename T>
__device__ __forceinline__ void load_tile(T* dst, const T* src, int hd, int stride) {
  constexpr int VN = Vec16<T>::N;
  const int chunks_per_row = hd / VN;
  const int total = TILE * chunks_per_row;
  for (int c = threadIdx.x; c < total; c += THREADS) {
    const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
    cp_async_16(dst + (size_t)r * stride + cc * VN, src + (size_t)r * hd + cc * VN);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_decode_split_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ seq_len, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int H, int K, int hd, int window, float scale,
                         int n_splits) {
  constexpr int VN = Vec16<T>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = hd + VN;  // padded row: consecutive keys fall into different banks
  T* k_s[2];
  T* v_s[2];
  k_s[0] = reinterpret_cast<T*>(smem_raw);
  v_s[0] = k_s[0] + (size_t)TILE * stride;
  k_s[1] = v_s[0] + (size_t)TILE * stride;
  v_s[1] = k_s[1] + (size_t)TILE * stride;
  float* q_s = reinterpret_cast<float*>(v_s[1] + (size_t)TILE * stride);  // [GT][hd]
  float* sc = q_s + GT * hd;                                               // [GT][TILE]
  __shared__ float alpha_s[GT];

  const int G = H / K;
  const int groups_per_kv = (G + GT - 1) / GT;
  const int split = blockIdx.x;
  const int kh = blockIdx.y / groups_per_kv;
  const int g0 = (blockIdx.y - kh * groups_per_kv) * GT;  // first head of this block within the group
  const int n_heads = min(GT, G - g0);
  const int h0 = kh * G + g0;
  const int s = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  const int kv_len = seq_len[s];
  const int pos = kv_len - 1;
  const int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int tile_lo = first / TILE, tile_hi = pos / TILE;  // inclusive
  const int n_tiles = tile_hi - tile_lo + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int my_lo = tile_lo + split * per_split;
  const int my_hi = min(my_lo + per_split - 1, tile_hi);

  float m_run = -INFINITY, l_run = 0.f;  // meaningful in warp g (< n_heads), all lanes equal
  float acc[GT][2];
#pragma unroll
  for (int g = 0; g < GT; ++g) acc[g][0] = acc[g][1] = 0.f;

  if (my_lo <= my_hi) {
    const int* table = block_table + (size_t)s * table_width;
    for (int i = tid; i < GT * hd; i += THREADS) {
      const int g = i / hd, d = i - g * hd;
      q_s[i] = (g < n_heads) ? to_f32(q[(size_t)s * q_stride + (size_t)(h0 + g) * hd + d]) : 0.f;
    }
    {
      const size_t base = ((size_t)table[my_lo] * K + kh) * TILE * hd;
      load_tile(k_s[0], k_pages + base, hd, stride);
      load_tile(v_s[0], v_pages + base, hd, stride);
      cp_async_commit();
    }
    for (int tile = my_lo; tile <= my_hi; ++tile) {
      const int buf = (tile - my_lo) & 1;
      if (tile + 1 <= my_hi) {
        const size_t base = ((size_t)table[tile + 1] * K + kh) * TILE * hd;
        load_tile(k_s[buf ^ 1], k_pages + base, hd, stride);
        load_tile(v_s[buf ^ 1], v_pages + base, hd, stride);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();  // tile `buf` (and q_s) visible to all

      // ---- scores: thread = (key, pair of heads)
      {
        const int key = tid & (TILE - 1);
        const int hp = tid >> 6;  // 0: heads 0,1   1: heads 2,3
        const T* kr = k_s[buf] + (size_t)key * stride;
        const float* qa = q_s + (2 * hp) * hd;
        const float* qb = qa + hd;
        float sa = 0.f, sb = 0.f;
        for (int c = 0; c < hd; c += VN) {
          float kf[VN];
          load_vec_f32<T>(kr + c, kf);
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            sa += qa[c + e] * kf[e];
            sb += qb[c + e] * kf[e];
          }
        }
        const int kpos = tile * TILE + key;
        const bool seen = kpos >= first && kpos <= pos;
        sc[(2 * hp) * TILE + key] = seen ? sa * scale : -INFINITY;
        sc[(2 * hp + 1) * TILE + key] = seen ? sb * scale : -INFINITY;
      }
      __syncthreads();

      // ---- online softmax: warp g owns head g
      if (warp < n_heads) {
        float* row = sc + warp * TILE;
        const float s0 = row[lane], s1 = row[lane + 32];
        const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));  // finite: every tile holds a seen key
        const float alpha = expf(m_run - m_new);
        const float p0 = expf(s0 - m_new), p1 = expf(s1 - m_new);  // exp(-inf) = 0 for unseen keys
        row[lane] = p0;
        row[lane + 32] = p1;
        l_run = l_run * alpha + warp_sum(p0 + p1);
        m_run = m_new;
        if (lane == 0) alpha_s[warp] = alpha;
      }
      __syncthreads();

      // ---- values: thread = output dimension(s) tid, tid + 128
      {
        const int n_valid = min(TILE, pos - tile * TILE + 1);  // rows past the last position are not read
#pragma unroll
        for (int dd = 0; dd < 2; ++dd) {
          const int d = tid + dd * THREADS;
          if (d < hd) {
            float a[GT];
#pragma unroll
            for (int g = 0; g < GT; ++g) a[g] = acc[g][dd] * ((g < n_heads) ? alpha_s[g] : 0.f);
            const T* vc = v_s[buf] + d;
            for (int key = 0; key < n_valid; ++key) {
              const float v = to_f32(vc[(size_t)key * stride]);
#pragma unroll
              for (int g = 0; g < GT; ++g) a[g] += sc[g * TILE + key] * v;
            }
#pragma unroll
            for (int g = 0; g < GT; ++g) acc[g][dd] = a[g];
          }
        }
      }
      __syncthreads();  // before the next iteration overwrites sc and the other buffer
    }
  }

  // ---- partial results
  if (warp < n_heads && lane == 0) {
    float* ml = part_ml + (((size_t)s * H + h0 + warp) * n_splits + split) * 2;
    ml[0] = m_run;
    ml[1] = l_run;
  }
#pragma unroll
  for (int dd = 0; dd < 2; ++dd) {
    const int d = tid + dd * THREADS;
    if (d < hd) {
#pragma unroll
      for (int g = 0; g < GT; ++g)
        if (g < n_heads) part_o[(((size_t)s * H + h0 + g) * n_splits + split) * hd + d] = acc[g][dd];
    }
  }
}

// out[s, h, :] = sum_split exp(m_split - M) o_split / sum_split exp(m_split - M) l_split
template <typename T>
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int out_stride, int H, int hd, int n_splits) {
  const int h = blockIdx.x, s = blockIdx.y;
  const float* ml = part_ml + ((size_t)s * H + h) * n_splits * 2;
  const float* po = part_o + ((size_t)s * H + h) * n_splits * hd;
  float M = -INFINITY;
  for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
  float L = 0.f;
  for (int i = 0; i < n_splits; ++i) {
    const float m = ml[2 * i];
    if (m != -INFINITY) L += expf(m - M) * ml[2 * i + 1];
  }
  const float inv = 1.0f / L;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float m = ml[2 * i];
      if (m != -INFINITY) o += expf(m - M) * po[(size_t)i * hd + d];
    }
    out[(size_t)s * out_stride + (size_t)h * hd + d] = from_f32<T>(o * inv);
  }
}

template <typename T>
static size_t split_smem_bytes(int hd) {
  const int stride = hd + Vec16<T>::N;
  return (size_t)4 * TILE * stride * sizeof(T) + (size_t)GT * hd * sizeof(float) + (size_t)GT * TILE * sizeof(float);
}

template <typename T>
static int launch_decode(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                         const int* block_table, int table_width, const int* seq_len, float* part_o,
                         float* part_ml, void* out, int out_stride, int n_seqs, int H, int K, int hd, int window,
                         float scale, int n_splits, cudaStream_t stream) {
  const size_t smem = split_smem_bytes<T>(hd);
  auto kern = attn_decode_split_kernel<T>;
  if (smem > 220 * 1024) RL_REFUSE(7, "attn_decode: head size %d needs %zu bytes of shared memory", hd, smem);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(8, "attn_decode: cannot get %zu bytes of shared memory", smem);
  }
  const int G = H / K;
  dim3 grid(n_splits, K * ((G + GT - 1) / GT), n_seqs);
  kern<<<grid, THREADS, smem, stream>>>((const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table,
                                        table_width, seq_len, part_o, part_ml, H, K, hd, window, scale, n_splits);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(e));
    return (int)e;
  }
  dim3 grid2(H, n_seqs);
  attn_decode_merge_kernel<T><<<grid2, 128, 0, stream>>>(part_o, part_ml, (T*)out, out_stride, H, hd, n_splits);
  RL_LAUNCH_RESULT();
}

// Scratch needed, in floats: n_seqs * H * n_splits * (hd + 2); the caller passes
// part_o of n_seqs*H*n_splits*hd floats and part_ml of n_seqs*H*n_splits*2.
RL_API int rl_attn_decode(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages,
                          const int* block_table, int table_width, const int* seq_len, float* part_o,
                          float* part_ml, void* out, int out_stride, int n_seqs, int H, int K, int hd,
                          int page_size, int window, float scale, int n_splits, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || K <= 0 || hd <= 0) RL_REFUSE(1, "attn_decode: S=%d H=%d K=%d hd=%d", n_seqs, H, K, hd);
  if (H % K) RL_REFUSE(2, "attn_decode: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != TILE) RL_REFUSE(3, "attn_decode: page size %d, this kernel is built for %d", page_size, TILE);
  if (hd > 2 * THREADS) RL_REFUSE(4, "attn_decode: head size %d exceeds %d", hd, 2 * THREADS);
  if (n_splits <= 0 || n_splits > 65535 || n_seqs > 65535) RL_REFUSE(5, "attn_decode: splits=%d seqs=%d", n_splits, n_seqs);
  if (window < 0) RL_REFUSE(6, "attn_decode: negative window");
  if (dtype == RL_BF16) {
    if (hd % 8) RL_REFUSE(9, "attn_decode: head size %d is not a multiple of 8", hd);
    return launch_decode<bf16>(q, q_stride, k_pages, v_pages, block_table, table_width, seq_len, part_o, part_ml, out,
                               out_stride, n_seqs, H, K, hd, window, scale, n_splits, stream);
  }
  if (dtype == RL_F32) {
    if (hd % 4) RL_REFUSE(9, "attn_decode: head size %d is not a multiple of 4", hd);
    return launch_decode<float>(q, q_stride, k_pages, v_pages, block_table, table_width, seq_len, part_o, part_ml,
                                out, out_stride, n_seqs, H, K, hd, window, scale, n_splits, stream);
  }
  RL_REFUSE(10, "attn_decode: unknown dtype %d", dtype);
}
