// Causal flash attention for prompts (and any step with more than one token per
// sequence) in bfloat16, reading keys and values from the paged cache.
//
// The reference's prefill attention is its scalar `attention_kernel`
// (src/backend/cuda.rs:157-232): one block per (row, head), FMA dot products.
// Here a block of four warps owns 64 query rows of one head of one sequence;
// Q K^T and P V run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit
// accumulate), the online softmax (max, sum, rescale) stays in 32-bit
// registers, and a key tile is exactly one cache page, copied to shared memory
// with cp.async while the previous page is being used.
//
// Works for a ragged batch: sequence s contributes q_len = seq_start[s+1] -
// seq_start[s] packed rows whose positions begin at seq_pos0[s]; its keys
// 0 .. pos are already in the cache (the rotary kernel ran before).  Head sizes
// are padded with zeros to HD in shared memory, so any multiple of 8 up to 256
// is served.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BM 64   // query rows per block
#define BN 64   // keys per tile = page size
#define NTHREADS 128

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
// d += a(16x16, row) * b(16x8, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy a page tile [BN][hd] (contiguous) into rows of STRIDE elements.
__device__ __forceinline__ void load_kv_tile(bf16* dst, const bf16* src, int hd, int stride) {
  const int chunks_per_row = hd >> 3;
  const int total = BN * chunks_per_row;
  for (int c = threadIdx.x; c < total; c += NTHREADS) {
    const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
    cp_async_16(dst + (size_t)r * stride + cc * 8, src + (size_t)r * hd + cc * 8);
  }
}

template <int HD>
__global__ void __launch_bounds__(NTHREADS)
flash_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_pages,
                     const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                     const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                     bf16* __restrict__ out, int out_stride, int H, int K, int hd, int window,
                     float scale_log2) {
  constexpr int STRIDE = HD + 8;  // 16 bytes of padding per row keeps ldmatrix free of bank conflicts
  constexpr int KSTEPS = HD / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [BM][STRIDE]
  bf16* k_s0 = q_s + BM * STRIDE;                 // two stages of K and V, [BN][STRIDE] each
  bf16* v_s0 = k_s0 + BN * STRIDE;
  bf16* k_s1 = v_s0 + BN * STRIDE;
  bf16* v_s1 = k_s1 + BN * STRIDE;

  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int tok0 = seq_start[s];
  const int q_len = seq_start[s + 1] - tok0;
  // first query row of this block within the sequence's rows: blocks go out in the order of blockIdx.x, then
  // y, so the last row tiles of all heads and sequences, which have the most keys to visit, start first
  const int row0 = (int)(gridDim.y - 1 - blockIdx.y) * BM;
  if (row0 >= q_len) return;
  const int pos0 = seq_pos0[s];
  const int kh = h / (H / K);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int rows_here = min(BM, q_len - row0);

  // ---- zero everything once (padding columns, rows past the end), then load Q
  {
    uint4 z = make_uint4(0, 0, 0, 0);
    uint4* p = reinterpret_cast<uint4*>(smem_raw);
    const int n16 = (5 * BM * STRIDE * (int)sizeof(bf16)) / 16;
    for (int i = tid; i < n16; i += NTHREADS) p[i] = z;
  }
  __syncthreads();
  {
    const int chunks_per_row = hd >> 3;
    const int total = rows_here * chunks_per_row;
    for (int c = tid; c < total; c += NTHREADS) {
      const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
      cp_async_16(q_s + (size_t)r * STRIDE + cc * 8,
                  q + (size_t)(tok0 + row0 + r) * q_stride + (size_t)h * hd + cc * 8);
    }
  }
  const int* table = block_table + (size_t)s * table_width;
  // positions: query row r of this block sits at pos0 + row0 + r
  const int last_pos = pos0 + row0 + rows_here - 1;
  const int first_pos = pos0 + row0;
  const int lowest_key = (window != 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
  const int tile_lo = lowest_key / BN, tile_hi = last_pos / BN;
  {
    const size_t base = ((size_t)table[tile_lo] * K + kh) * BN * hd;
    load_kv_tile(k_s0, k_pages + base, hd, STRIDE);
    load_kv_tile(v_s0, v_pages + base, hd, STRIDE);
  }
  cp_async_commit();

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};  // per-thread partial sums, reduced over the quad at the end
  const int qpos[2] = {first_pos + warp * 16 + g, first_pos + warp * 16 + g + 8};

  for (int tile = tile_lo; tile <= tile_hi; ++tile) {
    const int buf = (tile - tile_lo) & 1;
    bf16* k_s = buf ? k_s1 : k_s0;
    bf16* v_s = buf ? v_s1 : v_s0;
    if (tile + 1 <= tile_hi) {
      const size_t base = ((size_t)table[tile + 1] * K + kh) * BN * hd;
      load_kv_tile(buf ? k_s0 : k_s1, k_pages + base, hd, STRIDE);
      load_kv_tile(buf ? v_s0 : v_s1, v_pages + base, hd, STRIDE);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // ---- S = Q K^T for this warp's 16 rows and the tile's 64 keys
    float s_acc[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s_acc[i][0] = s_acc[i][1] = s_acc[i][2] = s_acc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (size_t)(warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, k_s + (size_t)(np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + kk * 16 + 8 * ((lane >> 3) & 1));
        mma_bf16(s_acc[2 * np], a, b[0], b[1]);
        mma_bf16(s_acc[2 * np + 1], a, b[2], b[3]);
      }
    }

    // ---- mask, scale (to base-2 exponents) and the online softmax
    const int key0 = tile * BN;
    const bool need_mask = (key0 + BN - 1 > first_pos + warp * 16) || (window != 0);
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        float v = s_acc[n][e] * scale_log2;
        if (need_mask) {
          const int key = key0 + n * 8 + 2 * t4 + (e & 1);
          const bool seen = key <= qpos[r] && (window == 0 || qpos[r] - key < window);
          if (!seen) v = -INFINITY;
        }
        s_acc[n][e] = v;
        tile_max[r] = fmaxf(tile_max[r], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = tile_max[r];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      // a row that has seen no key yet keeps exponent base 0 so that nothing becomes NaN
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = exp2f(m_run[r] - m_use[r]);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int n = 0; n < BN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = exp2f(s_acc[n][e] - m_use[r]);
        s_acc[n][e] = p;
        l_run[r] += p;
      }
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[0];
      o_acc[i][2] *= alpha[1];
      o_acc[i][3] *= alpha[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s_acc[2 * kk][0], s_acc[2 * kk][1]);
      a[1] = pack_bf16(s_acc[2 * kk][2], s_acc[2 * kk][3]);
      a[2] = pack_bf16(s_acc[2 * kk + 1][0], s_acc[2 * kk + 1][1]);
      a[3] = pack_bf16(s_acc[2 * kk + 1][2], s_acc[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_s + (size_t)(kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 + 8 * (lane >> 4));
        mma_bf16(o_acc[2 * dp], a, b[0], b[1]);
        mma_bf16(o_acc[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // all warps done with this stage before it is refilled
  }

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_run[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = (l > 0.f) ? 1.0f / l : 0.f;
    const int row = warp * 16 + g + 8 * r;
    if (row < rows_here) {
      bf16* o = out + (size_t)(tok0 + row0 + row) * out_stride + (size_t)h * hd;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        const int d = n * 8 + 2 * t4;
        if (d < hd) {
          __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[n][2 * r] * inv, o_acc[n][2 * r + 1] * inv);
          *reinterpret_cast<__nv_bfloat162*>(o + d) = v;
        }
      }
    }
  }
}

template <int HD>
static int launch_prefill(const bf16* q, int q_stride, const bf16* k_pages, const bf16* v_pages,
                          const int* block_table, int table_width, const int* seq_start, const int* seq_pos0,
                          bf16* out, int out_stride, int n_seqs, int max_q_len, int H, int K, int hd, int window,
                          float scale, cudaStream_t stream) {
  const size_t smem = (size_t)5 * BM * (HD + 8) * sizeof(bf16);
  auto kern = flash_prefill_kernel<HD>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(8, "flash_prefill: cannot get %zu bytes of shared memory", smem);
  }
  dim3 grid(H * n_seqs, (max_q_len + BM - 1) / BM);
  kern<<<grid, NTHREADS, smem, stream>>>(q, q_stride, k_pages, v_pages, block_table, table_width, seq_start, seq_pos0,
                                         out, out_stride, H, K, hd, window, scale * 1.4426950408889634f);
  RL_LAUNCH_RESULT();
}

RL_API int rl_flash_prefill(const void* q, int q_stride, const void* k_pages, const void* v_pages,
                            const int* block_table, int table_width, const int* seq_start, const int* seq_pos0,
                            void* out, int out_stride, int n_seqs, int max_q_len, int H, int K, int hd,
                            int page_size, int window, float scale, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || H <= 0 || K <= 0 || hd <= 0)
    RL_REFUSE(1, "flash_prefill: S=%d max_q=%d H=%d K=%d hd=%d", n_seqs, max_q_len, H, K, hd);
  if (H % K) RL_REFUSE(2, "flash_prefill: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != BN) RL_REFUSE(3, "flash_prefill: page size %d, this kernel is built for %d", page_size, BN);
  if (hd % 8) RL_REFUSE(4, "flash_prefill: head size %d is not a multiple of 8", hd);
  if (q_stride % 8 || out_stride % 2) RL_REFUSE(5, "flash_prefill: strides %d/%d break 16-byte alignment", q_stride, out_stride);
  if ((long long)H * n_seqs > 0x7fffffffLL || max_q_len / 16 > 65535)
    RL_REFUSE(6, "flash_prefill: H=%d x S=%d blocks or %d query rows exceed the grid", H, n_seqs, max_q_len);
  if (window < 0) RL_REFUSE(7, "flash_prefill: negative window");
  const bf16* qq = (const bf16*)q;
  const bf16* kp = (const bf16*)k_pages;
  const bf16* vp = (const bf16*)v_pages;
  bf16* oo = (bf16*)out;
#define RL_PREFILL(HDV)                                                                                          \
  return launch_prefill<HDV>(qq, q_stride, kp, vp, block_table, table_width, seq_start, seq_pos0, oo, out_stride, \
                             n_seqs, max_q_len, H, K, hd, window, scale, stream)
  if (hd <= 32) RL_PREFILL(32);
  if (hd <= 64) RL_PREFILL(64);
  if (hd <= 128) RL_PREFILL(128);
  if (hd <= 256) RL_PREFILL(256);
#undef RL_PREFILL
  RL_REFUSE(9, "flash_prefill: head size %d exceeds 256", hd);
}
