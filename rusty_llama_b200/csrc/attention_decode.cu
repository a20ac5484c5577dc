// Decode attention over the paged cache in bfloat16: one new token per sequence, keys and
// values streamed from HBM once per (sequence, kv head) for all query heads of the group, the
// key range cut into splits so that a small batch still fills the GPU (flash-decoding).  The
// reference runs its one scalar kernel with a single row here (src/backend/cuda.rs:1189-1192),
// one block per query head, which reads every key `group size` times.
//
// Kernel 1 (grid: splits x (kv heads * groups of 8 query heads) x sequences, one warp each).
// A decode step has few queries and many keys, so the keys are the rows of the tensor-core
// tiles: S^T[32 keys x 8 heads] = K_tile . Q^T and O^T[head size x 8 heads] += V_tile^T . P^T
// (mma.sync m16n8k16, bfloat16 in, 32-bit accumulate).  The probabilities leave the first product
// as accumulator fragments indexed (key, head) and enter the second as B fragments indexed
// (head, key); `movmatrix` transposes them inside the warp.  A tile is half a cache page (32
// positions), copied to shared memory with cp.async while the previous tile is in use; max, sum and rescaling of
// the online softmax are per head (per column) in 32-bit registers.  Each warp writes its partial
// (max as a base-2 exponent, sum, unnormalised output) to scratch.
// Kernel 2 (grid: query heads x sequences) merges the splits in split order.
//
// Scratch layout: part_o[seq][head][split][hd] floats, part_ml[seq][head][split][2].
// Head sizes are padded with zeros to HD in shared memory: any multiple of 8 up to 256.
#include <stdlib.h>

#include "common.cuh"
#include "attention_merge.cuh"

RL_DEFINE_ERROR_TEXT()

#define HEADS 8    // query heads per warp (the N of the MMA)
#define PAGE 64    // positions per cache page
#define BK 32      // keys per tile

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
// 8x8 matrix of 16-bit values held one 32-bit register per lane (row lane/4, columns 2*(lane%4), +1): its transpose
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
  return r;
}
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

// Copy BK rows of hd values (contiguous in global memory) into rows of `stride` elements, by one warp.
__device__ __forceinline__ void load_rows(bf16* dst, const bf16* src, int hd, int stride, int lane) {
  const int cpr = hd >> 3;  // 16-byte pieces per row
  const int total = BK * cpr;
  int r = lane / cpr, cc = lane - r * cpr;
  const int dr = 32 / cpr, dc = 32 - dr * cpr;
  for (int c = lane; c < total; c += 32) {
    cp_async_16(dst + (size_t)r * stride + cc * 8, src + (size_t)r * hd + cc * 8);
    r += dr;
    cc += dc;
    if (cc >= cpr) {
      cc -= cpr;
      ++r;
    }
  }
}

// STAGES: tiles in shared memory per warp (2 or 3): 3 keeps more bytes in flight per warp, 2 lets six
// instead of four warps share an SM.
template <int HD, int STAGES>
__global__ void __launch_bounds__(32)
attn_decode_split_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ k_pages,
                         const bf16* __restrict__ v_pages, const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ seq_len, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int H, int K, int hd, int window, float scale_log2,
                         int n_splits) {
  constexpr int STRIDE = HD + 8;  // 16 bytes of padding per row keep ldmatrix free of bank conflicts
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 16;
  constexpr int TILE_ELEMS = BK * STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);  // [HEADS][STRIDE]
  bf16* kv_s = q_s + HEADS * STRIDE;              // STAGES x (K tile, V tile), [BK][STRIDE] each

  const int G = H / K;
  const int groups_per_kv = (G + HEADS - 1) / HEADS;
  const int split = blockIdx.x;
  const int kh = blockIdx.y / groups_per_kv;
  const int g0 = (blockIdx.y - kh * groups_per_kv) * HEADS;
  const int n_heads = min(HEADS, G - g0);
  const int h0 = kh * G + g0;
  const int s = blockIdx.z;
  const int lane = threadIdx.x;
  const int g = lane >> 2, t4 = lane & 3;

  float o_acc[DTILES][4];  // (dim dt*16 + g [+8], head 2*t4 [+1])
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // heads 2*t4, 2*t4+1
  float l_run[2] = {0.f, 0.f};              // per-thread partial sums over this thread's keys

  // (no explicit trigger: the next kernel is released when this one's blocks have finished)
  // zero the padding (columns past hd, rows past the group's heads) once; this needs nothing from
  // the kernel before, so it runs while that kernel finishes
  {
    uint4 z = make_uint4(0, 0, 0, 0);
    uint4* p = reinterpret_cast<uint4*>(smem_raw);
    const int n16 = ((HEADS + 2 * STAGES * BK) * STRIDE * (int)sizeof(bf16)) / 16;
    for (int i = lane; i < n16; i += 32) p[i] = z;
  }
  __syncwarp();
  pdl_trigger();
  pdl_wait();
  const int kv_len = seq_len[s];
  const int pos = kv_len - 1;
  const int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int tile_lo = first / BK, tile_hi = pos / BK;  // inclusive, in tiles of BK keys
  const int n_tiles = tile_hi - tile_lo + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int my_lo = tile_lo + split * per_split;
  const int my_hi = min(my_lo + per_split - 1, tile_hi);


  if (my_lo <= my_hi) {

    {
      const int cpr = hd >> 3;
      for (int c = lane; c < n_heads * cpr; c += 32) {
        const int r = c / cpr, cc = c - r * cpr;
        cp_async_16(q_s + (size_t)r * STRIDE + cc * 8, q + (size_t)s * q_stride + (size_t)(h0 + r) * hd + cc * 8);
      }
    }
    cp_async_commit();
    const int* table = block_table + (size_t)s * table_width;
    auto fetch = [&](int tile) {
      if (tile <= my_hi) {
        const int stage = (tile - my_lo) % STAGES;
        const size_t base = (((size_t)table[tile >> 1] * K + kh) * PAGE + (tile & 1) * BK) * hd;
        load_rows(kv_s + (size_t)(2 * stage) * TILE_ELEMS, k_pages + base, hd, STRIDE, lane);
        load_rows(kv_s + (size_t)(2 * stage + 1) * TILE_ELEMS, v_pages + base, hd, STRIDE, lane);
      }
      cp_async_commit();  // also when there was nothing to fetch: the group count stays uniform
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) fetch(my_lo + i);
    cp_async_wait<STAGES - 1>();  // the queries have arrived
    __syncwarp();
    uint32_t qf[KSTEPS][2];  // Q^T as B fragments: (dims kk*16 + 2*t4 [+8], head g)
#pragma unroll
    for (int k2 = 0; k2 < KSTEPS / 2; ++k2) {
      uint32_t r[4];
      ldmatrix_x4(r, q_s + (size_t)(lane & 7) * STRIDE + k2 * 32 + 8 * (lane >> 3));
      qf[2 * k2][0] = r[0];
      qf[2 * k2][1] = r[1];
      qf[2 * k2 + 1][0] = r[2];
      qf[2 * k2 + 1][1] = r[3];
    }

    for (int tile = my_lo; tile <= my_hi; ++tile) {
      fetch(tile + STAGES - 1);
      cp_async_wait<STAGES - 1>();  // tile `tile` has arrived
      __syncwarp();
      const int stage = (tile - my_lo) % STAGES;
      const bf16* k_s = kv_s + (size_t)(2 * stage) * TILE_ELEMS;
      const bf16* v_s = k_s + TILE_ELEMS;

      // ---- S^T = K Q^T: 32 keys (two 16-row tiles) x 8 heads
      float s_acc[2][4];  // (key mt*16 + g [+8], head 2*t4 [+1])
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) s_acc[mt][0] = s_acc[mt][1] = s_acc[mt][2] = s_acc[mt][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          uint32_t a[4];
          ldmatrix_x4(a, k_s + (size_t)(mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + kk * 16 + 8 * (lane >> 4));
          mma_bf16(s_acc[mt], a, qf[kk][0], qf[kk][1]);
        }
      }

      // ---- mask by position, scale to base-2 exponents, online softmax per head (column)
      const int key0 = tile * BK;
      const bool need_mask = key0 < first || key0 + BK - 1 > pos;
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s_acc[mt][e] * scale_log2;
          if (need_mask) {
            const int key = key0 + mt * 16 + g + 8 * (e >> 1);
            if (key < first || key > pos) v = -INFINITY;
          }
          s_acc[mt][e] = v;
          tmax[e & 1] = fmaxf(tmax[e & 1], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float mx = tmax[j];
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run[j], mx);  // finite: every tile of the range holds a seen key
        m_use[j] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[j] = exp2f(m_run[j] - m_use[j]);
        m_run[j] = m_new;
        l_run[j] *= alpha[j];
      }
      uint32_t pb[2][2];  // P^T as B fragments of the two 16-key steps
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = exp2f(s_acc[mt][e] - m_use[e & 1]);
          l_run[e & 1] += p[e];
        }
        pb[mt][0] = movmatrix_trans(pack_bf16(p[0], p[1]));  // keys mt*16 + 0..7
        pb[mt][1] = movmatrix_trans(pack_bf16(p[2], p[3]));  // keys mt*16 + 8..15
      }
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        o_acc[i][0] *= alpha[0];
        o_acc[i][1] *= alpha[1];
        o_acc[i][2] *= alpha[0];
        o_acc[i][3] *= alpha[1];
      }

      // ---- O^T += V^T P^T: head size (16-row tiles) x 8 heads over the tile's 32 keys
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, v_s + (size_t)(mt * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + dt * 16 + 8 * ((lane >> 3) & 1));
          mma_bf16(o_acc[dt], a, pb[mt][0], pb[mt][1]);
        }
      }
      __syncwarp();  // the stage may be refilled by the next fetch
    }
  }

  // ---- partial results: max (base-2 exponent), sum, unnormalised output
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float l = l_run[j];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    const int head = 2 * t4 + j;
    if (head < n_heads) {
      const size_t slot = ((size_t)s * H + h0 + head) * n_splits + split;
      if (g == 0) {
        part_ml[slot * 2] = m_run[j];
        part_ml[slot * 2 + 1] = l;
      }
      float* po = part_o + slot * hd;
#pragma unroll
      for (int dt = 0; dt < DTILES; ++dt) {
        const int d = dt * 16 + g;
        if (d < hd) po[d] = o_acc[dt][j];
        if (d + 8 < hd) po[d + 8] = o_acc[dt][2 + j];
      }
    }
  }
}

template <int HD, int STAGES>
static int launch_decode_stages(const bf16* q, int q_stride, const bf16* k_pages, const bf16* v_pages,
                         const int* block_table, int table_width, const int* seq_len, float* part_o,
                         float* part_ml, bf16* out, int out_stride, int n_seqs, int H, int K, int hd, int window,
                         float scale, int n_splits, cudaStream_t stream) {
  const size_t smem = (size_t)(HEADS + 2 * STAGES * BK) * (HD + 8) * sizeof(bf16);
  auto kern = attn_decode_split_kernel<HD, STAGES>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) RL_REFUSE(8, "attn_decode: cannot get %zu bytes of shared memory", smem);
  }
  const int G = H / K;
  dim3 grid(n_splits, K * ((G + HEADS - 1) / HEADS), n_seqs);
  RL_LAUNCH_CHECK(rl_launch(kern, grid, 32, smem, stream, q, q_stride, k_pages, v_pages, block_table, table_width, seq_len,
                            part_o, part_ml, H, K, hd, window, scale * 1.4426950408889634f, n_splits));
  dim3 grid2(H, n_seqs);
  RL_LAUNCH_CHECK(rl_launch(attn_decode_merge_kernel, grid2, 128, 0, stream, (const float*)part_o, (const float*)part_ml,
                            out, out_stride, H, hd, n_splits));
  return 0;
}

template <int HD>
static int launch_decode(const bf16* q, int q_stride, const bf16* k_pages, const bf16* v_pages,
                         const int* block_table, int table_width, const int* seq_len, float* part_o,
                         float* part_ml, bf16* out, int out_stride, int n_seqs, int H, int K, int hd, int window,
                         float scale, int n_splits, cudaStream_t stream) {
  // Three stages (measured best at batch 8 and 64 once the splits are chosen to fill the GPU once);
  // RL_ATTN_STAGES=2 in the environment selects two, for measurements.
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("RL_ATTN_STAGES");
    forced = e ? atoi(e) : 0;
  }
  const int stages = forced == 2 ? 2 : 3;
  if (stages == 2)
    return launch_decode_stages<HD, 2>(q, q_stride, k_pages, v_pages, block_table, table_width, seq_len, part_o, part_ml,
                                       out, out_stride, n_seqs, H, K, hd, window, scale, n_splits, stream);
  return launch_decode_stages<HD, 3>(q, q_stride, k_pages, v_pages, block_table, table_width, seq_len, part_o, part_ml,
                                     out, out_stride, n_seqs, H, K, hd, window, scale, n_splits, stream);
}

// Scratch needed, in floats: n_seqs * H * n_splits * (hd + 2); the caller passes part_o of
// n_seqs*H*n_splits*hd floats and part_ml of n_seqs*H*n_splits*2.
RL_API int rl_attn_decode(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages,
                          const int* block_table, int table_width, const int* seq_len, float* part_o,
                          float* part_ml, void* out, int out_stride, int n_seqs, int H, int K, int hd,
                          int page_size, int window, float scale, int n_splits, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || K <= 0 || hd <= 0) RL_REFUSE(1, "attn_decode: S=%d H=%d K=%d hd=%d", n_seqs, H, K, hd);
  if (H % K) RL_REFUSE(2, "attn_decode: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != PAGE) RL_REFUSE(3, "attn_decode: page size %d, this kernel is built for %d", page_size, PAGE);
  if (dtype != RL_BF16) RL_REFUSE(4, "attn_decode: bfloat16 only (32-bit runs use attn_generic), got dtype %d", dtype);
  if (hd % 8) RL_REFUSE(9, "attn_decode: head size %d is not a multiple of 8", hd);
  if (q_stride % 8) RL_REFUSE(9, "attn_decode: query row stride %d breaks 16-byte alignment", q_stride);
  if (n_splits <= 0 || n_splits > 64 || n_seqs > 65535) RL_REFUSE(5, "attn_decode: splits=%d (1..64) seqs=%d", n_splits, n_seqs);
  if (window < 0) RL_REFUSE(6, "attn_decode: negative window");
  const bf16* qq = (const bf16*)q;
  const bf16* kp = (const bf16*)k_pages;
  const bf16* vp = (const bf16*)v_pages;
  bf16* oo = (bf16*)out;
#define RL_DECODE(HDV)                                                                                              \
  return launch_decode<HDV>(qq, q_stride, kp, vp, block_table, table_width, seq_len, part_o, part_ml, oo, out_stride, \
                            n_seqs, H, K, hd, window, scale, n_splits, stream)
  if (hd <= 32) RL_DECODE(32);
  if (hd <= 64) RL_DECODE(64);
  if (hd <= 128) RL_DECODE(128);
  if (hd <= 256) RL_DECODE(256);
#undef RL_DECODE
  RL_REFUSE(10, "attn_decode: head size %d exceeds 256", hd);
}

// ------------------------------------------------------------------ the same, with built-in scratch
// See attention_decode_static.h for what this is for and what its limits are.
#include "attention_decode_static.h"

// The split partials of rl_attn_decode_static live here.  In host code this name is only a handle
// for the runtime: the address a kernel can use is asked for with cudaGetSymbolAddress below.
static __device__ __align__(256) float rl_static_scratch[RL_ATTN_DECODE_STATIC_FLOATS];

#define RL_STATIC_MAX_DEVICES 64
static float* rl_static_scratch_addr[RL_STATIC_MAX_DEVICES] = {nullptr};

RL_API int rl_attn_decode_static(const void* q, int dtype, int q_stride, const void* k_pages, const void* v_pages,
                                 const int* block_table, int table_width, const int* seq_len, void* out,
                                 int out_stride, int n_seqs, int H, int K, int hd, int page_size, int window,
                                 float scale, int n_splits, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || hd <= 0 || n_splits <= 0)
    RL_REFUSE(1, "attn_decode_static: S=%d H=%d hd=%d splits=%d", n_seqs, H, hd, n_splits);
  const unsigned long long need = (unsigned long long)n_seqs * H * n_splits * (hd + 2);
  if (need > RL_ATTN_DECODE_STATIC_FLOATS)
    RL_REFUSE(11, "attn_decode_static: %d sequences x %d heads x %d splits x (%d + 2) = %llu floats of scratch, "
              "the built-in array holds %u; use fewer splits or rl_attn_decode with scratch of your own",
              n_seqs, H, n_splits, hd, need, (unsigned)RL_ATTN_DECODE_STATIC_FLOATS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= RL_STATIC_MAX_DEVICES)
    RL_REFUSE(12, "attn_decode_static: cannot tell the current device (%s)", cudaGetErrorString(e));
  if (rl_static_scratch_addr[dev] == nullptr) {
    // once per device, with that device current: the array's address on this GPU
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, rl_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      RL_REFUSE(13, "attn_decode_static: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
    rl_static_scratch_addr[dev] = p;
  }
  float* part_o = rl_static_scratch_addr[dev];
  float* part_ml = part_o + (size_t)n_seqs * H * n_splits * hd;
  return rl_attn_decode(q, dtype, q_stride, k_pages, v_pages, block_table, table_width, seq_len, part_o, part_ml, out,
                        out_stride, n_seqs, H, K, hd, page_size, window, scale, n_splits, stream);
}
