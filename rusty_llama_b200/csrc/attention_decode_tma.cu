// Decode attention over the paged cache in bfloat16 for head sizes 64 and 128, the form for small batches
// whose key range is cut into splits: the same mathematics and the same scratch layout as
// `attn_decode` (attention_decode.cu; the reference runs its scalar kernel with a single row here,
// src/backend/cuda.rs:1189-1192), another way of feeding it.
//
// There a block is one warp that copies its own tiles with cp.async, four blocks to an SM, and the
// warp's instruction stream (about a thousand instructions per 16 KB of keys and values) sets the
// pace.  Here a block is four product warps and one copying lane on a ring of whole cache pages:
//   warp 4 (one lane)  TMA: page after page of the split (64 keys: K and V, 32 KB, four tensor
//                      copies straight from the page, 128-byte swizzled) into a three-stage ring;
//   warps 0-3          warp w owns keys 16w .. 16w + 15 of every page: S^T[16 keys x 8 heads] =
//                      K Q^T and O^T[128 x 8 heads] += V^T P^T with mma.sync.m16n8k16, operands by
//                      ldmatrix from the swizzled tiles, online softmax per head in 32-bit
//                      registers, P^T by movmatrix; its own running maximum, sum and output.
// At the end the four warps' partial results are merged in shared memory (in warp order) and the
// block writes one partial (max as a base-2 exponent, sum, unnormalised output) per head to
// scratch; the merge kernel adds the splits in split order.
// Fused position encoding and cache write (fuse > 0): the step's rotary kernel is left out and this
// kernel does its work where the data passes anyway.  The queries are turned by their position's
// angles as they are put into shared memory; the block whose split holds the sequence's last page
// takes the new token's raw key and value from the projection's output, turns the key, puts both
// into its copy of the page in shared memory (the warp that owns that row does it, nobody else
// reads the row) and, for the next steps, into the cache.  Same formulas as rope.cu.
// Two blocks share an SM (99 KB of shared memory each): 192 KB of keys and values in flight per SM,
// eight product warps.  At head size 64 a page's keys and values are half as many bytes, so the ring
// has six stages instead of three and the same bytes are in flight.
//
// Every mbarrier wait is bounded; on expiry a code goes to status[0] and the block drains.
#include "tc_common.cuh"
#include "attention_merge.cuh"

RL_DEFINE_ERROR_TEXT()

#define HEADS 8     // query heads per block (the N of the MMA)
#define PAGE 64     // positions per cache page = keys per tile
#define PRODUCT_WARPS 4
#define NUM_THREADS ((PRODUCT_WARPS + 1) * 32)
#define HALF_BYTES (PAGE * 64 * 2)            // one [64 keys][64 dims] swizzled box: 8 KB
#define MAX_STAGES 6

// What follows from the head size HD (64 or 128): a stage holds a page's keys and then its values, each as
// HD / 64 boxes of 64 dims; the ring has 96 KB whatever the head size.
template <int HD>
struct Shape {
  static constexpr int BOXES = HD / 64;                     // boxes per page of keys (and of values)
  static constexpr int STAGE_BYTES = 2 * BOXES * HALF_BYTES;
  static constexpr int STAGES = 3 * 128 / HD;               // 3 at head size 128, 6 at 64
  static constexpr int Q_STRIDE = HD + 8;                   // bf16 elements per row of the query tile
  static constexpr int O_STRIDE = HD + 4;                   // floats per head in the merge buffer
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + HEADS * Q_STRIDE * 2 + 1024;
  static constexpr int DPL = HD / 32;                       // dims of the new key and value per lane of the patching warp
};

struct DecodeBarriers {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES];
  int abort_flag;
  int last;  // this block is the last of its group's splits to finish
  float cs[64], sn[64];  // cosine and sine of the new position's angles (fused rotary), HD / 2 of each
};
static_assert(sizeof(DecodeBarriers) <= 1024, "the small items must fit their area");

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
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
__device__ __forceinline__ void product_warps_sync() { asm volatile("bar.sync 1, %0;" ::"n"(PRODUCT_WARPS * 32) : "memory"); }

// byte offset, inside a [64 keys][64 dims] box, of the 16-byte piece `piece` (0..7) of row `row`
__device__ __forceinline__ uint32_t swz(int row, int piece) { return (uint32_t)(row * 128 + ((piece ^ (row & 7)) << 4)); }

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 2)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const bf16* __restrict__ q, int q_stride, const int* __restrict__ block_table, int table_width,
                       const int* __restrict__ seq_len, float* __restrict__ part_o, float* __restrict__ part_ml, int H,
                       int K, int window, float scale_log2, int n_splits, int* __restrict__ status,
                       int fuse, bf16* __restrict__ k_pages_w, bf16* __restrict__ v_pages_w,
                       const float* __restrict__ inv_freq, int rot, int interleaved,
                       unsigned int* __restrict__ counters, bf16* __restrict__ out, int out_stride,
                       const float* __restrict__ q_parts, int n_parts, long long part_stride, int test_role,
                       uint32_t test_ns) {
  // all shared memory is dynamic, so that the ring starts at the block's first byte (1024-byte
  // aligned, as the 128-byte swizzle needs)
  constexpr int STAGES = Shape<HD>::STAGES, STAGE_BYTES = Shape<HD>::STAGE_BYTES, BOXES = Shape<HD>::BOXES;
  constexpr int Q_STRIDE = Shape<HD>::Q_STRIDE, O_STRIDE = Shape<HD>::O_STRIDE, DPL = Shape<HD>::DPL;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* ring = smem;
  bf16* q_s = reinterpret_cast<bf16*>(ring + STAGES * STAGE_BYTES);  // [HEADS][Q_STRIDE]
  DecodeBarriers& bars = *reinterpret_cast<DecodeBarriers*>(reinterpret_cast<unsigned char*>(q_s) + HEADS * Q_STRIDE * 2);
  // after the last page the ring is free and holds the four warps' partial results
  float* merge_o = reinterpret_cast<float*>(ring);                      // [warps][HEADS][O_STRIDE]
  float* merge_ml = merge_o + PRODUCT_WARPS * HEADS * O_STRIDE;         // [warps][HEADS][2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = H / K;
  const int groups_per_kv = (G + HEADS - 1) / HEADS;
  const int split = blockIdx.x;
  const int kh = blockIdx.y / groups_per_kv;
  const int g0 = (blockIdx.y - kh * groups_per_kv) * HEADS;
  const int n_heads = min(HEADS, G - g0);
  const int h0 = kh * G + g0;
  const int s = blockIdx.z;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;
  const WaitCtl ctl = {&bars.abort_flag, test_role, test_ns};

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&bars.full[i], 1);
      mbar_init(&bars.empty[i], PRODUCT_WARPS);
    }
    bars.abort_flag = aligned ? 0 : 1;
    if (!aligned) give_up_code(status, 56);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // rows of the query tile past the group's heads are zero
  for (int i = threadIdx.x; i < HEADS * Q_STRIDE / 2; i += NUM_THREADS) reinterpret_cast<uint32_t*>(q_s)[i] = 0u;
  __syncthreads();
  pdl_trigger();

  // Lengths and page tables were uploaded before the step's first kernel; the kernel before this one
  // writes the queries and the newest position's key and value, nothing else that is read here.
  const int kv_len = seq_len[s];
  const int pos = kv_len - 1;
  const int first = (window != 0 && pos + 1 > window) ? pos + 1 - window : 0;
  const int tile_lo = first / PAGE, tile_hi = pos / PAGE;  // inclusive, in pages
  const int n_tiles = tile_hi - tile_lo + 1;
  const int per_split = (n_tiles + n_splits - 1) / n_splits;
  const int my_lo = tile_lo + split * per_split;
  const int my_hi = min(my_lo + per_split - 1, tile_hi);
  const int* table = block_table + (size_t)s * table_width;

  if (warp == PRODUCT_WARPS) {
    // ---------------- copies
    int issued = 0;
    if (lane == 0 && !*(volatile int*)&bars.abort_flag) {
      bool waited = false;
      for (int tile = my_lo; tile <= my_hi; ++tile, ++issued) {
        const int st = issued % STAGES, round = issued / STAGES;
        // pages before the sequence's last one are older than this step: their copies start while the
        // kernel before this one is still running
        if (!waited && (tile == tile_hi || round > 0)) {
          pdl_wait();
          waited = true;
        }
        if (round > 0 && !mbar_wait_role(&bars.empty[st], (round - 1) & 1, ctl, 51)) {
          give_up_code(status, 51);
          bars.abort_flag = 1;
          break;
        }
        if (*(volatile int*)&bars.abort_flag) break;
        const int page = table[tile];
        unsigned char* dst = ring + (size_t)st * STAGE_BYTES;
        mbar_expect_tx(&bars.full[st], STAGE_BYTES);
#pragma unroll
        for (int b = 0; b < BOXES; ++b) {
          tma_load_4d(dst + b * HALF_BYTES, &map_k, &bars.full[st], 64 * b, 0, kh, page);
          tma_load_4d(dst + (BOXES + b) * HALF_BYTES, &map_v, &bars.full[st], 64 * b, 0, kh, page);
        }
      }
    }
    // The copying warp stays until the product warps have left their loop over the pages (they arrive at
    // this barrier without waiting).  Nothing may still be writing shared memory when the block ends, or
    // when the ring is reused for the merge... which only happens when nobody gave up: if someone did, the
    // copying lane now waits (bounded, with the long limit) for the copies that were started.
    __syncwarp();
    asm volatile("bar.sync 2, %0;" ::"n"(NUM_THREADS) : "memory");
    if (lane == 0 && *(volatile int*)&bars.abort_flag)
      for (int j = max(0, issued - STAGES); j < issued; ++j) mbar_wait(&bars.full[j % STAGES], (j / STAGES) & 1);
    return;  // the product warps meet at a barrier of their own
  }

  const int half_rot = rot >> 1;
  if (fuse) {
    // angles of the new token's position, once per block (32-bit product, accurate sincosf); they depend
    // on the position alone, so this runs while the kernel before this one is still at work
    for (int j = threadIdx.x; j < half_rot; j += PRODUCT_WARPS * 32) {
      float sn, cs;
      sincosf((float)pos * inv_freq[j], &sn, &cs);
      bars.cs[j] = cs;
      bars.sn[j] = sn;
    }
  }
  pdl_wait();  // the queries are the previous kernel's output, and it may still read this one's scratch
  // ---------------- products
  const int g = lane >> 2, t4 = lane & 3;
  {
    // this block's queries: HEADS rows of HD values, 16 bytes per thread
    constexpr int PIECES = HD / 8;
    const int r = threadIdx.x / PIECES, piece = threadIdx.x % PIECES;  // 128 threads = 8 (or 16) rows x 16 (or 8) pieces
    if (r < n_heads) {
      const size_t at = (size_t)s * q_stride + (size_t)(h0 + r) * HD + piece * 8;
      if (n_parts == 0) {
        *reinterpret_cast<uint4*>(q_s + (size_t)r * Q_STRIDE + piece * 8) = __ldcg(reinterpret_cast<const uint4*>(q + at));
      } else {
        // the projection came as partial sums over slices of k: add them up (32-bit) and round once
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int p = 0; p < n_parts; ++p) {
          const float4 x0 = __ldcg(reinterpret_cast<const float4*>(q_parts + (size_t)p * part_stride + at));
          const float4 x1 = __ldcg(reinterpret_cast<const float4*>(q_parts + (size_t)p * part_stride + at + 4));
          v[0] += x0.x; v[1] += x0.y; v[2] += x0.z; v[3] += x0.w;
          v[4] += x1.x; v[5] += x1.y; v[6] += x1.z; v[7] += x1.w;
        }
        uint4 packed;
        packed.x = pack_bf16(v[0], v[1]);
        packed.y = pack_bf16(v[2], v[3]);
        packed.z = pack_bf16(v[4], v[5]);
        packed.w = pack_bf16(v[6], v[7]);
        *reinterpret_cast<uint4*>(q_s + (size_t)r * Q_STRIDE + piece * 8) = packed;
      }
    }
  }
  if (fuse) {
    product_warps_sync();  // the queries and the angles are in shared memory
    for (int idx = threadIdx.x; idx < n_heads * half_rot; idx += PRODUCT_WARPS * 32) {
      const int r = idx / half_rot, j = idx - r * half_rot;
      const int d0 = interleaved ? 2 * j : j, d1 = interleaved ? 2 * j + 1 : j + half_rot;
      bf16* row = q_s + (size_t)r * Q_STRIDE;
      const float a = __bfloat162float(row[d0]), b = __bfloat162float(row[d1]);
      row[d0] = __float2bfloat16_rn(a * bars.cs[j] - b * bars.sn[j]);
      row[d1] = __float2bfloat16_rn(a * bars.sn[j] + b * bars.cs[j]);
    }
  }
  product_warps_sync();
  uint32_t qf[HD / 16][2];  // Q^T as B fragments: (dims kk*16 + 2*t4 [+8], head g)
#pragma unroll
  for (int k2 = 0; k2 < HD / 32; ++k2) {
    uint32_t r[4];
    ldmatrix_x4(r, smem_u32(q_s + (size_t)(lane & 7) * Q_STRIDE + k2 * 32 + 8 * (lane >> 3)));
    qf[2 * k2][0] = r[0];
    qf[2 * k2][1] = r[1];
    qf[2 * k2 + 1][0] = r[2];
    qf[2 * k2 + 1][1] = r[3];
  }

  float o_acc[HD / 16][4];  // (dim dt*16 + g [+8], head 2*t4 [+1])
#pragma unroll
  for (int i = 0; i < HD / 16; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // heads 2*t4, 2*t4+1
  float l_run[2] = {0.f, 0.f};              // per-thread partial sums over this thread's keys

  // rows this lane addresses in the ldmatrix calls: K as A operand (16 keys x 16 dims), V transposed
  const int k_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), k_piece = lane >> 4;      // + 2 * kk
  const int v_row = warp * 16 + (lane & 7) + 8 * (lane >> 4), v_piece = (lane >> 3) & 1;      // + 2 * dt
  // The warp that owns the new position's row in the sequence's last page reads the new token's raw key
  // and value now, so that the loads are long done when that page arrives: lane l takes DPL = HD / 32
  // dimensions of both, from DPL l on, one load each (or one per partial sum, all independent).
  const bool patch_here = fuse == 2 && my_lo <= my_hi && my_hi == tile_hi && warp == ((pos & (PAGE - 1)) >> 4);
  float new_k[DPL], new_v[DPL];
#pragma unroll
  for (int e = 0; e < DPL; ++e) new_k[e] = new_v[e] = 0.f;
  if (patch_here) {
    const size_t k_at = (size_t)s * q_stride + (size_t)(H + kh) * HD + DPL * lane, v_at = k_at + (size_t)K * HD;
    if (n_parts == 0) {
      if (DPL == 4) {
        const uint2 kr = __ldcg(reinterpret_cast<const uint2*>(q + k_at)), vr = __ldcg(reinterpret_cast<const uint2*>(q + v_at));
        const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr.x)), k1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr.y));
        const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.x)), v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.y));
        new_k[0] = k0.x; new_k[1] = k0.y; new_k[DPL - 2] = k1.x; new_k[DPL - 1] = k1.y;
        new_v[0] = v0.x; new_v[1] = v0.y; new_v[DPL - 2] = v1.x; new_v[DPL - 1] = v1.y;
      } else {
        const uint32_t kr = __ldcg(reinterpret_cast<const uint32_t*>(q + k_at)), vr = __ldcg(reinterpret_cast<const uint32_t*>(q + v_at));
        const float2 k0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&kr));
        const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr));
        new_k[0] = k0.x; new_k[1] = k0.y;
        new_v[0] = v0.x; new_v[1] = v0.y;
      }
    } else {
      for (int p = 0; p < n_parts; ++p) {
        const float* kp = q_parts + (size_t)p * part_stride + k_at;
        const float* vp = q_parts + (size_t)p * part_stride + v_at;
#pragma unroll
        for (int e = 0; e < DPL; e += 2) {
          const float2 kk2 = __ldcg(reinterpret_cast<const float2*>(kp + e)), vv2 = __ldcg(reinterpret_cast<const float2*>(vp + e));
          new_k[e] += kk2.x; new_k[e + 1] += kk2.y;
          new_v[e] += vv2.x; new_v[e + 1] += vv2.y;
        }
      }
#pragma unroll
      for (int e = 0; e < DPL; ++e) {  // rounded to bfloat16 as the projection would have stored them
        new_k[e] = __bfloat162float(__float2bfloat16_rn(new_k[e]));
        new_v[e] = __bfloat162float(__float2bfloat16_rn(new_v[e]));
      }
    }
  }
  bool ok = true;
  int done = 0;
  for (int tile = my_lo; tile <= my_hi && ok; ++tile, ++done) {
    const int st = done % STAGES;
    if (!mbar_wait_role(&bars.full[st], (done / STAGES) & 1, ctl, 52)) {
      if (lane == 0) {
        give_up_code(status, 52);
        bars.abort_flag = 1;
      }
      ok = false;
      break;
    }
    if (*(volatile int*)&bars.abort_flag) {
      ok = false;
      break;
    }
    const uint32_t k_s = smem_u32(ring) + st * STAGE_BYTES, v_s = k_s + BOXES * HALF_BYTES;
    if (patch_here && tile == tile_hi) {
      // the new token's key and value (read before the loop): the key turned by the position's angles,
      // both into this block's copy of the page and (one block per kv head) into the cache
      const int row = pos & (PAGE - 1);
      const int hq = half_rot / DPL;  // lanes between the two halves of a pair (neighbour layout)
      float o[DPL];
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int d = DPL * lane + e;
        // the partner's raw value: from the lane that holds dimension d + half_rot or d - half_rot
        const float up = __shfl_sync(0xffffffffu, new_k[e], (lane + hq) & 31), dn = __shfl_sync(0xffffffffu, new_k[e], (lane - hq) & 31);
        float r = new_k[e];
        if (d < rot) {
          if (interleaved) {
            const int j = d >> 1;
            const float other = new_k[e ^ 1];
            r = (d & 1) ? other * bars.sn[j] + new_k[e] * bars.cs[j] : new_k[e] * bars.cs[j] - other * bars.sn[j];
          } else if (d < half_rot) {
            r = new_k[e] * bars.cs[d] - up * bars.sn[d];
          } else {
            r = dn * bars.sn[d - half_rot] + new_k[e] * bars.cs[d - half_rot];
          }
        }
        o[e] = r;
      }
      const int d0 = DPL * lane;
      const uint32_t in_tile = (d0 >> 6) * HALF_BYTES + swz(row, (d0 & 63) >> 3) + (d0 & 7) * 2;
      unsigned char* k_tile = ring + (size_t)st * STAGE_BYTES;
      const size_t cache_at = (((size_t)table[tile] * K + kh) * PAGE + row) * HD + d0;
      if (DPL == 4) {
        const uint2 k_packed = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[DPL - 2], o[DPL - 1]));
        const uint2 v_packed = make_uint2(pack_bf16(new_v[0], new_v[1]), pack_bf16(new_v[DPL - 2], new_v[DPL - 1]));
        *reinterpret_cast<uint2*>(k_tile + in_tile) = k_packed;
        *reinterpret_cast<uint2*>(k_tile + BOXES * HALF_BYTES + in_tile) = v_packed;
        if (g0 == 0) {
          *reinterpret_cast<uint2*>(k_pages_w + cache_at) = k_packed;
          *reinterpret_cast<uint2*>(v_pages_w + cache_at) = v_packed;
        }
      } else {
        const uint32_t k_packed = pack_bf16(o[0], o[1]), v_packed = pack_bf16(new_v[0], new_v[1]);
        *reinterpret_cast<uint32_t*>(k_tile + in_tile) = k_packed;
        *reinterpret_cast<uint32_t*>(k_tile + BOXES * HALF_BYTES + in_tile) = v_packed;
        if (g0 == 0) {
          *reinterpret_cast<uint32_t*>(k_pages_w + cache_at) = k_packed;
          *reinterpret_cast<uint32_t*>(v_pages_w + cache_at) = v_packed;
        }
      }
      __syncwarp();
    }

    // ---- S^T = K Q^T: this warp's 16 keys x 8 heads
    float s_acc[4] = {0.f, 0.f, 0.f, 0.f};  // (key g [+8], head 2*t4 [+1])
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t a[4];
      ldmatrix_x4(a, k_s + (kk >> 2) * HALF_BYTES + swz(k_row, ((kk & 3) << 1) | k_piece));
      mma_bf16(s_acc, a, qf[kk][0], qf[kk][1]);
    }

    // ---- mask by position, scale to base-2 exponents, online softmax per head (column)
    const int key0 = tile * PAGE + warp * 16;
    const bool need_mask = key0 < first || key0 + 15 > pos;
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v = s_acc[e] * scale_log2;
      if (need_mask) {
        const int key = key0 + g + 8 * (e >> 1);
        if (key < first || key > pos) v = -INFINITY;
      }
      s_acc[e] = v;
      tmax[e & 1] = fmaxf(tmax[e & 1], v);
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float mx = tmax[j];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[j], mx);
      m_use[j] = (m_new == -INFINITY) ? 0.f : m_new;  // a warp whose 16 keys are all masked so far
      alpha[j] = exp2f(m_run[j] - m_use[j]);
      m_run[j] = m_new;
      l_run[j] *= alpha[j];
    }
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      p[e] = exp2f(s_acc[e] - m_use[e & 1]);
      l_run[e & 1] += p[e];
    }
    const uint32_t pb0 = movmatrix_trans(pack_bf16(p[0], p[1]));  // keys 0..7 of the warp's 16
    const uint32_t pb1 = movmatrix_trans(pack_bf16(p[2], p[3]));  // keys 8..15
#pragma unroll
    for (int i = 0; i < HD / 16; ++i) {
      o_acc[i][0] *= alpha[0];
      o_acc[i][1] *= alpha[1];
      o_acc[i][2] *= alpha[0];
      o_acc[i][3] *= alpha[1];
    }

    // ---- O^T += V^T P^T: head size (16-row tiles) x 8 heads over the warp's 16 keys
#pragma unroll
    for (int dt = 0; dt < HD / 16; ++dt) {
      uint32_t a[4];
      ldmatrix_x4_trans(a, v_s + (dt >> 2) * HALF_BYTES + swz(v_row, ((dt & 3) << 1) | v_piece));
      mma_bf16(o_acc[dt], a, pb0, pb1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars.empty[st]);
  }

  // ---- the four warps' partial results meet in the ring's memory, which nobody reads any more once
  // every product warp is here (a warp that gave up comes here too)
  asm volatile("bar.arrive 2, %0;" ::"n"(NUM_THREADS) : "memory");  // lets the copying warp go (see there)
  product_warps_sync();
  if (*(volatile int*)&bars.abort_flag) return;  // the same answer for all four warps: nothing changes it after the barrier
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    float l = l_run[j];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    const int head = 2 * t4 + j;
    if (g == 0) {
      merge_ml[(warp * HEADS + head) * 2] = m_run[j];
      merge_ml[(warp * HEADS + head) * 2 + 1] = l;
    }
    float* mo = merge_o + (size_t)(warp * HEADS + head) * O_STRIDE;
#pragma unroll
    for (int dt = 0; dt < HD / 16; ++dt) {
      mo[dt * 16 + g] = o_acc[dt][j];
      mo[dt * 16 + g + 8] = o_acc[dt][2 + j];
    }
  }
  product_warps_sync();
  {
    const int head = threadIdx.x >> 4, d0 = threadIdx.x & 15;  // 128 threads = 8 heads x 16 lanes of dims
    if (head < n_heads) {
      float mw[PRODUCT_WARPS], M = -INFINITY;
#pragma unroll
      for (int w = 0; w < PRODUCT_WARPS; ++w) {
        mw[w] = merge_ml[(w * HEADS + head) * 2];
        M = fmaxf(M, mw[w]);
      }
      float l = 0.f;
#pragma unroll
      for (int w = 0; w < PRODUCT_WARPS; ++w) {
        mw[w] = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - M);
        l += mw[w] * merge_ml[(w * HEADS + head) * 2 + 1];
      }
      if (counters != nullptr && n_splits == 1) {
        // the only split: this is the result
        const float inv = 1.0f / l;
        bf16* orow = out + (size_t)s * out_stride + (size_t)(h0 + head) * HD;
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
          const int d = d0 + 16 * j;
          float o = 0.f;
#pragma unroll
          for (int w = 0; w < PRODUCT_WARPS; ++w) o += mw[w] * merge_o[(size_t)(w * HEADS + head) * O_STRIDE + d];
          orow[d] = __float2bfloat16_rn(o * inv);
        }
      } else {
        const size_t slot = ((size_t)s * H + h0 + head) * n_splits + split;
        if (d0 == 0) {
          part_ml[slot * 2] = M;  // -inf when the split held no key at all (an empty split)
          part_ml[slot * 2 + 1] = l;
        }
        float* po = part_o + slot * HD;
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
          const int d = d0 + 16 * j;
          float o = 0.f;
#pragma unroll
          for (int w = 0; w < PRODUCT_WARPS; ++w) o += mw[w] * merge_o[(size_t)(w * HEADS + head) * O_STRIDE + d];
          po[d] = o;
        }
      }
    }
  }
  if (counters == nullptr || n_splits == 1) return;

  // ---- the block that finishes last among the splits of its (sequence, head group) adds them up, in
  // split order, exactly as the merge kernel would: out = sum_i 2^(m_i - M) o_i / sum_i 2^(m_i - M) l_i.
  // Its partial results are made visible before the ticket is drawn, and the last one reads the others'
  // only after it has seen every ticket drawn.
  __threadfence();
  product_warps_sync();
  unsigned int* counter = counters + (size_t)s * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) bars.last = (atomicAdd(counter, 1u) == (unsigned int)n_splits - 1u) ? 1 : 0;
  product_warps_sync();
  if (!bars.last) return;
  __threadfence();
  {
    const int head = threadIdx.x >> 4, d0 = threadIdx.x & 15;
    if (head < n_heads) {
      const float* ml = part_ml + ((size_t)s * H + h0 + head) * n_splits * 2;
      const float* po = part_o + ((size_t)s * H + h0 + head) * n_splits * HD;
      float M = -INFINITY;
      for (int i = 0; i < n_splits; ++i) M = fmaxf(M, __ldcg(ml + 2 * i));
      float denom = 0.f;
      for (int i = 0; i < n_splits; ++i) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(ml + 2 * i));
        denom += ((v.x == -INFINITY) ? 0.f : exp2f(v.x - M)) * v.y;
      }
      const float inv = 1.0f / denom;
      float o[HD / 16];
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) o[j] = 0.f;
      for (int i = 0; i < n_splits; ++i) {
        const float mi = __ldcg(ml + 2 * i);
        const float wi = ((mi == -INFINITY) ? 0.f : exp2f(mi - M)) * inv;
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) o[j] += wi * __ldcg(po + (size_t)i * HD + d0 + 16 * j);
      }
      bf16* orow = out + (size_t)s * out_stride + (size_t)(h0 + head) * HD;
#pragma unroll
      for (int j = 0; j < HD / 16; ++j) orow[d0 + 16 * j] = __float2bfloat16_rn(o[j]);
    }
  }
  if (threadIdx.x == 0) *counter = 0u;  // ready for the next call
}

// ------------------------------------------------------------------ host side
// Head sizes this kernel is built for: 64 and 128 (1 if `hd` is one of them).
RL_API int rl_attn_decode_tma_takes(int hd) { return hd == 64 || hd == 128; }

// Same arguments as rl_attn_decode (scratch: part_o of n_seqs*H*n_splits*hd floats, part_ml of
// n_seqs*H*n_splits*2), plus the number of cache pages and a status word: one int in device memory,
// 0 before the call; non-zero afterwards means that a bounded wait expired (51 the copying lane, 52 a
// product warp; 56: shared memory not aligned) and the output is not valid.
// fuse: 0 = the queries are already position-encoded and the new key and value already in the cache;
// 1 = turn the queries here (the cache is another layer's and complete); 2 = turn the queries, and take
// the new token's key and value from q's rows (keys at column H * hd, values at (H + K) * hd), turn the
// key and store both (k_pages and v_pages are written).  inv_freq: rot / 2 angles per position; rot = 0
// means no rotation at all (then fuse = 2 only stores).
// q_parts (with fuse > 0 only): the projection's rows as n_parts float32 partial sums, part p at
// q_parts + p * part_stride, rows of q_stride values; q is then not read.
// counters: null, or n_seqs * (K * groups of 8 heads) zeros in device memory: the splits are then added
// up by the block that finishes last (no merge kernel is launched) and the counters are zeros again
// when the kernel ends.
// wait_test_role, wait_test_ns: 0, 0 in normal use; a test names 51 or 52 and a limit in nanoseconds, and
// that role's waits give up after that long instead of a second.
template <int HD>
static int launch_decode_tma(const void* q, int q_stride, const void* k_pages, const void* v_pages, int n_pages,
                             const int* block_table, int table_width, const int* seq_len, float* part_o, float* part_ml,
                             void* out, int out_stride, int n_seqs, int H, int K, int window, float scale, int n_splits,
                             int* status, int fuse, const float* inv_freq, int rot, int interleaved, unsigned int* counters,
                             const float* q_parts, int n_parts, long long part_stride, int wait_test_role,
                             unsigned int wait_test_ns, cudaStream_t stream) {
  CUtensorMap map_k, map_v;
  if (make_page_map(&map_k, k_pages, n_pages, K, PAGE, HD, PAGE) || make_page_map(&map_v, v_pages, n_pages, K, PAGE, HD, PAGE))
    RL_REFUSE(10, "attn_decode_tma: cannot describe the cache pages to TMA");
  auto kern = attn_decode_tma_kernel<HD>;
  constexpr int smem = Shape<HD>::SMEM_BYTES;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    RL_REFUSE(11, "attn_decode_tma: cannot get %d bytes of shared memory", smem);
  const int G = H / K;
  dim3 grid(n_splits, K * ((G + HEADS - 1) / HEADS), n_seqs);
  RL_LAUNCH_CHECK(rl_launch(kern, grid, NUM_THREADS, smem, stream, map_k, map_v, (const bf16*)q, q_stride, block_table,
                            table_width, seq_len, part_o, part_ml, H, K, window, scale * 1.4426950408889634f, n_splits, status,
                            fuse, (bf16*)const_cast<void*>(k_pages), (bf16*)const_cast<void*>(v_pages), inv_freq, fuse ? rot : 0,
                            interleaved, counters, (bf16*)out, out_stride, q_parts, n_parts, part_stride, wait_test_role,
                            (uint32_t)wait_test_ns));
  if (counters != nullptr) return 0;
  dim3 grid2(H, n_seqs);
  RL_LAUNCH_CHECK(rl_launch(attn_decode_merge_kernel, grid2, 128, 0, stream, (const float*)part_o, (const float*)part_ml,
                            (bf16*)out, out_stride, H, HD, n_splits));
  return 0;
}

RL_API int rl_attn_decode_tma(const void* q, int q_stride, const void* k_pages, const void* v_pages, int n_pages,
                              const int* block_table, int table_width, const int* seq_len, float* part_o, float* part_ml,
                              void* out, int out_stride, int n_seqs, int H, int K, int hd, int page_size, int window,
                              float scale, int n_splits, int* status, int fuse, const float* inv_freq, int rot,
                              int interleaved, unsigned int* counters, const float* q_parts, int n_parts,
                              long long part_stride, int wait_test_role, unsigned int wait_test_ns, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0 || K <= 0 || n_pages <= 0) RL_REFUSE(1, "attn_decode_tma: S=%d H=%d K=%d pages=%d", n_seqs, H, K, n_pages);
  if (!rl_attn_decode_tma_takes(hd)) RL_REFUSE(2, "attn_decode_tma: head size %d, this kernel is built for 64 and 128", hd);
  if (H % K) RL_REFUSE(3, "attn_decode_tma: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != PAGE) RL_REFUSE(4, "attn_decode_tma: page size %d, this kernel is built for %d", page_size, PAGE);
  if (q_stride % 8) RL_REFUSE(5, "attn_decode_tma: query row stride %d breaks 16-byte alignment", q_stride);
  if (((n_parts > 0 ? (uintptr_t)0 : (uintptr_t)q) | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15) RL_REFUSE(6, "attn_decode_tma: operands must be 16-byte aligned");
  if (n_splits <= 0 || n_splits > 64 || n_seqs > 65535) RL_REFUSE(7, "attn_decode_tma: splits=%d (1..64) seqs=%d", n_splits, n_seqs);
  if (window < 0 || status == nullptr || !(scale > 0.f)) RL_REFUSE(8, "attn_decode_tma: bad window or scale, or no status word");
  if (fuse < 0 || fuse > 2 || rot < 0 || rot > hd || (rot & 7) || (fuse && rot > 0 && inv_freq == nullptr))
    RL_REFUSE(12, "attn_decode_tma: fuse=%d with a rotary size of %d (a multiple of 8 up to the head size)%s", fuse, rot, inv_freq ? "" : " and no angles");
  if (n_parts < 0 || n_parts > 64 || (n_parts > 0 && (q_parts == nullptr || fuse == 0 || ((uintptr_t)q_parts & 15) || part_stride % 4 || q_stride % 4)))
    RL_REFUSE(14, "attn_decode_tma: %d partial sums need fuse > 0 and 16-byte aligned rows", n_parts);
  if (fuse == 2 && q_stride < (H + 2 * K) * hd) RL_REFUSE(13, "attn_decode_tma: rows of %d hold no key and value behind %d query heads", q_stride, H);
#define RL_DECODE_TMA(HDV)                                                                                                  \
  return launch_decode_tma<HDV>(q, q_stride, k_pages, v_pages, n_pages, block_table, table_width, seq_len, part_o, part_ml, out, \
                                out_stride, n_seqs, H, K, window, scale, n_splits, status, fuse, inv_freq, rot, interleaved,      \
                                counters, q_parts, n_parts, part_stride, wait_test_role, wait_test_ns, stream)
  if (hd == 64) RL_DECODE_TMA(64);
  RL_DECODE_TMA(128);
#undef RL_DECODE_TMA
}
