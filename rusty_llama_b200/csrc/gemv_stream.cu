// Matrix products of the decode step in bfloat16, out[M, N] = x[M, K] . w[N, K]^T for M <= 16,
// as a persistent kernel that keeps the copy engine busy: every weight is read from HBM once, and
// what limits the step is how many bytes are in flight, so the weights never pass through registers
// on their way in.  Counterpart of the reference's warp-per-row GEMV family
// (src/backend/cuda.rs:354-442).
//
// Work: the matrix is cut into items of 8 weight rows x one slice of k (at most 4096, or 5120 when k is longer than 4096; the whole of
// k unless the caller asks for partial sums); the items, slice by slice, are dealt out to one block
// per SM in contiguous, equally long ranges.  In a block
//   warp 16 (one lane)  copies stage after stage of weights, 8 rows x 1024 k = 16 KB each, into a
//                       ring of shared memory (13 stages, about 200 KB in flight per SM), each stage
//                       with an mbarrier that counts its bytes.  A stage is ONE tensor copy: the
//                       weight matrix is described to TMA as [row][k / 64][64 k], so that a box of
//                       8 x 16 x 64 is eight rows of 1024 k (copies of a row's 2 KB at a time were
//                       measured at 2.7 TB/s over the GPU: the copy engine wants large requests).
//                       The weights depend on no other kernel, so the copies start before the
//                       programmatic-dependency wait.
//   warps 0-15          hold the activations of the slice in registers for the whole range of items:
//                       warp w owns the 32-wide k blocks w and w + 16 of every stage.  The
//                       activations are the A operand of mma.sync.m16n8k16 (16 batch rows x 16 k),
//                       the weights the B operand (16 k x 8 features), 32-bit accumulators.  A lane
//                       reads 16 contiguous bytes of a row and uses them as its k elements of two
//                       consecutive MMAs; both operands follow the same rule, so the sum over k is
//                       unchanged.  Per stage a warp issues two 16-byte shared-memory loads and
//                       four MMAs into four independent accumulators.
//   warps 17-20         At the end of an item the sixteen warps leave their partial sums in one of two
//                       buffers of shared memory and go on with the next item at once; these four
//                       warps add them in warp order (no atomics, the same bits every run) and
//                       store the 16 x 8 results: as they are, or through SwiGLU when the rows
//                       alternate gate and up, or as one of k_slices partial results.  (With the
//                       sum done by the product warps themselves, every item cost them about half
//                       a microsecond of waiting for one another.)
// An RMSNorm between two such products can be folded into them (up to 8 rows).  The norm is
// y = x * w / sqrt(mean(x^2) + eps): the product BEFORE it (whose sums go into the residual stream x) adds
// them to x where it stores, writes x * w in bfloat16 beside it and leaves each block's share of the rows'
// sums of squares; the product AFTER it takes x * w as its activations and multiplies its 32-bit sums by the
// row's 1 / sqrt(...) before they are stored or go through the activation.  A row's scale is a scalar, so
// scaling the sums is scaling the activations; the kernel between the two products, with its pass over the
// stream and its two boundaries, is gone.
// Every wait is bounded: on expiry a code goes to status[0] and the block drains.
#include "tc_common.cuh"

RL_DEFINE_ERROR_TEXT()

#define CONSUMER_WARPS 16
#define STORE_WARPS 4
#define NUM_THREADS ((CONSUMER_WARPS + 1 + STORE_WARPS) * 32)
#define UNIT_ROWS 8
#define KC 1024                           // k per stage
#define STAGE_BYTES (UNIT_ROWS * KC * 2)  // [8 rows][16 blocks of 64 k][128 bytes, swizzled]
// k per slice: a warp keeps a slice's activations in registers, one 16-byte fragment per 512 k and row half.  Two
// builds of the kernel: slices of up to 4096 (four stages), and of up to 5120 (five stages) for products whose k
// is longer than 4096, which then come in fewer slices or, up to 5120, in one (the 13B sizes' width): with five
// stages' worth of fragments the compiler is one register short, and the products of k <= 4096 measured 1 % slower.
#define MAX_SLICE 5120
#define SHORT_SLICE 4096
#define KB_PER_WARP (KC / 32 / CONSUMER_WARPS)   // 2
#define STAGES 13
#define MAX_M 16
#define RED_BYTES (2 * CONSUMER_WARPS * 32 * 16)
#define SMALL_BYTES 1024
#define SMEM_BYTES (STAGES * STAGE_BYTES + RED_BYTES + SMALL_BYTES)
static_assert(SMEM_BYTES <= 227 * 1024, "more shared memory than a block can have");

struct StreamBarriers {
  uint64_t full[STAGES], empty[STAGES];
  uint64_t red_full[2], red_free[2];
  int abort_flag;
  float row_scale[8];  // (a folded norm after this product) 1 / sqrt(mean(x^2) + eps) per row
};

// A norm folded into this product (see the header); all pointers null: none.
struct Fold {
  // the norm comes BEFORE this product: its rows' sums of squares as [scale_blocks][8] shares, the row length
  // they were taken over, eps; the activations are x * w already
  const float* sumsq_in;
  int scale_blocks, norm_k;
  float eps;
  // the norm comes AFTER this product, whose sums belong to the residual stream: resid[m, n] += sum (32-bit, in
  // place), xw[m, n] = bfloat16(resid[m, n] * next_w[n]), sumsq_out[block][m] = the block's share of sum(resid^2)
  float* resid;
  const void* next_w;
  bf16* xw;
  float* sumsq_out;
  int resid_ld, xw_ld, next_w_f32;
};
static_assert(sizeof(StreamBarriers) <= SMALL_BYTES, "barriers must fit their area");

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <typename TO>
__device__ __forceinline__ void store_out(TO* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// slice_len: k per slice, a multiple of KC and at most MAX_SLICE (the last slice may be shorter);
// units = ceil(N / 8); items = units * slices, numbered slice by slice.  HI: more than 8 batch rows.
template <typename TO, bool SWIGLU, bool HI, int SLICE_STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemv_stream_kernel(const bf16* __restrict__ x, int ldx, const __grid_constant__ CUtensorMap map_w, TO* __restrict__ out, int ldo,
                   int M, int N, int K, int slice_len, int units, int items, int* __restrict__ status, int test_role,
                   uint32_t test_ns, const Fold fold) {
  // all shared memory is dynamic, so that the ring starts at the block's first byte (1024-byte
  // aligned, as the 128-byte swizzle needs)
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* ring = smem;                                                       // [STAGES][8][16][128 bytes]
  float4* red = reinterpret_cast<float4*>(ring + (size_t)STAGES * STAGE_BYTES);     // [2][warps][32]
  StreamBarriers& bars = *reinterpret_cast<StreamBarriers*>(reinterpret_cast<unsigned char*>(red) + RED_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // uniform over the block; nothing has been set up yet
    if (threadIdx.x == 0) give_up_code(status, 36);
    return;
  }
  const WaitCtl ctl = {&bars.abort_flag, test_role, test_ns};

  pdl_trigger();
  if (threadIdx.x == 32) rl_trace_event(1);  // (profiling aid, see common.cuh) block 0 is running
  if (threadIdx.x == CONSUMER_WARPS * 32)  // the copying lane: have the tensor map on its way before the barriers are set up
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
  int issued = 0;  // (the copying lane) stages whose copies were started
  const int first_item = (int)((long long)blockIdx.x * items / gridDim.x);
  const int end_item = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&bars.full[i], 1);
      mbar_init(&bars.empty[i], CONSUMER_WARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.red_full[i], CONSUMER_WARPS);
      mbar_init(&bars.red_free[i], STORE_WARPS);
    }
    bars.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == CONSUMER_WARPS) {
    // ---------------- copies
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      const uint32_t ring_addr = smem_u32(ring);
      const uint32_t full0 = smem_u32(&bars.full[0]);
      int it = 0;
      uint32_t st = 0, parity = 1, dst = ring_addr;  // the stage of copy `it`; the parity of its `empty` barrier once the ring has gone round
      int slice = first_item / units, unit = first_item - slice * units;
      bool ok = true;
      for (int item = first_item; item < end_item && ok; ++item) {
        const int kbeg = slice * slice_len, klen = min(slice_len, K - kbeg);
        for (int k0 = 0; k0 < klen; k0 += KC, ++it) {
          // (the wait looks at the abort flag itself when it has to wait; the copies of the first round, which
          // need no wait, are issued whatever the other roles do, and the drain waits for them)
          if (it >= STAGES && !mbar_wait_role(&bars.empty[st], parity, ctl, 32)) {
            give_up_code(status, 32);
            bars.abort_flag = 1;
            ok = false;
            break;
          }
          // rows past N and k past K arrive as zeros and count like the rest
          mbar_expect_tx_s(full0 + 8 * st, STAGE_BYTES);
          tma_load_3d(dst, &map_w, full0 + 8 * st, 0, (kbeg + k0) >> 6, unit * UNIT_ROWS, pol_w);
          if (it == 0) rl_trace_event(2);            // first copy issued
          if (it == STAGES - 1) rl_trace_event(3);   // the ring is full of requests
          dst += STAGE_BYTES;
          if (++st == STAGES) {
            st = 0;
            dst = ring_addr;
            parity ^= 1;
          }
        }
        if (++unit == units) {
          unit = 0;
          ++slice;
        }
      }
      rl_trace_event(7);  // last copy issued
      issued = it;
    }
  } else if (warp > CONSUMER_WARPS) {
    // ---------------- sums and stores
    const int e = threadIdx.x - (CONSUMER_WARPS + 1) * 32;  // 0..127
    pdl_wait();  // the kernel before this one may still read the output buffer
    float scale = 1.0f;  // (a folded norm before this product) this thread's row's 1 / sqrt(mean(x^2) + eps)
    if (fold.sumsq_in != nullptr) {
      // 8 rows x 16 threads: thread (m, t) adds the shares of blocks t, t + 16, ...; the sixteen partial sums of a
      // row meet by shuffles in a fixed order, so every block computes the same bits
      const int m = e >> 4, t = e & 15;
      float part = 0.f;
      for (int b = t; b < fold.scale_blocks; b += 16) part += __ldcg(fold.sumsq_in + (size_t)b * 8 + m);
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (t == 0) bars.row_scale[m] = 1.0f / sqrtf(part / (float)fold.norm_k + fold.eps);
      asm volatile("bar.sync 3, %0;" ::"n"(STORE_WARPS * 32) : "memory");
      scale = bars.row_scale[SWIGLU ? ((e >> 1) >> 2) & 7 : ((e >> 2) >> 2)];
    }
    // (a folded norm after this product) the stream's old values and the norm's weights at this thread's place in the
    // block's first items, asked for before the sums are waited for
    float x_old[4] = {0.f, 0.f, 0.f, 0.f}, w_next[4] = {0.f, 0.f, 0.f, 0.f};
    float ss = 0.f;
    if (!SWIGLU && fold.resid != nullptr) {
      const int l = e >> 2, c = e & 3;
      const int m = (l >> 2) + 8 * (c >> 1);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int item = first_item + i;
        const int n = (item % units) * UNIT_ROWS + 2 * (l & 3) + (c & 1);
        if (item < end_item && m < M && n < N) {
          x_old[i] = __ldcg(fold.resid + (size_t)m * fold.resid_ld + n);
          w_next[i] = fold.next_w_f32 ? __ldg(reinterpret_cast<const float*>(fold.next_w) + n)
                                      : __bfloat162float(reinterpret_cast<const bf16*>(fold.next_w)[n]);
        }
      }
    }
    int done_items = 0;
    for (int item = first_item; item < end_item; ++item, ++done_items) {
      const int slice = item / units, unit = item - slice * units;
      const int buf = done_items & 1;
      if (!mbar_wait_role(&bars.red_full[buf], (done_items >> 1) & 1, ctl, 35)) {
        if (lane == 0) {
          give_up_code(status, 35);
          bars.abort_flag = 1;
        }
        break;
      }
      if (*(volatile int*)&bars.abort_flag) break;
      const float* red_f = reinterpret_cast<const float*>(red + buf * (CONSUMER_WARPS * 32));
      TO* out_slice = out + (size_t)slice * M * ldo;
      if (SWIGLU) {
        if (e < 64) {
          const int l = e >> 1, hi = e & 1;
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int wq = 0; wq < CONSUMER_WARPS; ++wq) {
            gate += red_f[(wq * 32 + l) * 4 + 2 * hi];
            up += red_f[(wq * 32 + l) * 4 + 2 * hi + 1];
          }
          gate *= scale;
          up *= scale;
          const int m = (l >> 2) + 8 * hi, col = unit * (UNIT_ROWS / 2) + (l & 3);
          if (m < M && col < (N >> 1)) store_out<TO>(out_slice + (size_t)m * ldo + col, gate * (1.0f / (1.0f + expf(-gate))) * up);
        }
      } else {
        const int l = e >> 2, c = e & 3;
        float sum = 0.f;
#pragma unroll
        for (int wq = 0; wq < CONSUMER_WARPS; ++wq) sum += red_f[(wq * 32 + l) * 4 + c];
        sum *= scale;
        const int m = (l >> 2) + 8 * (c >> 1), n = unit * UNIT_ROWS + 2 * (l & 3) + (c & 1);
        if (m < M && n < N) {
          if (fold.resid != nullptr) {
            float* px = fold.resid + (size_t)m * fold.resid_ld + n;
            float old, wn;
            if (done_items < 4) {
              old = done_items == 0 ? x_old[0] : done_items == 1 ? x_old[1] : done_items == 2 ? x_old[2] : x_old[3];
              wn = done_items == 0 ? w_next[0] : done_items == 1 ? w_next[1] : done_items == 2 ? w_next[2] : w_next[3];
            } else {
              old = __ldcg(px);
              wn = fold.next_w_f32 ? __ldg(reinterpret_cast<const float*>(fold.next_w) + n) : __bfloat162float(reinterpret_cast<const bf16*>(fold.next_w)[n]);
            }
            const float v = old + sum;
            *px = v;
            fold.xw[(size_t)m * fold.xw_ld + n] = __float2bfloat16_rn(v * wn);
            ss += v * v;
          } else {
            store_out<TO>(out_slice + (size_t)m * ldo + n, sum);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.red_free[buf]);
      if (e == 0 && item == end_item - 1) rl_trace_event(8);  // last result stored
    }
    if (!SWIGLU && fold.resid != nullptr) {
      // row m's values sit in the 16 lanes [16 (m & 1), +16) of storing warp m >> 1 (those of rows 8..15 hold zeros):
      // added up in a fixed order, one number per row and block
#pragma unroll
      for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((lane & 15) == 0) fold.sumsq_out[(size_t)blockIdx.x * 8 + 2 * (e >> 5) + (lane >> 4)] = ss;
    }
  } else {
    // ---------------- products
    const int g = lane >> 2, t4 = lane & 3;
    // row g of a stage; k block kb = warp + 16 j lies in 64-k block kb / 2 as 16-byte pieces
    // (kb & 1) * 4 + t4, swizzled by the 64-k block's number
    uint32_t w_off[KB_PER_WARP];
#pragma unroll
    for (int j = 0; j < KB_PER_WARP; ++j) {
      const int kb = warp + CONSUMER_WARPS * j;
      w_off[j] = smem_u32(ring) + g * (KC * 2) + (kb >> 1) * 128 + (((((kb & 1) << 2) | t4) ^ ((kb >> 1) & 7)) << 4);
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 xa[SLICE_STAGES][KB_PER_WARP], xb[HI ? SLICE_STAGES : 1][KB_PER_WARP];
    int loaded_slice = -1, done_items = 0;
    bool ok = true;
    auto give_up = [&](int code) {
      if (lane == 0) {
        give_up_code(status, code);
        bars.abort_flag = 1;
      }
      ok = false;
    };
    pdl_wait();  // the activations are the previous kernel's output, and it may still read ours
    // The loop over stages keeps counters and addresses (no division, no pointer conversion) and leaves the
    // abort flag to the wait that has to wait: every instruction here is paid by every product warp for every
    // stage, and at 16 KB a stage the SM has 640 cycles for all of them together.
    const uint32_t full0 = smem_u32(&bars.full[0]), empty0 = smem_u32(&bars.empty[0]);
    uint32_t st = 0, parity = 0, st_off = 0;  // the stage to consume next, the parity of its `full` barrier, its offset in the ring
    int slice = first_item / units, unit = first_item - slice * units;
    for (int item = first_item; item < end_item && ok; ++item, ++done_items) {
      const int kbeg = slice * slice_len, klen = min(slice_len, K - kbeg);
      if (slice != loaded_slice) {
        // this lane's pieces of the activations of the slice, zero where there is no row or no k
#pragma unroll
        for (int s = 0; s < SLICE_STAGES; ++s)
#pragma unroll
          for (int j = 0; j < KB_PER_WARP; ++j) {
            const int k = s * KC + (warp + CONSUMER_WARPS * j) * 32 + t4 * 8;
            const bool k_ok = k + 8 <= klen;
            xa[s][j] = (k_ok && g < M) ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)g * ldx + kbeg + k)) : zero;
            if (HI) xb[s][j] = (k_ok && g + 8 < M) ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)(g + 8) * ldx + kbeg + k)) : zero;
          }
        loaded_slice = slice;
        if (warp == 0 && lane == 0 && item == first_item) rl_trace_event(4);  // activations requested
      }
      if (++unit == units) {  // (for the next item)
        unit = 0;
        ++slice;
      }
      float acc[2 * KB_PER_WARP][4];
#pragma unroll
      for (int i = 0; i < 2 * KB_PER_WARP; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
      for (int s = 0; s < SLICE_STAGES; ++s) {
        if (s * KC < klen && ok) {
          if (!mbar_wait_role_s(full0 + 8 * st, parity, ctl, 34)) {
            give_up(34);
          } else {
            uint4 b[KB_PER_WARP];
#pragma unroll
            for (int j = 0; j < KB_PER_WARP; ++j) b[j] = lds128(w_off[j] + st_off);
#pragma unroll
            for (int j = 0; j < KB_PER_WARP; ++j) {
              const uint4 lo = xa[s][j], hi = HI ? xb[s][j] : zero;
              mma_bf16_16x8x16(acc[2 * j], lo.x, hi.x, lo.y, hi.y, b[j].x, b[j].y);
              mma_bf16_16x8x16(acc[2 * j + 1], lo.z, hi.z, lo.w, hi.w, b[j].z, b[j].w);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_s(empty0 + 8 * st);
            if (warp == 0 && lane == 0 && item == first_item && s == 0) rl_trace_event(5);  // first stage consumed
            st_off += STAGE_BYTES;
            if (++st == STAGES) {
              st = 0;
              st_off = 0;
              parity ^= 1;
            }
          }
        }
      }
      if (!ok) break;
      // leave the partial sums to the storing warps; the buffer was last read two items ago
      const int buf = done_items & 1;
      if (done_items >= 2 && !mbar_wait_role(&bars.red_free[buf], ((done_items >> 1) - 1) & 1, ctl, 37)) {
        give_up(37);
        break;
      }
      float4 sum4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 2 * KB_PER_WARP; ++i) {
        sum4.x += acc[i][0];
        sum4.y += acc[i][1];
        sum4.z += acc[i][2];
        sum4.w += acc[i][3];
      }
      red[buf * (CONSUMER_WARPS * 32) + warp * 32 + lane] = sum4;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.red_full[buf]);
      if (warp == 0 && lane == 0 && item == end_item - 1) rl_trace_event(6);  // last item's sums handed over
    }
  }
  // Every role is done or has given up.  Nothing may still be writing shared memory when the block ends: if
  // someone gave up, the copying lane waits (bounded, with the long limit) for the copies that were started.
  // It does so here, after the roles have met, because it may have left its loop before another role gave up.
  __syncthreads();
  if (threadIdx.x == CONSUMER_WARPS * 32 && *(volatile int*)&bars.abort_flag)
    for (int j = max(0, issued - STAGES); j < issued; ++j) mbar_wait(&bars.full[j % STAGES], (j / STAGES) & 1);
}

// How the kernel cuts k: k per slice (a multiple of KC, at most MAX_SLICE) and the slices that
// result from at least k_slices of them.
static void plan(int K, int k_slices, int* slice_len, int* slices) {
  const int chunks = (K + KC - 1) / KC;
  const int want = k_slices < chunks ? k_slices : chunks;
  int per = (chunks + want - 1) / want;
  const int longest = (K > SHORT_SLICE ? MAX_SLICE : SHORT_SLICE) / KC;
  if (per > longest) per = longest;
  *slice_len = per * KC;
  *slices = (chunks + per - 1) / per;
}

RL_API int rl_gemv_stream_max_rows() { return MAX_M; }

// The slices of k that a call with these arguments produces (1: a finished result; more: partial
// sums), or 0 when the kernel does not take the shape.  A block keeps a slice of the activations in
// registers, so a slice is at most 5120 long and longer k always comes in slices.
RL_API int rl_gemv_stream_slices(int M, int K, int k_slices) {
  if (M <= 0 || M > MAX_M || K <= 0 || K % 64 || k_slices < 1 || k_slices > 64) return 0;
  int slice_len, slices;
  plan(K, k_slices, &slice_len, &slices);
  return slices;
}

// swiglu != 0: w holds N rows alternating gate and up, out gets N / 2 columns.
// k_slices > 1: out is [slices_used][M][ldo] float32 partial results that the consumer adds up.
// status: one int in device memory, 0 before the call; non-zero afterwards means that a bounded
// wait expired (32 the copying lane, 34 a product warp waiting for weights, 35 a storing warp, 37 a product
// warp waiting for a free sum buffer; 36: shared memory not aligned) and the output is not valid.
// wait_test_role, wait_test_ns: 0, 0 in normal use; a test names one of these codes and a limit in
// nanoseconds, and that role's waits give up after that long instead of a second.
static int launch_gemv_stream(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                              int K, int swiglu, int k_slices, int* slices_used, int* status, int wait_test_role,
                              unsigned int wait_test_ns, const Fold& fold, int* blocks_used, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemv_stream: M=%d N=%d K=%d", M, N, K);
  if (M > MAX_M) RL_REFUSE(2, "gemv_stream: %d rows, this kernel takes at most %d", M, MAX_M);
  if (K % 64 || ldx % 8 || ldw % 8) RL_REFUSE(3, "gemv_stream: K=%d must be a multiple of 64, ldx=%d and ldw=%d of 8", K, ldx, ldw);
  if (((uintptr_t)x | (uintptr_t)w) & 15) RL_REFUSE(9, "gemv_stream: operands must be 16-byte aligned");
  if (swiglu && (N & 1)) RL_REFUSE(6, "gemv_stream: %d gate/up rows are not pairs", N);
  if (k_slices < 1 || k_slices > 64) RL_REFUSE(7, "gemv_stream: %d k slices", k_slices);
  if (ldx < K || ldw < K || ldo < (swiglu ? N / 2 : N)) RL_REFUSE(4, "gemv_stream: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  if (out_dtype != RL_F32 && out_dtype != RL_BF16) RL_REFUSE(5, "gemv_stream: unknown output dtype %d", out_dtype);
  if (status == nullptr) RL_REFUSE(10, "gemv_stream: no status word");
  int slice_len, slices;
  plan(K, k_slices, &slice_len, &slices);
  // (a caller that did not ask for slices has room for one result only)
  if (slices > 1 && (swiglu || out_dtype != RL_F32 || k_slices == 1))
    RL_REFUSE(8, "gemv_stream: k = %d comes in %d slices of at most %d, whose partial sums are float32, cannot go through the activation and have to be asked for (k_slices > 1)", K, slices, MAX_SLICE);
  if (slices_used) *slices_used = slices;
  const int units = (N + UNIT_ROWS - 1) / UNIT_ROWS;
  const long long items_ll = (long long)units * slices;
  if (items_ll > 0x7fffffffLL) RL_REFUSE(12, "gemv_stream: too many work items");
  const int items = (int)items_ll;
  static int sm_count[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) RL_REFUSE(13, "gemv_stream: cannot tell the device");
  if (!sm_count[dev] && cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    RL_REFUSE(13, "gemv_stream: cannot count the SMs");
  const int blocks = items < sm_count[dev] ? items : sm_count[dev];
  if (blocks_used) *blocks_used = blocks;
  if (fold.sumsq_in != nullptr || fold.resid != nullptr) {
    if (M > 8) RL_REFUSE(20, "gemv_stream: a folded norm takes at most 8 rows, got %d", M);
    if (fold.resid != nullptr && (slices != 1 || swiglu)) RL_REFUSE(21, "gemv_stream: sums that go into the stream must be whole (k = %d comes in %d slices) and plain", K, slices);
    if (fold.sumsq_in != nullptr && slices != 1) RL_REFUSE(22, "gemv_stream: a row scale cannot be applied to partial sums (k = %d comes in %d slices)", K, slices);
    if (fold.sumsq_in != nullptr && (fold.scale_blocks <= 0 || fold.norm_k <= 0)) RL_REFUSE(23, "gemv_stream: a row scale needs its shares and the row length");
    if (fold.resid != nullptr && (fold.next_w == nullptr || fold.xw == nullptr || fold.sumsq_out == nullptr || fold.resid_ld < N || fold.xw_ld < N))
      RL_REFUSE(24, "gemv_stream: sums that go into the stream need the stream, the next norm's weight, a place for x * w and one for the sums of squares");
  }
  // the weights as [row][k / 64][64 k]: a box of 8 x 16 x 64 is eight rows of 1024 k
  EncodeTiledFn enc = encode_tiled();
  if (!enc) RL_REFUSE(15, "gemv_stream: cuTensorMapEncodeTiled is not available");
  CUtensorMap map_w;
  {
    cuuint64_t dims[3] = {64, (cuuint64_t)(K / 64), (cuuint64_t)N};
    cuuint64_t strides[2] = {128, (cuuint64_t)ldw * 2};
    cuuint32_t box[3] = {64, KC / 64, UNIT_ROWS};
    cuuint32_t estr[3] = {1, 1, 1};
    if (enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      RL_REFUSE(16, "gemv_stream: cannot describe the weights to TMA");
  }
#define LAUNCH(TO, SW, HI)                                                                                                  \
  do {                                                                                                                      \
    auto kern = slice_len > SHORT_SLICE ? gemv_stream_kernel<TO, SW, HI, MAX_SLICE / KC> : gemv_stream_kernel<TO, SW, HI, SHORT_SLICE / KC>;    \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)                 \
      RL_REFUSE(14, "gemv_stream: cannot get %d bytes of shared memory", SMEM_BYTES);                                       \
    RL_LAUNCH_CHECK(rl_launch<true>(kern, dim3(blocks), NUM_THREADS, SMEM_BYTES, stream, (const bf16*)x, ldx, map_w,       \
                                    (TO*)out, ldo, M, N, K, slice_len, units, items, status, wait_test_role,              \
                                    (uint32_t)wait_test_ns, fold));                                                       \
  } while (0)
#define LAUNCH_ROWS(TO, SW)      \
  do {                           \
    if (M > 8) LAUNCH(TO, SW, true); \
    else LAUNCH(TO, SW, false);  \
  } while (0)
  if (swiglu && out_dtype == RL_F32) LAUNCH_ROWS(float, true);
  else if (swiglu) LAUNCH_ROWS(bf16, true);
  else if (out_dtype == RL_F32) LAUNCH_ROWS(float, false);
  else LAUNCH_ROWS(bf16, false);
#undef LAUNCH_ROWS
#undef LAUNCH
  return 0;
}

RL_API int rl_gemv_stream(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                          int K, int swiglu, int k_slices, int* slices_used, int* status, int wait_test_role,
                          unsigned int wait_test_ns, cudaStream_t stream) {
  const Fold none = {};
  return launch_gemv_stream(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, swiglu, k_slices, slices_used, status, wait_test_role,
                            wait_test_ns, none, nullptr, stream);
}

// Blocks that a call with these sizes runs: the shares of the rows' sums of squares that `rl_gemv_stream_into_stream`
// leaves are that many.
RL_API int rl_gemv_stream_blocks(int N, int K) {
  if (N <= 0 || K <= 0 || K % 64) return 0;
  int slice_len, slices, dev = 0, sms = 0;
  plan(K, 1, &slice_len, &slices);
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  const long long items = (long long)((N + UNIT_ROWS - 1) / UNIT_ROWS) * slices;
  return (int)(items < sms ? items : sms);
}

// The product before a folded RMSNorm (at most 8 rows, k in one slice): resid[M, N] (32-bit, in place) += x . w^T;
// xw[M, N] = bfloat16(resid * next_w) for the product after the norm; sumsq[blocks][8] = each block's share of the
// rows' sum(resid^2), `blocks` being what rl_gemv_stream_blocks(N, K) says.
RL_API int rl_gemv_stream_into_stream(const void* x, int ldx, const void* w, int ldw, float* resid, int resid_ld, const void* next_w,
                                      int next_w_dtype, void* xw, int xw_ld, float* sumsq, int M, int N, int K, int* blocks_used,
                                      int* status, int wait_test_role, unsigned int wait_test_ns, cudaStream_t stream) {
  if (next_w_dtype != RL_F32 && next_w_dtype != RL_BF16) RL_REFUSE(25, "gemv_stream: unknown norm weight dtype %d", next_w_dtype);
  if (((uintptr_t)resid | (uintptr_t)xw) & 3) RL_REFUSE(26, "gemv_stream: the stream and x * w must be aligned to their elements");
  Fold fold = {};
  fold.resid = resid;
  fold.resid_ld = resid_ld;
  fold.next_w = next_w;
  fold.next_w_f32 = next_w_dtype == RL_F32;
  fold.xw = (bf16*)xw;
  fold.xw_ld = xw_ld;
  fold.sumsq_out = sumsq;
  int slices = 0;
  // (the ordinary output is not written in this form; the stream stands in for it in the argument checks)
  return launch_gemv_stream(x, ldx, w, ldw, resid, RL_F32, resid_ld, M, N, K, 0, 1, &slices, status, wait_test_role, wait_test_ns, fold,
                            blocks_used, stream);
}

// The product after a folded RMSNorm (at most 8 rows, k in one slice): as rl_gemv_stream with x = the `xw` left by
// rl_gemv_stream_into_stream, every row's sums multiplied by 1 / sqrt(sum(shares) / norm_k + eps) before they are
// stored or go through the activation.
RL_API int rl_gemv_stream_scaled(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M, int N, int K,
                                 int swiglu, const float* sumsq, int scale_blocks, int norm_k, float eps, int* status,
                                 int wait_test_role, unsigned int wait_test_ns, cudaStream_t stream) {
  Fold fold = {};
  fold.sumsq_in = sumsq;
  fold.scale_blocks = scale_blocks;
  fold.norm_k = norm_k;
  fold.eps = eps;
  int slices = 0;
  return launch_gemv_stream(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, swiglu, 1, &slices, status, wait_test_role, wait_test_ns, fold,
                            nullptr, stream);
}
