// bfloat16 matrix product for prompts on the 5th-generation tensor cores:
//   out[M, N] = x[M, K] . w[N, K]^T,  32-bit accumulation in tensor memory.
// The reference hands these products to cuBLASLt (src/backend/cuda.rs:717-758); this is the
// library's own kernel for the same shapes (M tokens of a prompt step, N output features).
//
// The kernel is persistent: one block per SM walks over 128 x 256 output tiles (tiles that share
// a w tile are neighbours in the walk, so they run at the same time and w is fetched from HBM
// once).  Warp 0 (one lane) is the producer: it asks the TMA unit for 64-wide k slices of the x
// tile (128 rows) and the w tile (256 rows), 128-byte swizzled, into a ring of 4 shared-memory
// stages, and arms each stage's `full` mbarrier with the byte count; it runs ahead across tile
// borders.  Warp 1 (one lane) issues tcgen05.mma (M 128, N 256, K 16, four per slice) on shared-
// memory descriptors of the stage, accumulating in one of two 256-column halves of tensor memory,
// and commits each slice to the stage's `empty` mbarrier, which hands the stage back to the
// producer when the tensor core has read it.  After a tile's last slice a commit arms the half's
// `acc_full`; warps 2..5 then read that half with tcgen05.ld (each warp owns 32 of the 128 lanes
// = rows), round to the output type, store 64-byte row pieces and release the half through
// `acc_empty`, while the tensor core already fills the other half with the next tile.  Rows and
// columns past M, N and K are zero-filled by TMA on the way in and masked on the way out, so any
// M and N work; K and the row strides of x and w must be multiples of 8 (16-byte TMA rows).
//
// Tile width.  With few rows (a decode step of 9 to 128 sequences) the product is a stream of
// weights, and 256-wide tiles may be too few to give every SM one (6144 features: 24 tiles).  The
// launcher then narrows the tiles (`bn`, a multiple of 16 from 16 to 256) so that they fill one wave.
// The stages and accumulators keep their places for 256 columns and a narrower tile uses part of them.
//
// Every wait on an mbarrier is bounded (about one second of polling): on expiry the waiter
// records a code in `status[0]`, the block drains, frees its tensor memory and returns.
#include "tc_common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BM 128
#define BN 256
#define BK 64
#define STAGES 4           // (5 when the rows fit a half tile of activations, see SMALL_A)
#define MAX_STAGES 5
#define UMMA_K 16
#define TMEM_COLS 512  // two accumulators of BN columns
#define NUM_THREADS 192
#define STAGE_A_BYTES (BM * BK * 2)
#define STAGE_B_BYTES (BN * BK * 2)
#define STAGE_BYTES (STAGE_A_BYTES + STAGE_B_BYTES)
#define SMALL_A_ROWS 64
#define SMALL_A_BYTES (SMALL_A_ROWS * BK * 2)

template <typename TO>
__device__ __forceinline__ void store_row32(TO* dst, const uint32_t (&r)[32], int n_valid, bool vec);
template <>
__device__ __forceinline__ void store_row32<bf16>(bf16* dst, const uint32_t (&r)[32], int n_valid, bool vec) {
  if (vec && n_valid >= 32) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
      __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
      __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
      __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
      v.x = *reinterpret_cast<uint32_t*>(&p0);
      v.y = *reinterpret_cast<uint32_t*>(&p1);
      v.z = *reinterpret_cast<uint32_t*>(&p2);
      v.w = *reinterpret_cast<uint32_t*>(&p3);
      d4[i] = v;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < n_valid) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
  }
}
template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const uint32_t (&r)[32], int n_valid, bool vec) {
  if (vec && n_valid >= 32) {
    float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      d4[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                          __uint_as_float(r[4 * i + 3]));
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < n_valid) dst[i] = __uint_as_float(r[i]);
  }
}

// 32 accumulator columns that alternate gate and up -> 16 values silu(gate) * up
template <typename TO>
__device__ __forceinline__ void store_swiglu16(TO* dst, const uint32_t (&r)[32], int n_valid, bool vec) {
  float h[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
    // exp and the division by the hardware's approximations (a few units in the last place of 32 bits,
    // far below the bfloat16 rounding that follows): the accurate forms cost a row's thread about 8 us per
    // tile, which a step with one tile per SM cannot hide behind the next tile's products
    h[i] = __fdividef(g, 1.0f + __expf(-g)) * u;
  }
  if (vec && n_valid >= 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) store4<TO>(dst + 4 * i, h + 4 * i);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n_valid) dst[i] = from_f32<TO>(h[i]);
  }
}

// ------------------------------------------------------------------ the epilogue's way out for bfloat16
// A thread of the epilogue holds a ROW of the accumulator (its lane of tensor memory), so stores straight from
// its registers put 16 bytes into each of 32 different lines per instruction.  For whole groups of columns the
// warp turns its 32 x 64 (or, after SwiGLU, 32 x 32) piece through 4 KB of shared memory instead and writes whole
// 128-byte (64-byte) rows, eight (four) lanes to a row.  Pieces of 16 bytes are swizzled by the row so that
// neither the row-wise writes nor the line-wise reads conflict.
#define OUT_STAGE_BYTES ROW_STAGE_BYTES  // per epilogue warp (pack2 and store_rows64_bf16 live in tc_common.cuh)
// the same for float32 results (partial sums over a slice of k): 32 columns are a row's 128 bytes
__device__ __forceinline__ void store_rows32_f32(float* out_tile, int ldo, int rows_valid, const uint32_t (&r)[32], uint32_t stage, int lane) {
#pragma unroll
  for (int p = 0; p < 8; ++p)
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + ((p ^ (lane & 7)) << 4)), "r"(r[4 * p]), "r"(r[4 * p + 1]),
                 "r"(r[4 * p + 2]), "r"(r[4 * p + 3])
                 : "memory");
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3), pc = lane & 7;
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(stage + rr * 128 + ((pc ^ (rr & 7)) << 4)));
    if (rr < rows_valid) *reinterpret_cast<uint4*>(out_tile + (size_t)rr * ldo + pc * 4) = v;
  }
  __syncwarp();
}
// the same after SwiGLU: 64 accumulator columns (gate and up alternating) -> 32 outputs = 64 bytes a row
__device__ __forceinline__ void store_rows32_swiglu_bf16(bf16* out_tile, int ldo, int rows_valid, const uint32_t (&r0)[32], const uint32_t (&r1)[32],
                                                         uint32_t stage, int lane) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t* r = p < 2 ? r0 : r1;
    const int b = (p & 1) * 16;
    float h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g = __uint_as_float(r[b + 2 * i]), u = __uint_as_float(r[b + 2 * i + 1]);
      h[i] = __fdividef(g, 1.0f + __expf(-g)) * u;  // (as in store_swiglu16)
    }
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 64 + ((p ^ ((lane >> 1) & 3)) << 4)), "r"(pack2(h[0], h[1])),
                 "r"(pack2(h[2], h[3])), "r"(pack2(h[4], h[5])), "r"(pack2(h[6], h[7]))
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int rr = it * 8 + (lane >> 2), pc = lane & 3;
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(stage + rr * 64 + ((pc ^ ((rr >> 1) & 3)) << 4)));
    if (rr < rows_valid) *reinterpret_cast<uint4*>(out_tile + (size_t)rr * ldo + pc * 8) = v;
  }
  __syncwarp();
}

// ------------------------------------------------------------------ the kernel

// SWIGLU: w's rows alternate gate and up (row 2i gate i, row 2i+1 up i); the epilogue writes
// h[m, i] = silu(gate) * up from the 32-bit accumulators, N / 2 columns per row.
// SMALL_A: at most 64 rows (a decode step of 9 to 64 sequences, bound by the weights' bytes).  A block then
// streams 2 MB of weights through four stages of 32 KB at 49 GB/s, well under what an SM can take, so the
// activations' half of a stage shrinks to the 64 rows that exist and a fifth stage takes the room (measured
// at 64 x 28672 x 4096: 43.0 -> 41.0 us).  The MMA still spans 128 rows: its rows 64..127 read the first 8 KB of the
// stage's weights as if they were activations and fill accumulator rows that are never stored.
template <typename TO, bool SWIGLU, bool SMALL_A>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               TO* __restrict__ out, int ldo, int M, int N, int K, int vec_store, int k_splits, int bn,
               int* __restrict__ status, int test_role, uint32_t test_ns) {
  extern __shared__ unsigned char smem_dyn[];
  // the swizzled stages must start on a 1024-byte boundary
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  constexpr int N_STAGES = SMALL_A ? 5 : STAGES;
  constexpr int A_BYTES = SMALL_A ? SMALL_A_BYTES : STAGE_A_BYTES;
  constexpr int STG_BYTES = A_BYTES + STAGE_B_BYTES;
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ __align__(8) uint64_t drain_bar;  // an issuer that gives up waits here for the MMAs it has issued
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const WaitCtl ctl = {&abort_flag, test_role, test_ns};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t issued = 0;  // (the producer's lane) slices whose copies were started
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + bn - 1) / bn;
  const int n_tiles = tiles_m * tiles_n;
  // a unit of work is one output tile and one slice of the k range (k_splits > 1: each slice
  // writes its own partial result, out[slice][M][ldo], and the consumer adds them)
  const int n_units = n_tiles * k_splits;
  const int slices_total = (K + BK - 1) / BK;
  const int slices_per_split = (slices_total + k_splits - 1) / k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < N_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);  // one arrival per epilogue warp
    }
    mbar_init(&drain_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // Barriers and tensor memory are set up.  The weights are no kernel's output, so the producer asks for
  // the first ring of them before the dependency wait (they arrive while the kernel before this one
  // finishes); the activations, and everything the other warps do, come after it.
  pdl_trigger();

  if (warp == 0) {
    // ---------------- producer
    // This lane and the tensor-core issuer's are single threads whose loop bodies are chains of dependent
    // instructions: what one trip costs is what a k slice costs whenever the data is near, and in a prompt it
    // comes close to the tensor core's own 512 cycles per slice.  So the loops keep counters instead of
    // dividing (an integer division by a run-time value measured 40 ns in such a thread), get shared-memory
    // addresses by adding, and look at the abort flag only inside a wait that has to wait (2048 x 6144 x 4096:
    // 87.7 -> 83.2 us).
    if (lane == 0) {
      // the same walk over (unit, k block) twice: at most STAGES steps of it for the early weights, then all of it
      const uint32_t stage0 = smem_u32(stages), full0 = smem_u32(&full_bar[0]);
      const uint32_t tx_bytes = A_BYTES + bn * BK * 2;
      uint32_t early = 0;
      for (int unit = blockIdx.x; unit < n_units && early < N_STAGES; unit += gridDim.x) {
        const int tile = unit % n_tiles, ks = unit / n_tiles;
        const int n0 = (tile / tiles_m) * bn;
        const int kb0 = ks * slices_per_split, kb1 = min(slices_total, kb0 + slices_per_split);
        for (int kb = kb0; kb < kb1 && early < N_STAGES; ++kb, ++early) {
          mbar_expect_tx_s(full0 + 8 * early, tx_bytes);
          tma_load_2d_s(stage0 + early * STG_BYTES + A_BYTES, &map_w, full0 + 8 * early, kb * BK, n0);
        }
      }
      pdl_wait();
      uint32_t it = 0;             // slices requested so far, over all tiles of this block
      uint32_t s = 0, parity = 1;  // the stage of slice `it`; the parity of its `empty` barrier once the ring has gone round
      uint32_t a_dst = stage0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
        const int tile = unit % n_tiles, ks = unit / n_tiles;
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * bn;
        const int kb0 = ks * slices_per_split, kb1 = min(slices_total, kb0 + slices_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          // (Slices of the first round, some with their weights already on the way, are requested without a
          // wait, whatever the other roles do: their barriers then complete and the drain can wait for them.)
          if (it >= N_STAGES && !mbar_wait_role(&empty_bar[s], parity, ctl, 1)) {
            give_up_code(status, 1);
            abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t bar = full0 + 8 * s;
          if (it >= early) {
            mbar_expect_tx_s(bar, tx_bytes);
            tma_load_2d_s(a_dst + A_BYTES, &map_w, bar, kb * BK, n0);
          }
          tma_load_2d_s(a_dst, &map_x, bar, kb * BK, m0);
          a_dst += STG_BYTES;
          if (++s == N_STAGES) {
            s = 0;
            a_dst = stage0;
            parity ^= 1;
          }
        }
      }
      issued = it;
    }
  } else if (warp == 1) {
    // ---------------- tensor-core issuer (reads shared and tensor memory only: no wait of its own)
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, bn);
      // descriptors differ from stage to stage only in their address field (bytes / 16)
      const uint64_t a_desc0 = make_smem_desc(smem_u32(stages)), b_desc0 = make_smem_desc(smem_u32(stages) + A_BYTES);
      uint64_t stage_off = 0;
      uint32_t s = 0, phase = 0;  // the stage and the parity of its `full` barrier
      bool ok = true;
      int local = 0;  // tiles done by this block
      for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x, ++local) {
        const int ks = unit / n_tiles;
        const int kb0 = ks * slices_per_split, kb1 = min(slices_total, kb0 + slices_per_split);
        const int acc = local & 1;
        const uint32_t use = local >> 1;  // how often this half was used before
        if (use > 0 && !mbar_wait_role(&acc_empty[acc], (use - 1) & 1, ctl, 4)) {
          give_up_code(status, 4);
          abort_flag = 1;
          ok = false;
          break;
        }
        if (*(volatile int*)&abort_flag) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_role(&full_bar[s], phase, ctl, 2)) {
            give_up_code(status, 2);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          // (Issuing the slice as one block of instructions, with the next stage's wait asked ahead by a
          // mbarrier.test_wait and skipped when the answer was yes, took a single tile from 0.785 to 0.975 of the tensor
          // core's nominal rate; in long runs of decode steps at batch 64 about one launch in 10^5 then gave up on a stage
          // that never arrived, and the cause was not found: the loop waits, issues and commits in turn.)
          umma_bf16_x4(tmem_d, a_desc0 + stage_off, b_desc0 + stage_off, idesc, kb > kb0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
          stage_off += (uint64_t)(STG_BYTES >> 4);
          if (++s == N_STAGES) {
            s = 0;
            stage_off = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[acc]);  // arrives when the whole tile has been accumulated
      }
      if (!ok) {
        // the tensor core may still be at work on slices issued before the wait that failed: tensor memory
        // is not given back, and the block does not end, before they are done (bounded like the drain)
        umma_commit(&drain_bar);
        mbar_wait(&drain_bar, 0);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5, each on its quarter of the 128 lanes
    pdl_wait();  // the kernel before this one may still read the output buffer
    const int quarter = warp & 3;
    const uint32_t out_stage = smem_u32(stages) + (uint32_t)(N_STAGES * STG_BYTES) + (uint32_t)(quarter * OUT_STAGE_BYTES);
    int local = 0;
    for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++local) {
      const int tile = unit % n_tiles, ks = unit / n_tiles;
      TO* out_k = out + (size_t)ks * M * ldo;
      const int acc = local & 1;
      // One warp polls the tile's barrier and the other three wait for it at a hardware barrier, where they take
      // no issue slots: the pollers of a whole tile's products share their SM sub-partitions with the two single
      // threads that feed the copy engine and the tensor core.
      if (quarter == 2 && !mbar_wait_role(&acc_full[acc], (local >> 1) & 1, ctl, 3) && lane == 0) {
        give_up_code(status, 3);
        abort_flag = 1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*(volatile int*)&abort_flag) break;
      tc_fence_after();
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * bn;
      const int row = m0 + quarter * 32 + lane;
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      int c = 0;
      // (a warp whose 32 rows do not all exist stores from registers as before: with few rows the turn through shared
      // memory costs more than it saves, 9.4 against 9.0 us for 16 x 4096 x 4096)
      const bool whole_rows = m0 + quarter * 32 + 32 <= M;
      if (sizeof(TO) == 2 && vec_store && whole_rows) {
        // whole groups of 64 accumulator columns go out through shared memory as whole rows (see above)
        const int rows_valid = 32;
#pragma unroll 1
        for (; (c + 2) * 32 <= bn && n0 + (c + 2) * 32 <= N; c += 2) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(lane_base + (uint32_t)(c * 32), r0);
          tmem_ld_32x32b_x32(lane_base + (uint32_t)(c * 32 + 32), r1);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          bf16* tile_out = reinterpret_cast<bf16*>(out_k) + (size_t)(m0 + quarter * 32) * ldo + (SWIGLU ? (col >> 1) : col);
          if (SWIGLU)
            store_rows32_swiglu_bf16(tile_out, ldo, rows_valid, r0, r1, out_stage, lane);
          else
            store_rows64_bf16(tile_out, ldo, rows_valid, r0, r1, out_stage, lane);
        }
      }
#pragma unroll 1
      for (; c < (bn + 31) / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(lane_base + (uint32_t)(c * 32), r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        const int n_valid = min(N - col, bn - c * 32);  // columns of this piece that belong to the tile and the matrix
        if (sizeof(TO) == 4 && !SWIGLU && vec_store && whole_rows && n_valid >= 32) {
          store_rows32_f32(reinterpret_cast<float*>(out_k) + (size_t)(m0 + quarter * 32) * ldo + col, ldo, 32, r, out_stage, lane);
          continue;
        }
        if (row < M && n_valid > 0) {
          if (SWIGLU)
            store_swiglu16<TO>(out_k + (size_t)row * ldo + (col >> 1), r, n_valid >> 1, vec_store != 0);
          else
            store_row32<TO>(out_k + (size_t)row * ldo + col, r, n_valid, vec_store != 0);
        }
      }
      // this half may be overwritten once all four warps have read it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  // Every role is done or has given up.  Nothing may still be writing shared memory when the block ends: if
  // someone gave up, the producer's lane waits (bounded, with the long limit) for the copies that were
  // started and not consumed.  It does so here, after the roles have met, because the producer may have
  // left its loop before another role gave up.
  if (threadIdx.x == 0 && *(volatile int*)&abort_flag) {
    const uint32_t first = issued > N_STAGES ? issued - N_STAGES : 0;
    for (uint32_t j = first; j < issued; ++j) mbar_wait(&full_bar[j % N_STAGES], (j / N_STAGES) & 1);
  }
}

// ------------------------------------------------------------------ host side
// status: one int in device memory, 0 before the call; non-zero afterwards means a bounded wait expired
// (1 producer, 2 tensor-core issuer waiting for data, 3 epilogue, 4 tensor-core issuer waiting for the
// epilogue) and the output is not valid.
// swiglu != 0: w holds N rows alternating gate and up, out gets N / 2 columns (see the kernel).
// k_splits > 1: the k range is cut into that many slices (rounded so that none is empty; the number
// used is returned through *k_splits_used), out is [slices][M][ldo] float32 partial results.
// wait_test_role, wait_test_ns: 0, 0 in normal use.  A test names one of the codes above and a limit in
// nanoseconds: the waits of that role then give up after that long instead of a second.
// tile_n: 0, or the tile width the caller wants (a multiple of 16 up to 256) in the place of the launcher's choice.
RL_API int rl_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                      int K, int swiglu, int k_splits, int* k_splits_used, int tile_n, int* status, int wait_test_role,
                      unsigned int wait_test_ns, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemm_tc: M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8) RL_REFUSE(2, "gemm_tc: K=%d, ldx=%d, ldw=%d must be multiples of 8 (16-byte TMA rows)", K, ldx, ldw);
  if (swiglu && (N & 1)) RL_REFUSE(11, "gemm_tc: %d gate/up rows are not pairs", N);
  if (ldx < K || ldw < K || ldo < (swiglu ? N / 2 : N)) RL_REFUSE(3, "gemm_tc: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) RL_REFUSE(4, "gemm_tc: operands must be 16-byte aligned");
  const int vec_store = (out_dtype == RL_BF16 ? (ldo % 8) : (ldo % 4)) == 0;  // else the epilogue stores element by element
  if (out_dtype != RL_BF16 && out_dtype != RL_F32) RL_REFUSE(6, "gemm_tc: unknown output dtype %d", out_dtype);
  if (status == nullptr) RL_REFUSE(7, "gemm_tc: no status word");
  if (k_splits < 1) RL_REFUSE(12, "gemm_tc: %d k slices", k_splits);
  if (k_splits > 1 && (swiglu || out_dtype != RL_F32)) RL_REFUSE(13, "gemm_tc: partial sums over k slices are float32 and cannot go through the activation");
  if (tile_n != 0 && (tile_n < 16 || tile_n > BN || tile_n % 16)) RL_REFUSE(14, "gemm_tc: a tile width of %d (a multiple of 16 up to %d)", tile_n, BN);
  {
    const int slices = (K + BK - 1) / BK;
    if (k_splits > slices) k_splits = slices;
    const int per = (slices + k_splits - 1) / k_splits;
    k_splits = (slices + per - 1) / per;  // no empty slice
    if (k_splits_used) *k_splits_used = k_splits;
  }
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0) n_sms = 148;
  }
  // the tile width: see the header
  int bn = BN;
  {
    const long long tiles_m = (M + BM - 1) / BM;
    const long long at_full_width = tiles_m * ((N + BN - 1) / BN) * k_splits;
    // (every tile reads its rows of x again, so narrower tiles cost L2 traffic: measured at 64 rows, a product
    // with 24 full tiles gains from 128 narrow ones, 29 -> 24 us, one with 112 full tiles does not)
    if (tile_n != 0) {
      bn = tile_n;
    } else if (at_full_width < n_sms / 2) {
      const long long per_row = n_sms / (tiles_m * k_splits);  // tiles that one row of tiles may have
      if (per_row >= 1) {
        long long want = (N + per_row - 1) / per_row;
        want = ((want + 15) / 16) * 16;
        bn = (int)(want < 16 ? 16 : (want > BN ? BN : want));
      }
    }
    // (Narrowing the tiles of a product with several rounds of tiles, so that the last round is fuller, was
    // measured and does not pay: at 2048 rows a width of 240 instead of 256 took 390 us instead of 350.)
  }
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + bn - 1) / bn) * k_splits;
  CUtensorMap map_x, map_w;
  const bool small_a = M <= SMALL_A_ROWS;
  int e1 = make_matrix_map(&map_x, x, M, K, ldx, small_a ? SMALL_A_ROWS : BM), e2 = make_matrix_map(&map_w, w, N, K, ldw, bn);
  if (e1 || e2) RL_REFUSE(9, "gemm_tc: cuTensorMapEncodeTiled unavailable or failed (%d, %d)", e1, e2);
  const size_t smem = (small_a ? (size_t)5 * (SMALL_A_BYTES + STAGE_B_BYTES) : (size_t)STAGES * STAGE_BYTES) + 4 * OUT_STAGE_BYTES + 1024;
  dim3 grid((unsigned)(tiles < n_sms ? tiles : n_sms));
#define RL_TC_LAUNCH(TOUT, SW)                                                                                      \
  do {                                                                                                            \
    auto kern = small_a ? gemm_tc_kernel<TOUT, SW, true> : gemm_tc_kernel<TOUT, SW, false>;                       \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)        \
      RL_REFUSE(10, "gemm_tc: cannot get %zu bytes of shared memory", smem);                                      \
    RL_LAUNCH_CHECK(rl_launch(kern, grid, NUM_THREADS, smem, stream, map_x, map_w, (TOUT*)out, ldo, M, N, K, vec_store,  \
                              k_splits, bn, status, wait_test_role, (uint32_t)wait_test_ns));                         \
  } while (0)
  if (out_dtype == RL_BF16 && swiglu) RL_TC_LAUNCH(bf16, true);
  else if (out_dtype == RL_BF16) RL_TC_LAUNCH(bf16, false);
  else if (swiglu) RL_TC_LAUNCH(float, true);
  else RL_TC_LAUNCH(float, false);
#undef RL_TC_LAUNCH
  return 0;
}
