// bfloat16 matrix product for prompts with PAIRS of SMs on one tile (tcgen05 cta_group::2):
//   out[M, N] = x[M, K] . w[N, K]^T,  32-bit accumulation in tensor memory.
// Same contract as `gemm_tc`; the reference hands these products to cuBLASLt
// (src/backend/cuda.rs:717-758).
//
// Why pairs: with one SM per 128 x 256 tile every 64-wide k slice brings 48 KB into shared memory
// and the tensor core reads 48 KB back out of it in the 512 cycles the slice's four MMAs take,
// 192 bytes a cycle against the 128 a cycle that shared memory delivers: the tensor pipe of
// `gemm_tc` is busy 76 % of the time.  A cluster of two blocks shares a 256 x 256 tile: each block
// loads its own 128 rows of x and HALF of the w tile (128 rows), 32 KB a slice, and the
// pair's tensor cores read each other's half of w.
//
// A cluster = blocks 2p (the leader) and 2p + 1 on neighbouring SMs, persistent over tiles.  In
// each block
//   warp 0 (one lane)  waits for its own stage to be free and asks TMA for its x rows and its half
//                      of w; both blocks' copies count their bytes on the LEADER's `full` barrier;
//   warp 1 (one lane)  in the leader only: waits for `full`, issues tcgen05.mma.cta_group::2
//                      (M 256, N 256, K 16), commits to the `empty` barrier of the stage in both
//                      blocks, and after a tile's last slice to `acc_full` in both blocks;
//   warps 2..5         read their block's 128 rows of the accumulator from tensor memory, store
//                      them, and arrive on the leader's `acc_empty` (eight arrivals free a half).
// Accumulators are double-buffered (2 x 256 columns) as in `gemm_tc`.
//
// Measured on a B200 (2048 x 28672 x 4096, power-capped, clocks near 1.5 GHz): 1.35 PFLOP/s against
// 1.36 for `gemm_tc`; 2048 x 4096 x 14336: 1.33 against 1.29.  Both sit at the same level, which the
// shared-memory argument above does not explain away, so `linear()` keeps the simpler single-SM
// kernel and this one is reached through `ops.gemm_tc(pair=True)` only.
//
// Every wait on an mbarrier is bounded; on expiry the waiter records a code in `status[0]`, tells
// both blocks, and everybody drains to the common end: no thread leaves before the cluster's
// closing barrier, because the partner may still signal this block's barriers.
#include <cooperative_groups.h>

#include "tc_common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BM 128            // rows of x per block (the pair's tile has 256)
#define BN 256            // columns of the pair's tile; a block loads BN / 2 rows of w
#define BK 64
#define STAGES 6
#define UMMA_K 16
#define TMEM_COLS 512     // two accumulators of BN columns
#define NUM_THREADS 192
#define STAGE_A_BYTES (BM * BK * 2)
#define STAGE_B_BYTES ((BN / 2) * BK * 2)
#define STAGE_BYTES (STAGE_A_BYTES + STAGE_B_BYTES)

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
    h[i] = g * (1.0f / (1.0f + expf(-g))) * u;
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


// ------------------------------------------------------------------ pair plumbing
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of this block's `p` in the block of rank `rank`
__device__ __forceinline__ uint32_t in_block(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_remote_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// a TMA tile copy of one block of a pair; the bytes count on the barrier at `bar_cluster_addr`,
// which may lie in the partner
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols));
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// one arrival on the barrier at `bar_cluster_addr` when every tcgen05.mma issued before by this
// thread has completed in both blocks
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// the same, arriving on the barrier at this offset in both blocks of the pair (a commit is no copy:
// nothing but the barrier's arrival crosses to the partner)
__device__ __forceinline__ void umma_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}

// ------------------------------------------------------------------ the kernel
template <typename TO, bool SWIGLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                TO* __restrict__ out, int ldo, int M, int N, int K, int vec_store, int k_splits,
                int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  // the swizzled stages must start on a 1024-byte boundary (the same offset in both blocks: the
  // dynamic area starts at the same address in every block of a kernel)
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];   // used in the leader
  __shared__ __align__(8) uint64_t empty_bar[STAGES];  // one in each block
  __shared__ __align__(8) uint64_t acc_full[2];        // one in each block
  __shared__ __align__(8) uint64_t acc_empty[2];       // used in the leader
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_units = n_tiles * k_splits;
  const int slices_total = (K + BK - 1) / BK;
  const int slices_per_split = (slices_total + k_splits - 1) / k_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);  // one arrival per epilogue warp of both blocks
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both blocks' barriers exist before anybody signals the partner's
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  pdl_wait();

  auto give_up = [&](int code) {
    atomicExch(status, code);
    abort_flag = 1;
    st_remote_u32(in_block(&abort_flag, rank ^ 1), 1);
  };

  if (warp == 0) {
    // ---------------- producer (both blocks)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      uint32_t full_addr[STAGES];
#pragma unroll
      for (int s = 0; s < STAGES; ++s) full_addr[s] = in_block(&full_bar[s], 0);
      for (int unit = pair; unit < n_units && ok; unit += n_pairs) {
        const int tile = unit % n_tiles, ks = unit / n_tiles;
        const int m0 = (tile % tiles_m) * (2 * BM) + (int)rank * BM;
        const int n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
        const int kb0 = ks * slices_per_split, kb1 = min(slices_total, kb0 + slices_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1)) {
            give_up(41);
            ok = false;
            break;
          }
          if (*(volatile int*)&abort_flag) {
            ok = false;
            break;
          }
          unsigned char* a_dst = stages + (size_t)s * STAGE_BYTES;
          unsigned char* b_dst = a_dst + STAGE_A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);  // both blocks' copies
          tma_load_2d_pair(a_dst, &map_x, full_addr[s], kb * BK, m0);
          tma_load_2d_pair(b_dst, &map_w, full_addr[s], kb * BK, n0);
        }
      }
      // nothing may still be writing shared memory when the block ends.  What this block requested
      // was consumed (the `empty` waits above) except for the last ring, whose `full` barriers
      // (in the leader) flip when both blocks' copies have landed: the leader waits for them here if
      // someone gave up, and the partner stays until the closing cluster barrier.
      if (!ok && leader) {
        const uint32_t first = it > STAGES ? it - STAGES : 0;
        for (uint32_t j = first; j < it; ++j) mbar_wait(&full_bar[j % STAGES], (j / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- tensor-core issuer (leader only)
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc(2 * BM, BN);
      // descriptors differ from stage to stage and k step to k step only in their address field (bytes / 16)
      const uint64_t a_desc0 = make_smem_desc(smem_u32(stages)), b_desc0 = make_smem_desc(smem_u32(stages) + STAGE_A_BYTES);
      uint32_t it = 0, s = 0, phase = 0;  // slices so far; the stage and the parity of its `full` barrier
      bool ok = true;
      int local = 0;
      for (int unit = pair; unit < n_units && ok; unit += n_pairs, ++local) {
        const int ks = unit / n_tiles;
        const int kb0 = ks * slices_per_split, kb1 = min(slices_total, kb0 + slices_per_split);
        const int acc = local & 1;
        const uint32_t use = local >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[acc], (use - 1) & 1)) {
          give_up(44);
          ok = false;
          break;
        }
        if (*(volatile int*)&abort_flag) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (!mbar_wait(&full_bar[s], phase)) {
            give_up(42);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t stage_off = (uint64_t)(s * (STAGE_BYTES >> 4));
          umma_bf16_x4_pair(tmem_d, a_desc0 + stage_off, b_desc0 + stage_off, idesc, kb > kb0 ? 1u : 0u);
          umma_commit_both(&empty_bar[s]);
          if (++s == STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit_both(&acc_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 of both blocks, each on its quarter of the block's 128 rows
    const int quarter = warp & 3;
    const uint32_t acc_empty_leader[2] = {in_block(&acc_empty[0], 0), in_block(&acc_empty[1], 0)};
    int local = 0;
    for (int unit = pair; unit < n_units; unit += n_pairs, ++local) {
      const int tile = unit % n_tiles, ks = unit / n_tiles;
      TO* out_k = out + (size_t)ks * M * ldo;
      const int acc = local & 1;
      if (!mbar_wait(&acc_full[acc], (local >> 1) & 1)) {
        if (lane == 0) give_up(43);
        break;
      }
      if (*(volatile int*)&abort_flag) break;
      tc_fence_after();
      const int m0 = (tile % tiles_m) * (2 * BM) + (int)rank * BM, n0 = (tile / tiles_m) * BN;
      const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row < M && col < N) {
          if (SWIGLU)
            store_swiglu16<TO>(out_k + (size_t)row * ldo + (col >> 1), r, (N - col) >> 1, vec_store != 0);
          else
            store_row32<TO>(out_k + (size_t)row * ldo + col, r, N - col, vec_store != 0);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_leader[acc]);
    }
  }
  // nobody leaves while the partner may still signal this block's barriers or read its half of w
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side
// Same arguments and meanings as rl_gemm_tc.  status codes 41-44: producer, tensor-core issuer
// waiting for data, epilogue, tensor-core issuer waiting for the epilogue.
RL_API int rl_gemm_tc2(const void* x, int ldx, const void* w, int ldw, void* out, int out_dtype, int ldo, int M, int N,
                       int K, int swiglu, int k_splits, int* k_splits_used, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) RL_REFUSE(1, "gemm_tc2: M=%d N=%d K=%d", M, N, K);
  if (K % 8 || ldx % 8 || ldw % 8) RL_REFUSE(2, "gemm_tc2: K=%d, ldx=%d, ldw=%d must be multiples of 8 (16-byte TMA rows)", K, ldx, ldw);
  if (swiglu && (N & 1)) RL_REFUSE(11, "gemm_tc2: %d gate/up rows are not pairs", N);
  if (ldx < K || ldw < K || ldo < (swiglu ? N / 2 : N)) RL_REFUSE(3, "gemm_tc2: leading sizes %d/%d/%d too small", ldx, ldw, ldo);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) RL_REFUSE(4, "gemm_tc2: operands must be 16-byte aligned");
  const int vec_store = (out_dtype == RL_BF16 ? (ldo % 8) : (ldo % 4)) == 0;
  if (out_dtype != RL_BF16 && out_dtype != RL_F32) RL_REFUSE(6, "gemm_tc2: unknown output dtype %d", out_dtype);
  if (status == nullptr) RL_REFUSE(7, "gemm_tc2: no status word");
  if (k_splits < 1) RL_REFUSE(12, "gemm_tc2: %d k slices", k_splits);
  if (k_splits > 1 && (swiglu || out_dtype != RL_F32)) RL_REFUSE(13, "gemm_tc2: partial sums over k slices are float32 and cannot go through the activation");
  {
    const int slices = (K + BK - 1) / BK;
    if (k_splits > slices) k_splits = slices;
    const int per = (slices + k_splits - 1) / k_splits;
    k_splits = (slices + per - 1) / per;
    if (k_splits_used) *k_splits_used = k_splits;
  }
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0) n_sms = 148;
  }
  const long long units = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN) * k_splits;
  CUtensorMap map_x, map_w;
  int e1 = make_matrix_map(&map_x, x, M, K, ldx, BM), e2 = make_matrix_map(&map_w, w, N, K, ldw, BN / 2);
  if (e1 || e2) RL_REFUSE(9, "gemm_tc2: cuTensorMapEncodeTiled unavailable or failed (%d, %d)", e1, e2);
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  const long long max_pairs = n_sms / 2;
  const unsigned pairs = (unsigned)(units < max_pairs ? units : max_pairs);
#define RL_TC_LAUNCH(TOUT, SW)                                                                                    \
  do {                                                                                                            \
    auto kern = gemm_tc2_kernel<TOUT, SW>;                                                                        \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)        \
      RL_REFUSE(10, "gemm_tc2: cannot get %zu bytes of shared memory", smem);                                     \
    cudaLaunchConfig_t cfg = {};                                                                                  \
    cfg.gridDim = dim3(2 * pairs);                                                                                \
    cfg.blockDim = dim3(NUM_THREADS);                                                                             \
    cfg.dynamicSmemBytes = smem;                                                                                  \
    cfg.stream = stream;                                                                                          \
    cudaLaunchAttribute attr[1];                                                                                  \
    attr[0].id = cudaLaunchAttributeClusterDimension;                                                             \
    attr[0].val.clusterDim.x = 2;                                                                                 \
    attr[0].val.clusterDim.y = 1;                                                                                 \
    attr[0].val.clusterDim.z = 1;                                                                                 \
    cfg.attrs = attr;                                                                                             \
    cfg.numAttrs = 1;                                                                                             \
    RL_LAUNCH_CHECK(cudaLaunchKernelEx(&cfg, kern, map_x, map_w, (TOUT*)out, ldo, M, N, K, vec_store, k_splits, status)); \
  } while (0)
  if (out_dtype == RL_BF16 && swiglu) RL_TC_LAUNCH(bf16, true);
  else if (out_dtype == RL_BF16) RL_TC_LAUNCH(bf16, false);
  else if (swiglu) RL_TC_LAUNCH(float, true);
  else RL_TC_LAUNCH(float, false);
#undef RL_TC_LAUNCH
  return 0;
}
