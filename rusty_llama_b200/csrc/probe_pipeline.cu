// Two measuring aids for the TMA / mbarrier pipelines of the other kernels (not used by the engine):
//
// rl_probe_tma_stream: one block per SM streams a buffer through a ring of shared-memory stages with TMA tensor
// copies and does nothing with the data: what HBM delivers to such a ring, as a function of the stage's shape
// (rows x contiguous bytes per row), the ring's depth and the walk (rows in groups along k, as the streaming
// product does, or tiles of many rows and 128 bytes along k, as a GEMM's operand).
//
// rl_probe_handshake: a producer thread and a consumer thread hand stages to each other through mbarriers, with
// or without a TMA copy per stage, with counters or with divisions by the ring's depth, with or without a read of
// the global timer per wait: what one trip of such a single-thread loop costs.
//
// rl_probe_mma_rate: one thread per block issues a run of tcgen05.mma (M 128, N n, K 16, bfloat16) on operands that
// already lie in shared memory (or, for A, in tensor memory), and notes the SM's cycles from the first issue to
// the arrival of the commit: what the tensor core takes per instruction, by N, with one accumulator or two in
// turn, with A from shared or from tensor memory, with or without TMA copies landing in the same shared memory.
//
// Every wait gives up after 2^22 polls and sets *err.
#include "tc_common.cuh"

RL_DEFINE_ERROR_TEXT()

#define PROBE_MAX_STAGES 32

__device__ __forceinline__ bool probe_wait(uint64_t* bar, uint32_t parity, int* err) {
  for (uint32_t i = 0; i < (1u << 22); ++i)
    if (mbar_try_wait(bar, parity)) return true;
  *err = 1;
  return false;
}
__device__ __forceinline__ void probe_tma_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// The buffer as a matrix [N][K] of bfloat16.  gemm_walk == 0: the map is [row][k / 64][64], a stage is `rows` rows x
// `kc` k, a block takes a contiguous range of row groups and walks each along k.  gemm_walk != 0: the map is
// [k / 64][row][64], a stage is `rows` rows x kc / 64 blocks of 64 k (each row of a block 128 bytes), row groups are
// dealt out round robin.
__global__ void __launch_bounds__(128, 1)
probe_stream_kernel(const __grid_constant__ CUtensorMap map, int N, int K, int rows, int kc, int stages, int stage_bytes,
                    int gemm_walk, int* err) {
  extern __shared__ __align__(1024) unsigned char ring[];
  __shared__ __align__(8) uint64_t full[PROBE_MAX_STAGES], empty[PROBE_MAX_STAGES];
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int groups = N / rows, per_group = K / kc;
  int g0, g1, gstep;
  if (gemm_walk) {
    g0 = blockIdx.x;
    g1 = groups;
    gstep = gridDim.x;
  } else {
    g0 = (int)((long long)groups * blockIdx.x / gridDim.x);
    g1 = (int)((long long)groups * (blockIdx.x + 1) / gridDim.x);
    gstep = 1;
  }
  int n = 0;
  for (int g = g0; g < g1; g += gstep) n += per_group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    const uint32_t ring0 = smem_u32(ring), full0 = smem_u32(&full[0]);
    int s = 0, g = g0, kk = 0;
    uint32_t parity = 1;
    for (int i = 0; i < n; ++i) {
      if (!probe_wait(&empty[s], parity, err)) break;
      mbar_expect_tx_s(full0 + 8 * s, stage_bytes);
      if (gemm_walk)
        probe_tma_3d(ring0 + s * stage_bytes, &map, full0 + 8 * s, 0, g * rows, kk * (kc / 64));
      else
        probe_tma_3d(ring0 + s * stage_bytes, &map, full0 + 8 * s, 0, kk * (kc / 64), g * rows);
      if (++kk == per_group) {
        kk = 0;
        g += gstep;
      }
      if (++s == stages) {
        s = 0;
        parity ^= 1;
      }
    }
  } else if (warp == 1 && lane == 0) {
    int s = 0;
    uint32_t parity = 0;
    for (int i = 0; i < n; ++i) {
      if (!probe_wait(&full[s], parity, err)) break;
      mbar_arrive(&empty[s]);
      if (++s == stages) {
        s = 0;
        parity ^= 1;
      }
    }
  }
  __syncthreads();
}

// buf: `bytes` of device memory (a multiple of K * rows * 2); err: one int, 0 before the call.
RL_API int rl_probe_tma_stream(const void* buf, long long bytes, int K, int rows, int kc, int stages, int gemm_walk, int l2_promotion,
                               int* err, cudaStream_t stream) {
  if (buf == nullptr || err == nullptr || bytes <= 0 || K <= 0 || K % 64 || rows <= 0 || rows > 256 || kc <= 0 || kc % 64 || kc > K ||
      K % kc || kc / 64 > 256 || stages < 1 || stages > PROBE_MAX_STAGES)
    RL_REFUSE(1, "probe_tma_stream: bytes=%lld K=%d rows=%d kc=%d stages=%d", bytes, K, rows, kc, stages);
  const long long N = bytes / 2 / K;
  const int stage_bytes = rows * kc * 2;
  if (N < rows || N > 0x7fffffffLL || stage_bytes % 1024 || (long long)stage_bytes * stages > 216 * 1024)
    RL_REFUSE(2, "probe_tma_stream: %lld rows, stages of %d bytes", N, stage_bytes);
  EncodeTiledFn enc = encode_tiled();
  if (!enc) RL_REFUSE(3, "probe_tma_stream: cuTensorMapEncodeTiled is not available");
  CUtensorMap map;
  cuuint64_t dims[3], strides[2];
  cuuint32_t box[3], estr[3] = {1, 1, 1};
  if (gemm_walk) {
    dims[0] = 64; dims[1] = (cuuint64_t)N; dims[2] = (cuuint64_t)(K / 64);
    strides[0] = (cuuint64_t)K * 2; strides[1] = 128;
    box[0] = 64; box[1] = (cuuint32_t)rows; box[2] = (cuuint32_t)(kc / 64);
  } else {
    dims[0] = 64; dims[1] = (cuuint64_t)(K / 64); dims[2] = (cuuint64_t)N;
    strides[0] = 128; strides[1] = (cuuint64_t)K * 2;
    box[0] = 64; box[1] = (cuuint32_t)(kc / 64); box[2] = (cuuint32_t)rows;
  }
  const CUtensorMapL2promotion promo = l2_promotion == 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                       : l2_promotion == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_NONE;
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(buf), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    RL_REFUSE(4, "probe_tma_stream: cannot describe the buffer to TMA");
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    RL_REFUSE(5, "probe_tma_stream: cannot count the SMs");
  const size_t smem = (size_t)stage_bytes * stages;
  if (cudaFuncSetAttribute(probe_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    RL_REFUSE(6, "probe_tma_stream: cannot get %zu bytes of shared memory", smem);
  RL_LAUNCH_CHECK(rl_launch<false>(probe_stream_kernel, dim3(sms), 128, smem, stream, map, (int)N, K, rows, kc, stages, stage_bytes,
                                   gemm_walk, err));
  return 0;
}

// mode bits: 1 = a TMA copy of one 32 x 128-byte box per stage (else a plain arrival), 2 = a second box, 4 = stage and
// parity by division instead of counters, 8 = both threads read the global timer before every wait.
template <int mode>
__global__ void __launch_bounds__(256, 1)
probe_handshake_kernel(const __grid_constant__ CUtensorMap map, int stages, int n_iters, int k_blocks, long long* out_ns, int* err) {
  extern __shared__ __align__(1024) unsigned char ring[];
  __shared__ __align__(8) uint64_t full[PROBE_MAX_STAGES], empty[PROBE_MAX_STAGES];
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int box_bytes = 32 * 128;
  if (warp == 0 && lane == 0) {
    const uint32_t ring0 = smem_u32(ring), full0 = smem_u32(&full[0]);
    int s = 0, kx = blockIdx.x % k_blocks;
    uint32_t parity = 1;
    uint64_t psink = 0;
    for (int i = 0; i < n_iters; ++i) {
      if (mode & 4) {
        s = i % stages;
        parity = ((i / stages) & 1) ^ 1;
        kx = (i + blockIdx.x) % k_blocks;
      }
      if (mode & 8) psink += global_ns();
      if (!probe_wait(&empty[s], parity, err)) break;
      if (mode & 1) {
        mbar_expect_tx_s(full0 + 8 * s, (mode & 2) ? 2 * box_bytes : box_bytes);
        tma_load_2d_s(ring0 + s * box_bytes, &map, full0 + 8 * s, kx * 64, 0);
        if (mode & 2) tma_load_2d_s(ring0 + s * box_bytes, &map, full0 + 8 * s, kx * 64, 32);
      } else {
        mbar_arrive(&full[s]);
      }
      if (!(mode & 4)) {
        if (++s == stages) {
          s = 0;
          parity ^= 1;
        }
        if (++kx == k_blocks) kx = 0;
      }
    }
    if (psink == 1) *err = 2;  // (keeps the timer reads)
  } else if (warp == 7 && lane == 0) {
    const uint64_t t0 = global_ns();
    uint64_t sink = 0;
    int s = 0;
    uint32_t parity = 0;
    for (int i = 0; i < n_iters; ++i) {
      if (mode & 4) {
        s = i % stages;
        parity = (i / stages) & 1;
      }
      if (mode & 8) sink += global_ns();
      if (!probe_wait(&full[s], parity, err)) break;
      mbar_arrive(&empty[s]);
      if (!(mode & 4) && ++s == stages) {
        s = 0;
        parity ^= 1;
      }
    }
    out_ns[blockIdx.x] = (long long)(global_ns() - t0);
    if (sink == 1) *err = 2;  // (keeps the timer reads)
  }
  __syncthreads();
}

// buf: at least 64 rows x k_blocks * 64 bfloat16 (row stride k_blocks * 64); out_ns: one value per block (n_blocks of them).
RL_API int rl_probe_handshake(const void* buf, int k_blocks, int mode, int stages, int n_iters, int n_blocks, long long* out_ns, int* err,
                              cudaStream_t stream) {
  if (buf == nullptr || out_ns == nullptr || err == nullptr || k_blocks < 1 || stages < 1 || stages > PROBE_MAX_STAGES || n_iters < 1 ||
      n_blocks < 1 || mode < 0 || mode > 15)
    RL_REFUSE(1, "probe_handshake: k_blocks=%d mode=%d stages=%d iterations=%d blocks=%d", k_blocks, mode, stages, n_iters, n_blocks);
  CUtensorMap map;
  if (make_matrix_map(&map, buf, 64, k_blocks * 64, k_blocks * 64, 32)) RL_REFUSE(2, "probe_handshake: cannot describe the buffer to TMA");
  const size_t smem = (size_t)stages * 32 * 128;
#define RL_PROBE_MODE(MODE)                                                                                                          \
  case MODE:                                                                                                                         \
    if (cudaFuncSetAttribute(probe_handshake_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)   \
      RL_REFUSE(3, "probe_handshake: cannot get %zu bytes of shared memory", smem);                                                  \
    RL_LAUNCH_CHECK(rl_launch<false>(probe_handshake_kernel<MODE>, dim3(n_blocks), 256, smem, stream, map, stages, n_iters, k_blocks, \
                                     out_ns, err));                                                                                  \
    break
  switch (mode) {
    RL_PROBE_MODE(0);
    RL_PROBE_MODE(1);
    RL_PROBE_MODE(3);
    RL_PROBE_MODE(4);
    RL_PROBE_MODE(5);
    RL_PROBE_MODE(8);
    RL_PROBE_MODE(9);
    default:
      RL_REFUSE(4, "probe_handshake: mode %d is not one of 0, 1, 3, 4, 5, 8, 9", mode);
  }
#undef RL_PROBE_MODE
  return 0;
}


// form bit 0: two accumulators in turn (else one); bit 1: A from tensor memory (n <= 128); bit 2: a second thread keeps
// three TMA copies of 32 KB in flight into the block's shared memory meanwhile (what a GEMM's producer does); bits 3
// and 4 (with A from shared memory and one accumulator): a commit after every fourth instruction, a wait and a fence
// before every fourth (bit 5: the wait without the fence); bit 6: the slice as `umma_bf16_x4_commit_peek` issues it.
__global__ void __launch_bounds__(128, 1)
probe_mma_kernel(const __grid_constant__ CUtensorMap map, int k_blocks, int n, int form, int n_mma, long long* out_cycles, int* err) {
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* a_s = base;               // 128 rows x 64 k, 16 KB
  unsigned char* b_s = base + 16 * 1024;   // 256 rows x 64 k, 32 KB
  unsigned char* ring = base + 48 * 1024;  // 3 x 32 KB for the copies
  __shared__ __align__(8) uint64_t done_bar, copy_bar[3], slice_bar, ready_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int stop;
  for (int i = threadIdx.x; i < 48 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(&done_bar, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&copy_bar[i], 1);
    mbar_init(&slice_bar, 1);
    mbar_init(&ready_bar, 1);
    mbar_arrive(&ready_bar);  // its first phase is complete from the start
    stop = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fence_async_shared();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) tmem_alloc(&tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0 && lane == 0) {
    const uint32_t idesc = make_idesc_bf16(128, n, 0, 0);
    const uint32_t acc1 = (form & 2) ? 128u : 256u, a_tmem = tmem_base + 256;
    const uint64_t a_desc = make_smem_desc(smem_u32(a_s)), b_desc = make_smem_desc(smem_u32(b_s));
    long long t0, t1;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t0)::"memory");
    // (eight at a time with everything but the instruction itself hoisted: the loop must not be what is measured)
    const uint32_t d0 = tmem_base, d1 = tmem_base + ((form & 1) ? acc1 : 0u);
    if (form & 2) {
      for (int i = 0; i < n_mma; i += 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) umma_bf16_ts((u & 1) ? d1 : d0, a_tmem + (u & 3) * 8, b_desc + 2 * (u & 3), idesc, 1u);
      }
    } else if (form & 64) {
      // the same slice with the question about the next stage asked before the MMAs and read after the commit
      uint32_t not_ready = 0;
      const uint32_t slice_b = smem_u32(&slice_bar), ready_b = smem_u32(&ready_bar);
      for (int i = 0; i < n_mma; i += 4) not_ready += 1u - umma_bf16_x4_commit_peek(d0, a_desc, b_desc, idesc, 1u, slice_b, ready_b, 0u);
      if (not_ready) *err = 3;
    } else if (form & 56) {
      // what a GEMM's issuer does between two k slices, after every fourth instruction: bit 3 a commit (to a barrier
      // nobody waits on), bit 4 a wait on a barrier that is complete and the fence that follows it
      uint32_t spins = 0;
      for (int i = 0; i < n_mma; i += 4) {
        if (form & 16) {
          while (!mbar_try_wait(&ready_bar, 0) && ++spins < (1u << 22)) {
          }
          if (!(form & 32)) tc_fence_after();
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) umma_bf16(d0, a_desc + 2 * u, b_desc + 2 * u, idesc, 1u);
        if (form & 8) umma_commit(&slice_bar);
      }
      if (spins >= (1u << 22)) *err = 1;
    } else {
      for (int i = 0; i < n_mma; i += 8) {
#pragma unroll
        for (int u = 0; u < 8; ++u) umma_bf16((u & 1) ? d1 : d0, a_desc + 2 * (u & 3), b_desc + 2 * (u & 3), idesc, 1u);
      }
    }
    umma_commit(&done_bar);
    probe_wait(&done_bar, 0, err);
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t1)::"memory");
    out_cycles[blockIdx.x] = t1 - t0;
    *(volatile int*)&stop = 1;
  } else if (warp == 1 && lane == 0 && (form & 4)) {
    // copies of 256 rows x 64 k (32 KB) each, three in flight, until the issuer is done (and at most 2^16 of them)
    int kx = blockIdx.x % k_blocks, issued = 0;
    for (int i = 0; i < (1 << 16) && !*(volatile int*)&stop; ++i) {
      const int st = i % 3;
      if (i >= 3 && !probe_wait(&copy_bar[st], ((i / 3) - 1) & 1, err)) break;
      mbar_expect_tx(&copy_bar[st], 32 * 1024);
      tma_load_2d(ring + st * 32 * 1024, &map, &copy_bar[st], kx * 64, 0);
      issued = i + 1;
      if (++kx == k_blocks) kx = 0;
    }
    // nothing may still be landing in shared memory when the block ends
    for (int i = issued > 3 ? issued - 3 : 0; i < issued; ++i) probe_wait(&copy_bar[i % 3], (i / 3) & 1, err);
    out_cycles[gridDim.x + blockIdx.x] = issued;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// buf: at least 256 rows x k_blocks * 64 bfloat16 (row stride k_blocks * 64); out_cycles: 2 x n_blocks values, each block's
// cycles and then each block's count of copies.
RL_API int rl_probe_mma_rate(const void* buf, int k_blocks, int n, int form, int n_mma, int n_blocks, long long* out_cycles, int* err,
                             cudaStream_t stream) {
  if (buf == nullptr || out_cycles == nullptr || err == nullptr || k_blocks < 1 || n < 16 || n > 256 || n % 16 || form < 0 || form > 127 ||
      n_mma < 8 || n_mma % 8 || n_blocks < 1 || ((form & 2) && n > 128))
    RL_REFUSE(1, "probe_mma_rate: k_blocks=%d n=%d form=%d MMAs=%d blocks=%d", k_blocks, n, form, n_mma, n_blocks);
  CUtensorMap map;
  if (make_matrix_map(&map, buf, 256, k_blocks * 64, k_blocks * 64, 256)) RL_REFUSE(2, "probe_mma_rate: cannot describe the buffer to TMA");
  const size_t smem = (48 + 96 + 1) * 1024;
  if (cudaFuncSetAttribute(probe_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    RL_REFUSE(3, "probe_mma_rate: cannot get %zu bytes of shared memory", smem);
  RL_LAUNCH_CHECK(rl_launch<false>(probe_mma_kernel, dim3(n_blocks), 128, smem, stream, map, k_blocks, n, form, n_mma, out_cycles, err));
  return 0;
}
