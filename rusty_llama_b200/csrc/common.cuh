// Shared helpers of the sm_100a kernels: element types, conversions, reductions
// and the convention of the exported launchers.
//
// Every launcher is `extern "C"`, takes raw device pointers, sizes and the
// stream to launch on, allocates nothing and returns 0 or an error code:
// a positive code is a CUDA error (cudaError_t) seen right after the launch,
// a negative one means the launcher refused its arguments before launching;
// `rl_error_text()` then holds the reason.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define RL_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// dtype codes shared with the Python side
#define RL_F32 0
#define RL_BF16 1

static thread_local char rl_error_buf[512] = {0};

#define RL_REFUSE(code, ...)                                         \
  do {                                                               \
    snprintf(rl_error_buf, sizeof(rl_error_buf), __VA_ARGS__);       \
    return -(code);                                                  \
  } while (0)

#define RL_LAUNCH_RESULT()                                                         \
  do {                                                                             \
    cudaError_t rl_e = cudaGetLastError();                                         \
    if (rl_e != cudaSuccess) {                                                     \
      snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(rl_e)); \
      return (int)rl_e;                                                            \
    }                                                                              \
    return 0;                                                                      \
  } while (0)

// Profiling aid, compiled in only with -DRL_TRACE (RUSTY_LLAMA_NVCC_EXTRA="-DRL_TRACE"): the first
// thread of a kernel's first block notes the time at which its dependency wait returned, i.e. when the
// kernel before it had finished, in a buffer that the host hands to every library with rl_trace_set.
// The differences between successive notes are the kernels' durations inside a replayed graph, where
// no profiler can look without serialising them.
#ifdef RL_TRACE
static __device__ unsigned long long* rl_trace_buf = nullptr;
static __device__ unsigned int* rl_trace_count = nullptr;
static __device__ unsigned int rl_trace_cap = 0;
#define RL_DEFINE_TRACE()                                                                             \
  RL_API int rl_trace_set(void* buf, void* count, unsigned int cap) {                                 \
    cudaError_t e = cudaMemcpyToSymbol(rl_trace_buf, &buf, sizeof(void*));                            \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(rl_trace_count, &count, sizeof(void*));              \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(rl_trace_cap, &cap, sizeof(unsigned int));           \
    return (int)e;                                                                                    \
  }
__device__ __forceinline__ void rl_trace_mark() {
  if (threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && rl_trace_buf != nullptr) {
    const unsigned int i = atomicAdd(rl_trace_count, 1u);
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (i < rl_trace_cap) rl_trace_buf[i] = t & 0x00ffffffffffffffull;
  }
}
// a note with a number in its top byte, from whichever single thread calls it (block 0 only)
__device__ __forceinline__ void rl_trace_event(unsigned int id) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && rl_trace_buf != nullptr) {
    const unsigned int i = atomicAdd(rl_trace_count, 1u);
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (i < rl_trace_cap) rl_trace_buf[i] = ((unsigned long long)id << 56) | (t & 0x00ffffffffffffffull);
  }
}
#else
#define RL_DEFINE_TRACE()
__device__ __forceinline__ void rl_trace_mark() {}
__device__ __forceinline__ void rl_trace_event(unsigned int) {}
#endif

#define RL_DEFINE_ERROR_TEXT()                                 \
  RL_API const char* rl_error_text() { return rl_error_buf; } \
  RL_DEFINE_TRACE()

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block whose size is a multiple of 32 and at most 1024.  The order
// of the additions depends on the block size only, so equal inputs give equal
// bits.  `red` is 32 floats of shared memory.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarps; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[0];
  for (int w = 1; w < nwarps; ++w) t = fmaxf(t, red[w]);
  return t;
}

// 8 bf16 values (16 bytes) to 8 floats.
__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = __bfloat1622float2(p[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// Four consecutive elements as floats and back (16 bytes of float, 8 of bfloat16); the address
// must be aligned to that size.  load4 works on any address (shared memory included); load4_g is
// for global memory only and goes to L2 (ld.global.cg), never through the read-only path: a
// kernel that was started early (see pdl_wait below) reads what its predecessor wrote while both
// were running, which the non-coherent path does not allow.
template <typename T>
__device__ __forceinline__ void load4(const T* p, float* f);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float* f) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16* p, float* f) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void load4_g(const T* p, float* f);
template <>
__device__ __forceinline__ void load4_g<float>(const float* p, float* f) {
  const float4 v = __ldcg(reinterpret_cast<const float4*>(p));
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <>
__device__ __forceinline__ void load4_g<bf16>(const bf16* p, float* f) {
  const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float* f);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* p, const float* f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
  __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ------------------------------------------------------------------ programmatic dependent launch
// The kernels of a decode step are short (a few microseconds each), so the gap between one kernel's
// last block and the next kernel's first load is a visible share of the step.  Kernels launched with
// rl_launch may start while their predecessor in the stream is still running: everything a kernel
// does before pdl_wait() (index arithmetic, shared-memory set-up, requests for weights, which no
// kernel writes) overlaps the predecessor's tail; pdl_wait() returns once the predecessor has
// finished and its writes are visible.  Rules: every block calls pdl_wait() before it touches memory
// that another kernel writes, and before any early return; nothing is written to global memory
// before it.  The kernels of a decode step release their successor first thing (pdl_trigger): the
// successor becomes resident as soon as every block of its predecessor has started, and the
// persistent streaming product then requests its first ring of weights (200 KB per SM) while the
// norm, rotary or attention kernel before it is still at work.  Measured on the decode step of an
// 8B model at batch 8: 4.43 ms without, 4.01 ms with.  RL_PDL=0 in the environment turns it off.
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  rl_trace_mark();
}
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Called first thing by the kernels of a decode step: once every block of a kernel has started, its
// successor (if launched with the programmatic attribute) may become resident and do what does not
// depend on other kernels, which for a streaming product is requesting its first ring of weights.
__device__ __forceinline__ void pdl_trigger() { pdl_launch_dependents(); }

static bool rl_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("RL_PDL");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on != 0;
}

template <bool EARLY_START = true, typename... KArgs, typename... Args>
static cudaError_t rl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (EARLY_START && rl_pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define RL_LAUNCH_CHECK(expr)                                                      \
  do {                                                                             \
    cudaError_t rl_e = (expr);                                                     \
    if (rl_e == cudaSuccess) rl_e = cudaGetLastError();                            \
    if (rl_e != cudaSuccess) {                                                     \
      snprintf(rl_error_buf, sizeof(rl_error_buf), "%s", cudaGetErrorString(rl_e)); \
      return (int)rl_e;                                                            \
    }                                                                              \
  } while (0)
