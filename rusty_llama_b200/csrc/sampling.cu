// Choosing the next token on the device, with the reference's rules
// (src/sampler.rs:801-819): temperature 0 is the argmax with the last of equal
// maxima (:78-84); otherwise logits / t (:101-106), an optional nucleus (:116-164)
// and one inverse-CDF draw (:190-216) from an xorshift64* stream (:176-187) that
// is kept per sequence.  The reference samples on the host after copying the
// logits back; here only the chosen token ids leave the device.
//
// One block per row.  The nucleus is found without sorting: the probability
// that closes it is located by a bisection over the bit patterns of positive
// floats (their integer order is their numeric order), each probe being one
// masked sum over the row; equal probabilities are taken in index order.
// Sums are tree sums, so a draw that lands within rounding of a boundary of the
// cumulative distribution may pick the neighbouring token of the sequential
// 32-bit sum the reference does.
#include "common.cuh"

RL_DEFINE_ERROR_TEXT()

#define SAMPLE_THREADS 1024

// ---------------------------------------------------------------- argmax
struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; among equal values the larger index (last of ties)
  if (b.v > a.v || (b.v == a.v && b.i > a.i)) return b;
  return a;
}

__device__ int block_argmax(const float* row, int n, float t, ArgMax* sh) {
  ArgMax best = {-INFINITY, -1};
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // four values per load, four loads in flight: a row of 128k logits is scanned by one block,
    // which would otherwise wait for one load after the other
    const int n4 = n >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = r4[i + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int base = 4 * (i + u * blockDim.x);
        best = better(best, ArgMax{v[u].x / t, base});
        best = better(best, ArgMax{v[u].y / t, base + 1});
        best = better(best, ArgMax{v[u].z / t, base + 2});
        best = better(best, ArgMax{v[u].w / t, base + 3});
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = r4[i];
      best = better(best, ArgMax{v.x / t, 4 * i});
      best = better(best, ArgMax{v.y / t, 4 * i + 1});
      best = better(best, ArgMax{v.z / t, 4 * i + 2});
      best = better(best, ArgMax{v.w / t, 4 * i + 3});
    }
    for (int j = 4 * n4 + threadIdx.x; j < n; j += blockDim.x) best = better(best, ArgMax{row[j] / t, j});
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) best = better(best, ArgMax{row[i] / t, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = best;
  __syncthreads();
  ArgMax r = sh[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = better(r, sh[w]);
  return r.i < 0 ? n - 1 : r.i;  // all NaN: the reference ends on the last index
}

__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int n, int* __restrict__ out) {
  __shared__ ArgMax sh[32];
  const int r = blockIdx.x;
  const int idx = block_argmax(logits + (size_t)r * row_stride, n, 1.0f, sh);
  if (threadIdx.x == 0) out[r] = idx;
}

RL_API int rl_argmax(const float* logits, long long row_stride, int n_rows, int n, int* out, cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0) RL_REFUSE(1, "argmax: rows=%d n=%d", n_rows, n);
  argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, row_stride, n, out);
  RL_LAUNCH_RESULT();
}

// ---------------------------------------------------------------- sampling

// Sum and count of the probabilities p[i] >= lo (as bit patterns) that also pass `floor_bits`.
__device__ __forceinline__ void masked_sum(const float* p, int n, uint32_t lo_bits, float* red, float& sum,
                                           int& count) {
  float s = 0.f;
  float c = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = p[i];
    if (__float_as_uint(v) >= lo_bits) {
      s += v;
      c += 1.f;
    }
  }
  sum = block_sum(s, red);
  count = (int)block_sum(c, red);
}

// Largest bit pattern b in [lo, hi) such that the mass of {p >= b} exceeds `limit`;
// the caller guarantees that lo qualifies and hi does not.
__device__ uint32_t bisect_mass(const float* p, int n, uint32_t lo, uint32_t hi, float limit, float* red) {
  while (hi - lo > 1) {
    const uint32_t mid = lo + ((hi - lo) >> 1);
    float s;
    int c;
    masked_sum(p, n, mid, red, s, c);
    if (s > limit) lo = mid; else hi = mid;
  }
  return lo;
}

// Smallest probability that is >= the pattern `b` (the value that closes the set).
__device__ float min_at_least(const float* p, int n, uint32_t b, float* red) {
  float m = INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = p[i];
    if (__float_as_uint(v) >= b) m = fminf(m, v);
  }
  return -block_max(-m, red);
}

// Index of the j-th (from 0) element equal to `v`, in index order; -1 if there are fewer.
__device__ int kth_equal(const float* p, int n, float v, int j, int* sh_int) {
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int begin = threadIdx.x * per, end = min(n, begin + per);
  int mine = 0;
  for (int i = begin; i < end; ++i) mine += (p[i] == v);
  __syncthreads();
  sh_int[threadIdx.x] = mine;
  __syncthreads();
  // the thread whose range holds the j-th match finds it; a serial prefix over 1024 counts is cheap
  if (threadIdx.x == 0) {
    int before = 0, owner = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (j < before + sh_int[t]) { owner = t; break; }
      before += sh_int[t];
    }
    sh_int[blockDim.x] = owner;
    sh_int[blockDim.x + 1] = before;
  }
  __syncthreads();
  const int owner = sh_int[blockDim.x], before = sh_int[blockDim.x + 1];
  __syncthreads();
  if (owner < 0) return -1;
  if ((int)threadIdx.x == owner) {
    int seen = before, found = -1;
    for (int i = begin; i < end; ++i)
      if (p[i] == v) {
        if (seen == j) { found = i; break; }
        ++seen;
      }
    sh_int[blockDim.x + 2] = found;
  }
  __syncthreads();
  const int found = sh_int[blockDim.x + 2];
  __syncthreads();
  return found;
}

// First index, in index order, whose running sum of p exceeds `target`; n-1 if none.
__device__ int first_cdf_above(const float* p, int n, float target, float* sh_f, int* sh_int) {
  const int per = (n + blockDim.x - 1) / blockDim.x;
  const int begin = threadIdx.x * per, end = min(n, begin + per);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) mine += p[i];
  __syncthreads();
  sh_f[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float before = 0.f;
    int owner = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (target < before + sh_f[t]) { owner = t; break; }
      before += sh_f[t];
    }
    sh_int[0] = owner;
    sh_f[blockDim.x] = before;
  }
  __syncthreads();
  const int owner = sh_int[0];
  const float before = sh_f[blockDim.x];
  __syncthreads();
  if (owner < 0) return n - 1;
  if ((int)threadIdx.x == owner) {
    float cdf = before;
    int found = end - 1;
    for (int i = begin; i < end; ++i) {
      cdf += p[i];
      if (target < cdf) { found = i; break; }
    }
    sh_int[1] = found;
  }
  __syncthreads();
  const int found = sh_int[1];
  __syncthreads();
  return found;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int n, float temperature, float top_p,
              unsigned long long* __restrict__ rng_states, const int* __restrict__ rng_index,
              float* __restrict__ probs, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ ArgMax sh_arg[32];
  __shared__ float sh_f[SAMPLE_THREADS + 1];
  __shared__ int sh_int[SAMPLE_THREADS + 3];
  __shared__ float coin_s;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* p = probs + (size_t)r * n;

  // one draw per sampled token (src/sampler.rs:176-187)
  if (threadIdx.x == 0) {
    unsigned long long* st = rng_states + rng_index[r];
    unsigned long long s = *st;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *st = s;
    const uint32_t u = (uint32_t)((s * 0x2545F4914F6CDD1DULL) >> 32);
    coin_s = (float)(u >> 8) / 16777216.0f;
  }

  // softmax of logits / t (src/sampler.rs:58-73, :101-106)
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, row[i] / temperature);
  mx = block_max(mx, red);
  float part = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float e = expf(row[i] / temperature - mx);
    p[i] = e;
    part += e;
  }
  const float inv = 1.0f / block_sum(part, red);
  for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] *= inv;
  __syncthreads();
  const float coin = coin_s;

  int chosen;
  if (!(top_p > 0.f && top_p < 1.f)) {
    chosen = first_cdf_above(p, n, coin, sh_f, sh_int);
  } else {
    // candidates must reach (1 - top_p) / (n - 1) (src/sampler.rs:127-134)
    const float cutoff = (1.0f - top_p) / (float)max(n - 1, 1);
    const uint32_t cutoff_bits = __float_as_uint(cutoff);
    float kept_mass;
    int kept;
    masked_sum(p, n, cutoff_bits, red, kept_mass, kept);
    if (kept == 0) {
      chosen = block_argmax(row, n, temperature, sh_arg);  // (src/sampler.rs:135-144)
    } else {
      float pmax = 0.f;
      for (int i = threadIdx.x; i < n; i += blockDim.x) pmax = fmaxf(pmax, p[i]);
      pmax = block_max(pmax, red);
      const uint32_t top_bits = __float_as_uint(pmax) + 1u;
      // the value that closes the nucleus, the mass above it, and how many of its equals are in
      float v_min, mass_gt;
      int ties_in;
      if (!(kept_mass > top_p)) {  // the mass never exceeds top_p: everything kept stays (:150-158)
        v_min = min_at_least(p, n, cutoff_bits, red);
        float s_ge; int c_ge, c_gt;
        masked_sum(p, n, __float_as_uint(v_min), red, s_ge, c_ge);
        masked_sum(p, n, __float_as_uint(v_min) + 1u, red, mass_gt, c_gt);
        ties_in = c_ge - c_gt;
      } else {
        const uint32_t b = bisect_mass(p, n, cutoff_bits, top_bits, top_p, red);
        v_min = min_at_least(p, n, b, red);
        float s_ge; int c_ge, c_gt;
        masked_sum(p, n, __float_as_uint(v_min), red, s_ge, c_ge);
        masked_sum(p, n, __float_as_uint(v_min) + 1u, red, mass_gt, c_gt);
        const int ties = c_ge - c_gt;
        int need = (int)floorf((top_p - mass_gt) / v_min) + 1;  // smallest count whose sum exceeds top_p
        ties_in = min(max(need, 1), ties);
      }
      const float nucleus_mass = mass_gt + (float)ties_in * v_min;
      const float target = coin * nucleus_mass;  // (src/sampler.rs:199-204)
      if (!(mass_gt > target)) {
        // falls among the equals that close the nucleus
        int j = (int)floorf((target - mass_gt) / v_min);
        j = min(max(j, 0), ties_in - 1);
        chosen = kth_equal(p, n, v_min, j, sh_int);
      } else {
        // largest value whose "at least" mass exceeds the target, within the part above v_min
        const uint32_t b = bisect_mass(p, n, __float_as_uint(v_min) + 1u, top_bits, target, red);
        const float v_sel = min_at_least(p, n, b, red);
        float s_ge, s_gt; int c_ge, c_gt;
        masked_sum(p, n, __float_as_uint(v_sel), red, s_ge, c_ge);
        masked_sum(p, n, __float_as_uint(v_sel) + 1u, red, s_gt, c_gt);
        int j = (int)floorf((target - s_gt) / v_sel);
        j = min(max(j, 0), c_ge - c_gt - 1);
        chosen = kth_equal(p, n, v_sel, j, sh_int);
      }
      if (chosen < 0) chosen = block_argmax(row, n, temperature, sh_arg);
    }
  }
  if (threadIdx.x == 0) out[r] = chosen;
}

// probs: scratch of n_rows * n floats.  rng_states[rng_index[r]] is read and advanced for row r.
RL_API int rl_sample(const float* logits, long long row_stride, int n_rows, int n, float temperature, float top_p,
                     unsigned long long* rng_states, const int* rng_index, float* probs, int* out,
                     cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0) RL_REFUSE(1, "sample: rows=%d n=%d", n_rows, n);
  if (!(temperature > 0.f)) RL_REFUSE(2, "sample: temperature %f is not positive (0 is the argmax kernel's)", temperature);
  if (!rng_states || !rng_index || !probs) RL_REFUSE(3, "sample: missing random state or scratch");
  sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, row_stride, n, temperature, top_p, rng_states,
                                                        rng_index, probs, out);
  RL_LAUNCH_RESULT();
}
