// Choosing the next token on the device, with the reference's rules
// (src/sampler.rs:801-819): temperature 0 is the argmax with the last of equal
// maxima (:78-84); otherwise logits / t (:101-106), an optional nucleus (:116-164)
// and one inverse-CDF draw (:190-216) from an xorshift64* stream (:176-187) that
// is kept per sequence.  The reference samples on the host after copying the
// logits back; here only the chosen token ids leave the device.
//
// One block per row.  The nucleus is found without sorting: the probability
// that closes it is located digit by digit in the bit patterns of positive
// floats (their integer order is their numeric order): four sweeps over the
// row, each a histogram of probability mass over the next eight bits, instead
// of one sweep per bit.  The masses are added as 64-bit fixed-point numbers
// (2^-44), so the histogram's atomic additions give the same sums in whatever
// order they happen and a row of 128k probabilities is summed more exactly than
// in 32-bit floats; equal probabilities are taken in index order.  A draw that
// lands within rounding of a boundary of the cumulative distribution may pick
// the neighbouring token of the sequential 32-bit sum the reference does.
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

// ---------------------------------------------------------------- sweeps over a row
// f(value, index) for every element of p[0..n), every thread of the block taking part.  A block that
// scans a row of 128k values alone is bound by how many loads it has in flight, so an aligned row is
// read four values per load, four loads ahead.  The order in which a thread meets its elements is not
// the index order.
template <typename F>
__device__ __forceinline__ void sweep(const float* p, int n, F f) {
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const int n4 = n >> 2;
    const float4* p4 = reinterpret_cast<const float4*>(p);
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = p4[i + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int base = 4 * (i + u * blockDim.x);
        f(v[u].x, base);
        f(v[u].y, base + 1);
        f(v[u].z, base + 2);
        f(v[u].w, base + 3);
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = p4[i];
      f(v.x, 4 * i);
      f(v.y, 4 * i + 1);
      f(v.z, 4 * i + 2);
      f(v.w, 4 * i + 3);
    }
    for (int j = 4 * n4 + threadIdx.x; j < n; j += blockDim.x) f(p[j], j);
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) f(p[i], i);
  }
}

// The part of a row that one warp owns when the row is cut into 32 contiguous parts (index order matters).
__device__ __forceinline__ void warp_range(int n, int warp, int n_warps, int& begin, int& end) {
  const int per = (((n + n_warps - 1) / n_warps) + 31) & ~31;  // whole tiles of 32
  begin = min(n, warp * per);
  end = min(n, begin + per);
}

// ---------------------------------------------------------------- sampling

// Sum and count of the probabilities p[i] >= lo (as bit patterns) that also pass `floor_bits`.
__device__ __forceinline__ void masked_sum(const float* p, int n, uint32_t lo_bits, float* red, float& sum,
                                           int& count) {
  float s = 0.f;
  float c = 0.f;
  sweep(p, n, [&](float v, int) {
    if (__float_as_uint(v) >= lo_bits) {
      s += v;
      c += 1.f;
    }
  });
  sum = block_sum(s, red);
  count = (int)block_sum(c, red);
}

// Fixed-point masses: a probability as a multiple of 2^-44 (the sum of a whole row stays below 2^45).
#define MASS_ONE 17592186044416.0  // 2^44
__device__ __forceinline__ unsigned long long to_mass(float v) { return (unsigned long long)((double)v * MASS_ONE + 0.5); }
__device__ __forceinline__ float from_mass(unsigned long long m) { return (float)((double)m / MASS_ONE); }

#define HIST_COPIES 16   // two warps share a copy of the histogram
#define HIST_BINS 256

// Among the probabilities whose bit pattern is at least `lo_bits`: the value v* with
// mass{p > v*} <= limit < mass{p >= v*} (the caller guarantees that their whole mass exceeds `limit`;
// if rounding says otherwise the smallest of them is returned).  Returns v*'s bit pattern and leaves
// mass{p > v*} in *mass_gt.  hist: HIST_COPIES * HIST_BINS 64-bit words of shared memory; bins: HIST_BINS more.
__device__ uint32_t select_mass(const float* p, int n, uint32_t lo_bits, float limit, unsigned long long* hist,
                                unsigned long long* bins, float* mass_gt) {
  __shared__ uint32_t sel_prefix;
  __shared__ unsigned long long sel_above;
  const unsigned long long limit_m = to_mass(fmaxf(limit, 0.f));
  uint32_t prefix = 0, prefix_mask = 0;
  unsigned long long above = 0;  // mass of the candidates above the prefix's range
  unsigned long long* mine = hist + (threadIdx.x >> 6) * HIST_BINS;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < HIST_COPIES * HIST_BINS; i += blockDim.x) hist[i] = 0ull;
    __syncthreads();
    sweep(p, n, [&](float v, int) {
      const uint32_t key = __float_as_uint(v);
      if (key >= lo_bits && (key & prefix_mask) == prefix) atomicAdd(&mine[(key >> shift) & (HIST_BINS - 1)], to_mass(v));
    });
    __syncthreads();
    if (threadIdx.x < HIST_BINS) {
      unsigned long long m = 0;
#pragma unroll
      for (int c = 0; c < HIST_COPIES; ++c) m += hist[c * HIST_BINS + threadIdx.x];
      bins[threadIdx.x] = m;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long acc = above;
      int chosen = -1, lowest = -1;
      for (int d = HIST_BINS - 1; d >= 0; --d) {
        if (bins[d] == 0ull) continue;
        lowest = d;
        if (acc + bins[d] > limit_m) {
          chosen = d;
          break;
        }
        acc += bins[d];
      }
      if (chosen < 0) {  // rounding: the candidates' mass does not exceed the limit after all
        chosen = max(lowest, 0);
        acc -= lowest >= 0 ? bins[lowest] : 0ull;
      }
      sel_prefix = prefix | ((uint32_t)chosen << shift);
      sel_above = acc;
    }
    __syncthreads();
    prefix = sel_prefix;
    above = sel_above;
    prefix_mask |= (uint32_t)(HIST_BINS - 1) << shift;
    __syncthreads();
  }
  *mass_gt = from_mass(above);
  return prefix;
}

// How many probabilities have exactly the bit pattern `bits`.
__device__ int count_equal(const float* p, int n, uint32_t bits, float* red) {
  float c = 0.f;
  sweep(p, n, [&](float v, int) { c += (__float_as_uint(v) == bits) ? 1.f : 0.f; });
  return (int)block_sum(c, red);
}

// Smallest probability that is >= the pattern `b` (the value that closes the set).
__device__ float min_at_least(const float* p, int n, uint32_t b, float* red) {
  float m = INFINITY;
  sweep(p, n, [&](float v, int) {
    if (__float_as_uint(v) >= b) m = fminf(m, v);
  });
  return -block_max(-m, red);
}

// Index of the j-th (from 0) element equal to `v`, in index order; -1 if there are fewer.
// Each warp counts the matches in its contiguous part of the row (coalesced loads); the warp whose part
// holds the j-th match then walks it in tiles of 32, a ballot per tile.
__device__ int kth_equal(const float* p, int n, float v, int j, int* sh_int) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  int begin, end;
  warp_range(n, warp, n_warps, begin, end);
  int mine = 0;
  for (int i = begin + lane; i < end; i += 32) mine += (p[i] == v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  __syncthreads();
  if (lane == 0) sh_int[warp] = mine;
  if (threadIdx.x == 0) sh_int[n_warps + 2] = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    int before = 0, owner = -1;
    for (int w = 0; w < n_warps; ++w) {
      if (j < before + sh_int[w]) { owner = w; break; }
      before += sh_int[w];
    }
    sh_int[n_warps] = owner;
    sh_int[n_warps + 1] = before;
  }
  __syncthreads();
  const int owner = sh_int[n_warps];
  if (warp == owner) {
    int seen = sh_int[n_warps + 1];
    for (int base = begin; base < end; base += 32) {
      const int i = base + lane;
      const unsigned hits = __ballot_sync(0xffffffffu, i < end && p[i] == v);
      const int c = __popc(hits);
      if (j < seen + c) {
        // the (j - seen)-th set bit of hits
        unsigned h = hits;
        for (int k = 0; k < j - seen; ++k) h &= h - 1;
        if (lane == 0) sh_int[n_warps + 2] = base + __ffs(h) - 1;
        break;
      }
      seen += c;
    }
  }
  __syncthreads();
  const int found = sh_int[n_warps + 2];
  __syncthreads();
  return found;
}

// First index, in index order, whose running sum of p exceeds `target`; n-1 if none.
// The same two levels: sums of the warps' parts, then the owning warp walks its part in tiles of 32
// with a prefix sum by shuffles.
__device__ int first_cdf_above(const float* p, int n, float target, float* sh_f, int* sh_int) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  int begin, end;
  warp_range(n, warp, n_warps, begin, end);
  float mine = 0.f;
  for (int i = begin + lane; i < end; i += 32) mine += p[i];
  mine = warp_sum(mine);
  __syncthreads();
  if (lane == 0) sh_f[warp] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float before = 0.f;
    int owner = -1;
    for (int w = 0; w < n_warps; ++w) {
      if (target < before + sh_f[w]) { owner = w; break; }
      before += sh_f[w];
    }
    sh_int[0] = owner;
    sh_int[1] = n - 1;
    sh_f[n_warps] = before;
  }
  __syncthreads();
  const int owner = sh_int[0];
  if (warp == owner) {
    float before = sh_f[n_warps];
    int found = end - 1;  // rounding may leave the target just above the part's own sum
    for (int base = begin; base < end; base += 32) {
      const int i = base + lane;
      float x = i < end ? p[i] : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {  // inclusive prefix sum over the tile
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      const unsigned over = __ballot_sync(0xffffffffu, i < end && target < before + x);
      if (over) {
        found = base + __ffs(over) - 1;
        break;
      }
      before += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) sh_int[1] = found;
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
  __shared__ unsigned long long hist[HIST_COPIES * HIST_BINS];
  __shared__ unsigned long long hist_bins[HIST_BINS];
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
  float mx = -INFINITY;  // the largest logit / t is the largest logit, divided (t > 0): one division, not n
  sweep(row, n, [&](float v, int) { mx = fmaxf(mx, v); });
  mx = block_max(mx, red) / temperature;
  float part = 0.f;
  sweep(row, n, [&](float v, int i) {
    const float e = expf(v / temperature - mx);
    p[i] = e;
    part += e;
  });
  const float inv = 1.0f / block_sum(part, red);
  __syncthreads();
  sweep(p, n, [&](float v, int i) { p[i] = v * inv; });
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
        const uint32_t v_bits = select_mass(p, n, cutoff_bits, top_p, hist, hist_bins, &mass_gt);
        v_min = __uint_as_float(v_bits);
        const int ties = count_equal(p, n, v_bits, red);
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
        float s_gt;
        const uint32_t sel_bits = select_mass(p, n, __float_as_uint(v_min) + 1u, target, hist, hist_bins, &s_gt);
        const float v_sel = __uint_as_float(sel_bits);
        const int equals = count_equal(p, n, sel_bits, red);
        int j = (int)floorf((target - s_gt) / v_sel);
        j = min(max(j, 0), equals - 1);
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
