// Choosing the next token on the device, with the reference's rules
// (src/sampler.rs:801-819): temperature 0 is the argmax with the last of equal
// maxima (:78-84); otherwise logits / t (:101-106), an optional nucleus (:116-164)
// and one inverse-CDF draw (:190-216) from an xorshift64* stream (:176-187) that
// is kept per sequence.  The reference samples on the host after copying the
// logits back; here only the chosen token ids leave the device.
//
// A row is shared by a team of blocks (a thread-block cluster of up to 8, each on an SM of its own,
// each sweeping its part of the row; sums, histograms and counts meet through distributed shared
// memory): one block alone took 0.29 ms for a row of 128k, a quarter of it per sweep waiting on its
// own loads.  The nucleus is found without sorting: the probability
// that closes it is located digit by digit in the bit patterns of positive
// floats (their integer order is their numeric order): four sweeps over the
// row, each a histogram of probability mass over the next eight bits, instead
// of one sweep per bit.  The masses are added as 64-bit fixed-point numbers
// (2^-44), so the histogram's atomic additions give the same sums in whatever
// order they happen and a row of 128k probabilities is summed more exactly than
// in 32-bit floats; equal probabilities are taken in index order.  A draw that
// lands within rounding of a boundary of the cumulative distribution may pick
// the neighbouring token of the sequential 32-bit sum the reference does.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

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

// The reference's argmax compares with `!(best > candidate)`, which a NaN on either side makes true: a NaN
// takes the running maximum's place and is itself replaced by whatever follows it (src/sampler.rs:76-84, test
// :983-988).  The result is therefore the last of the equal maxima among the elements AFTER the row's last NaN,
// or that NaN's own index when it is the row's last element.  Only a broken model produces NaN logits, so
// the first scan also looks for the last NaN and a second scan over the elements after it runs only then.
__device__ int block_argmax_scan(const float* row, int lo, int n, float t, ArgMax* sh, int* last_nan_out) {
  ArgMax best = {-INFINITY, -1};
  int last_nan = -1;
  auto see = [&](float v, int i) {
    if (v != v) last_nan = max(last_nan, i);
    else best = better(best, ArgMax{v / t, i});
  };
  if (lo == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
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
        see(v[u].x, base);
        see(v[u].y, base + 1);
        see(v[u].z, base + 2);
        see(v[u].w, base + 3);
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = r4[i];
      see(v.x, 4 * i);
      see(v.y, 4 * i + 1);
      see(v.z, 4 * i + 2);
      see(v.w, 4 * i + 3);
    }
    for (int j = 4 * n4 + threadIdx.x; j < n; j += blockDim.x) see(row[j], j);
  } else {
    for (int i = lo + threadIdx.x; i < n; i += blockDim.x) see(row[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
    last_nan = max(last_nan, __shfl_xor_sync(0xffffffffu, last_nan, o));
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = best;
  __syncthreads();
  ArgMax r = sh[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) r = better(r, sh[w]);
  __syncthreads();
  if (lane == 0) sh[warp].i = last_nan;
  __syncthreads();
  int ln = sh[0].i;
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) ln = max(ln, sh[w].i);
  *last_nan_out = ln;
  return r.i;
}

__device__ int block_argmax(const float* row, int n, float t, ArgMax* sh) {
  int last_nan;
  const int idx = block_argmax_scan(row, 0, n, t, sh, &last_nan);
  if (last_nan < 0) return idx;
  if (last_nan == n - 1) return n - 1;
  int none;
  return block_argmax_scan(row, last_nan + 1, n, t, sh, &none);
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

// ---------------------------------------------------------------- sweeps over a part of a row
// f(value, index) for every element of p[begin..end), every thread of the block taking part.  A block
// that scans its part alone is bound by how many loads it has in flight, so an aligned part is read
// four values per load, four loads ahead.  The order in which a thread meets its elements is not the
// index order.
template <typename F>
__device__ __forceinline__ void sweep(const float* p, int begin, int end, F f) {
  const float* q = p + begin;
  const int n = end - begin;
  if ((reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    const int n4 = n >> 2;
    const float4* q4 = reinterpret_cast<const float4*>(q);
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < n4; i += 4 * blockDim.x) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = q4[i + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int base = begin + 4 * (i + u * blockDim.x);
        f(v[u].x, base);
        f(v[u].y, base + 1);
        f(v[u].z, base + 2);
        f(v[u].w, base + 3);
      }
    }
    for (; i < n4; i += blockDim.x) {
      const float4 v = q4[i];
      const int base = begin + 4 * i;
      f(v.x, base);
      f(v.y, base + 1);
      f(v.z, base + 2);
      f(v.w, base + 3);
    }
    for (int j = 4 * n4 + threadIdx.x; j < n; j += blockDim.x) f(q[j], begin + j);
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) f(q[i], begin + i);
  }
}

// ---------------------------------------------------------------- the team of blocks that shares a row
#define TEAM_MAX 8
#define HIST_COPIES 16   // two warps share a copy of the histogram
#define HIST_BINS 256
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
static_assert(SAMPLE_WARPS == 32, "the warps' totals are scanned by one warp, a lane each");

// What the blocks of a team leave for one another in their own shared memory.  Everything that is
// exchanged has two places used in turn, so that one cluster barrier per exchange is enough: a block can
// only write a place for the second time after a later barrier, which every reader of the first round
// has reached.
struct Exchange {
  float f[2][4];
  int i[2][4];
  unsigned long long bins[2][HIST_BINS];
};

struct Team {
  cg::cluster_group cluster;
  int rank, size;
  int begin, end;   // this block's part of the row, in index order by rank
  Exchange* x;      // this block's own
  int turn;
  float* red;       // 32 floats for block-wide reductions

  __device__ __forceinline__ const Exchange* of(int r) const { return cluster.map_shared_rank(x, r); }

  // sums of a and b over the whole row (every block gets the same values: added in rank order)
  __device__ void sum2(float a, float b, float& A, float& B) {
    a = block_sum(a, red);
    b = block_sum(b, red);
    if (threadIdx.x == 0) {
      x->f[turn][0] = a;
      x->f[turn][1] = b;
    }
    cluster.sync();
    A = 0.f;
    B = 0.f;
    for (int r = 0; r < size; ++r) {
      A += of(r)->f[turn][0];
      B += of(r)->f[turn][1];
    }
    turn ^= 1;
  }
  __device__ float sum(float a) {
    float A, B;
    sum2(a, 0.f, A, B);
    return A;
  }
  // the largest of unsigned values over the whole row
  __device__ uint32_t umax(uint32_t a) {
    a = __reduce_max_sync(0xffffffffu, a);
    uint32_t* redu = reinterpret_cast<uint32_t*>(red);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) redu[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x < 32) {
      a = __reduce_max_sync(0xffffffffu, redu[threadIdx.x]);  // SAMPLE_WARPS == 32
      if (threadIdx.x == 0) x->i[turn][2] = (int)a;
    }
    cluster.sync();
    uint32_t A = 0;
    for (int r = 0; r < size; ++r) A = max(A, (uint32_t)of(r)->i[turn][2]);
    turn ^= 1;
    return A;
  }
  __device__ float maximum(float a) {
    a = block_max(a, red);
    if (threadIdx.x == 0) x->f[turn][0] = a;
    cluster.sync();
    float A = -INFINITY;
    for (int r = 0; r < size; ++r) A = fmaxf(A, of(r)->f[turn][0]);
    turn ^= 1;
    return A;
  }
};

// ---------------------------------------------------------------- sampling

// Sum and count of the probabilities whose bit pattern is at least `lo_bits`.
__device__ __forceinline__ void masked_sum(Team& tm, const float* p, uint32_t lo_bits, float& sum, int& count) {
  float s = 0.f;
  float c = 0.f;
  sweep(p, tm.begin, tm.end, [&](float v, int) {
    if (__float_as_uint(v) >= lo_bits) {
      s += v;
      c += 1.f;
    }
  });
  float C;
  tm.sum2(s, c, sum, C);
  count = (int)C;
}

// Fixed-point masses: a probability as a multiple of 2^-44 (the sum of a whole row stays below 2^45).
#define MASS_ONE 17592186044416.0  // 2^44
__device__ __forceinline__ unsigned long long to_mass(float v) { return (unsigned long long)((double)v * MASS_ONE + 0.5); }
__device__ __forceinline__ float from_mass(unsigned long long m) { return (float)((double)m / MASS_ONE); }

// The elements of a[begin..end) carry a 32-bit key (0: not a candidate) and a 64-bit weight, both from
// kw(value, index, key, weight).  Finds the key k* with weight{key > k*} <= limit < weight{key >= k*}, digit
// by digit (8 bits a sweep).  If the candidates' whole weight does not exceed the limit, *fell is set and
// the smallest key among them is returned (0 if there is no candidate).  Leaves weight{key > k*} in
// *above_out.  hist: HIST_COPIES * HIST_BINS 64-bit words of shared memory.
// Every block of the team walks the same bins in the same order and so takes the same decisions.
template <typename KW>
__device__ uint32_t select_desc(Team& tm, const float* p, KW kw, unsigned long long limit_m, unsigned long long* hist,
                                unsigned long long* total_bins, unsigned long long* above_out, bool* fell) {
  __shared__ uint32_t sel_prefix;
  __shared__ unsigned long long sel_above;
  __shared__ int sel_fell;
  uint32_t prefix = 0, prefix_mask = 0;
  unsigned long long above = 0;  // mass of the candidates above the prefix's range
  unsigned long long* mine = hist + (threadIdx.x >> 6) * HIST_BINS;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < HIST_COPIES * HIST_BINS; i += blockDim.x) hist[i] = 0ull;
    __syncthreads();
    sweep(p, tm.begin, tm.end, [&](float v, int i) {
      uint32_t key;
      unsigned long long w;
      kw(v, i, key, w);
      if (key != 0u && (key & prefix_mask) == prefix) atomicAdd(&mine[(key >> shift) & (HIST_BINS - 1)], w);
    });
    __syncthreads();
    if (threadIdx.x < HIST_BINS) {
      unsigned long long m = 0;
#pragma unroll
      for (int c = 0; c < HIST_COPIES; ++c) m += hist[c * HIST_BINS + threadIdx.x];
      tm.x->bins[tm.turn][threadIdx.x] = m;
    }
    tm.cluster.sync();
    if (threadIdx.x < HIST_BINS) {
      unsigned long long m = 0;
      for (int r = 0; r < tm.size; ++r) m += tm.of(r)->bins[tm.turn][threadIdx.x];
      total_bins[threadIdx.x] = m;
    }
    tm.turn ^= 1;
    __syncthreads();
    if (threadIdx.x < 32) {
      // warp 0 walks the bins from the top: lane l owns bins 8l .. 8l+7; the masses above a lane's bins
      // come from a suffix sum over the lanes, then each lane walks its own eight
      const int lane = threadIdx.x;
      unsigned long long own[8], lane_total = 0;
      unsigned nonzero = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        own[e] = total_bins[8 * lane + e];
        lane_total += own[e];
        nonzero |= (own[e] != 0ull) << e;
      }
      unsigned long long higher = lane_total;  // inclusive suffix sum over lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long y = __shfl_down_sync(0xffffffffu, higher, o);
        if (lane + o < 32) higher += y;
      }
      unsigned long long acc = above + higher - lane_total;
      int hit = -1;
      unsigned long long acc_hit = 0;
#pragma unroll
      for (int e = 7; e >= 0; --e) {
        if (hit < 0 && own[e] != 0ull && acc + own[e] > limit_m) {
          hit = e;
          acc_hit = acc;
        }
        acc += own[e];
      }
      const unsigned hits = __ballot_sync(0xffffffffu, hit >= 0);
      const unsigned filled = __ballot_sync(0xffffffffu, nonzero != 0u);
      if (hits) {
        if (lane == 31 - __clz(hits)) {  // the highest lane with a hit holds the first bin from the top
          sel_prefix = prefix | ((uint32_t)(8 * lane + hit) << shift);
          sel_above = acc_hit;
          sel_fell = 0;
        }
      } else if (filled) {  // rounding: the candidates' mass does not exceed the limit after all
        if (lane == __ffs(filled) - 1) {
          const int e = __ffs(nonzero) - 1;  // the lowest bin that holds anything
          // (the bins below e in this lane and all lower lanes are empty, so `higher` is all the mass)
          sel_prefix = prefix | ((uint32_t)(8 * lane + e) << shift);
          sel_above = above + higher - own[e];
          sel_fell = 1;
        }
      } else if (lane == 0) {  // no candidate at all
        sel_prefix = prefix;
        sel_above = above;
        sel_fell = 1;
      }
    }
    __syncthreads();
    prefix = sel_prefix;
    above = sel_above;
    prefix_mask |= (uint32_t)(HIST_BINS - 1) << shift;
    __syncthreads();
  }
  *above_out = above;
  *fell = sel_fell != 0;
  return prefix;
}

// Among the probabilities whose bit pattern is at least `lo_bits`: the value v* with
// mass{p > v*} <= limit < mass{p >= v*} (the caller guarantees that their whole mass exceeds `limit`;
// if rounding says otherwise the smallest of them is returned).  Returns v*'s bit pattern and leaves
// mass{p > v*} in *mass_gt.
__device__ uint32_t select_mass(Team& tm, const float* p, uint32_t lo_bits, float limit, unsigned long long* hist,
                                unsigned long long* total_bins, float* mass_gt) {
  unsigned long long above;
  bool fell;
  const uint32_t bits = select_desc(
      tm, p,
      [&](float v, int, uint32_t& key, unsigned long long& w) {
        const uint32_t b = __float_as_uint(v);
        key = b >= lo_bits ? b : 0u;
        w = to_mass(v);
      },
      to_mass(fmaxf(limit, 0.f)), hist, total_bins, &above, &fell);
  *mass_gt = from_mass(above);
  return bits;
}

// How many probabilities have exactly the bit pattern `bits`.
__device__ int count_equal(Team& tm, const float* p, uint32_t bits) {
  float c = 0.f;
  sweep(p, tm.begin, tm.end, [&](float v, int) { c += (__float_as_uint(v) == bits) ? 1.f : 0.f; });
  return (int)tm.sum(c);
}

// Smallest probability whose bit pattern is at least `b` (the value that closes the set).
__device__ float min_at_least(Team& tm, const float* p, uint32_t b) {
  float m = INFINITY;
  sweep(p, tm.begin, tm.end, [&](float v, int) {
    if (__float_as_uint(v) >= b) m = fminf(m, v);
  });
  return -tm.maximum(-m);
}

// The part of a block's part that one of its warps owns (contiguous, whole tiles of 32: index order matters).
__device__ __forceinline__ void warp_range(const Team& tm, int warp, int& begin, int& end) {
  const int n = tm.end - tm.begin;
  const int per = (((n + SAMPLE_WARPS - 1) / SAMPLE_WARPS) + 31) & ~31;
  begin = tm.begin + min(n, warp * per);
  end = min(tm.end, begin + per);
}

// Index of the j-th (from 0) element equal to `v`, in index order; -1 if there are fewer.  With
// `clamp`, j is first brought into 0 .. (number of equals - 1).
// Every warp of every block counts the matches in its contiguous part (coalesced loads).  The counts are
// added up in index order on two levels, the warps of a block by a scan in its first warp and the blocks
// by a scan that every warp makes for itself from the exchanged totals; the warp whose part holds the
// j-th match walks it in tiles of 32, a ballot per tile, and the whole team reads the answer from that block.
__device__ int kth_equal(Team& tm, const float* p, float v, int j, bool clamp) {
  __shared__ int found_s;
  __shared__ int warp_incl[SAMPLE_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int begin, end;
  warp_range(tm, warp, begin, end);
  int mine = 0;
  for (int i = begin + lane; i < end; i += 32) mine += (p[i] == v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
  if (lane == 0) warp_incl[warp] = mine;
  if (threadIdx.x == 0) found_s = -1;
  __syncthreads();
  if (warp == 0) {
    int x = warp_incl[lane];  // SAMPLE_WARPS == 32
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    warp_incl[lane] = x;
    if (lane == 31) tm.x->i[tm.turn][1] = x;
  }
  tm.cluster.sync();
  const int tot = lane < tm.size ? tm.of(lane)->i[tm.turn][1] : 0;
  int incl = tot;
#pragma unroll
  for (int o = 1; o < TEAM_MAX; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  const int total = __shfl_sync(0xffffffffu, incl, tm.size - 1);
  if (clamp) j = min(max(j, 0), total - 1);
  const unsigned hit = __ballot_sync(0xffffffffu, lane < tm.size && j >= incl - tot && j < incl);
  const int owner_rank = hit ? __ffs(hit) - 1 : -1;
  if (owner_rank == tm.rank) {
    const int jj = j - __shfl_sync(0xffffffffu, incl - tot, owner_rank);
    int seen = warp ? warp_incl[warp - 1] : 0;
    if (jj >= seen && jj < warp_incl[warp]) {
      for (int base = begin; base < end; base += 32) {
        const int i = base + lane;
        const unsigned hits = __ballot_sync(0xffffffffu, i < end && p[i] == v);
        const int c = __popc(hits);
        if (jj < seen + c) {
          unsigned h = hits;
          for (int k = 0; k < jj - seen; ++k) h &= h - 1;  // drop the matches before the wanted one
          if (lane == 0) found_s = base + __ffs(h) - 1;
          break;
        }
        seen += c;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tm.x->i[tm.turn][0] = found_s;
  tm.cluster.sync();
  const int found = owner_rank < 0 ? -1 : tm.of(owner_rank)->i[tm.turn][0];
  tm.turn ^= 1;
  return found;
}

// First index, in index order, whose running sum of p exceeds `target`; n-1 if none.
// The same two levels with sums in the place of counts; the owning warp walks its part in tiles of 32
// with a prefix sum by shuffles.
__device__ int first_cdf_above(Team& tm, const float* p, int n, float target) {
  __shared__ int found_s;
  __shared__ float warp_incl[SAMPLE_WARPS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int begin, end;
  warp_range(tm, warp, begin, end);
  float mine = 0.f;
  for (int i = begin + lane; i < end; i += 32) mine += p[i];
  mine = warp_sum(mine);
  if (lane == 0) warp_incl[warp] = mine;
  if (threadIdx.x == 0) found_s = n - 1;
  __syncthreads();
  if (warp == 0) {
    float x = warp_incl[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    warp_incl[lane] = x;
    if (lane == 31) tm.x->f[tm.turn][1] = x;
  }
  tm.cluster.sync();
  const float tot = lane < tm.size ? tm.of(lane)->f[tm.turn][1] : 0.f;
  float incl = tot;
#pragma unroll
  for (int o = 1; o < TEAM_MAX; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  const float excl = __shfl_up_sync(0xffffffffu, incl, 1);
  const unsigned hit = __ballot_sync(0xffffffffu, lane < tm.size && target < incl);
  const int owner_rank = hit ? __ffs(hit) - 1 : -1;
  if (owner_rank == tm.rank) {
    const float before_rank = owner_rank ? __shfl_sync(0xffffffffu, excl, owner_rank) : 0.f;
    // the first warp whose running sum passes the target (rounding may leave it just above the block's
    // own sum: then the last warp, and the last index of its part)
    const unsigned whit = __ballot_sync(0xffffffffu, target < before_rank + warp_incl[lane]);
    const int owner_warp = whit ? __ffs(whit) - 1 : SAMPLE_WARPS - 1;
    if (warp == owner_warp) {
      float before = before_rank + (warp ? warp_incl[warp - 1] : 0.f);
      int found = max(end - 1, 0);
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
      if (lane == 0) found_s = found;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tm.x->i[tm.turn][0] = found_s;
  tm.cluster.sync();
  const int found = owner_rank < 0 ? n - 1 : tm.of(owner_rank)->i[tm.turn][0];
  tm.turn ^= 1;
  return found;
}

// The argmax of logits / t over the whole row, last of equal maxima.
__device__ int team_argmax(Team& tm, const float* row, float t, ArgMax* sh) {
  ArgMax best = {-INFINITY, -1};
  sweep(row, tm.begin, tm.end, [&](float v, int i) { best = better(best, ArgMax{v / t, i}); });
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other;
    other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
    other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
    best = better(best, other);
  }
  __syncthreads();
  if (lane == 0) sh[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgMax r = sh[0];
    for (int w = 1; w < SAMPLE_WARPS; ++w) r = better(r, sh[w]);
    tm.x->f[tm.turn][0] = r.v;
    tm.x->i[tm.turn][0] = r.i;
  }
  tm.cluster.sync();
  ArgMax all = {-INFINITY, -1};
  for (int r = 0; r < tm.size; ++r) all = better(all, ArgMax{tm.of(r)->f[tm.turn][0], tm.of(r)->i[tm.turn][0]});
  tm.turn ^= 1;
  return all.i;
}

// grid: (team size, rows), clusters of (team size, 1, 1)
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int n, float temperature, float top_p,
              unsigned long long* __restrict__ rng_states, const int* __restrict__ rng_index,
              float* __restrict__ probs, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ ArgMax sh_arg[32];
  __shared__ Exchange exchange;
  __shared__ unsigned long long hist[HIST_COPIES * HIST_BINS];
  __shared__ unsigned long long total_bins[HIST_BINS];
  Team tm = {cg::this_cluster(), 0, 0, 0, 0, &exchange, 0, red};
  tm.rank = (int)tm.cluster.block_rank();
  tm.size = (int)tm.cluster.num_blocks();
  {
    const int per = (((n + tm.size - 1) / tm.size) + 3) & ~3;  // parts that keep the row's 16-byte alignment
    tm.begin = min(n, tm.rank * per);
    tm.end = min(n, tm.begin + per);
  }
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * row_stride;
  float* p = probs + (size_t)r * n;

  // one draw per sampled token (src/sampler.rs:176-187): the first block draws, the others read it after
  // the first exchange below
  if (tm.rank == 0 && threadIdx.x == 0) {
    unsigned long long* st = rng_states + rng_index[r];
    unsigned long long s = *st;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *st = s;
    const uint32_t u = (uint32_t)((s * 0x2545F4914F6CDD1DULL) >> 32);
    exchange.f[0][3] = (float)(u >> 8) / 16777216.0f;
  }

  // softmax of logits / t (src/sampler.rs:58-73, :101-106)
  float mx = -INFINITY;  // the largest logit / t is the largest logit, divided (t > 0): one division, not n
  sweep(row, tm.begin, tm.end, [&](float v, int) { mx = fmaxf(mx, v); });
  mx = tm.maximum(mx) / temperature;  // (turn 0: the coin lies in the same place of the first block)
  const float coin = tm.of(0)->f[0][3];
  float part = 0.f;
  sweep(row, tm.begin, tm.end, [&](float v, int i) {
    const float e = expf(v / temperature - mx);
    p[i] = e;
    part += e;
  });
  const float inv = 1.0f / tm.sum(part);
  __syncthreads();
  sweep(p, tm.begin, tm.end, [&](float v, int i) { p[i] = v * inv; });
  __syncthreads();

  int chosen;
  if (!(top_p > 0.f && top_p < 1.f)) {
    chosen = first_cdf_above(tm, p, n, coin);
  } else {
    // candidates must reach (1 - top_p) / (n - 1) (src/sampler.rs:127-134)
    const float cutoff = (1.0f - top_p) / (float)max(n - 1, 1);
    const uint32_t cutoff_bits = __float_as_uint(cutoff);
    float kept_mass;
    int kept;
    masked_sum(tm, p, cutoff_bits, kept_mass, kept);
    if (kept == 0) {
      chosen = team_argmax(tm, row, temperature, sh_arg);  // (src/sampler.rs:135-144)
    } else {
      // the value that closes the nucleus, the mass above it, and how many of its equals are in
      float v_min, mass_gt;
      int ties_in;
      if (!(kept_mass > top_p)) {  // the mass never exceeds top_p: everything kept stays (:150-158)
        v_min = min_at_least(tm, p, cutoff_bits);
        float s_ge; int c_ge, c_gt;
        masked_sum(tm, p, __float_as_uint(v_min), s_ge, c_ge);
        masked_sum(tm, p, __float_as_uint(v_min) + 1u, mass_gt, c_gt);
        ties_in = c_ge - c_gt;
      } else {
        const uint32_t v_bits = select_mass(tm, p, cutoff_bits, top_p, hist, total_bins, &mass_gt);
        v_min = __uint_as_float(v_bits);
        const int ties = count_equal(tm, p, v_bits);
        int need = (int)floorf((top_p - mass_gt) / v_min) + 1;  // smallest count whose sum exceeds top_p
        ties_in = min(max(need, 1), ties);
      }
      const float nucleus_mass = mass_gt + (float)ties_in * v_min;
      const float target = coin * nucleus_mass;  // (src/sampler.rs:199-204)
      if (!(mass_gt > target)) {
        // falls among the equals that close the nucleus
        int j = (int)floorf((target - mass_gt) / v_min);
        j = min(max(j, 0), ties_in - 1);
        chosen = kth_equal(tm, p, v_min, j, false);
      } else {
        // largest value whose "at least" mass exceeds the target, within the part above v_min
        float s_gt;
        const uint32_t sel_bits = select_mass(tm, p, __float_as_uint(v_min) + 1u, target, hist, total_bins, &s_gt);
        const float v_sel = __uint_as_float(sel_bits);
        const int j = (int)floorf((target - s_gt) / v_sel);
        chosen = kth_equal(tm, p, v_sel, j, true);  // j brought into the number of equals
      }
      if (chosen < 0) chosen = team_argmax(tm, row, temperature, sh_arg);
    }
  }
  if (tm.rank == 0 && threadIdx.x == 0) out[r] = chosen;
  tm.cluster.sync();  // nobody leaves while a team mate may still read its shared memory
}

// ---------------------------------------------------------------- the longer chain
// penalties -> DRY -> top-k -> top-p -> min-p -> XTC -> temperature -> draw (or argmax), the order of the reference's
// chain when any of its further knobs is set (src/sampler.rs:821-931); with mirostat, penalties -> DRY ->
// temperature -> mirostat's own cut and draw (:829-866).  Every filter of that chain keeps
// a prefix of the candidates in descending order, so the survivors are always "all logits above a
// threshold, and the first E (by index) of those equal to it": the kernel carries (threshold key, E)
// from stage to stage and never sorts.  Equal logits are taken in index order where the reference's
// unstable sorts leave the order open.

// Keys: the bit pattern of a float made monotone (larger float, larger key); 0 is never a finite float's.
__device__ __forceinline__ uint32_t okey(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unkey(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct ChainParams {
  float temperature, top_p, min_p;
  float repeat_penalty, frequency_penalty, presence_penalty;
  int top_k, last_n;
  int mirostat;             // 0, or 1 / 2: the mode that replaces top-k, top-p and min-p (src/sampler.rs:829-866)
  float mirostat_tau, mirostat_eta;
  float xtc_probability, xtc_threshold;  // "exclude top choices", after min-p (src/sampler.rs:569-602); 0 = off
  // DRY, after the penalties (src/sampler.rs:683-733): off when the multiplier is 0, the base below 1 or the window 0
  float dry_multiplier, dry_base;
  int dry_allowed_length, dry_last_n, dry_n_breakers;
  int dry_breakers[8];  // tokens that a repeat may not cross
};

#define MIROSTAT_M 100  // candidates of the Zipf estimate of mirostat 1 (the reference's mirostat_m)
#define MIROSTAT_LIST 128

#define HISTORY_MAX 1024  // tokens of history that the penalties and DRY can look back on
#define DRY_MAX_BREAKERS 8

// f(value, index, sum, count) adds to two running sums; their totals over the whole row come back.
template <typename F>
__device__ __forceinline__ void team_sum2(Team& tm, const float* a, F f, float& A, float& B) {
  float s = 0.f, c = 0.f;
  sweep(a, tm.begin, tm.end, [&](float v, int i) { f(v, i, s, c); });
  tm.sum2(s, c, A, B);
}

// grid: (team size, rows), clusters of (team size, 1, 1).  work: per row 2 * n_pad floats (the penalised
// logits, then the weights of the current softmax).  history[slot][HISTORY_MAX] is a ring of the sequence's
// chosen tokens, the p-th of them at p % HISTORY_MAX, history_count[slot] of them so far: the penalties read
// its last `last_n` (src/sampler.rs:339-347), DRY its last `dry_last_n` (:735-743).
// mirostat_mu[slot]: the surprise ceiling that mirostat adapts, NaN for a sequence that has not drawn yet.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_chain_kernel(const float* __restrict__ logits, long long row_stride, int n, int n_pad, ChainParams cp,
                    unsigned long long* __restrict__ rng_states, const int* __restrict__ slot_of_row,
                    int* __restrict__ history, int* __restrict__ history_count, float* __restrict__ mirostat_mu,
                    unsigned long long* __restrict__ xtc_states, float* __restrict__ work, int* __restrict__ out) {
  __shared__ float red[32];
  __shared__ ArgMax sh_arg[32];
  __shared__ Exchange exchange;
  __shared__ unsigned long long hist[HIST_COPIES * HIST_BINS];
  __shared__ unsigned long long total_bins[HIST_BINS];
  __shared__ int ring[HISTORY_MAX];
  Team tm = {cg::this_cluster(), 0, 0, 0, 0, &exchange, 0, red};
  tm.rank = (int)tm.cluster.block_rank();
  tm.size = (int)tm.cluster.num_blocks();
  {
    const int per = (((n + tm.size - 1) / tm.size) + 3) & ~3;
    tm.begin = min(n, tm.rank * per);
    tm.end = min(n, tm.begin + per);
  }
  const int r = blockIdx.y;
  const int slot = slot_of_row[r];
  const float* row = logits + (size_t)r * row_stride;
  float* L = work + (size_t)r * 2 * n_pad;
  float* q = L + n_pad;
  const bool draws = cp.temperature != 0.f;

  // one draw per sampled token, none for the argmax (src/sampler.rs:190-193, :225-228)
  if (draws && tm.rank == 0 && threadIdx.x == 0) {
    unsigned long long* st = rng_states + slot;
    unsigned long long s = *st;
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    *st = s;
    const uint32_t u = (uint32_t)((s * 0x2545F4914F6CDD1DULL) >> 32);
    exchange.f[0][3] = (float)(u >> 8) / 16777216.0f;
  }

  // ---- penalties over the ring of accepted tokens (src/sampler.rs:314-337)
  sweep(row, tm.begin, tm.end, [&](float v, int i) { L[i] = v; });
  const bool penalties_on = cp.repeat_penalty != 1.f || cp.frequency_penalty != 0.f || cp.presence_penalty != 0.f;
  const bool dry_on = cp.dry_multiplier != 0.f && !(cp.dry_base < 1.f) && cp.dry_last_n > 0;
  const bool records = cp.last_n > 0 || dry_on;
  const int accepted = records ? history_count[slot] : 0;
  const int* past = history + (size_t)slot * HISTORY_MAX;
  const int valid = min(accepted, cp.last_n);
  if (penalties_on && valid > 0) {
    for (int j = threadIdx.x; j < valid; j += blockDim.x) ring[j] = past[(accepted - valid + j) % HISTORY_MAX];
    __syncthreads();  // (also orders the writes of L above before the changes below)
    for (int j = threadIdx.x; j < valid; j += blockDim.x) {
      const int t = ring[j];
      if (t < tm.begin || t >= tm.end) continue;  // another block's, or no token of this vocabulary
      int cnt = 0;
      bool first = true;
      for (int jj = 0; jj < valid; ++jj) {
        if (ring[jj] == t) {
          ++cnt;
          if (jj < j) first = false;
        }
      }
      if (first) {
        float l = L[t];
        l = l > 0.f ? l / cp.repeat_penalty : l * cp.repeat_penalty;
        l -= (float)cnt * cp.frequency_penalty;
        l -= cp.presence_penalty;
        L[t] = l;
      }
    }
  }
  __syncthreads();

  // ---- DRY: a token that would make the end of the history repeat an earlier stretch of it loses
  // multiplier * base^(length of the repeat - allowed length) (src/sampler.rs:683-733)
  const int dry_n = dry_on ? min(accepted, cp.dry_last_n) : 0;
  if (dry_n > max(cp.dry_allowed_length, 1)) {
    __shared__ int rep_limit_s;
    const int allowed = max(cp.dry_allowed_length, 1);
    int* rev = ring;                                 // the window, newest first
    int* rep_len = reinterpret_cast<int*>(hist);     // [k]: length of the repeat that rev[k - 1] would complete, or 0
    if (threadIdx.x == 0) rep_limit_s = dry_n;
    for (int i = threadIdx.x; i < dry_n; i += blockDim.x) rev[i] = past[(accepted - 1 - i) % HISTORY_MAX];
    __syncthreads();
    // the window ends before the most recent breaker
    for (int i = threadIdx.x; i < dry_n; i += blockDim.x)
      for (int b = 0; b < cp.dry_n_breakers; ++b)
        if (rev[i] == cp.dry_breakers[b]) atomicMin(&rep_limit_s, i);
    __syncthreads();
    const int limit = rep_limit_s;
    if (limit > allowed) {
      // z[k]: how far the window from k on agrees with the window from 0 on (the reference's Z array of
      // the reversed window, here by direct comparison: the window has at most 1024 tokens)
      for (int k = threadIdx.x; k < limit; k += blockDim.x) {
        int z = 0;
        if (k >= 1) {
          while (k + z < limit && rev[z] == rev[k + z]) ++z;
          rep_len[k] = (z + 1 >= allowed) ? z + 1 : 0;
        } else {
          rep_len[k] = 0;
        }
      }
      __syncthreads();
      for (int k = 1 + (int)threadIdx.x; k < limit; k += blockDim.x) {
        const int len = rep_len[k];
        const int t = rev[k - 1];  // the token that followed the earlier stretch
        if (len == 0 || t < tm.begin || t >= tm.end) continue;
        bool longest = true;  // of all places with this continuation, the longest repeat (the first of equals) counts
        for (int kk = 1; kk < limit; ++kk)
          if (rev[kk - 1] == t && (rep_len[kk] > len || (rep_len[kk] == len && kk < k))) longest = false;
        if (longest) {
          float pw = 1.f, b = cp.dry_base;  // base^(len - allowed) by squaring, as powi does
          for (int e = len - allowed; e > 0; e >>= 1) {
            if (e & 1) pw *= b;
            b *= b;
          }
          L[t] -= cp.dry_multiplier * pw;
        }
      }
    }
    __syncthreads();
  }

  float mx_l = -INFINITY;
  sweep(L, tm.begin, tm.end, [&](float v, int) { mx_l = fmaxf(mx_l, v); });
  mx_l = tm.maximum(mx_l);
  const float coin = draws ? tm.of(0)->f[0][3] : 0.f;

  // survivors: key > T, and the first E (by index) of key == T; N of them
  uint32_t T = 0;
  int E = 0, N = n;
  bool filtered = false, collapsed = false;

  // ---- mirostat: temperature first, then its own cut in the place of top-k, top-p and min-p
  float mu = 0.f;
  if (cp.mirostat != 0) {
    __shared__ float cand[MIROSTAT_LIST], all[MIROSTAT_LIST], sorted[MIROSTAT_LIST];
    __shared__ int cand_n, keep_s;
    mu = mirostat_mu[slot];
    if (!(mu == mu)) mu = 2.0f * cp.mirostat_tau;  // a new sequence (src/sampler.rs:379, :451-453)
    const float t = cp.temperature, mx_t = mx_l / t;
    float sum_all, unused;
    team_sum2(tm, L, [&](float v, int, float& s, float&) { s += expf(v / t - mx_t); }, sum_all, unused);
    const float inv_all = 1.0f / sum_all;
    sweep(L, tm.begin, tm.end, [&](float v, int i) { q[i] = expf(v / t - mx_t) * inv_all; });
    __syncthreads();
    if (cp.mirostat == 2) {
      // the candidates, in descending order, up to the first whose surprise -log2 p exceeds mu; at least
      // one (src/sampler.rs:501-506)
      uint32_t inv_key = 0;
      sweep(L, tm.begin, tm.end, [&](float v, int i) { if (!(-log2f(q[i]) > mu)) inv_key = max(inv_key, ~okey(v)); });
      const uint32_t lowest = tm.umax(inv_key);
      if (lowest != 0u) {
        T = ~lowest;
        float cnt, unused2;
        team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) == T ? 1.f : 0.f; }, cnt, unused2);
        E = (int)cnt;
      } else {  // none: the first of the sorted candidates stays
        T = okey(mx_l);
        E = 1;
      }
    } else {
      // mirostat 1: the Zipf exponent from the ratios of the MIROSTAT_M largest probabilities, and from it
      // the number of candidates that keeps the expected surprise near mu (src/sampler.rs:401-431)
      const int mm = min(MIROSTAT_M, n);
      unsigned long long above;
      bool fell;
      const uint32_t key_m = select_desc(
          tm, L, [&](float v, int, uint32_t& key, unsigned long long& w) { key = okey(v); w = 1ull; },
          (unsigned long long)(mm - 1), hist, total_bins, &above, &fell);
      if (threadIdx.x == 0) cand_n = 0;
      __syncthreads();
      sweep(L, tm.begin, tm.end, [&](float v, int i) {
        if (okey(v) > key_m) {
          const int at = atomicAdd(&cand_n, 1);
          if (at < MIROSTAT_LIST) cand[at] = q[i];
        }
      });
      tm.cluster.sync();
      // every block gathers all blocks' candidates (fewer than mm) and fills up with the mm-th largest value
      const float q_m = expf(unkey(key_m) / t - mx_t) * inv_all;
      if (threadIdx.x < MIROSTAT_LIST) {
        int j = threadIdx.x;
        float v = threadIdx.x < mm ? q_m : -1.f;  // (places past mm sort to the end)
        for (int rk = 0; rk < tm.size; ++rk) {
          const int c = min(*tm.cluster.map_shared_rank(&cand_n, rk), MIROSTAT_LIST);
          if (j < c) {
            v = tm.cluster.map_shared_rank(cand, rk)[j];
            break;
          }
          j -= c;
        }
        all[threadIdx.x] = v;
      }
      __syncthreads();
      if (threadIdx.x < MIROSTAT_LIST) {
        // descending order by counting, for each value, the larger ones and the equal ones before it
        const float mine = all[threadIdx.x];
        int place = 0;
        for (int k = 0; k < MIROSTAT_LIST; ++k) place += (all[k] > mine || (all[k] == mine && k < (int)threadIdx.x)) ? 1 : 0;
        sorted[place] = mine;
      }
      tm.cluster.sync();  // (also: nobody leaves this part while a team mate still reads its list)
      if (threadIdx.x == 0) {
        const int bound = min(max(MIROSTAT_M - 1, 0), max(n - 1, 0));
        double sum_ti_bi = 0.0, sum_ti_sq = 0.0;
        for (int i = 0; i < bound; ++i) {
          const double t_i = log((double)(i + 2) / (double)(i + 1));
          const double b_i = log((double)sorted[i] / (double)sorted[i + 1]);
          sum_ti_bi += t_i * b_i;
          sum_ti_sq += t_i * t_i;
        }
        const double s_hat = sum_ti_bi / sum_ti_sq;
        const double epsilon_hat = s_hat - 1.0;
        const double k = pow((epsilon_hat * pow(2.0, (double)mu)) / (1.0 - pow(-epsilon_hat, (double)n)), 1.0 / s_hat);
        long long keep = isfinite(k) ? (k >= 9.2e18 ? 0x7fffffffffffffffLL : (k <= -9.2e18 ? -0x7fffffffffffffffLL - 1 : (long long)k)) : 1;
        keep = keep < 1 ? 1 : keep;
        keep_s = (int)(keep > n ? n : keep);
      }
      __syncthreads();
      const int keep = keep_s;
      if (keep < n) {
        T = select_desc(
            tm, L, [&](float v, int, uint32_t& key, unsigned long long& w) { key = okey(v); w = 1ull; },
            (unsigned long long)(keep - 1), hist, total_bins, &above, &fell);
        E = keep - (int)above;
      }
    }
    filtered = true;
  }

  // ---- top-k (src/sampler.rs:239-251)
  if (cp.mirostat == 0 && cp.top_k > 0 && cp.top_k < N) {
    unsigned long long above;
    bool fell;
    T = select_desc(
        tm, L, [&](float v, int, uint32_t& key, unsigned long long& w) { key = okey(v); w = 1ull; },
        (unsigned long long)(cp.top_k - 1), hist, total_bins, &above, &fell);
    E = cp.top_k - (int)above;
    N = cp.top_k;
    filtered = true;
  }

  // ---- top-p over the softmax of the survivors (src/sampler.rs:120-160)
  if (cp.mirostat == 0 && cp.top_p > 0.f && cp.top_p < 1.f) {
    float sum_gt, unused;
    team_sum2(tm, L, [&](float v, int, float& s, float&) { if (okey(v) > T) s += expf(v - mx_l); }, sum_gt, unused);
    const float e_t = E > 0 ? expf(unkey(T) - mx_l) : 0.f;
    const float inv = 1.0f / (sum_gt + (float)E * e_t);
    sweep(L, tm.begin, tm.end, [&](float v, int i) { q[i] = expf(v - mx_l) * inv; });
    __syncthreads();
    const float q_t = e_t * inv;
    const float cutoff = (1.0f - cp.top_p) / (float)max(N - 1, 1);
    float kept_gt_mass, kept_gt_count;
    team_sum2(tm, L, [&](float v, int i, float& s, float& c) {
      if (okey(v) > T && q[i] >= cutoff) { s += q[i]; c += 1.f; }
    }, kept_gt_mass, kept_gt_count);
    const bool t_in = E > 0 && q_t >= cutoff;
    const int kept = (int)kept_gt_count + (t_in ? E : 0);
    const float kept_mass = kept_gt_mass + (t_in ? (float)E * q_t : 0.f);
    if (kept == 0) {
      collapsed = true;  // the argmax alone (:135-144)
    } else if (!(kept_mass > cp.top_p)) {
      // the mass never exceeds top_p: everything kept stays (:150-158)
      if (!t_in) {
        uint32_t inv_key = 0;
        sweep(L, tm.begin, tm.end, [&](float v, int i) { if (okey(v) > T && q[i] >= cutoff) inv_key = max(inv_key, ~okey(v)); });
        T = ~tm.umax(inv_key);
        float cnt, unused2;
        team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) == T ? 1.f : 0.f; }, cnt, unused2);
        E = (int)cnt;
      }
    } else {
      unsigned long long above;
      bool fell;
      const uint32_t k_sel = select_desc(
          tm, L, [&](float v, int i, uint32_t& key, unsigned long long& w) {
            const uint32_t k = okey(v);
            key = (k > T && q[i] >= cutoff) ? k : 0u;
            w = to_mass(q[i]);
          },
          to_mass(cp.top_p), hist, total_bins, &above, &fell);
      if (fell && t_in) {
        // the nucleus closes among the equals at the old threshold
        const int need = (int)floorf((cp.top_p - kept_gt_mass) / q_t) + 1;
        E = min(max(need, 1), E);
      } else {
        const float q_sel = expf(unkey(k_sel) - mx_l) * inv;
        float cnt, unused2;
        team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) == k_sel ? 1.f : 0.f; }, cnt, unused2);
        const int need = (int)floorf((cp.top_p - from_mass(above)) / q_sel) + 1;
        E = min(max(need, 1), (int)cnt);
        T = k_sel;
      }
    }
    if (!collapsed) {
      float cnt_gt, unused3;
      team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) > T ? 1.f : 0.f; }, cnt_gt, unused3);
      N = (int)cnt_gt + E;
    }
    filtered = true;
  }

  // ---- min-p in logit space: logit >= max + ln p, at least one (src/sampler.rs:265-281)
  if (cp.mirostat == 0 && !collapsed && cp.min_p > 0.f && N >= 2) {
    const uint32_t tk = okey(mx_l + logf(cp.min_p));
    if (tk > T) {
      float c_ge, unused;
      team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) >= tk ? 1.f : 0.f; }, c_ge, unused);
      if ((int)c_ge == 0) {
        collapsed = true;  // p > 1: the first of the sorted candidates stays, a largest logit
      } else {
        uint32_t inv_key = 0;
        sweep(L, tm.begin, tm.end, [&](float v, int) { if (okey(v) >= tk) inv_key = max(inv_key, ~okey(v)); });
        T = ~tm.umax(inv_key);
        float cnt, unused2;
        team_sum2(tm, L, [&](float v, int, float& s, float&) { s += okey(v) == T ? 1.f : 0.f; }, cnt, unused2);
        E = (int)cnt;
        N = (int)c_ge;
      }
    }
    filtered = true;
  }

  // ---- XTC: with a probability of its own, all but the least likely of the candidates above a threshold go
  // (src/sampler.rs:569-602).  What goes is struck from the working logits (minus infinity), so the stages
  // below need no upper bound.
  if (cp.mirostat == 0 && !collapsed && cp.xtc_probability > 0.f && !(cp.xtc_threshold > 0.5f) && N >= 2) {
    // its own generator, started from the same seed; one draw whether or not the filter then acts
    if (tm.rank == 0 && threadIdx.x == 0) {
      unsigned long long* st = xtc_states + slot;
      unsigned long long z = *st;
      z ^= z >> 12;
      z ^= z << 25;
      z ^= z >> 27;
      *st = z;
      exchange.f[tm.turn][2] = (float)((uint32_t)((z * 0x2545F4914F6CDD1DULL) >> 32) >> 8) / 16777216.0f;
    }
    tm.cluster.sync();
    const float chance = tm.of(0)->f[tm.turn][2];
    tm.turn ^= 1;
    if (!(chance > cp.xtc_probability)) {
      float sum_gt, unused;
      team_sum2(tm, L, [&](float v, int, float& s, float&) { if (okey(v) > T) s += expf(v - mx_l); }, sum_gt, unused);
      const float e_t = E > 0 ? expf(unkey(T) - mx_l) : 0.f;
      const float inv = 1.0f / (sum_gt + (float)E * e_t);
      float above_gt, unused2;
      team_sum2(tm, L, [&](float v, int, float& s, float&) { if (okey(v) > T && expf(v - mx_l) * inv >= cp.xtc_threshold) s += 1.f; },
                above_gt, unused2);
      const bool t_in = E > 0 && e_t * inv >= cp.xtc_threshold;
      const int pos_last = (int)above_gt + (t_in ? E : 0) - 1;  // how many of the leading candidates go
      const float ninf = -INFINITY;
      if (pos_last > 0) {
        if (t_in) {
          // every candidate is above the threshold: only the last of them stays
          const int keep_idx = kth_equal(tm, L, unkey(T), E - 1, false);
          sweep(L, tm.begin, tm.end, [&](float v, int i) { if (okey(v) > T || (okey(v) == T && i != keep_idx)) L[i] = ninf; });
          mx_l = unkey(T);
          E = 1;
        } else {
          unsigned long long above;
          bool fell;
          const uint32_t U = select_desc(
              tm, L, [&](float v, int, uint32_t& key, unsigned long long& w) { const uint32_t k = okey(v); key = k > T ? k : 0u; w = 1ull; },
              (unsigned long long)pos_last, hist, total_bins, &above, &fell);
          const int first_kept = kth_equal(tm, L, unkey(U), pos_last - (int)above, false);
          sweep(L, tm.begin, tm.end, [&](float v, int i) { if (okey(v) > U || (okey(v) == U && i < first_kept)) L[i] = ninf; });
          mx_l = unkey(U);
        }
        __syncthreads();
        if (T < okey(ninf)) {  // everything had survived so far: now what was struck must not
          T = okey(ninf);
          E = 0;
        }
      }
      filtered = true;
    }
  }

  // ---- the choice: argmax (:225-228), or temperature and a draw in the candidates' order (:101-106, :190-215)
  int chosen;
  float inv_final = 0.f;
  if (collapsed || !draws) {
    chosen = team_argmax(tm, L, 1.0f, sh_arg);
  } else {
    const float t = cp.temperature, mx_t = mx_l / t;
    float sum_gt, unused;
    team_sum2(tm, L, [&](float v, int, float& s, float&) { if (okey(v) > T) s += expf(v / t - mx_t); }, sum_gt, unused);
    const float e_t = E > 0 ? expf(unkey(T) / t - mx_t) : 0.f;
    const float inv = 1.0f / (sum_gt + (float)E * e_t);
    inv_final = inv;
    sweep(L, tm.begin, tm.end, [&](float v, int i) { q[i] = okey(v) > T || !filtered ? expf(v / t - mx_t) * inv : 0.f; });
    __syncthreads();
    const float q_t = e_t * inv;
    const float target = coin;  // the softmax was just renewed, so the coin is the target (:199-204)
    if (!filtered) {
      chosen = first_cdf_above(tm, q, n, target);  // untouched order: by index
    } else {
      // descending order: the largest value whose "at least" mass exceeds the target
      unsigned long long above;
      bool fell;
      const uint32_t k_sel = select_desc(
          tm, L, [&](float v, int i, uint32_t& key, unsigned long long& w) {
            const uint32_t k = okey(v);
            key = k > T ? k : 0u;
            w = to_mass(q[i]);
          },
          to_mass(target), hist, total_bins, &above, &fell);
      if (fell && E > 0) {
        // among the equals at the threshold (or past the end: the last of them)
        const float gt_mass = sum_gt * inv;
        int j = q_t > 0.f ? (int)floorf((target - gt_mass) / q_t) : E - 1;
        j = min(max(j, 0), E - 1);
        chosen = kth_equal(tm, L, unkey(T), j, false);
      } else if (fell) {
        chosen = kth_equal(tm, L, unkey(k_sel), 0x7fffffff, true);  // past the end: the last candidate
      } else {
        const float q_sel = expf(unkey(k_sel) / t - mx_t) * inv;
        const int j = (int)floorf((target - from_mass(above)) / q_sel);
        chosen = kth_equal(tm, L, unkey(k_sel), j, true);
      }
    }
    if (chosen < 0) chosen = team_argmax(tm, L, 1.0f, sh_arg);
  }
  if (tm.rank == 0 && threadIdx.x == 0) {
    out[r] = chosen;
    if (cp.mirostat != 0) {
      // mu moves toward the surprise that was observed (src/sampler.rs:446-448, :521-523)
      const float p_sel = expf(L[chosen] / cp.temperature - mx_l / cp.temperature) * inv_final;
      mirostat_mu[slot] = mu - cp.mirostat_eta * (-log2f(p_sel) - cp.mirostat_tau);
    }
    if (records) {  // the chosen token joins the history (src/sampler.rs:339-347, :735-743)
      history[(size_t)slot * HISTORY_MAX + accepted % HISTORY_MAX] = chosen;
      history_count[slot] = accepted + 1;
    }
  }
  tm.cluster.sync();  // nobody leaves while a team mate may still read its shared memory
}

// probs: scratch of n_rows * n floats.  rng_states[rng_index[r]] is read and advanced for row r.
RL_API int rl_sample(const float* logits, long long row_stride, int n_rows, int n, float temperature, float top_p,
                     unsigned long long* rng_states, const int* rng_index, float* probs, int* out,
                     cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0) RL_REFUSE(1, "sample: rows=%d n=%d", n_rows, n);
  if (!(temperature > 0.f)) RL_REFUSE(2, "sample: temperature %f is not positive (0 is the argmax kernel's)", temperature);
  if (!rng_states || !rng_index || !probs) RL_REFUSE(3, "sample: missing random state or scratch");
  if (n_rows > 65535) RL_REFUSE(4, "sample: %d rows exceed 65535", n_rows);
  // a team member should have a few thousand values to sweep, or the exchanges cost more than they save
  int team = 1;
  while (team < TEAM_MAX && n / (2 * team) >= 4096) team *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(team, n_rows);
  cfg.blockDim = dim3(SAMPLE_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = team;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RL_LAUNCH_CHECK(cudaLaunchKernelEx(&cfg, sample_kernel, logits, row_stride, n, temperature, top_p, rng_states, rng_index, probs, out));
  return 0;
}

// The longer chain.  work: n_rows * 2 * n_pad floats with n_pad = n rounded up to 4.  history: int
// [slots][1024], history_count: int [slots], mirostat_mu: float [slots] (may be null without mirostat) and
// xtc_states: the second generator's states (may be null without XTC), all indexed by slot_of_row[r], like
// rng_states.
RL_API int rl_sample_chain(const float* logits, long long row_stride, int n_rows, int n, float temperature, float top_p,
                           int top_k, float min_p, float repeat_penalty, int last_n, float frequency_penalty,
                           float presence_penalty, int mirostat, float mirostat_tau, float mirostat_eta,
                           float xtc_probability, float xtc_threshold, float dry_multiplier, float dry_base,
                           int dry_allowed_length, int dry_last_n, const int* dry_breakers, int dry_n_breakers,
                           unsigned long long* rng_states,
                           const int* slot_of_row, int* history, int* history_count, float* mirostat_mu,
                           unsigned long long* xtc_states, float* work, int* out, cudaStream_t stream) {
  if (n_rows <= 0 || n <= 0) RL_REFUSE(1, "sample_chain: rows=%d n=%d", n_rows, n);
  if (!(temperature >= 0.f)) RL_REFUSE(2, "sample_chain: temperature %f is negative", temperature);
  if (!rng_states || !slot_of_row || !work || !history || !history_count) RL_REFUSE(3, "sample_chain: missing random state, history or scratch");
  if (n_rows > 65535) RL_REFUSE(4, "sample_chain: %d rows exceed 65535", n_rows);
  if (last_n < 0 || last_n > HISTORY_MAX) RL_REFUSE(5, "sample_chain: a history of %d tokens is outside 0..%d", last_n, HISTORY_MAX);
  if (top_k < 0 || !(repeat_penalty > 0.f)) RL_REFUSE(6, "sample_chain: top_k %d or repeat penalty %f out of range", top_k, repeat_penalty);
  if (mirostat < 0 || mirostat > 2) RL_REFUSE(7, "sample_chain: mirostat %d is none of 0, 1, 2", mirostat);
  if (mirostat != 0 && (!(temperature > 0.f) || mirostat_mu == nullptr))
    RL_REFUSE(8, "sample_chain: mirostat needs a positive temperature (got %f) and its state", temperature);
  if (xtc_probability > 0.f && xtc_states == nullptr) RL_REFUSE(9, "sample_chain: XTC needs its random states");
  ChainParams cp = {temperature, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty, top_k, last_n,
                    mirostat, mirostat_tau, mirostat_eta, xtc_probability, xtc_threshold,
                    dry_multiplier, dry_base, dry_allowed_length, dry_last_n, dry_n_breakers, {0, 0, 0, 0, 0, 0, 0, 0}};
  if (dry_last_n < 0 || dry_last_n > HISTORY_MAX || dry_allowed_length < 0)
    RL_REFUSE(10, "sample_chain: a DRY window of %d tokens is outside 0..%d, or its allowed length %d is negative", dry_last_n, HISTORY_MAX, dry_allowed_length);
  if (dry_n_breakers < 0 || dry_n_breakers > DRY_MAX_BREAKERS || (dry_n_breakers > 0 && dry_breakers == nullptr))
    RL_REFUSE(11, "sample_chain: %d DRY sequence breakers, at most %d are taken", dry_n_breakers, DRY_MAX_BREAKERS);
  for (int b = 0; b < dry_n_breakers; ++b) cp.dry_breakers[b] = dry_breakers[b];  // (a host array)
  int team = 1;
  while (team < TEAM_MAX && n / (2 * team) >= 4096) team *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(team, n_rows);
  cfg.blockDim = dim3(SAMPLE_THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = team;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int n_pad = (n + 3) & ~3;
  RL_LAUNCH_CHECK(cudaLaunchKernelEx(&cfg, sample_chain_kernel, logits, row_stride, n, n_pad, cp, rng_states, slot_of_row, history,
                                     history_count, mirostat_mu, xtc_states, work, out));
  return 0;
}
