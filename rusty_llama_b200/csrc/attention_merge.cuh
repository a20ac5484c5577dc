// The second kernel of split decode attention, shared by its two first kernels (attention_decode.cu,
// attention_decode_tma.cu).  Scratch layout: part_o[seq][head][split][hd] floats (unnormalised outputs),
// part_ml[seq][head][split][2] (maximum as a base-2 exponent, sum).
#pragma once

#include "common.cuh"

// out[s, h, :] = sum_split 2^(m_split - M) o_split / sum_split 2^(m_split - M) l_split
// One block per (sequence, head).  Warp 0 takes the splits' (max, sum) pairs side by side and leaves
// each split's normalised weight in shared memory; then every thread owns output dimensions and adds
// the splits up in split order, four loads in flight at a time.  At most 64 splits.
__global__ void attn_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         bf16* __restrict__ out, int out_stride, int H, int hd, int n_splits) {
  __shared__ float w_s[64];
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, s = blockIdx.y;
  const float* ml = part_ml + ((size_t)s * H + h) * n_splits * 2;
  const float* po = part_o + ((size_t)s * H + h) * n_splits * hd;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
    if (lane < n_splits) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(ml + 2 * lane));
      m0 = v.x;
      l0 = v.y;
    }
    if (lane + 32 < n_splits) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(ml + 2 * (lane + 32)));
      m1 = v.x;
      l1 = v.y;
    }
    const float M = warp_max(fmaxf(m0, m1));
    const float w0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M);
    const float w1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - M);
    const float inv = 1.0f / warp_sum(w0 * l0 + w1 * l1);
    w_s[lane] = w0 * inv;
    w_s[lane + 32] = w1 * inv;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
    int i = 0;
    for (; i + 4 <= n_splits; i += 4) {
      const float v0 = __ldcg(po + (size_t)i * hd + d), v1 = __ldcg(po + (size_t)(i + 1) * hd + d);
      const float v2 = __ldcg(po + (size_t)(i + 2) * hd + d), v3 = __ldcg(po + (size_t)(i + 3) * hd + d);
      o += w_s[i] * v0;
      o += w_s[i + 1] * v1;
      o += w_s[i + 2] * v2;
      o += w_s[i + 3] * v3;
    }
    for (; i < n_splits; ++i) o += w_s[i] * __ldcg(po + (size_t)i * hd + d);
    out[(size_t)s * out_stride + (size_t)h * hd + d] = __float2bfloat16_rn(o);
  }
}

