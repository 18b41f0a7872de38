// Pieces that the decode attention kernels share: one key folded into a running softmax.
#pragma once

#include "common.cuh"

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// One key (its 16-byte part of K and of V) folded into a stream's running softmax.
template <int LPK>
__device__ __forceinline__ void fold_key(const uint4& kraw, const uint4& vraw, bool have, const float (&q)[8], float scale,
                                         float& m, float& l, float (&acc)[8]) {
  float k[8], v[8];
  unpack8(kraw, k);
  unpack8(vraw, v);
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) dot = fmaf(q[i], k[i], dot);
#pragma unroll
  for (int off = LPK / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
  const float sc = have ? dot * scale : -INFINITY;
  const float m_new = fmaxf(m, sc);
  const float corr = m_new == -INFINITY ? 0.f : __expf(m - m_new);
  const float pj = m_new == -INFINITY ? 0.f : __expf(sc - m_new);
  l = l * corr + pj;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = fmaf(pj, v[i], acc[i] * corr);
  m = m_new;
}

