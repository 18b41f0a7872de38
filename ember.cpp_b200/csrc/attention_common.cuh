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

// Packed float32 pairs (sm_100: one instruction, two results).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
        "l"(reinterpret_cast<unsigned long long&>(c)));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ void unpack8(const uint4& raw, float2 (&f)[4]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __bfloat1622float2(h[i]);
}

// N keys folded into a stream's running softmax together: their scores first, then one new
// maximum, one correction of the sums so far and N weighted values, in packed pairs.  The same
// sums as N calls of fold_key up to the order of additions; about a third fewer instructions.
// q and acc hold the lane's 8 dims as 4 pairs.
template <int LPK, int N>
__device__ __forceinline__ void fold_keys(const uint4 (&kraw)[N], const uint4 (&vraw)[N], const bool (&have)[N],
                                          const float2 (&q)[4], float scale, float& m, float& l, float2 (&acc)[4]) {
  float sc[N];
#pragma unroll
  for (int u = 0; u < N; ++u) {
    float2 k[4];
    unpack8(kraw[u], k);
    float2 d = mul2(q[0], k[0]);
#pragma unroll
    for (int i = 1; i < 4; ++i) d = fma2(q[i], k[i], d);
    sc[u] = d.x + d.y;
  }
#pragma unroll
  for (int off = LPK / 2; off > 0; off >>= 1) {
#pragma unroll
    for (int u = 0; u < N; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], off);
  }
  float m_new = m;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    sc[u] = have[u] ? sc[u] * scale : -INFINITY;
    m_new = fmaxf(m_new, sc[u]);
  }
  const bool none = m_new == -INFINITY;
  const float corr = none ? 0.f : __expf(m - m_new);
  float p[N], sum = 0.f;
#pragma unroll
  for (int u = 0; u < N; ++u) {
    p[u] = none ? 0.f : __expf(sc[u] - m_new);
    sum += p[u];
  }
  l = l * corr + sum;
  const float2 c2 = make_float2(corr, corr);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = mul2(acc[i], c2);
#pragma unroll
  for (int u = 0; u < N; ++u) {
    float2 v[4];
    unpack8(vraw[u], v);
    const float2 p2 = make_float2(p[u], p[u]);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = fma2(v[i], p2, acc[i]);
  }
  m = m_new;
}

