// Fitness functors shared by the swarm kernels: per-element accumulation + per-row finalisation of
// ackley_func / rastrigin_func / sphere_func (evox/problems/numerical/basic.py:52-69, 115-116).
#pragma once
#include <math.h>

#include "common.cuh"

namespace evox {

struct FitParams {
  float a, b, c;
};

// --------------------------------------------------------------------------------------------
// Fitness functors: per-element accumulation + per-row finalisation. The sums use fused
// multiply-adds and a lane-strided order, so fitness values agree with the reference to
// rounding (relative 1e-5 is the tested bound), not bit for bit.
// --------------------------------------------------------------------------------------------
// cos(t) for the fitness sums: Cody-Waite reduction to [-pi, pi] with 2*pi split in two floats,
// then the hardware cosine (absolute error 2^-21.4 on that interval). Per term the error is below
// 1e-6, i.e. below 1e-6 on mean(cos) for Ackley and below 1e-5 * d on Rastrigin's sum of 10*cos,
// an order of magnitude inside the 1e-5 relative tolerance of the fitness values.
// Valid for |t| <= 32768 (callers check, once per element or once per group of four).
__device__ __forceinline__ float fast_cos_core(float t) {
  const float magic = 12582912.0f;  // 1.5 * 2^23: adding and subtracting rounds to nearest integer
  const float k = __fadd_rn(__fmaf_rn(t, 0.15915494309189535f, magic), -magic);
  float r = __fmaf_rn(-k, 6.2831854820251465f, t);
  r = __fmaf_rn(-k, -1.7484555e-07f, r);
  return __cosf(r);
}
// Exact path for arguments far outside any benchmark's bounds; kept out of line so that its registers
// and code do not weigh on the loops that never take it.
static __device__ __noinline__ float slow_cos(float t) { return cosf(t); }
__device__ __forceinline__ float fast_cos(float t) {
  if (fabsf(t) > 32768.0f) return slow_cos(t);
  return fast_cos_core(t);
}
__device__ __forceinline__ float max_abs4(const float4& x) { return fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))); }

template <int FIT>
struct Fitness;

template <>
struct Fitness<EVOX_FIT_ACKLEY> {
  float s_sq = 0.f, s_cos = 0.f;
  __device__ __forceinline__ void add(float x, const FitParams& p) {
    s_sq = __fmaf_rn(x, x, s_sq);
    s_cos += fast_cos(__fmul_rn(p.c, x));
  }
  __device__ __forceinline__ void add4(const float4& x, const FitParams& p) {
    if (max_abs4(x) * fabsf(p.c) > 32768.0f) {  // also taken for NaN-free infinities; NaN falls through and propagates
      add(x.x, p);
      add(x.y, p);
      add(x.z, p);
      add(x.w, p);
      return;
    }
    s_sq = __fmaf_rn(x.x, x.x, s_sq);
    s_sq = __fmaf_rn(x.y, x.y, s_sq);
    s_sq = __fmaf_rn(x.z, x.z, s_sq);
    s_sq = __fmaf_rn(x.w, x.w, s_sq);
    s_cos += fast_cos_core(__fmul_rn(p.c, x.x));
    s_cos += fast_cos_core(__fmul_rn(p.c, x.y));
    s_cos += fast_cos_core(__fmul_rn(p.c, x.z));
    s_cos += fast_cos_core(__fmul_rn(p.c, x.w));
  }
  __device__ __forceinline__ void reduce() {
    s_sq = warp_sum(s_sq);
    s_cos = warp_sum(s_cos);
  }
  __device__ __forceinline__ float finish(int d, const FitParams& p) const {
    const float fd = (float)d;
    const float m_sq = __fdiv_rn(s_sq, fd);
    const float m_cos = __fdiv_rn(s_cos, fd);
    const float t1 = __fmul_rn(-p.a, expf(__fmul_rn(-p.b, sqrtf(m_sq))));
    const float t2 = expf(m_cos);
    return __fadd_rn(__fadd_rn(__fsub_rn(t1, t2), p.a), 2.718281828459045f);
  }
};

template <>
struct Fitness<EVOX_FIT_RASTRIGIN> {
  float s = 0.f, s_cos = 0.f;
  __device__ __forceinline__ void add(float x, const FitParams&) {
    s = __fmaf_rn(x, x, s);
    s_cos += fast_cos(__fmul_rn(6.283185307179586f, x));
  }
  __device__ __forceinline__ void add4(const float4& x, const FitParams& p) {
    if (max_abs4(x) > 5000.0f) {  // 2 pi x beyond the fast cosine's range
      add(x.x, p);
      add(x.y, p);
      add(x.z, p);
      add(x.w, p);
      return;
    }
    s = __fmaf_rn(x.x, x.x, s);
    s = __fmaf_rn(x.y, x.y, s);
    s = __fmaf_rn(x.z, x.z, s);
    s = __fmaf_rn(x.w, x.w, s);
    s_cos += fast_cos_core(__fmul_rn(6.283185307179586f, x.x));
    s_cos += fast_cos_core(__fmul_rn(6.283185307179586f, x.y));
    s_cos += fast_cos_core(__fmul_rn(6.283185307179586f, x.z));
    s_cos += fast_cos_core(__fmul_rn(6.283185307179586f, x.w));
  }
  __device__ __forceinline__ void reduce() {
    s = warp_sum(s);
    s_cos = warp_sum(s_cos);
  }
  __device__ __forceinline__ float finish(int d, const FitParams&) const {
    return __fadd_rn((float)(10 * (long long)d), __fmaf_rn(-10.0f, s_cos, s));
  }
};

template <>
struct Fitness<EVOX_FIT_SPHERE> {
  float s = 0.f;
  __device__ __forceinline__ void add(float x, const FitParams&) { s = __fmaf_rn(x, x, s); }
  __device__ __forceinline__ void add4(const float4& x, const FitParams&) {
    s = __fmaf_rn(x.x, x.x, s);
    s = __fmaf_rn(x.y, x.y, s);
    s = __fmaf_rn(x.z, x.z, s);
    s = __fmaf_rn(x.w, x.w, s);
  }
  __device__ __forceinline__ void reduce() { s = warp_sum(s); }
  __device__ __forceinline__ float finish(int, const FitParams&) const { return s; }
};

}  // namespace evox
