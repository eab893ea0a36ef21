// Shared device/host helpers for the evox_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/evox_b200.h"

namespace evox {

// ---------------------------------------------------------------------------
// Error plumbing: every C-ABI entry point returns 0 on success or a negative
// EVOX_ERR_* code; the message is kept per thread for evox_last_error().
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);

#define EVOX_REQUIRE(cond, code, ...)   \
  do {                                  \
    if (!(cond)) {                      \
      ::evox::set_error(__VA_ARGS__);   \
      return (code);                    \
    }                                   \
  } while (0)

#define EVOX_CUDA(call)                                                              \
  do {                                                                               \
    cudaError_t e__ = (call);                                                        \
    if (e__ != cudaSuccess) {                                                        \
      ::evox::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),     \
                        __FILE__, __LINE__);                                         \
      return EVOX_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)

#define EVOX_LAUNCH_CHECK()                                                          \
  do {                                                                               \
    cudaError_t e__ = cudaGetLastError();                                            \
    if (e__ != cudaSuccess) {                                                        \
      ::evox::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__), \
                        __FILE__, __LINE__);                                         \
      return EVOX_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)

int sm_count();  // cached multiprocessor count of the current device

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// Philox4x32-10. Same constants, round function and output order (c0..c3) as
// the reference generator (evox/triton_kernels/kernels/philox.py:35-112).
// ---------------------------------------------------------------------------
#define EVOX_PHILOX_M0 0xD2511F53u
#define EVOX_PHILOX_M1 0xCD9E8D57u
#define EVOX_PHILOX_W0 0x9E3779B9u
#define EVOX_PHILOX_W1 0xBB67AE85u

__device__ __forceinline__ uint4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(EVOX_PHILOX_M0, c0);
    const uint32_t lo0 = EVOX_PHILOX_M0 * c0;
    const uint32_t hi1 = __umulhi(EVOX_PHILOX_M1, c2);
    const uint32_t lo1 = EVOX_PHILOX_M1 * c2;
    c0 = hi1 ^ c1 ^ k0;
    c1 = lo1;
    c2 = hi0 ^ c3 ^ k1;
    c3 = lo0;
    k0 += EVOX_PHILOX_W0;
    k1 += EVOX_PHILOX_W1;
  }
  return make_uint4(c0, c1, c2, c3);
}

// The same generator with the key schedule taken out of the kernel: the ten (k0, k1) pairs depend only
// on the seed, so the host computes them once per launch and they travel as kernel arguments.
struct PhiloxKeys {
  uint32_t k[20];
};

static inline PhiloxKeys philox_round_keys(uint64_t seed) {
  PhiloxKeys rk;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    rk.k[2 * r] = k0;
    rk.k[2 * r + 1] = k1;
    k0 += EVOX_PHILOX_W0;
    k1 += EVOX_PHILOX_W1;
  }
  return rk;
}

__device__ __forceinline__ uint4 philox4x32_10_keyed(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxKeys& rk) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = (unsigned long long)EVOX_PHILOX_M0 * (unsigned long long)c0;
    const unsigned long long p1 = (unsigned long long)EVOX_PHILOX_M1 * (unsigned long long)c2;
    c0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk.k[2 * r];
    c1 = (uint32_t)p1;
    c2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk.k[2 * r + 1];
    c3 = (uint32_t)p0;
  }
  return make_uint4(c0, c1, c2, c3);
}

// 24-bit uniform in [0,1): (u >> 8) * 2^-24, as philox.py:108-110.
__device__ __forceinline__ float u24_to_unit(uint32_t u) {
  return __uint2float_rn(u >> 8) * 5.9604644775390625e-08f;
}

// ---------------------------------------------------------------------------
// (value, index) minimum with torch.argmin's semantics: NaN is smaller than
// every number, and among equal keys the lowest index wins.
// ---------------------------------------------------------------------------
struct MinIdx {
  float v;
  long long i;
};

__device__ __forceinline__ bool key_less(float a, float b) {
  const bool an = a != a, bn = b != b;
  if (an || bn) return an && !bn;
  return a < b;
}

__device__ __forceinline__ MinIdx min_idx_combine(MinIdx a, MinIdx b) {
  // returns the one that argmin would report first
  if (key_less(b.v, a.v)) return b;
  if (key_less(a.v, b.v)) return a;
  return (b.i < a.i) ? b : a;
}

__device__ __forceinline__ MinIdx warp_min_idx(MinIdx m) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    MinIdx o;
    o.v = __shfl_xor_sync(0xffffffffu, m.v, off);
    o.i = __shfl_xor_sync(0xffffffffu, m.i, off);
    m = min_idx_combine(m, o);
  }
  return m;
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

// relu-form clamp used by the reference everywhere instead of torch.clamp
// (evox/utils/jit_fix_operator.py:42-44): a + relu(lb - a) - relu(a - ub),
// each operation rounded on its own (no fused multiply-add can appear here).
__device__ __forceinline__ float relu_clamp(float a, float lb, float ub) {
  const float lo = fmaxf(__fsub_rn(lb, a), 0.0f);
  const float hi = fmaxf(__fsub_rn(a, ub), 0.0f);
  return __fsub_rn(__fadd_rn(a, lo), hi);
}

}  // namespace evox
