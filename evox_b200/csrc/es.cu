// P4 (part 1): Philox streams, virtual LoRA factors, the low-rank forward correction, the
// population gradient and the centre update of the evolution strategies, in fp32.
//
// Reference semantics:
//   philox_uniform / philox_normal          evox/triton_kernels/kernels/philox.py:52-112
//   generate_lora_factors, lora_delta_output, lora_gradient
//                                           evox/triton_kernels/kernels/lora_noise.py:86-196
//   VirtualLoRAProblem._virtual_forward     evox/problems/neuroevolution/virtual_lora_problem.py:126-201
//   OpenES.step                             evox/algorithms/so/es_variants/open_es.py:60-83
//   adam_single_tensor                      evox/algorithms/so/es_variants/adam_step.py:4-26
// The bf16 tensor-core path of the base product lives in lora_gemm_sm100.cu; the kernels here
// are the fp32 path (any shape) and everything around the product.
#include <math.h>

#include "common.cuh"

namespace evox {
namespace {

constexpr int kThreads = 256;

// Four uniforms of Philox call `call` of one individual's stream (philox.py:62-111): key = the
// two halves of the int64 seed, counter = (low32(counter) + call mod 2^32, high32(counter), 0, 0).
__device__ __forceinline__ float4 stream_uniform4(unsigned long long seed, unsigned long long counter, uint32_t call) {
  const uint4 r = philox4x32_10((uint32_t)counter + call, (uint32_t)(counter >> 32), 0u, 0u, (uint32_t)seed,
                                (uint32_t)(seed >> 32));
  return make_float4(u24_to_unit(r.x), u24_to_unit(r.y), u24_to_unit(r.z), u24_to_unit(r.w));
}

// Box-Muller on the pairs (u0, u1) and (u2, u3) (philox.py:103-111): z = sqrt(-2 log max(u1, 1e-10))
// * (cos, sin)(2 pi u2), interleaved.
__device__ __forceinline__ float4 stream_normal4(unsigned long long seed, unsigned long long counter, uint32_t call) {
  const float4 u = stream_uniform4(seed, counter, call);
  const float r0 = sqrtf(__fmul_rn(-2.0f, logf(fmaxf(u.x, 1e-10f))));
  const float r1 = sqrtf(__fmul_rn(-2.0f, logf(fmaxf(u.z, 1e-10f))));
  float s0, c0, s1, c1;
  sincosf(__fmul_rn(6.283185307179586f, u.y), &s0, &c0);
  sincosf(__fmul_rn(6.283185307179586f, u.w), &s1, &c1);
  return make_float4(__fmul_rn(r0, c0), __fmul_rn(r0, s0), __fmul_rn(r1, c1), __fmul_rn(r1, s1));
}

template <bool NORMAL>
__global__ void __launch_bounds__(kThreads)
    philox_fill_kernel(const long long* __restrict__ seeds, long long pop, long long n, unsigned long long counter,
                       float* __restrict__ out) {
  const long long n_call = (n + 3) >> 2;
  const long long total = pop * n_call;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long p = t / n_call, q = t - p * n_call;
    const unsigned long long seed = (unsigned long long)seeds[p];
    const float4 v = NORMAL ? stream_normal4(seed, counter, (uint32_t)q) : stream_uniform4(seed, counter, (uint32_t)q);
    float* o = out + p * n + 4 * q;
    const long long rem = n - 4 * q;
    if (rem >= 4 && ((reinterpret_cast<uintptr_t>(o) & 15u) == 0)) {
      *reinterpret_cast<float4*>(o) = v;
    } else {
      o[0] = v.x;
      if (rem > 1) o[1] = v.y;
      if (rem > 2) o[2] = v.z;
      if (rem > 3) o[3] = v.w;
    }
  }
}

// t[p][b][q] = sum_k x[p][b][k] * A[p][q][k]  — one warp per (p, b) row, rank <= 32.
__global__ void __launch_bounds__(kThreads)
    lora_down_kernel(const float* __restrict__ x, long long x_pop_stride, const float* __restrict__ A, long long pop,
                     long long batch, long long k, int r, float* __restrict__ t) {
  const int lane = threadIdx.x & 31;
  const long long gwarp = ((long long)blockIdx.x * kThreads + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * kThreads) >> 5;
  for (long long row = gwarp; row < pop * batch; row += n_warps) {
    const long long p = row / batch, b = row - p * batch;
    const float* xr = x + p * x_pop_stride + b * k;
    const float* Ap = A + p * (long long)r * k;
    for (int q = 0; q < r; ++q) {
      float acc = 0.f;
      for (long long c = lane; c < k; c += 32) acc = __fmaf_rn(xr[c], Ap[(long long)q * k + c], acc);
      acc = warp_sum(acc);
      if (lane == 0) t[row * r + q] = acc;
    }
  }
}

// out[p][b][n] = (base ? base : 0) + sigma * sum_q t[p][b][q] * B[p][n][q]   (lora_noise.py:151-153)
__global__ void __launch_bounds__(kThreads)
    lora_up_kernel(const float* __restrict__ t, const float* __restrict__ B, float sigma, long long pop, long long batch,
                   long long d, int r, float* __restrict__ out) {
  const long long total = pop * batch * d;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long row = e / d, n = e - row * d;
    const long long p = row / batch;
    const float* tr = t + row * r;
    const float* Bn = B + (p * d + n) * r;
    float acc = 0.f;
    for (int q = 0; q < r; ++q) acc = __fmaf_rn(tr[q], Bn[q], acc);
    out[e] = __fmul_rn(sigma, acc);
  }
}

// grad[j][l] = sum_i fitness[i] * sum_q B[i][j][q] * A[i][q][l] / (pop * sigma)   (lora_noise.py:195)
// 64 x 64 output tile per block, one individual's factors staged in shared memory per step.
template <int RMAX>
__global__ void __launch_bounds__(kThreads)
    lora_gradient_kernel(const float* __restrict__ fitness, const float* __restrict__ A, const float* __restrict__ B,
                         long long pop, float inv_scale, long long d, long long k, int r, float* __restrict__ grad) {
  __shared__ float sB[64][RMAX + 1];
  __shared__ float sA[RMAX][64];
  const long long j0 = (long long)blockIdx.y * 64, l0 = (long long)blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {};
  for (long long i = 0; i < pop; ++i) {
    const float fi = fitness[i];
    for (int t = threadIdx.x; t < 64 * r; t += kThreads) {
      const int jj = t / r, q = t - jj * r;
      const long long j = j0 + jj;
      sB[jj][q] = (j < d) ? __fmul_rn(fi, B[(i * d + j) * r + q]) : 0.f;
    }
    for (int t = threadIdx.x; t < 64 * r; t += kThreads) {
      const int q = t >> 6, ll = t & 63;
      const long long l = l0 + ll;
      sA[q][ll] = (l < k) ? A[(i * r + q) * k + l] : 0.f;
    }
    __syncthreads();
    for (int q = 0; q < r; ++q) {
      float bv[4], av[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        bv[u] = sB[ty * 4 + u][q];
        av[u] = sA[q][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[u][w] = __fmaf_rn(bv[u], av[w], acc[u][w]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const long long j = j0 + ty * 4 + u, l = l0 + tx * 4 + w;
      if (j < d && l < k) grad[j * k + l] = __fmul_rn(acc[u][w], inv_scale);
    }
}

// out[l] = sum_i scale_i * noise[i][l], scale_i = fitness[i] * inv_scale   (1-D blocks, lora_noise.py:190-192;
// also OpenES's noise^T fitness, open_es.py:70, with `sign_split` = pop/2 for mirrored sampling
// where row i >= sign_split reuses noise row i - sign_split negated).
// One block = 32 (or 128, as float4) columns x 8 warps; warp w walks rows w, w + 8, ... (a row's piece is one
// coalesced 128- or 512-byte read), the eight partial sums are folded in warp order. The number of blocks grows with the
// row length, the length of every dependent chain is pop / 8: short rows with many individuals no longer
// serialise on one thread per column.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
    weighted_rows_kernel(const float* __restrict__ fitness, const float* __restrict__ noise, long long pop, long long n,
                         long long noise_rows, float inv_scale, float* __restrict__ out) {
  constexpr int kWarps = kThreads / 32, kTile = 32 * VEC;
  __shared__ float part[kWarps][kTile];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long l0 = (long long)blockIdx.x * kTile; l0 < n; l0 += (long long)gridDim.x * kTile) {
    const long long l = l0 + (long long)lane * VEC;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    if (l < n) {
      // the warp's rows in ascending order, written as two loops (own noise rows, then the mirrored ones: the same
      // noise row with the fitness negated; f * (-z) and (-f) * z round alike) instead of one with a select per row
      auto add_row = [&](float f, const float* row) {
        if constexpr (VEC == 4) {
          const float4 z = __ldg(reinterpret_cast<const float4*>(row));
          acc[0] = __fmaf_rn(f, z.x, acc[0]);
          acc[1] = __fmaf_rn(f, z.y, acc[1]);
          acc[2] = __fmaf_rn(f, z.z, acc[2]);
          acc[3] = __fmaf_rn(f, z.w, acc[3]);
        } else {
          acc[0] = __fmaf_rn(f, __ldg(row), acc[0]);
        }
      };
      const long long plain_end = noise_rows < pop ? noise_rows : pop;
      long long i = warp;
#pragma unroll 4
      for (; i < plain_end; i += kWarps) add_row(fitness[i], noise + i * n + l);
#pragma unroll 4
      for (; i < pop; i += kWarps) add_row(-fitness[i], noise + (i - noise_rows) * n + l);
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) part[warp][lane * VEC + j] = acc[j];
    __syncthreads();
    for (int c = threadIdx.x; c < kTile; c += kThreads) {
      if (l0 + c < n) {
        float t = part[0][c];
        for (int w = 1; w < kWarps; ++w) t += part[w][c];
        out[l0 + c] = __fmul_rn(t, inv_scale);
      }
    }
    __syncthreads();
  }
}

int launch_weighted_rows(const float* fitness, const float* noise, long long pop, long long n, long long noise_rows, float inv_scale,
                         float* out, cudaStream_t s);

// pop[i][l] = center[l] + sigma * (+-) noise[i mod rows][l]   (open_es.py:64-68); with `accum` the same
// perturbation is also added to accum[i][l] (PersistentES, persistent_es.py:76-80).
// Rows on blockIdx.y, VEC consecutive columns per thread: no index division, 16-byte accesses when VEC = 4.
// MIRRORED (row i + noise_rows is row i with the perturbation negated: one read, two writes) and ACCUM are template
// arguments: as run-time conditions inside the column loop they cost the kernel a tenth of its bandwidth.
template <int VEC, bool MIRRORED, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
    openes_ask_kernel(const float* __restrict__ center, const float* __restrict__ noise, const float* __restrict__ sigma_p,
                      long long pop, long long n, long long noise_rows, float* __restrict__ out, float* __restrict__ accum) {
  const float sigma = *sigma_p;
  const long long nv = n / VEC;
  for (long long i = blockIdx.y; i < noise_rows; i += gridDim.y) {
    const float* zrow = noise + i * n;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nv; c += (long long)gridDim.x * blockDim.x) {
      float z[VEC], ce[VEC];
      if constexpr (VEC == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4*>(zrow) + c);
        const float4 u = __ldg(reinterpret_cast<const float4*>(center) + c);
        z[0] = t.x; z[1] = t.y; z[2] = t.z; z[3] = t.w;
        ce[0] = u.x; ce[1] = u.y; ce[2] = u.z; ce[3] = u.w;
      } else {
        z[0] = zrow[c];
        ce[0] = center[c];
      }
#pragma unroll
      for (int half = 0; half < (MIRRORED ? 2 : 1); ++half) {
        const long long row = i + half * noise_rows;
        float* orow = out + row * n;
        float* arow = ACCUM ? accum + row * n : nullptr;
        float ac[VEC], o[VEC];
        if constexpr (ACCUM) {
          if constexpr (VEC == 4) {
            const float4 q = __ldcs(reinterpret_cast<const float4*>(arow) + c);
            ac[0] = q.x; ac[1] = q.y; ac[2] = q.z; ac[3] = q.w;
          } else {
            ac[0] = arow[c];
          }
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const float pert = __fmul_rn(sigma, half ? -z[j] : z[j]);
          o[j] = __fadd_rn(ce[j], pert);
          if constexpr (ACCUM) ac[j] = __fadd_rn(ac[j], pert);
        }
        if constexpr (VEC == 4) {
          __stcs(reinterpret_cast<float4*>(orow) + c, make_float4(o[0], o[1], o[2], o[3]));
          if constexpr (ACCUM) __stcs(reinterpret_cast<float4*>(arow) + c, make_float4(ac[0], ac[1], ac[2], ac[3]));
        } else {
          orow[c] = o[0];
          if constexpr (ACCUM) arow[c] = ac[0];
        }
      }
    }
  }
}

// pop[i][l] = center[l] + noise[i][l] * sigma[l]: per-coordinate step sizes (snes.py:79, des.py:60).
template <int VEC>
__global__ void __launch_bounds__(kThreads)
    es_ask_diag_kernel(const float* __restrict__ center, const float* __restrict__ noise, const float* __restrict__ sigma, long long pop,
                       long long n, float* __restrict__ out) {
  const long long nv = n / VEC;
  for (long long i = blockIdx.y; i < pop; i += gridDim.y) {
    const float* zrow = noise + i * n;
    float* orow = out + i * n;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nv; c += (long long)gridDim.x * blockDim.x) {
      if constexpr (VEC == 4) {
        const float4 z = __ldcs(reinterpret_cast<const float4*>(zrow) + c);
        const float4 ce = __ldg(reinterpret_cast<const float4*>(center) + c), sg = __ldg(reinterpret_cast<const float4*>(sigma) + c);
        __stcs(reinterpret_cast<float4*>(orow) + c,
               make_float4(__fadd_rn(ce.x, __fmul_rn(z.x, sg.x)), __fadd_rn(ce.y, __fmul_rn(z.y, sg.y)),
                           __fadd_rn(ce.z, __fmul_rn(z.z, sg.z)), __fadd_rn(ce.w, __fmul_rn(z.w, sg.w))));
      } else {
        orow[c] = __fadd_rn(center[c], __fmul_rn(zrow[c], sigma[c]));
      }
    }
  }
}

// Grid of the row-by-column elementwise kernels: columns on x, a bounded number of row slots on y.
dim3 rows_by_cols_grid(long long pop, long long cols);

// Two row-weighted column sums of x (pop x n) in one pass:
//   first[l] = sum_i w[i] * x[i][l],   second[l] = sum_i w[i] * ((x[i][l] - shift[l])^2 + offset)
// (snes.py:83-84 with shift = 0, offset = -1 on the noise; des.py:66-67 with shift = center, offset = 0 on the
// population). w[i] is the weight of row i's fitness rank.
template <int VEC>
__global__ void __launch_bounds__(kThreads)
    rank_weighted_moments_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ shift, float offset,
                                 long long pop, long long n, float* __restrict__ first, float* __restrict__ second) {
  // same decomposition as weighted_rows_kernel: a tile of 32 * VEC columns per block, rows dealt to the 8 warps
  constexpr int kWarps = kThreads / 32, kTile = 32 * VEC;
  __shared__ float part[2][kWarps][kTile];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long l0 = (long long)blockIdx.x * kTile; l0 < n; l0 += (long long)gridDim.x * kTile) {
    const long long l = l0 + (long long)lane * VEC;
    float a[VEC], b[VEC], sh[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      a[j] = b[j] = 0.f;
      sh[j] = (shift && l + j < n) ? shift[l + j] : 0.f;
    }
    if (l < n) {
#pragma unroll 4
      for (long long i = warp; i < pop; i += kWarps) {
        const float wi = w[i];
        float v[VEC];
        if constexpr (VEC == 4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(x + i * n + l));
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
          v[0] = __ldg(x + i * n + l);
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const float dv = __fsub_rn(v[j], sh[j]);
          a[j] = __fmaf_rn(wi, v[j], a[j]);
          b[j] = __fmaf_rn(wi, __fadd_rn(__fmul_rn(dv, dv), offset), b[j]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      part[0][warp][lane * VEC + j] = a[j];
      part[1][warp][lane * VEC + j] = b[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < kTile; c += kThreads) {
      if (l0 + c < n) {
        float ta = part[0][0][c], tb = part[1][0][c];
        for (int q = 1; q < kWarps; ++q) {
          ta += part[0][q][c];
          tb += part[1][q][c];
        }
        first[l0 + c] = ta;
        second[l0 + c] = tb;
      }
    }
    __syncthreads();
  }
}

// SGD: center -= lr * grad. Adam (adam_step.py:20-26, no bias correction, eps added after the root):
// m = lerp(m, g, 1 - b1); v = v * b2 + g * g * (1 - b2); center -= lr * m / (sqrt(v) + eps).
__global__ void __launch_bounds__(kThreads)
    es_update_kernel(float* __restrict__ center, const float* __restrict__ grad, const float* __restrict__ lr_p,
                     float* __restrict__ m, float* __restrict__ v, const float* __restrict__ beta1_p,
                     const float* __restrict__ beta2_p, float eps, long long n) {
  const float lr = *lr_p;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
    const float g = grad[e];
    if (m == nullptr) {
      center[e] = __fsub_rn(center[e], __fmul_rn(lr, g));
    } else {
      const float b1 = *beta1_p, b2 = *beta2_p;
      const float w1 = __fsub_rn(1.0f, b1);
      // torch.lerp(start, end, w): fma(w, end - start, start) for |w| < 0.5, else fma(w - 1, end - start, end)
      const float mn = (w1 < 0.5f) ? __fmaf_rn(w1, __fsub_rn(g, m[e]), m[e])
                                   : __fmaf_rn(__fsub_rn(w1, 1.0f), __fsub_rn(g, m[e]), g);
      const float vn = __fadd_rn(__fmul_rn(v[e], b2), __fmul_rn(__fmul_rn(g, g), __fsub_rn(1.0f, b2)));
      m[e] = mn;
      v[e] = vn;
      center[e] = __fsub_rn(center[e], __fdiv_rn(__fmul_rn(lr, mn), __fadd_rn(sqrtf(vn), eps)));
    }
  }
}

// One virtual-LoRA linear layer in fp32 (virtual_lora_problem.py:160-193):
//   out[p][b][n] = act( sum_k h[p][b][k] W[n][k] + bias[n] + sigma * sum_q t[p][b][q] B[p][n][q]
//                       + sigma * bias_noise[p][n] )
// 64 x 64 tile per block over (rows = pop * batch, n); t (= h A^T), B and bias_noise are inputs.
__global__ void __launch_bounds__(kThreads)
    lora_linear_kernel(const float* __restrict__ h, long long h_pop_stride, const float* __restrict__ W,
                       const float* __restrict__ bias, const float* __restrict__ t, const float* __restrict__ B,
                       const float* __restrict__ bias_noise, float sigma, long long pop, long long batch, long long k,
                       long long d, int r, int relu, float* __restrict__ out) {
  __shared__ float sH[16][64 + 1];
  __shared__ float sW[16][64 + 1];
  const long long rows = pop * batch;
  const long long r0 = (long long)blockIdx.y * 64, n0 = (long long)blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (long long k0 = 0; k0 < k; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += kThreads) {
      const int rr = e >> 4, kk = e & 15;
      const long long row = r0 + rr, col = k0 + kk;
      float hv = 0.f, wv = 0.f;
      if (row < rows && col < k) {
        const long long p = row / batch, b = row - p * batch;
        hv = h[p * h_pop_stride + b * k + col];
      }
      const long long n = n0 + rr;
      if (n < d && col < k) wv = W[n * k + col];
      sH[kk][rr] = hv;
      sW[kk][rr] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float hv[4], wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        hv[u] = sH[kk][ty * 4 + u];
        wv[u] = sW[kk][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) acc[u][w] = __fmaf_rn(hv[u], wv[w], acc[u][w]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const long long row = r0 + ty * 4 + u;
    if (row >= rows) continue;
    const long long p = row / batch;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const long long n = n0 + tx * 4 + w;
      if (n >= d) continue;
      float y = acc[u][w];
      if (bias) y = __fadd_rn(y, bias[n]);
      if (t) {
        float dl = 0.f;
        for (int q = 0; q < r; ++q) dl = __fmaf_rn(t[row * r + q], B[(p * d + n) * r + q], dl);
        y = __fadd_rn(y, __fmul_rn(sigma, dl));
      }
      if (bias_noise) y = __fadd_rn(y, __fmul_rn(sigma, bias_noise[p * d + n]));
      out[row * d + n] = relu ? fmaxf(y, 0.f) : y;
    }
  }
}

int grid_for(long long work, int per);

dim3 rows_by_cols_grid(long long pop, long long cols) {
  long long gx = (cols + kThreads - 1) / kThreads;
  if (gx < 1) gx = 1;
  const long long cap = (long long)sm_count() * 16;
  if (gx > cap) gx = cap;
  long long gy = cap / gx;
  if (gy < 1) gy = 1;
  if (gy > pop) gy = pop;
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)gx, (unsigned)gy);
}

int launch_weighted_rows(const float* fitness, const float* noise, long long pop, long long n, long long noise_rows, float inv_scale,
                         float* out, cudaStream_t s) {
  // float4 tiles need 128 columns per block: only when that still leaves a block or more per SM
  if (n % 4 == 0 && aligned16(noise) && n >= 128ll * sm_count()) {
    weighted_rows_kernel<4><<<grid_for(n, 128), kThreads, 0, s>>>(fitness, noise, pop, n, noise_rows, inv_scale, out);
  } else {
    weighted_rows_kernel<1><<<grid_for(n, 32), kThreads, 0, s>>>(fitness, noise, pop, n, noise_rows, inv_scale, out);
  }
  return 0;
}

int grid_for(long long work, int per = kThreads) {
  long long want = (work + per - 1) / per;
  const long long cap = (long long)sm_count() * 16;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace
}  // namespace evox

using namespace evox;

static int philox_fill(bool normal, const int64_t* seeds, int64_t pop, int64_t n, uint64_t counter, float* out, void* stream) {
  EVOX_REQUIRE(seeds && out, EVOX_ERR_INVALID, "philox: NULL pointer");
  EVOX_REQUIRE(pop > 0 && n > 0, EVOX_ERR_INVALID, "philox: pop and n must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = grid_for(pop * ((n + 3) / 4));
  if (normal) philox_fill_kernel<true><<<grid, kThreads, 0, s>>>((const long long*)seeds, pop, n, counter, out);
  else philox_fill_kernel<false><<<grid, kThreads, 0, s>>>((const long long*)seeds, pop, n, counter, out);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_philox_uniform(const int64_t* seeds, int64_t pop, int64_t n, uint64_t counter, float* out, void* stream) {
  return philox_fill(false, seeds, pop, n, counter, out, stream);
}

extern "C" int evox_philox_normal(const int64_t* seeds, int64_t pop, int64_t n, uint64_t counter, float* out, void* stream) {
  // an odd n draws ceil(n / 2) pairs and drops the last value (philox.py:98-112): same as filling n values
  return philox_fill(true, seeds, pop, n, counter, out, stream);
}

extern "C" int evox_lora_down(const float* x, int32_t x_is_shared, const float* A, int64_t pop, int64_t batch, int64_t k,
                              int32_t r, float* t, void* stream) {
  EVOX_REQUIRE(x && A && t, EVOX_ERR_INVALID, "lora_down: NULL pointer");
  EVOX_REQUIRE(pop > 0 && batch > 0 && k > 0 && r > 0, EVOX_ERR_INVALID, "lora_down: sizes must be positive");
  lora_down_kernel<<<grid_for(pop * batch * 32), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      x, x_is_shared ? 0 : batch * k, A, pop, batch, k, r, t);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_lora_delta_output(const float* x, const float* A, const float* B, float sigma, int64_t pop,
                                      int64_t batch, int64_t k, int32_t r, int64_t d, float* out, float* t_scratch,
                                      void* stream) {
  EVOX_REQUIRE(x && A && B && out && t_scratch, EVOX_ERR_INVALID, "lora_delta_output: NULL pointer");
  EVOX_REQUIRE(pop > 0 && batch > 0 && k > 0 && r > 0 && d > 0, EVOX_ERR_INVALID, "lora_delta_output: sizes must be positive");
  if (int rc = evox_lora_down(x, 0, A, pop, batch, k, r, t_scratch, stream)) return rc;
  lora_up_kernel<<<grid_for(pop * batch * d), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(t_scratch, B, sigma, pop,
                                                                                                   batch, d, r, out);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_lora_gradient(const float* fitness, const float* A, const float* B, int64_t pop, float sigma,
                                  int64_t d, int64_t k, int32_t r, float* grad, void* stream) {
  EVOX_REQUIRE(fitness && A && grad, EVOX_ERR_INVALID, "lora_gradient: NULL pointer");
  EVOX_REQUIRE(pop > 0 && k > 0, EVOX_ERR_INVALID, "lora_gradient: sizes must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float inv_scale = 1.0f / ((float)pop * sigma);
  if (B == nullptr) {  // 1-D block: A is the (pop, k) noise
    launch_weighted_rows(fitness, A, pop, k, pop, inv_scale, grad, s);
  } else {
    EVOX_REQUIRE(d > 0 && r > 0 && r <= 64, EVOX_ERR_INVALID, "lora_gradient: rank must be in [1, 64], got %d", r);
    dim3 grid((unsigned)((k + 63) / 64), (unsigned)((d + 63) / 64));
    if (r <= 8) lora_gradient_kernel<8><<<grid, kThreads, 0, s>>>(fitness, A, B, pop, inv_scale, d, k, r, grad);
    else if (r <= 16) lora_gradient_kernel<16><<<grid, kThreads, 0, s>>>(fitness, A, B, pop, inv_scale, d, k, r, grad);
    else lora_gradient_kernel<64><<<grid, kThreads, 0, s>>>(fitness, A, B, pop, inv_scale, d, k, r, grad);
  }
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_lora_linear_forward(const float* h, int32_t h_is_shared, const float* W, const float* bias,
                                        const float* t, const float* B, const float* bias_noise, float sigma,
                                        int64_t pop, int64_t batch, int64_t k, int64_t d, int32_t r, int32_t relu,
                                        float* out, void* stream) {
  EVOX_REQUIRE(h && W && out, EVOX_ERR_INVALID, "lora_linear_forward: NULL pointer");
  EVOX_REQUIRE((t == nullptr) == (B == nullptr), EVOX_ERR_INVALID, "lora_linear_forward: t and B go together");
  EVOX_REQUIRE(pop > 0 && batch > 0 && k > 0 && d > 0, EVOX_ERR_INVALID, "lora_linear_forward: sizes must be positive");
  dim3 grid((unsigned)((d + 63) / 64), (unsigned)((pop * batch + 63) / 64));
  lora_linear_kernel<<<grid, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      h, h_is_shared ? 0 : batch * k, W, bias, t, B, bias_noise, sigma, pop, batch, k, d, r, relu, out);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_openes_ask(const float* center, const float* noise, const float* sigma, int64_t pop, int64_t dim,
                               int64_t noise_rows, float* population, void* stream) {
  EVOX_REQUIRE(center && noise && sigma && population, EVOX_ERR_INVALID, "openes_ask: NULL pointer");
  EVOX_REQUIRE(pop > 0 && dim > 0 && (noise_rows == pop || 2 * noise_rows == pop), EVOX_ERR_INVALID,
               "openes_ask: noise_rows must be pop or pop / 2");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = dim % 4 == 0 && aligned16(center) && aligned16(noise) && aligned16(population);
  const bool mirrored = noise_rows < pop;
  const dim3 grid = vec ? rows_by_cols_grid(noise_rows, dim / 4) : rows_by_cols_grid(noise_rows, dim);
  if (vec && mirrored) openes_ask_kernel<4, true, false><<<grid, kThreads, 0, s>>>(center, noise, sigma, pop, dim, noise_rows, population, nullptr);
  else if (vec) openes_ask_kernel<4, false, false><<<grid, kThreads, 0, s>>>(center, noise, sigma, pop, dim, noise_rows, population, nullptr);
  else if (mirrored) openes_ask_kernel<1, true, false><<<grid, kThreads, 0, s>>>(center, noise, sigma, pop, dim, noise_rows, population, nullptr);
  else openes_ask_kernel<1, false, false><<<grid, kThreads, 0, s>>>(center, noise, sigma, pop, dim, noise_rows, population, nullptr);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_pes_ask(const float* center, const float* noise, const float* sigma, int64_t pop, int64_t dim,
                            float* pert_accum, float* population, void* stream) {
  EVOX_REQUIRE(center && noise && sigma && pert_accum && population, EVOX_ERR_INVALID, "pes_ask: NULL pointer");
  EVOX_REQUIRE(pop > 0 && dim > 0 && pop % 2 == 0, EVOX_ERR_INVALID, "pes_ask: pop must be positive and even");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dim % 4 == 0 && aligned16(center) && aligned16(noise) && aligned16(population) && aligned16(pert_accum))
    openes_ask_kernel<4, true, true><<<rows_by_cols_grid(pop / 2, dim / 4), kThreads, 0, s>>>(center, noise, sigma, pop, dim, pop / 2, population, pert_accum);
  else
    openes_ask_kernel<1, true, true><<<rows_by_cols_grid(pop / 2, dim), kThreads, 0, s>>>(center, noise, sigma, pop, dim, pop / 2, population, pert_accum);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_es_ask_diag(const float* center, const float* noise, const float* sigma, int64_t pop, int64_t dim,
                                float* population, void* stream) {
  EVOX_REQUIRE(center && noise && sigma && population, EVOX_ERR_INVALID, "es_ask_diag: NULL pointer");
  EVOX_REQUIRE(pop > 0 && dim > 0, EVOX_ERR_INVALID, "es_ask_diag: sizes must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dim % 4 == 0 && aligned16(center) && aligned16(noise) && aligned16(sigma) && aligned16(population))
    es_ask_diag_kernel<4><<<rows_by_cols_grid(pop, dim / 4), kThreads, 0, s>>>(center, noise, sigma, pop, dim, population);
  else
    es_ask_diag_kernel<1><<<rows_by_cols_grid(pop, dim), kThreads, 0, s>>>(center, noise, sigma, pop, dim, population);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_rank_weighted_moments(const float* x, const float* row_weights, const float* shift, float offset, int64_t pop,
                                          int64_t dim, float* first, float* second, void* stream) {
  EVOX_REQUIRE(x && row_weights && first && second, EVOX_ERR_INVALID, "rank_weighted_moments: NULL pointer");
  EVOX_REQUIRE(pop > 0 && dim > 0, EVOX_ERR_INVALID, "rank_weighted_moments: sizes must be positive");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dim % 4 == 0 && aligned16(x) && dim >= 128ll * sm_count())
    rank_weighted_moments_kernel<4><<<grid_for(dim, 128), kThreads, 0, s>>>(x, row_weights, shift, offset, pop, dim, first, second);
  else
    rank_weighted_moments_kernel<1><<<grid_for(dim, 32), kThreads, 0, s>>>(x, row_weights, shift, offset, pop, dim, first, second);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_openes_gradient(const float* noise, const float* fitness, int64_t pop, int64_t dim, int64_t noise_rows,
                                    float sigma, float* grad, void* stream) {
  EVOX_REQUIRE(noise && fitness && grad, EVOX_ERR_INVALID, "openes_gradient: NULL pointer");
  EVOX_REQUIRE(pop > 0 && dim > 0 && (noise_rows == pop || 2 * noise_rows == pop), EVOX_ERR_INVALID,
               "openes_gradient: noise_rows must be pop or pop / 2");
  // grad = noise^T fitness / pop / sigma (open_es.py:70)
  launch_weighted_rows(fitness, noise, pop, dim, noise_rows, 1.0f / (float)pop / sigma, grad, reinterpret_cast<cudaStream_t>(stream));
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_es_update(float* center, const float* grad, const float* learning_rate, float* exp_avg,
                              float* exp_avg_sq, const float* beta1, const float* beta2, float eps, int64_t dim,
                              void* stream) {
  EVOX_REQUIRE(center && grad && learning_rate, EVOX_ERR_INVALID, "es_update: NULL pointer");
  EVOX_REQUIRE((exp_avg == nullptr) == (exp_avg_sq == nullptr), EVOX_ERR_INVALID, "es_update: both Adam moments or neither");
  EVOX_REQUIRE(exp_avg == nullptr || (beta1 && beta2), EVOX_ERR_INVALID, "es_update: Adam needs beta1 and beta2");
  EVOX_REQUIRE(dim > 0, EVOX_ERR_INVALID, "es_update: dim must be positive");
  es_update_kernel<<<grid_for(dim), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      center, grad, learning_rate, exp_avg, exp_avg_sq, beta1, beta2, eps, dim);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
