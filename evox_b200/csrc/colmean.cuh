// Mean position of a swarm (column mean of a (P, d) row-major matrix) with a fixed summation order,
// shared by the swarm kernels that need torch.mean(pop, dim=0) (CSO, SL-PSO). Partial column sums are
// written per block — by colsum_kernel here, or by an update kernel that sees every row anyway — and
// colmean_finish_kernel folds them.
#pragma once
#include "common.cuh"

namespace evox {
namespace {

constexpr int kColmeanWarps = 8;
constexpr int kColmeanThreads = kColmeanWarps * 32;
constexpr int kColmeanBlocksPerSM = 4;

// Column sums of a (P, d) matrix: block (x = column tile, y = row group) sums its rows, warps folded in
// warp order, into partial[blockIdx.y][column].
template <int VEC>
__global__ void __launch_bounds__(kColmeanThreads) colsum_kernel(const float* __restrict__ pop, long long P, int d, float* __restrict__ partial) {
  __shared__ float sh[kColmeanWarps][32 * VEC];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + lane) * VEC;
  float s[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) s[j] = 0.f;
  if (col < d) {
    for (long long row = (long long)blockIdx.y * kColmeanWarps + warp; row < P; row += (long long)gridDim.y * kColmeanWarps) {
      if constexpr (VEC == 4) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(pop + (size_t)row * d + col));
        s[0] += x.x;
        s[1] += x.y;
        s[2] += x.z;
        s[3] += x.w;
      } else {
        s[0] += pop[(size_t)row * d + col];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) sh[warp][lane * VEC + j] = s[j];
  __syncthreads();
  if (warp == 0 && col < d) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float t = sh[0][lane * VEC + j];
      for (int w = 1; w < kColmeanWarps; ++w) t += sh[w][lane * VEC + j];
      partial[(size_t)blockIdx.y * d + col + j] = t;
    }
  }
}

// center[col] = (sum over the n_partial rows of partial[.][col], 32 interleaved running sums folded by a
// fixed tree) / P   (torch.mean(pop, dim=0)).
__global__ void __launch_bounds__(1024) colmean_finish_kernel(const float* __restrict__ partial, int n_partial, int d, long long P,
                                                                  float* __restrict__ center) {
  __shared__ float sh[32][33];
  const int col = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (col < d)
    for (int b = threadIdx.y; b < n_partial; b += 32) s += partial[(size_t)b * d + col];
  sh[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  for (int off = 16; off > 0; off >>= 1) {
    if ((int)threadIdx.y < off) sh[threadIdx.y][threadIdx.x] += sh[threadIdx.y + off][threadIdx.x];
    __syncthreads();
  }
  if (threadIdx.y == 0 && col < d) center[col] = sh[0][threadIdx.x] / (float)P;
}

// workspace: center [d padded to 4] | partial [max_partials][d]
long long padded_dim(int d) { return ((long long)d + 3) / 4 * 4; }
int max_partials() { return sm_count() * kColmeanBlocksPerSM; }

// Full pass: center (d floats) = column mean of pop; partial is scratch of max_partials() * d floats.
int run_colmean(const float* pop, long long P, int d, float* center, float* partial, cudaStream_t s) {
  const bool vec = (d % 4 == 0) && aligned16(pop);
  const int tile = vec ? 128 : 32;
  const int gx = (d + tile - 1) / tile;
  int gy = (max_partials() + gx - 1) / gx;
  const long long row_groups = (P + kColmeanWarps - 1) / kColmeanWarps;
  if (gy > row_groups) gy = (int)row_groups;
  if (gy > max_partials()) gy = max_partials();
  if (gy < 1) gy = 1;
  if (vec)
    colsum_kernel<4><<<dim3(gx, gy), kColmeanThreads, 0, s>>>(pop, P, d, partial);
  else
    colsum_kernel<1><<<dim3(gx, gy), kColmeanThreads, 0, s>>>(pop, P, d, partial);
  EVOX_LAUNCH_CHECK();
  colmean_finish_kernel<<<(d + 31) / 32, dim3(32, 32), 0, s>>>(partial, gy, d, P, center);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

}  // namespace
}  // namespace evox
