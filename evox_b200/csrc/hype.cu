// Monte-Carlo hypervolume contributions of HypE.
//
// Reference semantics: cal_hv (evox/algorithms/mo/hype.py:12-39). For n objective rows and n_sample
// sampling points the reference materialises the (n_sample, n) table "row i is <= sample s in every
// objective" twice (as bool and as int64) and gathers alpha through it; here the table is never stored:
//   hv_sample_count_kernel    count_s = #rows that cover sample s (row slices on grid y, integer atomics)
//   hv_row_sum_kernel         partial[slice][i] = sum of weight_s = alpha[count_s - 1] (0 if nobody covers s)
//                             over the samples of the slice covered by row i
//   hv_finish_kernel          hv[i] = (sum over slices, in slice order) * volume / n_sample
// The counts are integers and the cover test is the reference's (f - s) <= 0 in fp32, so the only
// difference from the reference is the order in which the fp32 weights of one row are added.
#include "common.cuh"

namespace evox {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSamplesPerWarp = 4;
constexpr int kSamplesPerBlock = kWarps * kSamplesPerWarp;
constexpr int kMaxObjectives = 32;  // the generic row-sum kernel keeps 256 rows x m words of its own in the 48 KB
constexpr int kTileFloats = 12288;  // 48 KB of staged rows / samples per block
constexpr int kMaxSlices = 16;

__host__ __device__ inline int row_tile(int m) {
  int t = kTileFloats / m;
  t = t > 1024 ? 1024 : t;
  return t & ~31;
}

// The objectives of one row or one sample: registers when the count is known at compile time (M > 0),
// a strided view of shared memory otherwise.
template <int M>
struct Point {
  float v[M];
  __device__ __forceinline__ void load(const float* src, int stride, int) {
#pragma unroll
    for (int k = 0; k < M; ++k) v[k] = src[(size_t)k * stride];
  }
  __device__ __forceinline__ float get(int k) const { return v[k]; }
};
template <>
struct Point<0> {
  const float* p;
  int stride;
  __device__ __forceinline__ void load(const float* src, int stride_, int) {
    p = src;
    stride = stride_;
  }
  __device__ __forceinline__ float get(int k) const { return p[(size_t)k * stride]; }
};

// rows: tile[k * tile_rows + i] (structure of arrays, so that a warp reads consecutive words).
// blockIdx.y takes a slice of the rows; the integer counts of the slices meet in `count` (zeroed by the
// caller) with atomicAdd, which is exact in any order.
template <int M>
__global__ void __launch_bounds__(kThreads) hv_sample_count_kernel(const float* __restrict__ fit, const float* __restrict__ samples,
                                                                   long long n, int m_rt, long long n_sample, long long rows_per_slice,
                                                                   int* __restrict__ count) {
  extern __shared__ __align__(16) float smem[];
  const int m = M ? M : m_rt;
  const int tile_rows = row_tile(m);
  float* tile = smem;                            // m * tile_rows
  float* smp = smem + (size_t)m * tile_rows;     // kSamplesPerBlock * m, sample-major
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long s_block = (long long)blockIdx.x * kSamplesPerBlock;
  for (int e = threadIdx.x; e < kSamplesPerBlock * m; e += kThreads) {
    const long long s = s_block + e / m;
    smp[e] = s < n_sample ? samples[s * m + e % m] : 0.f;
  }
  __syncthreads();
  Point<M> pt[kSamplesPerWarp];
#pragma unroll
  for (int j = 0; j < kSamplesPerWarp; ++j) pt[j].load(smp + (warp * kSamplesPerWarp + j) * m, 1, m);
  int cnt[kSamplesPerWarp] = {0, 0, 0, 0};
  const long long r_begin = (long long)blockIdx.y * rows_per_slice;
  const long long r_end = (r_begin + rows_per_slice) < n ? (r_begin + rows_per_slice) : n;
  for (long long r0 = r_begin; r0 < r_end; r0 += tile_rows) {
    const int rows = (int)((r_end - r0) < tile_rows ? (r_end - r0) : tile_rows);
    __syncthreads();
    for (int e = threadIdx.x; e < rows * m; e += kThreads) {
      const int i = e / m, k = e - i * m;
      tile[k * tile_rows + i] = fit[r0 * m + e];
    }
    __syncthreads();
    for (int i = lane; i < rows; i += 32) {
      bool ok[kSamplesPerWarp] = {true, true, true, true};
      auto test = [&](int k) {
        const float f = tile[k * tile_rows + i];
#pragma unroll
        for (int j = 0; j < kSamplesPerWarp; ++j) ok[j] &= (__fsub_rn(f, pt[j].get(k)) <= 0.f);  // no short circuit: no branches
      };
      if constexpr (M > 0) {
#pragma unroll
        for (int k = 0; k < M; ++k) test(k);
      } else {
#pragma unroll 4
        for (int k = 0; k < m; ++k) test(k);
      }
#pragma unroll
      for (int j = 0; j < kSamplesPerWarp; ++j) cnt[j] += ok[j] ? 1 : 0;
    }
  }
#pragma unroll
  for (int j = 0; j < kSamplesPerWarp; ++j) {
    int c = cnt[j];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
    const long long s = s_block + warp * kSamplesPerWarp + j;
    if (lane == 0 && s < n_sample && c) atomicAdd(count + s, c);
  }
}

// Words per staged sample in hv_row_sum_kernel: the objectives, then the weight; padded to whole float4
// when the number of objectives is known at compile time, so that a sample is one or two 16-byte reads.
__host__ __device__ constexpr int sample_stride(int M, int m) { return M ? ((M + 1 + 3) & ~3) : (m + 1); }

// One thread per row, a slice of the samples per blockIdx.y. Every thread of the block reads the same
// staged sample at the same time (shared-memory broadcast).
template <int M>
__global__ void __launch_bounds__(kThreads) hv_row_sum_kernel(const float* __restrict__ fit, const float* __restrict__ samples,
                                                              const int* __restrict__ count, const float* __restrict__ alpha,
                                                              long long n, int m_rt, long long n_sample, long long slice_len,
                                                              float* __restrict__ partial) {
  extern __shared__ __align__(16) float smem[];
  const int m = M ? M : m_rt;
  const int stride = sample_stride(M, m);
  const int tile_samples = (kTileFloats - (M ? 0 : kThreads * m)) / stride;
  float* tile = smem;                                    // tile_samples * stride
  float* own = smem + (size_t)tile_samples * stride;     // generic m only: this block's rows, [k][thread]
  const long long i = (long long)blockIdx.x * kThreads + threadIdx.x;
  const bool live = i < n;
  Point<M> f;
  if constexpr (M > 0) {
    f.load(fit + (live ? i : 0) * m, 1, m);
  } else {
    for (int k = 0; k < m; ++k) own[k * kThreads + threadIdx.x] = fit[(live ? i : 0) * m + k];
    f.load(own + threadIdx.x, kThreads, m);
  }
  const long long s_begin = (long long)blockIdx.y * slice_len;
  const long long s_end = (s_begin + slice_len) < n_sample ? (s_begin + slice_len) : n_sample;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (long long s0 = s_begin; s0 < s_end; s0 += tile_samples) {
    const int cnt = (int)((s_end - s0) < tile_samples ? (s_end - s0) : tile_samples);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * stride; e += kThreads) {
      const int s = e / stride, k = e - s * stride;
      float v = 0.f;
      if (k < m) {
        v = samples[(s0 + s) * m + k];
      } else if (k == m) {
        // hype.py:32-35: ds - 1 where ds > 0, then alpha[ds]; a sample nobody covers adds nothing
        const int c = count[s0 + s];
        v = c > 0 ? alpha[c - 1] : 0.f;
      }
      tile[e] = v;
    }
    __syncthreads();
    // four accumulators dealt by sample number inside the tile: short chains, fixed order
    auto covered = [&](int s) -> float {
      if constexpr (M > 0) {
        constexpr int kWords = sample_stride(M, 0);
        float w[kWords];
#pragma unroll
        for (int q = 0; q < kWords / 4; ++q) {
          const float4 v = reinterpret_cast<const float4*>(tile + s * kWords)[q];
          w[4 * q] = v.x, w[4 * q + 1] = v.y, w[4 * q + 2] = v.z, w[4 * q + 3] = v.w;
        }
        bool ok = true;
#pragma unroll
        for (int k = 0; k < M; ++k) ok &= (__fsub_rn(f.get(k), w[k]) <= 0.f);
        return ok ? w[M] : 0.f;
      } else {
        const float* sp = tile + s * stride;
        bool ok = true;
#pragma unroll 4
        for (int k = 0; k < m; ++k) ok &= (__fsub_rn(f.get(k), sp[k]) <= 0.f);
        return ok ? sp[m] : 0.f;
      }
    };
    int s = 0;
    for (; s + 4 <= cnt; s += 4) {
      acc[0] += covered(s);
      acc[1] += covered(s + 1);
      acc[2] += covered(s + 2);
      acc[3] += covered(s + 3);
    }
    for (; s < cnt; ++s) acc[0] += covered(s);
  }
  if (live) partial[(size_t)blockIdx.y * n + i] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

__global__ void hv_finish_kernel(const float* __restrict__ partial, int slices, long long n, const float* __restrict__ volume,
                                 long long n_sample, float* __restrict__ hv) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += partial[(size_t)k * n + i];
  hv[i] = __fdiv_rn(__fmul_rn(s, *volume), (float)n_sample);  // hype.py:38
}

int slices_for(long long n, long long n_sample) {
  const long long row_blocks = (n + kThreads - 1) / kThreads;
  long long want = (2LL * sm_count() + row_blocks - 1) / row_blocks;
  const long long by_len = (n_sample + 255) / 256;  // at least 256 samples per slice
  want = want > by_len ? by_len : want;
  want = want > kMaxSlices ? kMaxSlices : want;
  return (int)(want < 1 ? 1 : want);
}

template <int M>
void launch_hv(const float* fit, const float* samples, const float* alpha, const float* volume, long long n, int m, long long n_sample,
               float* hv, int* count, float* partial, int slices, cudaStream_t s) {
  const size_t smem1 = ((size_t)m * row_tile(m) + (size_t)kSamplesPerBlock * m) * sizeof(float);
  const size_t smem2 = (size_t)kTileFloats * sizeof(float);
  if (smem1 > 48 * 1024) cudaFuncSetAttribute(hv_sample_count_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
  const long long g1 = (n_sample + kSamplesPerBlock - 1) / kSamplesPerBlock;
  // enough blocks for four per multiprocessor, but no row slice shorter than one staged tile
  long long row_slices = (4LL * sm_count() + g1 - 1) / g1;
  const long long max_slices = (n + row_tile(m) - 1) / row_tile(m);
  row_slices = row_slices > max_slices ? max_slices : row_slices;
  row_slices = row_slices > 65535 ? 65535 : (row_slices < 1 ? 1 : row_slices);
  const long long rows_per_slice = (n + row_slices - 1) / row_slices;
  cudaMemsetAsync(count, 0, sizeof(int) * (size_t)n_sample, s);
  hv_sample_count_kernel<M><<<dim3((unsigned)g1, (unsigned)row_slices), kThreads, smem1, s>>>(fit, samples, n, m, n_sample, rows_per_slice, count);
  const long long slice_len = (n_sample + slices - 1) / slices;
  const dim3 g2((unsigned)((n + kThreads - 1) / kThreads), (unsigned)slices);
  hv_row_sum_kernel<M><<<g2, kThreads, smem2, s>>>(fit, samples, count, alpha, n, m, n_sample, slice_len, partial);
  hv_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, slices, n, volume, n_sample, hv);
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_hv_workspace_bytes(int64_t n, int64_t n_sample) {
  if (n <= 0 || n_sample <= 0) return 0;
  return ((size_t)n_sample + (size_t)kMaxSlices * (size_t)n) * sizeof(float);
}

extern "C" int evox_hv_contribution(const float* fit, const float* samples, const float* alpha, const float* volume, int64_t n,
                                    int32_t m, int64_t n_sample, float* hv, void* workspace, size_t workspace_bytes, void* stream) {
  EVOX_REQUIRE(fit && samples && alpha && volume && hv && workspace, EVOX_ERR_INVALID, "hv_contribution: NULL pointer");
  EVOX_REQUIRE(n > 0 && n_sample > 0, EVOX_ERR_INVALID, "hv_contribution: sizes must be positive");
  EVOX_REQUIRE(m >= 1 && m <= kMaxObjectives, EVOX_ERR_INVALID, "hv_contribution: 1 <= m <= %d objectives, got %d", kMaxObjectives, m);
  EVOX_REQUIRE(workspace_bytes >= evox_hv_workspace_bytes(n, n_sample), EVOX_ERR_WORKSPACE, "hv_contribution: workspace too small");
  int* count = static_cast<int*>(workspace);
  float* partial = reinterpret_cast<float*>(count + n_sample);
  const int slices = slices_for(n, n_sample);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (m) {
    case 2: launch_hv<2>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 3: launch_hv<3>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 4: launch_hv<4>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 5: launch_hv<5>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 6: launch_hv<6>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 7: launch_hv<7>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    case 8: launch_hv<8>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
    default: launch_hv<0>(fit, samples, alpha, volume, n, m, n_sample, hv, count, partial, slices, s); break;
  }
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
