// Issue-rate microbenchmark behind the roofline of the non-dominated sort.
//
// The dominance phase of non_dominate_rank (evox/operators/selection/non_dominate.py:6-26) reads a few
// kilobytes and performs m * n^2 fp32 comparisons whose results are combined into predicates: its
// ceiling is the rate at which the SMs issue fp32 set-predicate instructions, which no vendor figure and
// no memory-copy measurement gives. This kernel measures that rate on the GPU it runs on: every thread
// keeps 4 values a[i] and 16 values b[j] in registers and evaluates, per iteration, the 64 comparisons
// a[i] <= b[j], AND-combined per i (the shape of "all(a <= b)" in the dominance test); the b[j] move by
// a float add per iteration (a different pipe) so that nothing is loop-invariant, and each of the four
// predicates is consumed by one integer select-add. The caller times the launch with CUDA events and
// divides 64 * iterations * threads by the duration.
#include "common.cuh"

namespace evox {
namespace {

__global__ void __launch_bounds__(256) compare_rate_kernel(const float* __restrict__ in, unsigned int* __restrict__ out,
                                                           int iterations) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  float a[4], b[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) a[i] = in[(tid + i) & 1023];
#pragma unroll
  for (int j = 0; j < 16; ++j) b[j] = in[(tid * 7 + j) & 1023];
  const float step = in[1023];
  unsigned int acc = 0;
  for (int it = 0; it < iterations; ++it) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      bool p = true;
#pragma unroll
      for (int j = 0; j < 16; ++j) p = p && (a[i] <= b[j]);
      acc += p ? 1u : 0u;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) b[j] = __fadd_rn(b[j], step);
  }
  out[tid] = acc;
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" int64_t evox_bench_compare_rate_threads(void) { return (int64_t)sm_count() * 8 * 256; }

extern "C" int evox_bench_compare_rate(const float* in, uint32_t* out, int32_t iterations, void* stream) {
  EVOX_REQUIRE(in && out, EVOX_ERR_INVALID, "bench_compare_rate: NULL pointer");
  EVOX_REQUIRE(iterations > 0, EVOX_ERR_INVALID, "bench_compare_rate: iterations must be positive");
  compare_rate_kernel<<<sm_count() * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, out, iterations);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
