// Mating and variation around the NSGA-II / RVEA selection: binary tournament on several keys,
// and simulated binary crossover + polynomial mutation + clamp as one kernel.
//
// Reference semantics: tournament_selection_multifit
// (evox/operators/selection/tournament_selection.py:8-29), simulated_binary
// (evox/operators/crossover/sbx.py:4-39), polynomial_mutation
// (evox/operators/mutation/pm_mutation.py:6-68) and the clamp that follows them in NSGA2.step /
// RVEA.step (evox/algorithms/mo/nsga2.py:94-97, rvea.py:138-141). The reference runs them as about
// forty elementwise launches; here parents are gathered, crossed, mutated and clamped in one pass
// (8 bytes read + 4 bytes written per offspring variable when the draws come from Philox).
#include <math.h>

#include "common.cuh"

namespace evox {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ uint32_t sort_key(float x) {
  if (x != x) return 0xffffffffu;  // NaN sorts last, like torch's ascending sort
  if (x == 0.0f) x = 0.0f;
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Winner of each round: lexicographic minimum over the keys, LAST key first (lexsort's convention,
// evox/utils/jit_fix_operator.py:216-252); among equal candidates the earlier slot wins (stable sort).
__global__ void tournament_kernel(const long long* __restrict__ parents, long long n_round, int k,
                                  const float* __restrict__ fitness, int n_keys, long long* __restrict__ out) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < n_round; r += (long long)gridDim.x * blockDim.x) {
    long long best = parents[r * k];
    for (int c = 1; c < k; ++c) {
      const long long cand = parents[r * k + c];
      bool wins = false;
      for (int q = n_keys - 1; q >= 0; --q) {
        const uint32_t a = sort_key(fitness[cand * n_keys + q]), b = sort_key(fitness[best * n_keys + q]);
        if (a != b) {
          wins = a < b;
          break;
        }
      }
      if (wins) best = cand;
    }
    out[r] = best;
  }
}

struct VarArgs {
  const float* pop;            // (n_pop, d)
  const long long* mating;     // (n) row numbers into pop, or null: parents are rows 0..n-1 of pop
  const float* lb;
  const float* ub;
  const float* sbx_mu;         // (n / 2, d) draws, or all six null -> in-kernel Philox
  const long long* sbx_sign;   // (n / 2, d) in {0, 1}
  const float* sbx_half;
  const float* sbx_pc;
  const float* pm_site;        // (2 * (n / 2), d)
  const float* pm_mu;
  long long n;
  int d;
  float pro_c, inv_dis_c, neg_inv_dis_c;   // 1 / (dis_c + 1), -1 / (dis_c + 1)
  float site_threshold, dis_m_plus_1, inv_dis_m;  // pro_m / d, dis_m + 1, 1 / (dis_m + 1)
  unsigned long long seed, generation;
  int flags;                   // bit 0 crossover, bit 1 mutation, bit 2 final clamp
  float* out;                  // (2 * (n / 2), d)
};

__device__ __forceinline__ float philox_draw(const VarArgs& a, long long element, uint32_t which) {
  const uint4 r = philox4x32_10((uint32_t)(element >> 2), (uint32_t)((unsigned long long)element >> 34), (uint32_t)a.generation,
                                which + 8u * (uint32_t)(a.generation >> 32), (uint32_t)a.seed, (uint32_t)(a.seed >> 32));
  const int lane = (int)(element & 3);
  const uint32_t u = lane == 0 ? r.x : (lane == 1 ? r.y : (lane == 2 ? r.z : r.w));
  return u24_to_unit(u);
}

// polynomial_mutation for one variable (pm_mutation.py:26-66); every operation rounded on its own.
__device__ __forceinline__ float mutate_one(float x, float lower, float upper, float r_site, float mu, const VarArgs& a) {
  const bool site = r_site < a.site_threshold;
  const float hi = __fsub_rn(x, fmaxf(__fsub_rn(x, upper), 0.f));    // minimum(x, upper), relu form
  float pop = __fadd_rn(hi, fmaxf(__fsub_rn(lower, hi), 0.f));         // maximum(., lower)
  const float span = __fsub_rn(upper, lower);
  if (site && mu <= 0.5f) {
    const float norm = __fdiv_rn(__fsub_rn(pop, lower), span);
    const float inner = __fadd_rn(__fmul_rn(2.f, mu),
                                  __fmul_rn(__fsub_rn(1.f, __fmul_rn(2.f, mu)), powf(__fsub_rn(1.f, norm), a.dis_m_plus_1)));
    pop = __fadd_rn(pop, __fmul_rn(span, __fsub_rn(powf(inner, a.inv_dis_m), 1.f)));
  }
  if (site && mu > 0.5f) {
    const float norm = __fdiv_rn(__fsub_rn(upper, pop), span);
    const float inner = __fadd_rn(__fmul_rn(2.f, __fsub_rn(1.f, mu)),
                                  __fmul_rn(__fmul_rn(2.f, __fsub_rn(mu, 0.5f)), powf(__fsub_rn(1.f, norm), a.dis_m_plus_1)));
    pop = __fadd_rn(pop, __fmul_rn(span, __fsub_rn(1.f, powf(inner, a.inv_dis_m))));
  }
  return pop;
}

__global__ void __launch_bounds__(kThreads) offspring_kernel(const VarArgs a) {
  const long long half = a.n / 2;
  const long long total = half * a.d;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long i = e / a.d;
    const int c = (int)(e - i * a.d);
    const long long r1 = a.mating ? a.mating[i] : i, r2 = a.mating ? a.mating[i + half] : i + half;
    const float p1 = a.pop[r1 * a.d + c], p2 = a.pop[r2 * a.d + c];
    float mu, r_half, r_pc, site1, site2, pmu1, pmu2;
    int sign;
    if (a.sbx_mu != nullptr) {
      mu = a.sbx_mu[e];
      sign = (int)a.sbx_sign[e];
      r_half = a.sbx_half[e];
      r_pc = a.sbx_pc[e];
      site1 = a.pm_site[e];
      site2 = a.pm_site[e + total];
      pmu1 = a.pm_mu[e];
      pmu2 = a.pm_mu[e + total];
    } else {
      mu = philox_draw(a, e, 0u);
      sign = philox_draw(a, e, 1u) < 0.5f ? 0 : 1;
      r_half = philox_draw(a, e, 2u);
      r_pc = philox_draw(a, e, 3u);
      site1 = philox_draw(a, e, 4u);
      site2 = philox_draw(a, e + total, 4u);
      pmu1 = philox_draw(a, e, 5u);
      pmu2 = philox_draw(a, e + total, 5u);
    }
    // simulated binary crossover (sbx.py:21-37)
    float beta = (mu <= 0.5f) ? powf(__fmul_rn(2.f, mu), a.inv_dis_c) : powf(__fsub_rn(2.f, __fmul_rn(2.f, mu)), a.neg_inv_dis_c);
    beta = __fmul_rn(beta, (float)(1 - sign * 2));
    if (r_half < 0.5f) beta = 1.f;
    if (r_pc > a.pro_c) beta = 1.f;
    const float mid = __fdiv_rn(__fadd_rn(p1, p2), 2.f);
    const float dev = __fdiv_rn(__fmul_rn(beta, __fsub_rn(p1, p2)), 2.f);
    const float lower = a.lb[c], upper = a.ub[c];
    float c1 = (a.flags & 1) ? __fadd_rn(mid, dev) : p1;
    float c2 = (a.flags & 1) ? __fsub_rn(mid, dev) : p2;
    if (a.flags & 2) {
      c1 = mutate_one(c1, lower, upper, site1, pmu1, a);
      c2 = mutate_one(c2, lower, upper, site2, pmu2, a);
    }
    if (a.flags & 4) {
      c1 = relu_clamp(c1, lower, upper);
      c2 = relu_clamp(c2, lower, upper);
    }
    a.out[e] = c1;
    a.out[e + total] = c2;
  }
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" int evox_tournament_multifit(const int64_t* parents, int64_t n_round, int32_t tournament_size, const float* fitness,
                                        int64_t n_candidates, int32_t n_keys, int64_t* selected, void* stream) {
  EVOX_REQUIRE(parents && fitness && selected, EVOX_ERR_INVALID, "tournament_multifit: NULL pointer");
  EVOX_REQUIRE(n_round > 0 && tournament_size > 0 && n_keys > 0 && n_candidates > 0, EVOX_ERR_INVALID,
               "tournament_multifit: sizes must be positive");
  const long long blocks = (n_round + kThreads - 1) / kThreads;
  tournament_kernel<<<(unsigned)(blocks < 4096 ? blocks : 4096), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const long long*)parents, n_round, tournament_size, fitness, n_keys, (long long*)selected);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_offspring(const float* pop, const int64_t* mating_pool, int64_t n, int32_t dim, const float* lb,
                              const float* ub, const float* sbx_mu, const int64_t* sbx_sign, const float* sbx_half,
                              const float* sbx_pc, const float* pm_site, const float* pm_mu, float pro_c, float dis_c,
                              float pro_m, float dis_m, int32_t flags, uint64_t seed, uint64_t generation, float* offspring,
                              void* stream) {
  EVOX_REQUIRE(pop && lb && ub && offspring, EVOX_ERR_INVALID, "offspring: NULL pointer");
  EVOX_REQUIRE(n >= 2 && dim > 0, EVOX_ERR_INVALID, "offspring: needs at least two parents and a positive dimension");
  const bool any = sbx_mu || sbx_sign || sbx_half || sbx_pc || pm_site || pm_mu;
  const bool all = sbx_mu && sbx_sign && sbx_half && sbx_pc && pm_site && pm_mu;
  EVOX_REQUIRE(any == all, EVOX_ERR_INVALID, "offspring: give all six draw tensors or none");
  VarArgs a;
  a.pop = pop;
  a.mating = (const long long*)mating_pool;
  a.lb = lb;
  a.ub = ub;
  a.sbx_mu = sbx_mu;
  a.sbx_sign = (const long long*)sbx_sign;
  a.sbx_half = sbx_half;
  a.sbx_pc = sbx_pc;
  a.pm_site = pm_site;
  a.pm_mu = pm_mu;
  a.n = n;
  a.d = dim;
  a.pro_c = pro_c;
  a.inv_dis_c = (float)(1.0 / ((double)dis_c + 1.0));
  a.neg_inv_dis_c = (float)(-1.0 / ((double)dis_c + 1.0));
  a.site_threshold = (float)((double)pro_m / (double)dim);
  a.dis_m_plus_1 = (float)((double)dis_m + 1.0);
  a.inv_dis_m = (float)(1.0 / ((double)dis_m + 1.0));
  a.seed = seed;
  a.generation = generation;
  a.flags = flags;
  a.out = offspring;
  const long long total = (n / 2) * (long long)dim;
  long long blocks = (total + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count() * 16;
  offspring_kernel<<<(unsigned)(blocks < cap ? blocks : cap), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
