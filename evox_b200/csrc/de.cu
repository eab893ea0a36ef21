// Differential evolution (rand/1/bin and best/1/bin): trial vectors fused with their evaluation, then the
// one-to-one selection.
//
// Reference semantics: DE.step (evox/algorithms/so/de_variants/de.py:105-157) with one difference vector:
//   mutant = base + F * (pop[r1] - pop[r2]),  base = pop[r0] or the best individual;
//   trial  = where(cross < CR or column == forced column, mutant, pop[i]), relu-form clamp;
//   pop[i], fit[i] <- trial, f(trial) where f(trial) < fit[i].
// Every mutant reads OTHER individuals' vectors of the generation before, so the trials go to a buffer of
// their own (de_trial_kernel: one warp per individual, up to four rows read + one written per
// individual-dimension, fitness fused) and a second launch copies the winners (de_select_kernel: 8 B per
// accepted individual-dimension).
#include "common.cuh"
#include "fitness.cuh"

namespace evox {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

struct DeArgs {
  const float* pop;
  float* trial;
  float* trial_fit;
  const long long* r0;     // base rows, or null: every mutant starts from row `best`
  const long long* r1;
  const long long* r2;
  const long long* best;   // device scalar: row of the best individual (base "best")
  const long long* forced; // column that always crosses over
  const float* lb;
  const float* ub;
  const float* weight;     // F (device scalar)
  const float* cr;         // CR (device scalar)
  const float* cross;      // (P, d) uniform draws or null: in-kernel Philox
  long long P;
  int d;
  FitParams fp;
  PhiloxKeys keys;
  unsigned long long generation;
  int write_fit;
};

// de.py:133-143 for one variable, each operation rounded on its own.
__device__ __forceinline__ float trial_one(float x, float base, float a, float b, float lb, float ub, float u, bool is_forced, float F,
                                           float cr) {
  const float mutant = __fadd_rn(base, __fmul_rn(F, __fsub_rn(a, b)));
  const float t = (u < cr || is_forced) ? mutant : x;
  return relu_clamp(t, lb, ub);
}

template <int VEC, bool PHILOX, int FIT>
__global__ void __launch_bounds__(kThreads, 4) de_trial_kernel(const DeArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  const float F = *a.weight, cr = *a.cr;
  const int d = a.d;
  const int n_call = (d + 3) >> 2;
  const long long best = a.r0 ? 0 : *a.best;
  auto row_of = [&](long long r) { return ((unsigned long long)r < (unsigned long long)a.P) ? r : 0; };
  for (long long row = warp0; row < a.P; row += n_warps) {
    const size_t base = (size_t)row * (size_t)d;
    const size_t b0 = (size_t)row_of(a.r0 ? a.r0[row] : best) * (size_t)d;
    const size_t b1 = (size_t)row_of(a.r1[row]) * (size_t)d, b2 = (size_t)row_of(a.r2[row]) * (size_t)d;
    const int forced = (int)a.forced[row];
    Fitness<FIT> acc;
    if constexpr (VEC == 4) {
      const float4* x4 = reinterpret_cast<const float4*>(a.pop + base);
      const float4* p0 = reinterpret_cast<const float4*>(a.pop + b0);
      const float4* p1 = reinterpret_cast<const float4*>(a.pop + b1);
      const float4* p2 = reinterpret_cast<const float4*>(a.pop + b2);
      float4* out4 = reinterpret_cast<float4*>(a.trial + base);
      const float4* lb4 = reinterpret_cast<const float4*>(a.lb);
      const float4* ub4 = reinterpret_cast<const float4*>(a.ub);
      for (int c = lane; c < n_call; c += 32) {
        const float4 x = __ldg(x4 + c), v0 = __ldg(p0 + c), v1 = __ldg(p1 + c), v2 = __ldg(p2 + c);
        float4 u;
        if constexpr (PHILOX) {
          // counter (q lo, q hi, generation lo, generation hi), q = row * ceil(d / 4) + column / 4
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)c;
          const uint4 r = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation, (uint32_t)(a.generation >> 32), a.keys);
          u = make_float4(u24_to_unit(r.x), u24_to_unit(r.y), u24_to_unit(r.z), u24_to_unit(r.w));
        } else {
          u = __ldcs(reinterpret_cast<const float4*>(a.cross + base) + c);
        }
        const float4 lb = __ldg(lb4 + c), ub = __ldg(ub4 + c);
        const int e = c * 4;
        float4 t;
        t.x = trial_one(x.x, v0.x, v1.x, v2.x, lb.x, ub.x, u.x, e == forced, F, cr);
        t.y = trial_one(x.y, v0.y, v1.y, v2.y, lb.y, ub.y, u.y, e + 1 == forced, F, cr);
        t.z = trial_one(x.z, v0.z, v1.z, v2.z, lb.z, ub.z, u.z, e + 2 == forced, F, cr);
        t.w = trial_one(x.w, v0.w, v1.w, v2.w, lb.w, ub.w, u.w, e + 3 == forced, F, cr);
        __stcs(out4 + c, t);
        acc.add4(t, a.fp);
      }
    } else {
      for (int e = lane; e < d; e += 32) {
        float u;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)(e >> 2);
          const uint4 r = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation, (uint32_t)(a.generation >> 32), a.keys);
          const int k = e & 3;
          u = u24_to_unit(k == 0 ? r.x : (k == 1 ? r.y : (k == 2 ? r.z : r.w)));
        } else {
          u = a.cross[base + e];
        }
        const float t = trial_one(a.pop[base + e], a.pop[b0 + e], a.pop[b1 + e], a.pop[b2 + e], a.lb[e], a.ub[e], u, e == forced, F, cr);
        a.trial[base + e] = t;
        acc.add(t, a.fp);
      }
    }
    acc.reduce();
    if (lane == 0 && a.write_fit) a.trial_fit[row] = acc.finish(d, a.fp);
  }
}

// de.py:152-157: individuals whose trial is strictly better are replaced by it.
__global__ void __launch_bounds__(kThreads)
    de_select_kernel(const float* __restrict__ trial, const float* __restrict__ trial_fit, float* __restrict__ pop, float* __restrict__ fit,
                     long long P, int d, int vec) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  for (long long row = warp0; row < P; row += n_warps) {
    const float f = trial_fit[row];
    if (!(f < fit[row])) continue;
    const size_t base = (size_t)row * (size_t)d;
    if (vec) {
      const float4* src = reinterpret_cast<const float4*>(trial + base);
      float4* dst = reinterpret_cast<float4*>(pop + base);
      for (int c = lane; c < (d >> 2); c += 32) __stcs(dst + c, __ldcs(src + c));
    } else {
      for (int e = lane; e < d; e += 32) pop[base + e] = trial[base + e];
    }
    __syncwarp();
    if (lane == 0) fit[row] = f;
  }
}

template <int VEC, bool PHILOX>
void launch_trial(int fitness_id, int grid, cudaStream_t s, const DeArgs& a) {
  switch (fitness_id) {
    case EVOX_FIT_ACKLEY:
      de_trial_kernel<VEC, PHILOX, EVOX_FIT_ACKLEY><<<grid, kThreads, 0, s>>>(a);
      break;
    case EVOX_FIT_RASTRIGIN:
      de_trial_kernel<VEC, PHILOX, EVOX_FIT_RASTRIGIN><<<grid, kThreads, 0, s>>>(a);
      break;
    default:
      de_trial_kernel<VEC, PHILOX, EVOX_FIT_SPHERE><<<grid, kThreads, 0, s>>>(a);
      break;
  }
}

int row_grid(long long rows) {
  const long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = (long long)sm_count() * 4;
  return (int)(blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" int evox_de_trial(const float* pop, float* trial, float* trial_fit, const int64_t* base_rows, const int64_t* best_row,
                             const int64_t* rows_a, const int64_t* rows_b, const int64_t* forced_column, const float* lb,
                             const float* ub, const float* differential_weight, const float* cross_probability, const float* cross,
                             int64_t pop_size, int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                             uint64_t generation, void* stream) {
  EVOX_REQUIRE(pop && trial && rows_a && rows_b && forced_column && lb && ub && differential_weight && cross_probability,
               EVOX_ERR_INVALID, "de_trial: NULL pointer");
  EVOX_REQUIRE((base_rows != nullptr) != (best_row != nullptr), EVOX_ERR_INVALID, "de_trial: give base_rows or best_row, not both");
  EVOX_REQUIRE(pop != trial, EVOX_ERR_INVALID, "de_trial: pop and trial must be different buffers");
  EVOX_REQUIRE(pop_size > 0 && dim > 0, EVOX_ERR_INVALID, "de_trial: sizes must be positive");
  EVOX_REQUIRE(fitness_id == -1 || (fitness_id >= EVOX_FIT_ACKLEY && fitness_id <= EVOX_FIT_SPHERE), EVOX_ERR_INVALID,
               "de_trial: unknown fitness id %d", fitness_id);
  EVOX_REQUIRE(fitness_id == -1 || trial_fit, EVOX_ERR_INVALID, "de_trial: trial_fit is NULL");
  EVOX_REQUIRE(fitness_id != EVOX_FIT_ACKLEY || params, EVOX_ERR_INVALID, "de_trial: Ackley needs params {a, b, c}");
  DeArgs a;
  a.pop = pop;
  a.trial = trial;
  a.trial_fit = trial_fit;
  a.r0 = (const long long*)base_rows;
  a.r1 = (const long long*)rows_a;
  a.r2 = (const long long*)rows_b;
  a.best = (const long long*)best_row;
  a.forced = (const long long*)forced_column;
  a.lb = lb;
  a.ub = ub;
  a.weight = differential_weight;
  a.cr = cross_probability;
  a.cross = cross;
  a.P = pop_size;
  a.d = dim;
  a.fp = (fitness_id == EVOX_FIT_ACKLEY) ? FitParams{params[0], params[1], params[2]} : FitParams{0.f, 0.f, 0.f};
  a.keys = philox_round_keys(seed);
  a.generation = generation;
  a.write_fit = fitness_id != -1;
  const int fid = fitness_id == -1 ? EVOX_FIT_SPHERE : fitness_id;
  const bool vec = (dim % 4 == 0) && aligned16(pop) && aligned16(trial) && aligned16(lb) && aligned16(ub) && (cross == nullptr || aligned16(cross));
  const int grid = row_grid(pop_size);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (vec) {
    if (cross) launch_trial<4, false>(fid, grid, s, a); else launch_trial<4, true>(fid, grid, s, a);
  } else {
    if (cross) launch_trial<1, false>(fid, grid, s, a); else launch_trial<1, true>(fid, grid, s, a);
  }
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_de_select(const float* trial, const float* trial_fit, float* pop, float* fit, int64_t pop_size, int32_t dim,
                              void* stream) {
  EVOX_REQUIRE(trial && trial_fit && pop && fit, EVOX_ERR_INVALID, "de_select: NULL pointer");
  EVOX_REQUIRE(pop_size > 0 && dim > 0, EVOX_ERR_INVALID, "de_select: sizes must be positive");
  EVOX_REQUIRE(pop != trial, EVOX_ERR_INVALID, "de_select: pop and trial must be different buffers");
  const int vec = (dim % 4 == 0) && aligned16(pop) && aligned16(trial);
  de_select_kernel<<<row_grid(pop_size), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(trial, trial_fit, pop, fit, pop_size, dim, vec);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
