// Comprehensive-learning PSO: personal-best update and the move fused with the fitness evaluation.
//
// Reference semantics: CLPSO.step (evox/algorithms/so/pso_variants/clpso.py:72-123). Each particle
// learns from ONE personal best per generation — its own, or with probability P_c the better of two
// randomly chosen particles' — so the move reads another particle's personal-best row, and that row
// must already be the updated one (clpso.py:101-116 update all personal bests first). Hence two launches:
//   clpso_pbest_kernel      rows whose fitness improved copy pop -> personal_best_location (8 B per
//                           improved particle-dimension) and their fitness;
//   clpso_move_eval_kernel  one warp per particle: v' = w v + c r (pbest[src] - x), relu-form clamps
//                           (clpso.py:119-122; the position uses the UNclamped v'), fitness of the moved
//                           particle: 12 B read + 8 B written per particle-dimension.
// The global best is only tracked (clpso.py:105-108): the PSO arg-min kernels do that.
#include "common.cuh"
#include "fitness.cuh"

namespace evox {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

__global__ void __launch_bounds__(kThreads)
    clpso_pbest_kernel(const float* __restrict__ pop, const float* __restrict__ fit, float* __restrict__ pbest_loc,
                       float* __restrict__ pbest_fit, long long P, int d, int vec) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  for (long long row = warp0; row < P; row += n_warps) {
    const float f = fit[row];
    if (!(pbest_fit[row] > f)) continue;  // clpso.py:101
    const size_t base = (size_t)row * (size_t)d;
    if (vec) {
      const float4* src = reinterpret_cast<const float4*>(pop + base);
      float4* dst = reinterpret_cast<float4*>(pbest_loc + base);
      for (int c = lane; c < (d >> 2); c += 32) __stcs(dst + c, __ldcs(src + c));
    } else {
      for (int e = lane; e < d; e += 32) pbest_loc[base + e] = pop[base + e];
    }
    __syncwarp();
    if (lane == 0) pbest_fit[row] = f;
  }
}

struct ClpsoArgs {
  float* pop;
  float* vel;
  const float* pbest_loc;
  float* fit;
  const long long* src_rows;  // row whose personal best particle i learns from
  const float* lb;
  const float* ub;
  const float* w;
  const float* c;
  const float* r;             // (P, d) uniform draws or null: in-kernel Philox
  long long P;
  int d;
  FitParams fp;
  PhiloxKeys keys;
  unsigned long long generation;
  int write_fit;
};

// clpso.py:119-122 for one variable; every operation rounded on its own.
__device__ __forceinline__ float clpso_one(float x, float& v, float pb, float lb, float ub, float r, float w, float c) {
  const float vn = __fadd_rn(__fmul_rn(w, v), __fmul_rn(__fmul_rn(c, r), __fsub_rn(pb, x)));
  v = relu_clamp(vn, lb, ub);
  return relu_clamp(__fadd_rn(x, vn), lb, ub);
}

template <int VEC, bool PHILOX, int FIT>
__global__ void __launch_bounds__(kThreads, 4) clpso_move_eval_kernel(const ClpsoArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  const float w = *a.w, cc = *a.c;
  const int d = a.d;
  const int n_call = (d + 3) >> 2;
  for (long long row = warp0; row < a.P; row += n_warps) {
    long long src = a.src_rows[row];
    if ((unsigned long long)src >= (unsigned long long)a.P) src = row;
    const size_t base = (size_t)row * (size_t)d, bsrc = (size_t)src * (size_t)d;
    Fitness<FIT> acc;
    if constexpr (VEC == 4) {
      float4* pop4 = reinterpret_cast<float4*>(a.pop + base);
      float4* vel4 = reinterpret_cast<float4*>(a.vel + base);
      const float4* pb4 = reinterpret_cast<const float4*>(a.pbest_loc + bsrc);
      const float4* lb4 = reinterpret_cast<const float4*>(a.lb);
      const float4* ub4 = reinterpret_cast<const float4*>(a.ub);
      for (int c = lane; c < n_call; c += 32) {
        const float4 x = __ldcs(pop4 + c);
        float4 v = __ldcs(vel4 + c);
        const float4 pb = __ldg(pb4 + c);  // another particle may read the same row: keep it cacheable
        float4 r;
        if constexpr (PHILOX) {
          // counter (q lo, q hi, generation lo, generation hi), q = row * ceil(d / 4) + column / 4
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)c;
          const uint4 u = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation, (uint32_t)(a.generation >> 32), a.keys);
          r = make_float4(u24_to_unit(u.x), u24_to_unit(u.y), u24_to_unit(u.z), u24_to_unit(u.w));
        } else {
          r = __ldcs(reinterpret_cast<const float4*>(a.r + base) + c);
        }
        const float4 lb = __ldg(lb4 + c), ub = __ldg(ub4 + c);
        float4 xo;
        xo.x = clpso_one(x.x, v.x, pb.x, lb.x, ub.x, r.x, w, cc);
        xo.y = clpso_one(x.y, v.y, pb.y, lb.y, ub.y, r.y, w, cc);
        xo.z = clpso_one(x.z, v.z, pb.z, lb.z, ub.z, r.z, w, cc);
        xo.w = clpso_one(x.w, v.w, pb.w, lb.w, ub.w, r.w, w, cc);
        __stcs(pop4 + c, xo);
        __stcs(vel4 + c, v);
        acc.add4(xo, a.fp);
      }
    } else {
      for (int e = lane; e < d; e += 32) {
        const float x = a.pop[base + e];
        float v = a.vel[base + e];
        float r;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)(e >> 2);
          const uint4 u = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation, (uint32_t)(a.generation >> 32), a.keys);
          const int k = e & 3;
          r = u24_to_unit(k == 0 ? u.x : (k == 1 ? u.y : (k == 2 ? u.z : u.w)));
        } else {
          r = a.r[base + e];
        }
        const float xo = clpso_one(x, v, a.pbest_loc[bsrc + e], a.lb[e], a.ub[e], r, w, cc);
        a.pop[base + e] = xo;
        a.vel[base + e] = v;
        acc.add(xo, a.fp);
      }
    }
    acc.reduce();
    if (lane == 0 && a.write_fit) a.fit[row] = acc.finish(d, a.fp);  // clpso.py:123
  }
}

template <int VEC, bool PHILOX>
void launch_clpso(int fitness_id, int grid, cudaStream_t s, const ClpsoArgs& a) {
  switch (fitness_id) {
    case EVOX_FIT_ACKLEY:
      clpso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_ACKLEY><<<grid, kThreads, 0, s>>>(a);
      break;
    case EVOX_FIT_RASTRIGIN:
      clpso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_RASTRIGIN><<<grid, kThreads, 0, s>>>(a);
      break;
    default:
      clpso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_SPHERE><<<grid, kThreads, 0, s>>>(a);
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

extern "C" int evox_clpso_update_pbest(const float* pop, const float* fit, float* personal_best_location, float* personal_best_fit,
                                       int64_t pop_size, int32_t dim, void* stream) {
  EVOX_REQUIRE(pop && fit && personal_best_location && personal_best_fit, EVOX_ERR_INVALID, "clpso_update_pbest: NULL pointer");
  EVOX_REQUIRE(pop_size > 0 && dim > 0, EVOX_ERR_INVALID, "clpso_update_pbest: sizes must be positive");
  EVOX_REQUIRE(pop != personal_best_location, EVOX_ERR_INVALID, "clpso_update_pbest: pop and personal_best_location must not alias");
  const int vec = (dim % 4 == 0) && aligned16(pop) && aligned16(personal_best_location);
  clpso_pbest_kernel<<<row_grid(pop_size), kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pop, fit, personal_best_location,
                                                                                               personal_best_fit, pop_size, dim, vec);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_clpso_move_eval(float* pop, float* velocity, const float* personal_best_location, float* fit,
                                    const int64_t* source_rows, const float* lb, const float* ub, const float* w, const float* c,
                                    const float* r, int64_t pop_size, int32_t dim, int32_t fitness_id, const float* params,
                                    uint64_t seed, uint64_t generation, void* stream) {
  EVOX_REQUIRE(pop && velocity && personal_best_location && fit && source_rows && lb && ub && w && c, EVOX_ERR_INVALID,
               "clpso_move_eval: NULL pointer");
  EVOX_REQUIRE(pop_size > 0 && dim > 0, EVOX_ERR_INVALID, "clpso_move_eval: sizes must be positive");
  EVOX_REQUIRE(fitness_id == -1 || (fitness_id >= EVOX_FIT_ACKLEY && fitness_id <= EVOX_FIT_SPHERE), EVOX_ERR_INVALID,
               "clpso_move_eval: unknown fitness id %d", fitness_id);
  EVOX_REQUIRE(fitness_id != EVOX_FIT_ACKLEY || params, EVOX_ERR_INVALID, "clpso_move_eval: Ackley needs params {a, b, c}");
  ClpsoArgs a;
  a.pop = pop;
  a.vel = velocity;
  a.pbest_loc = personal_best_location;
  a.fit = fit;
  a.src_rows = (const long long*)source_rows;
  a.lb = lb;
  a.ub = ub;
  a.w = w;
  a.c = c;
  a.r = r;
  a.P = pop_size;
  a.d = dim;
  a.fp = (fitness_id == EVOX_FIT_ACKLEY) ? FitParams{params[0], params[1], params[2]} : FitParams{0.f, 0.f, 0.f};
  a.keys = philox_round_keys(seed);
  a.generation = generation;
  a.write_fit = fitness_id != -1;
  const int fid = fitness_id == -1 ? EVOX_FIT_SPHERE : fitness_id;
  const bool vec = (dim % 4 == 0) && aligned16(pop) && aligned16(velocity) && aligned16(personal_best_location) && aligned16(lb) &&
                   aligned16(ub) && (r == nullptr || aligned16(r));
  const int grid = row_grid(pop_size);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (vec) {
    if (r) launch_clpso<4, false>(fid, grid, s, a); else launch_clpso<4, true>(fid, grid, s, a);
  } else {
    if (r) launch_clpso<1, false>(fid, grid, s, a); else launch_clpso<1, true>(fid, grid, s, a);
  }
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
