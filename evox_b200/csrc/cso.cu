// Competitive swarm optimiser: one generation fused with the fitness evaluation.
//
// Reference semantics: CSO.step (evox/algorithms/so/pso_variants/cso.py:71-105): a random pairing of the
// swarm, the loser of each pair (the student) learns from the winner (the teacher) and from the swarm's
// mean position, is clamped with the relu-form clamp (evox/utils/jit_fix_operator.py:42-44) and
// re-evaluated. The reference stores the students' new positions and fitness but NOT their new
// velocities (cso.py:98-105): by default `velocity` is read-only here too; store_velocity = 1 writes them
// (4 B more per student-dimension).
//
// One generation is two launches:
//   cso_update_kernel  one warp per pair: reads velocity[student], pop[teacher], pop[student] (12 B per
//                      student-dimension), writes pop[student] (4 B), evaluates the student and — since
//                      it thereby sees every row of the next swarm exactly once — accumulates the column
//                      sums of the next generation's mean in registers (rows of up to 1,024 floats);
//   cso_center_finish_kernel  sums the per-block partial column sums in a fixed order.
// That is 8 B per particle-dimension per generation; the separate column-sum pass (cso_colsum_kernel,
// 4 B more) only runs for the first generation, for longer rows, or when the swarm was changed from
// outside between two steps.
#include "colmean.cuh"
#include "common.cuh"
#include "fitness.cuh"

namespace evox {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kMaxChunks = 8;           // float4 chunks per lane whose column sums a warp keeps in shared memory
constexpr int kMaxFusedDim = kMaxChunks * 32 * 4;
constexpr int kBlocksPerSM = 4;  // = kColmeanBlocksPerSM: the partial rows are indexed by block

struct CsoArgs {
  float* pop;
  float* vel;
  int store_velocity;    // 0: velocity is read-only, as in the reference; 1: the students' new velocities are stored
  float* fit;
  const long long* perm;
  const float* lb;
  const float* ub;
  const float* phi;
  const float* center;
  const float* lambdas;  // (3, P / 2, d) draws, or null: in-kernel Philox
  long long P;
  int d;
  FitParams fp;
  PhiloxKeys keys;
  unsigned long long generation;
  int write_fit;
  float* candidates;     // optional (P / 2, d): the students' new positions, pair order
  long long* students;   // optional (P / 2): row of each pair's student
  float* partial;        // [gridDim.x][d] column sums of the updated swarm (SUMS variant)
};

// Uniform draws of the in-kernel stream: Philox4x32-10 keyed by the seed, counter
// (q lo, q hi, generation lo, which + 4 * generation hi), q = pair * ceil(d / 4) + column / 4, which = 0..2
// for lambda1..lambda3 (cso.py:90 draws them as one (3, P / 2, d) block).
__device__ __forceinline__ float4 cso_uniform4(const CsoArgs& a, unsigned long long q, uint32_t which) {
  const uint4 r = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation,
                                      which + 4u * (uint32_t)(a.generation >> 32), a.keys);
  return make_float4(u24_to_unit(r.x), u24_to_unit(r.y), u24_to_unit(r.z), u24_to_unit(r.w));
}

// cso.py:92-101 for one variable; every operation rounded on its own, in the reference's order.
__device__ __forceinline__ float learn_one(float& v, float pt, float ps, float ce, float lb, float ub, float l1, float l2, float l3,
                                           float phi) {
  const float inertia = __fmul_rn(l1, v);
  const float teach = __fmul_rn(l2, __fsub_rn(pt, ps));
  const float centre = __fmul_rn(__fmul_rn(phi, l3), __fsub_rn(ce, ps));
  const float range = __fsub_rn(ub, lb);
  const float sv = relu_clamp(__fadd_rn(__fadd_rn(inertia, teach), centre), -range, range);
  v = sv;
  return relu_clamp(__fadd_rn(ps, sv), lb, ub);
}

template <int VEC, bool PHILOX, int FIT, bool SUMS>
__global__ void __launch_bounds__(kThreads, kBlocksPerSM) cso_update_kernel(const CsoArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + warp;
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  const long long half = a.P / 2;
  const int d = a.d;
  const int n_call = (d + 3) >> 2;
  const float phi = *a.phi;
  // running column sums of the rows this warp has seen: slot [warp][chunk], each owned by one lane
  __shared__ float4 ssum[SUMS ? kWarpsPerBlock : 1][SUMS ? kMaxChunks * 32 : 1];
  if constexpr (SUMS) {
    for (int c = lane; c < kMaxChunks * 32; c += 32) ssum[warp][c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  // the pair after this one is looked up while this one is processed (perm -> fit is a dependent chain)
  long long left_n = 0, right_n = 0;
  if (warp0 < half) {
    left_n = a.perm[warp0];
    right_n = a.perm[warp0 + half];
  }
  for (long long pair = warp0; pair < half; pair += n_warps) {
    const long long left = left_n, right = right_n;
    if (pair + n_warps < half) {
      left_n = __ldg(a.perm + pair + n_warps);
      right_n = __ldg(a.perm + pair + n_warps + half);
    }
    if ((unsigned long long)left >= (unsigned long long)a.P || (unsigned long long)right >= (unsigned long long)a.P) continue;
    const bool mask = a.fit[left] < a.fit[right];  // cso.py:82: ties and NaN make the LEFT one the student
    const long long teacher = mask ? left : right, student = mask ? right : left;
    const size_t bs = (size_t)student * (size_t)d, bt = (size_t)teacher * (size_t)d, bp = (size_t)pair * (size_t)d;
    const size_t lam_stride = (size_t)half * (size_t)d;
    Fitness<FIT> acc;
    if constexpr (VEC == 4) {
      float4* ps4 = reinterpret_cast<float4*>(a.pop + bs);
      const float4* pt4 = reinterpret_cast<const float4*>(a.pop + bt);
      float4* v4 = reinterpret_cast<float4*>(a.vel + bs);
      const float4* ce4 = reinterpret_cast<const float4*>(a.center);
      const float4* lb4 = reinterpret_cast<const float4*>(a.lb);
      const float4* ub4 = reinterpret_cast<const float4*>(a.ub);
      auto chunk = [&](int c, float4 v, const float4 pt, const float4 ps) {
        const float4 ce = __ldg(ce4 + c), lb = __ldg(lb4 + c), ub = __ldg(ub4 + c);
        float4 l1, l2, l3;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)pair * (unsigned long long)n_call + (unsigned long long)c;
          l1 = cso_uniform4(a, q, 0u);
          l2 = cso_uniform4(a, q, 1u);
          l3 = cso_uniform4(a, q, 2u);
        } else {
          l1 = __ldcs(reinterpret_cast<const float4*>(a.lambdas + bp) + c);
          l2 = __ldcs(reinterpret_cast<const float4*>(a.lambdas + lam_stride + bp) + c);
          l3 = __ldcs(reinterpret_cast<const float4*>(a.lambdas + 2 * lam_stride + bp) + c);
        }
        float4 xo;
        xo.x = learn_one(v.x, pt.x, ps.x, ce.x, lb.x, ub.x, l1.x, l2.x, l3.x, phi);
        xo.y = learn_one(v.y, pt.y, ps.y, ce.y, lb.y, ub.y, l1.y, l2.y, l3.y, phi);
        xo.z = learn_one(v.z, pt.z, ps.z, ce.z, lb.z, ub.z, l1.z, l2.z, l3.z, phi);
        xo.w = learn_one(v.w, pt.w, ps.w, ce.w, lb.w, ub.w, l1.w, l2.w, l3.w, phi);
        __stcs(ps4 + c, xo);
        if (a.store_velocity) __stcs(v4 + c, v);
        if (a.candidates) __stcs(reinterpret_cast<float4*>(a.candidates + bp) + c, xo);
        acc.add4(xo, a.fp);
        if constexpr (SUMS) {  // both rows of the pair as they stand after this generation
          float4 s = ssum[warp][c];
          s.x += pt.x + xo.x;
          s.y += pt.y + xo.y;
          s.z += pt.z + xo.z;
          s.w += pt.w + xo.w;
          ssum[warp][c] = s;
        }
      };
      for (int c = lane; c < n_call; c += 32) chunk(c, __ldcs(v4 + c), __ldcs(pt4 + c), __ldcs(ps4 + c));
    } else {
      for (int e = lane; e < d; e += 32) {
        float v = a.vel[bs + e];
        const float pt = a.pop[bt + e], ps = a.pop[bs + e];
        float l1, l2, l3;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)pair * (unsigned long long)n_call + (unsigned long long)(e >> 2);
          const float4 u1 = cso_uniform4(a, q, 0u), u2 = cso_uniform4(a, q, 1u), u3 = cso_uniform4(a, q, 2u);
          const int k = e & 3;
          l1 = k == 0 ? u1.x : (k == 1 ? u1.y : (k == 2 ? u1.z : u1.w));
          l2 = k == 0 ? u2.x : (k == 1 ? u2.y : (k == 2 ? u2.z : u2.w));
          l3 = k == 0 ? u3.x : (k == 1 ? u3.y : (k == 2 ? u3.z : u3.w));
        } else {
          l1 = a.lambdas[bp + e];
          l2 = a.lambdas[lam_stride + bp + e];
          l3 = a.lambdas[2 * lam_stride + bp + e];
        }
        const float xo = learn_one(v, pt, ps, a.center[e], a.lb[e], a.ub[e], l1, l2, l3, phi);
        a.pop[bs + e] = xo;
        if (a.store_velocity) a.vel[bs + e] = v;
        if (a.candidates) a.candidates[bp + e] = xo;
        acc.add(xo, a.fp);
      }
    }
    acc.reduce();
    if (lane == 0) {
      if (a.write_fit) a.fit[student] = acc.finish(d, a.fp);  // cso.py:103-105
      if (a.students) a.students[pair] = student;
    }
  }

  if constexpr (SUMS) {
    // the warps' sums are folded in warp order and the block writes one partial row
    __syncthreads();
    float4* out = reinterpret_cast<float4*>(a.partial + (size_t)blockIdx.x * (size_t)d);
    for (int c = threadIdx.x; c < n_call; c += kThreads) {
      float4 s = ssum[0][c];
      for (int w = 1; w < kWarpsPerBlock; ++w) {
        const float4 o = ssum[w][c];
        s = make_float4(s.x + o.x, s.y + o.y, s.z + o.z, s.w + o.w);
      }
      out[c] = s;
    }
  }
}

template <int VEC, bool PHILOX, bool SUMS>
void launch_update(int fitness_id, int grid, cudaStream_t s, const CsoArgs& a) {
  switch (fitness_id) {
    case EVOX_FIT_ACKLEY:
      cso_update_kernel<VEC, PHILOX, EVOX_FIT_ACKLEY, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
    case EVOX_FIT_RASTRIGIN:
      cso_update_kernel<VEC, PHILOX, EVOX_FIT_RASTRIGIN, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
    default:
      cso_update_kernel<VEC, PHILOX, EVOX_FIT_SPHERE, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
  }
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_cso_workspace_bytes(int64_t pop_size, int32_t dim) {
  if (pop_size <= 0 || dim <= 0) return 0;
  return sizeof(float) * (size_t)padded_dim(dim) * (size_t)(1 + max_partials());
}

extern "C" int evox_cso_step(float* pop, float* velocity, int32_t store_velocity, float* fit, const int64_t* perm, const float* lb, const float* ub,
                             const float* phi, const float* lambdas, int64_t pop_size, int32_t dim, int32_t fitness_id,
                             const float* fit_params, uint64_t seed, uint64_t generation, int32_t center_ready, float* candidates,
                             int64_t* students, void* workspace, size_t workspace_bytes, int32_t* next_center_ready, void* stream) {
  EVOX_REQUIRE(pop && velocity && fit && perm && lb && ub && phi && workspace, EVOX_ERR_INVALID, "cso_step: NULL pointer");
  EVOX_REQUIRE(pop_size >= 2 && pop_size % 2 == 0 && dim > 0, EVOX_ERR_INVALID,
               "cso_step: the swarm must have an even number of particles (the reference pairs them all)");
  EVOX_REQUIRE(fitness_id == -1 || (fitness_id >= EVOX_FIT_ACKLEY && fitness_id <= EVOX_FIT_SPHERE), EVOX_ERR_INVALID,
               "cso_step: unknown fitness id %d", fitness_id);
  EVOX_REQUIRE(fitness_id == -1 || fit_params, EVOX_ERR_INVALID, "cso_step: fit_params is NULL");
  EVOX_REQUIRE(workspace_bytes >= evox_cso_workspace_bytes(pop_size, dim), EVOX_ERR_WORKSPACE, "cso_step: workspace too small");
  EVOX_REQUIRE(aligned16(workspace), EVOX_ERR_INVALID, "cso_step: workspace must be 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* center = reinterpret_cast<float*>(workspace);
  float* partial = center + padded_dim(dim);
  if (!center_ready) {
    if (int rc = run_colmean(pop, pop_size, dim, center, partial, s)) return rc;
  }
  CsoArgs a;
  a.pop = pop;
  a.vel = velocity;
  a.store_velocity = store_velocity;
  a.fit = fit;
  a.perm = (const long long*)perm;
  a.lb = lb;
  a.ub = ub;
  a.phi = phi;
  a.center = center;
  a.lambdas = lambdas;
  a.P = pop_size;
  a.d = dim;
  a.fp = fitness_id == -1 ? FitParams{0.f, 0.f, 0.f} : FitParams{fit_params[0], fit_params[1], fit_params[2]};
  a.keys = philox_round_keys(seed);
  a.generation = generation;
  a.write_fit = fitness_id != -1;
  a.candidates = candidates;
  a.students = (long long*)students;
  a.partial = partial;
  const bool vec = (dim % 4 == 0) && aligned16(pop) && aligned16(velocity) && aligned16(lb) && aligned16(ub) &&
                   (lambdas == nullptr || aligned16(lambdas)) && (candidates == nullptr || aligned16(candidates));
  const bool sums = vec && dim <= kMaxFusedDim;
  const long long half = pop_size / 2;
  long long blocks = (half + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = max_partials();
  const int grid = (int)(blocks < cap ? blocks : cap);
  const int fid = fitness_id == -1 ? EVOX_FIT_SPHERE : fitness_id;
  if (vec) {
    if (sums) {
      if (lambdas) launch_update<4, false, true>(fid, grid, s, a); else launch_update<4, true, true>(fid, grid, s, a);
    } else {
      if (lambdas) launch_update<4, false, false>(fid, grid, s, a); else launch_update<4, true, false>(fid, grid, s, a);
    }
  } else {
    if (lambdas) launch_update<1, false, false>(fid, grid, s, a); else launch_update<1, true, false>(fid, grid, s, a);
  }
  EVOX_LAUNCH_CHECK();
  if (sums) {
    colmean_finish_kernel<<<(dim + 31) / 32, dim3(32, 32), 0, s>>>(partial, grid, dim, pop_size, center);
    EVOX_LAUNCH_CHECK();
  }
  if (next_center_ready) *next_center_ready = sums ? 1 : 0;
  return EVOX_OK;
}
