// Social-learning PSO (both demonstrator-choice variants): one generation fused with the evaluation.
//
// Reference semantics: SLPSOGS.step / SLPSOUS.step (evox/algorithms/so/pso_variants/sl_pso_gs.py:72-104,
// sl_pso_us.py:72-110). The two differ only in how particle i picks its demonstrator's rank (Gaussian or
// uniform sampling over the fitness-sorted swarm: pop_size scalars, kept in torch ops on the host side);
// the update is the same:
//   v' = r1 * v + r2 * (X_k - x) + (r3 * epsilon) * (X_avg - x),   x' = clamp(x + v'),  v = clamp(v')
// with X_k another particle's position BEFORE this generation, X_avg the swarm's mean position before this
// generation, and the relu-form clamp with the POSITION bounds for both.
// Because X_k is a pre-update row of the swarm, the new positions go to a second buffer (the caller swaps
// the two afterwards). One launch, one warp per particle: 12 B read (x, v, X_k) + 8 B written per
// particle-dimension; the kernel also accumulates the column sums of the NEW swarm (rows of up to 1,024
// floats), so the next generation's X_avg costs no further pass.
#include "colmean.cuh"
#include "common.cuh"
#include "fitness.cuh"

namespace evox {
namespace {

constexpr int kWarpsPerBlock = kColmeanWarps;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kMaxChunks = 8;  // float4 chunks per lane whose column sums a warp keeps in shared memory
constexpr int kMaxFusedDim = kMaxChunks * 32 * 4;

struct SlpsoArgs {
  const float* pop;      // swarm before this generation (read only)
  float* pop_new;        // swarm after it
  float* vel;
  float* fit;
  const long long* demo; // row of each particle's demonstrator
  const float* lb;
  const float* ub;
  const float* eps;      // social influence factor (device scalar)
  const float* center;   // X_avg
  const float* r1;       // (P, d) draws each, or all null: in-kernel Philox
  const float* r2;
  const float* r3;
  long long P;
  int d;
  FitParams fp;
  PhiloxKeys keys;
  unsigned long long generation;
  int write_fit;
  float* partial;        // [gridDim.x][d] column sums of pop_new (SUMS variant)
};

// Uniform draws of the in-kernel stream: Philox4x32-10 keyed by the seed, counter
// (q lo, q hi, generation lo, which + 4 * generation hi), q = row * ceil(d / 4) + column / 4, which = 0..2.
__device__ __forceinline__ float4 slpso_uniform4(const SlpsoArgs& a, unsigned long long q, uint32_t which) {
  const uint4 r = philox4x32_10_keyed((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)a.generation,
                                      which + 4u * (uint32_t)(a.generation >> 32), a.keys);
  return make_float4(u24_to_unit(r.x), u24_to_unit(r.y), u24_to_unit(r.z), u24_to_unit(r.w));
}

// sl_pso_gs.py:94-97 for one variable; every operation rounded on its own, in the reference's order.
__device__ __forceinline__ float learn_one(float x, float& v, float xk, float xavg, float lb, float ub, float r1, float r2, float r3,
                                           float eps) {
  const float vn = __fadd_rn(__fadd_rn(__fmul_rn(r1, v), __fmul_rn(r2, __fsub_rn(xk, x))),
                             __fmul_rn(__fmul_rn(r3, eps), __fsub_rn(xavg, x)));
  v = relu_clamp(vn, lb, ub);
  return relu_clamp(__fadd_rn(x, vn), lb, ub);
}

template <int VEC, bool PHILOX, int FIT, bool SUMS>
__global__ void __launch_bounds__(kThreads, kColmeanBlocksPerSM) slpso_update_kernel(const SlpsoArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + warp;
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  const int d = a.d;
  const int n_call = (d + 3) >> 2;
  const float eps = *a.eps;
  // running column sums of the new rows this warp has written: slot [warp][chunk], each owned by one lane
  __shared__ float4 ssum[SUMS ? kWarpsPerBlock : 1][SUMS ? kMaxChunks * 32 : 1];
  if constexpr (SUMS) {
    for (int c = lane; c < kMaxChunks * 32; c += 32) ssum[warp][c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (long long row = warp0; row < a.P; row += n_warps) {
    long long k = a.demo[row];
    if ((unsigned long long)k >= (unsigned long long)a.P) k = row;
    const size_t base = (size_t)row * (size_t)d, bk = (size_t)k * (size_t)d;
    Fitness<FIT> acc;
    if constexpr (VEC == 4) {
      const float4* x4 = reinterpret_cast<const float4*>(a.pop + base);
      const float4* xk4 = reinterpret_cast<const float4*>(a.pop + bk);
      float4* out4 = reinterpret_cast<float4*>(a.pop_new + base);
      float4* v4 = reinterpret_cast<float4*>(a.vel + base);
      const float4* ce4 = reinterpret_cast<const float4*>(a.center);
      const float4* lb4 = reinterpret_cast<const float4*>(a.lb);
      const float4* ub4 = reinterpret_cast<const float4*>(a.ub);
      for (int c = lane; c < n_call; c += 32) {
        const float4 x = __ldg(x4 + c);    // rows of the old swarm are read twice (own row, someone's demonstrator)
        const float4 xk = __ldg(xk4 + c);
        float4 v = __ldcs(v4 + c);
        const float4 ce = __ldg(ce4 + c), lb = __ldg(lb4 + c), ub = __ldg(ub4 + c);
        float4 r1, r2, r3;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)c;
          r1 = slpso_uniform4(a, q, 0u);
          r2 = slpso_uniform4(a, q, 1u);
          r3 = slpso_uniform4(a, q, 2u);
        } else {
          r1 = __ldcs(reinterpret_cast<const float4*>(a.r1 + base) + c);
          r2 = __ldcs(reinterpret_cast<const float4*>(a.r2 + base) + c);
          r3 = __ldcs(reinterpret_cast<const float4*>(a.r3 + base) + c);
        }
        float4 xo;
        xo.x = learn_one(x.x, v.x, xk.x, ce.x, lb.x, ub.x, r1.x, r2.x, r3.x, eps);
        xo.y = learn_one(x.y, v.y, xk.y, ce.y, lb.y, ub.y, r1.y, r2.y, r3.y, eps);
        xo.z = learn_one(x.z, v.z, xk.z, ce.z, lb.z, ub.z, r1.z, r2.z, r3.z, eps);
        xo.w = learn_one(x.w, v.w, xk.w, ce.w, lb.w, ub.w, r1.w, r2.w, r3.w, eps);
        __stcs(out4 + c, xo);
        __stcs(v4 + c, v);
        acc.add4(xo, a.fp);
        if constexpr (SUMS) {
          float4 s = ssum[warp][c];
          s.x += xo.x;
          s.y += xo.y;
          s.z += xo.z;
          s.w += xo.w;
          ssum[warp][c] = s;
        }
      }
    } else {
      for (int e = lane; e < d; e += 32) {
        const float x = a.pop[base + e];
        float v = a.vel[base + e];
        float r1, r2, r3;
        if constexpr (PHILOX) {
          const unsigned long long q = (unsigned long long)row * (unsigned long long)n_call + (unsigned long long)(e >> 2);
          const float4 u1 = slpso_uniform4(a, q, 0u), u2 = slpso_uniform4(a, q, 1u), u3 = slpso_uniform4(a, q, 2u);
          const int j = e & 3;
          r1 = j == 0 ? u1.x : (j == 1 ? u1.y : (j == 2 ? u1.z : u1.w));
          r2 = j == 0 ? u2.x : (j == 1 ? u2.y : (j == 2 ? u2.z : u2.w));
          r3 = j == 0 ? u3.x : (j == 1 ? u3.y : (j == 2 ? u3.z : u3.w));
        } else {
          r1 = a.r1[base + e];
          r2 = a.r2[base + e];
          r3 = a.r3[base + e];
        }
        const float xo = learn_one(x, v, a.pop[bk + e], a.center[e], a.lb[e], a.ub[e], r1, r2, r3, eps);
        a.pop_new[base + e] = xo;
        a.vel[base + e] = v;
        acc.add(xo, a.fp);
      }
    }
    acc.reduce();
    if (lane == 0 && a.write_fit) a.fit[row] = acc.finish(d, a.fp);
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
void launch_slpso(int fitness_id, int grid, cudaStream_t s, const SlpsoArgs& a) {
  switch (fitness_id) {
    case EVOX_FIT_ACKLEY:
      slpso_update_kernel<VEC, PHILOX, EVOX_FIT_ACKLEY, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
    case EVOX_FIT_RASTRIGIN:
      slpso_update_kernel<VEC, PHILOX, EVOX_FIT_RASTRIGIN, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
    default:
      slpso_update_kernel<VEC, PHILOX, EVOX_FIT_SPHERE, SUMS><<<grid, kThreads, 0, s>>>(a);
      break;
  }
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_slpso_workspace_bytes(int64_t pop_size, int32_t dim) {
  if (pop_size <= 0 || dim <= 0) return 0;
  return sizeof(float) * (size_t)padded_dim(dim) * (size_t)(1 + max_partials());
}

extern "C" int evox_slpso_step(const float* pop, float* pop_new, float* velocity, float* fit, const int64_t* demonstrator_rows,
                               const float* lb, const float* ub, const float* social_influence_factor, const float* r1,
                               const float* r2, const float* r3, int64_t pop_size, int32_t dim, int32_t fitness_id,
                               const float* params, uint64_t seed, uint64_t generation, int32_t center_ready, void* workspace,
                               size_t workspace_bytes, int32_t* next_center_ready, void* stream) {
  EVOX_REQUIRE(pop && pop_new && velocity && fit && demonstrator_rows && lb && ub && social_influence_factor && workspace,
               EVOX_ERR_INVALID, "slpso_step: NULL pointer");
  EVOX_REQUIRE(pop != pop_new, EVOX_ERR_INVALID, "slpso_step: pop and pop_new must be different buffers");
  EVOX_REQUIRE(pop_size > 0 && dim > 0, EVOX_ERR_INVALID, "slpso_step: sizes must be positive");
  EVOX_REQUIRE(fitness_id == -1 || (fitness_id >= EVOX_FIT_ACKLEY && fitness_id <= EVOX_FIT_SPHERE), EVOX_ERR_INVALID,
               "slpso_step: unknown fitness id %d", fitness_id);
  EVOX_REQUIRE(fitness_id != EVOX_FIT_ACKLEY || params, EVOX_ERR_INVALID, "slpso_step: Ackley needs params {a, b, c}");
  const bool any = r1 || r2 || r3, all = r1 && r2 && r3;
  EVOX_REQUIRE(any == all, EVOX_ERR_INVALID, "slpso_step: give all three draw tensors or none");
  EVOX_REQUIRE(workspace_bytes >= evox_slpso_workspace_bytes(pop_size, dim), EVOX_ERR_WORKSPACE, "slpso_step: workspace too small");
  EVOX_REQUIRE(aligned16(workspace), EVOX_ERR_INVALID, "slpso_step: workspace must be 16-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* center = reinterpret_cast<float*>(workspace);
  float* partial = center + padded_dim(dim);
  if (!center_ready) {
    if (int rc = run_colmean(pop, pop_size, dim, center, partial, s)) return rc;
  }
  SlpsoArgs a;
  a.pop = pop;
  a.pop_new = pop_new;
  a.vel = velocity;
  a.fit = fit;
  a.demo = (const long long*)demonstrator_rows;
  a.lb = lb;
  a.ub = ub;
  a.eps = social_influence_factor;
  a.center = center;
  a.r1 = r1;
  a.r2 = r2;
  a.r3 = r3;
  a.P = pop_size;
  a.d = dim;
  a.fp = (fitness_id == EVOX_FIT_ACKLEY) ? FitParams{params[0], params[1], params[2]} : FitParams{0.f, 0.f, 0.f};
  a.keys = philox_round_keys(seed);
  a.generation = generation;
  a.write_fit = fitness_id != -1;
  a.partial = partial;
  const bool vec = (dim % 4 == 0) && aligned16(pop) && aligned16(pop_new) && aligned16(velocity) && aligned16(lb) && aligned16(ub) &&
                   (!all || (aligned16(r1) && aligned16(r2) && aligned16(r3)));
  const bool sums = vec && dim <= kMaxFusedDim;
  const long long blocks = (pop_size + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const long long cap = max_partials();
  const int grid = (int)(blocks < cap ? blocks : cap);
  const int fid = fitness_id == -1 ? EVOX_FIT_SPHERE : fitness_id;
  if (vec) {
    if (sums) {
      if (all) launch_slpso<4, false, true>(fid, grid, s, a); else launch_slpso<4, true, true>(fid, grid, s, a);
    } else {
      if (all) launch_slpso<4, false, false>(fid, grid, s, a); else launch_slpso<4, true, false>(fid, grid, s, a);
    }
  } else {
    if (all) launch_slpso<1, false, false>(fid, grid, s, a); else launch_slpso<1, true, false>(fid, grid, s, a);
  }
  EVOX_LAUNCH_CHECK();
  if (sums) {
    // the partial sums belong to pop_new: the mean the NEXT call needs, when pop_new is its pop
    colmean_finish_kernel<<<(dim + 31) / 32, dim3(32, 32), 0, s>>>(partial, grid, dim, pop_size, center);
    EVOX_LAUNCH_CHECK();
  }
  if (next_center_ready) *next_center_ready = sums ? 1 : 0;
  return EVOX_OK;
}
