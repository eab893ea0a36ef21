// P1: particle swarm generation step fused with the fitness evaluation.
//
// Reference semantics: PSO.step / PSO.init_step (evox/algorithms/so/pso_variants/pso.py:71-115),
// min_by (pso_variants/utils.py:6-25), clamp (evox/utils/jit_fix_operator.py:24-44),
// ackley_func / rastrigin_func (evox/problems/numerical/basic.py:66-69, 115-116).
//
// One generation is ONE launch (evox_pso_generation): pso_move_eval_kernel<.., FUSED = true>
//   head  — every warp folds the best-particle records left by the previous generation (one per
//           shard) into the running global best: the winner's row is the social attractor;
//   body  — one warp per particle, 128-bit loads: personal-best update, velocity / position
//           update, relu-form clamps and the fitness of the moved particle, with a fixed-order
//           shuffle reduction so results do not depend on scheduling;
//   tail  — per-block (min, row) of the NEW fitness; the last block to arrive (atomic ticket)
//           stores the folded global best and writes this shard's record for the next generation.
// The two-launch form (pso_local_best_kernel, then the un-fused move kernel) is kept: it starts a
// run (init_step), recovers when something else wrote to the swarm between two generations, and
// serves callers that evaluate the fitness themselves.
// HBM traffic per particle-dimension: 12 B read (pop, velocity, personal best) + 8 B written
// (pop, velocity), + 8 B read when rg / rp are supplied as tensors instead of Philox.
#include <math.h>
#include <type_traits>

#include "common.cuh"
#include "fitness.cuh"

namespace evox {

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;
constexpr int kMaxPartials = 2048;
// The generation kernel runs 32 warps per SM as ONE block of 1,024 threads: measured in one GPU call at
// 1,000,000 x 1,000, 282.5 generations/s against 279-282 with two blocks of 512 and 276 with four blocks of 256
// (fewer blocks also mean fewer partial minima for the last block to fold).
constexpr int kMoveWarps = 32;
constexpr int kMoveThreads = kMoveWarps * 32;
#ifndef MOVE_BLOCKS_PER_SM
#define MOVE_BLOCKS_PER_SM 1
#endif

// --------------------------------------------------------------------------------------------
// Uniform stream of the in-kernel generator. One Philox call covers 4 consecutive columns of
// one row for one of the two draws: counter = (q lo, q hi, generation lo, which + 2*generation hi)
// with q = global_row * ceil(dim/4) + column/4, key = (seed lo, seed hi).
// --------------------------------------------------------------------------------------------
struct RoundKeys {
  uint32_t k[20];  // (k0, k1) of each of the 10 rounds, computed once on the host
};

template <bool SCALED = true>
__device__ __forceinline__ float4 pso_uniform4(uint64_t q, uint64_t generation, uint32_t which,
                                               const RoundKeys& rk) {
  uint32_t c0 = (uint32_t)q, c1 = (uint32_t)(q >> 32), c2 = (uint32_t)generation;
  uint32_t c3 = which + 2u * (uint32_t)(generation >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    // one 32 x 32 -> 64 bit multiply per half instead of separate high / low products
    const unsigned long long p0 = (unsigned long long)EVOX_PHILOX_M0 * (unsigned long long)c0;
    const unsigned long long p1 = (unsigned long long)EVOX_PHILOX_M1 * (unsigned long long)c2;
    c0 = (uint32_t)(p1 >> 32) ^ c1 ^ rk.k[2 * r];
    c1 = (uint32_t)p1;
    c2 = (uint32_t)(p0 >> 32) ^ c3 ^ rk.k[2 * r + 1];
    c3 = (uint32_t)p0;
  }
  if (SCALED) return make_float4(u24_to_unit(c0), u24_to_unit(c1), u24_to_unit(c2), u24_to_unit(c3));
  // the 24-bit integers as floats; the caller folds the factor 2^-24 into phi (an exact power-of-two
  // scaling: phi * (m * 2^-24) and (phi * 2^-24) * m round to the same float)
  return make_float4(__uint2float_rn(c0 >> 8), __uint2float_rn(c1 >> 8), __uint2float_rn(c2 >> 8), __uint2float_rn(c3 >> 8));
}

static RoundKeys make_round_keys(uint64_t seed) {
  RoundKeys rk;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    rk.k[2 * r] = k0;
    rk.k[2 * r + 1] = k1;
    k0 += EVOX_PHILOX_W0;
    k1 += EVOX_PHILOX_W1;
  }
  return rk;
}

__device__ __forceinline__ float pick(const float4& v, int k) {
  return k == 0 ? v.x : (k == 1 ? v.y : (k == 2 ? v.z : v.w));
}

struct MoveArgs {
  float* pop;
  float* vel;
  float* pbest_loc;
  float* pbest_fit;
  float* fit;
  const float* gbest_loc;
  const float* lb;
  const float* ub;
  const float* w;
  const float* phi_p;
  const float* phi_g;
  const float* rg;
  const float* rp;
  long long P;
  int d;
  FitParams fp;
  RoundKeys rk;
  uint64_t generation;
  long long row_offset;
  // read only by the FUSED instantiations
  const uint32_t* cands;    // n_cands records of (4 + d) words left by the previous generation
  int n_cands;
  float* gbest_fit;         // running best fitness: read by every warp, stored by the last block
  float* gbest_loc_out;     // the array gbest_loc points at, writable
  uint32_t* cand_out;       // this shard's record of the new swarm (never inside cands)
  unsigned int* ticket;
  MinIdx* partials;
  // Sharded swarm with the records exchanged by the kernels themselves (n_peers > 0): every rank holds an
  // exchange buffer of the same layout — records[2][n_peers][4 + d] then flags[2][n_peers], all 32-bit words —
  // and peer_base[p] is rank p's buffer as THIS device addresses it (peer memory over NVLink). The tail stores
  // this shard's record into slot (tag_out & 1, my_rank) of every rank's buffer and then the flag tag_out; the
  // head waits until its own buffer's flags of parity tag_in & 1 all read tag_in. cands / cand_out are unused.
  unsigned long long peer_base[16];
  int n_peers;
  int my_rank;
  unsigned int tag_in;
  int* status;  // set to 1 when a wait for a peer's flag gave up
};

constexpr long long kNoRow = 0x7fffffffffffffffLL;
// A wait for another GPU's record ends after two seconds (or this many polls, whichever comes first): the kernel
// then sets its status word and goes on, and later launches that find the word set do not wait at all.
constexpr unsigned kPeerSpinLimit = 1u << 24;
constexpr unsigned long long kPeerWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ unsigned int load_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void store_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// true when argmin would report b before a (smaller key, then lower index)
__device__ __forceinline__ bool comes_first(const MinIdx& b, const MinIdx& a) {
  return key_less(b.v, a.v) || (!key_less(a.v, b.v) && b.i < a.i);
}

// min_by over [old best, records] (pso_variants/utils.py:18-25): the old best wins ties, then the lowest
// GLOBAL row index. Every lane returns the same answer: the attractor row, whether a record replaced the old
// best, and that record's fitness.
__device__ __forceinline__ const float* fold_candidates(const MoveArgs& a, int lane, bool* take, float* best_fit) {
  const int words = 4 + a.d;
  const uint32_t* cands = a.cands;
  int n_cands = a.n_cands;
  if (a.n_peers > 0) {
    // the records of the previous generation arrive from the other GPUs: wait (bounded) for every rank's flag
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(a.peer_base[a.my_rank]);
    const unsigned parity = a.tag_in & 1u;
    const unsigned int* flags = mine + (size_t)2 * a.n_peers * words + (size_t)parity * a.n_peers;
    for (int r = lane; r < a.n_peers; r += 32) {
      if (load_acquire_sys(flags + r) == a.tag_in) continue;
      if (*reinterpret_cast<const volatile int*>(a.status) != 0) continue;  // an earlier wait gave up: do not wait again
      const unsigned long long t0 = global_timer_ns();
      unsigned spins = 0;
      while (load_acquire_sys(flags + r) != a.tag_in) {
        if (++spins > kPeerSpinLimit || global_timer_ns() - t0 > kPeerWaitNs) {
          atomicExch(a.status, 1);
          break;
        }
        __nanosleep(200);
      }
    }
    __syncwarp();
    cands = mine + (size_t)parity * a.n_peers * words;
    n_cands = a.n_peers;
  }
  MinIdx m{INFINITY, kNoRow};
  int rec = 0;
  for (int r = lane; r < n_cands; r += 32) {
    const uint32_t* c = cands + (size_t)r * words;
    // plain loads: in peer mode another GPU wrote these words while this kernel may already have been running
    const MinIdx o{__uint_as_float(c[0]), (long long)(((unsigned long long)c[2] << 32) | c[1])};
    if (comes_first(o, m)) {
      m = o;
      rec = r;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    MinIdx o;
    o.v = __shfl_xor_sync(0xffffffffu, m.v, off);
    o.i = __shfl_xor_sync(0xffffffffu, m.i, off);
    const int orec = __shfl_xor_sync(0xffffffffu, rec, off);
    if (comes_first(o, m)) {
      m = o;
      rec = orec;
    }
  }
  *take = key_less(m.v, *a.gbest_fit);
  *best_fit = m.v;
  return *take ? reinterpret_cast<const float*>(cands + (size_t)rec * words + 4) : a.gbest_loc;
}

__device__ __forceinline__ MinIdx block_min_idx(MinIdx m, MinIdx* smem) {
  m = warp_min_idx(m);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) smem[wid] = m;
  __syncthreads();
  if (wid == 0) {
    MinIdx t = (lane < (int)(blockDim.x >> 5)) ? smem[lane] : MinIdx{INFINITY, kNoRow};
    t = warp_min_idx(t);
    if (lane == 0) smem[0] = t;
  }
  __syncthreads();
  MinIdx r = smem[0];
  __syncthreads();
  return r;
}

// One particle-dimension of PSO.step (pso.py:98-105). Returns the clamped position.
__device__ __forceinline__ float move_one(float x, float& v, float pb, float gb, float lb, float ub,
                                          float rg, float rp, float w, float phi_p, float phi_g) {
  const float inertia = __fmul_rn(w, v);
  const float cognitive = __fmul_rn(__fmul_rn(phi_p, rp), __fsub_rn(pb, x));
  const float social = __fmul_rn(__fmul_rn(phi_g, rg), __fsub_rn(gb, x));
  const float vn = __fadd_rn(__fadd_rn(inertia, cognitive), social);
  const float xn = __fadd_rn(x, vn);
  v = relu_clamp(vn, lb, ub);
  return relu_clamp(xn, lb, ub);
}

template <int VEC, bool PHILOX, int FIT, bool FUSED>
__global__ void __launch_bounds__(kMoveThreads, MOVE_BLOCKS_PER_SM) pso_move_eval_kernel(const MoveArgs a) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kMoveWarps + (threadIdx.x >> 5);
  __shared__ MinIdx s_warp_min[FUSED ? kMoveWarps : 1];
  const float* gbest_row = a.gbest_loc;
  if constexpr (FUSED) {
    bool take;
    float best;
    gbest_row = fold_candidates(a, lane, &take, &best);
    if (lane == 0) s_warp_min[threadIdx.x >> 5] = MinIdx{INFINITY, kNoRow};
  }
  const long long n_warps = (long long)gridDim.x * kMoveWarps;
  const float w = *a.w, phi_p = *a.phi_p, phi_g = *a.phi_g;
  // vector path in Philox mode: the draws arrive as 24-bit integers, 2^-24 rides on phi (exact)
  const float phi_p_v = (PHILOX && VEC == 4) ? phi_p * 5.9604644775390625e-08f : phi_p;
  const float phi_g_v = (PHILOX && VEC == 4) ? phi_g * 5.9604644775390625e-08f : phi_g;
  const int d = a.d;
  const int n_call = (d + 3) >> 2;  // Philox calls per row and draw

  for (long long row = warp0; row < a.P; row += n_warps) {
    const float f_old = a.fit[row];
    const float pbf = a.pbest_fit[row];
    const bool better = pbf > f_old;  // pso.py:89
    const size_t base = (size_t)row * (size_t)d;
    Fitness<FIT> acc;

    if constexpr (VEC == 4) {
      float4* pop4 = reinterpret_cast<float4*>(a.pop + base);
      float4* vel4 = reinterpret_cast<float4*>(a.vel + base);
      float4* pb4 = reinterpret_cast<float4*>(a.pbest_loc + base);
      const float4* gb4 = reinterpret_cast<const float4*>(gbest_row);
      const float4* lb4 = reinterpret_cast<const float4*>(a.lb);
      const float4* ub4 = reinterpret_cast<const float4*>(a.ub);
      const float4* rg4 = PHILOX ? nullptr : reinterpret_cast<const float4*>(a.rg + base);
      const float4* rp4 = PHILOX ? nullptr : reinterpret_cast<const float4*>(a.rp + base);
      const uint64_t q0 = (uint64_t)(a.row_offset + row) * (uint64_t)n_call;
      // The loop exists twice, for rows whose position becomes their personal best (no load of the old best, one
      // more store) and for the others: written out like this (instead of a select and a predicated store inside
      // one loop) the kernel is 10 % faster (0.78 -> 0.86 of the measured copy bandwidth at 1,000,000 x 1,000).
      // Plain loop: with 32 warps per SM the other warps cover a chunk's load latency. Measured
      // and dropped: a register double buffer (next chunk's loads issued ahead) 4 % slower; the loads of two chunks
      // issued together 3 % slower at four blocks per SM and 13 % slower at three; four chunks at two blocks per SM
      // 20 % slower; lanes holding half chunks (8-byte loads, 40 registers, six blocks per SM, the two lanes of a
      // chunk swapping halves of their Philox draws) 25 % slower; the two per-row scalars fetched one row ahead
      // 1 % slower. The pace follows the instruction count and the number of resident warps, not the bytes in flight.
      auto chunks = [&](auto tag) {
        constexpr bool BETTER = decltype(tag)::value;
#pragma unroll 1  // unrolled by two this loop is 10 % slower, by four 27 % (measured): one chunk per trip
      for (int c = lane; c < n_call; c += 32) {
        const float4 x = __ldcs(pop4 + c);
        float4 v = __ldcs(vel4 + c);
        const float4 pb = BETTER ? x : __ldcs(pb4 + c);
        float4 rg, rp;
        if constexpr (PHILOX) {
          rg = pso_uniform4<false>(q0 + c, a.generation, 0u, a.rk);
          rp = pso_uniform4<false>(q0 + c, a.generation, 1u, a.rk);
        } else {
          rg = __ldcs(rg4 + c);
          rp = __ldcs(rp4 + c);
        }
        const float4 gb = FUSED ? gb4[c] : __ldg(gb4 + c);  // fused: may be a record a peer wrote during this launch
        const float4 lb = __ldg(lb4 + c);
        const float4 ub = __ldg(ub4 + c);
        float4 xo;
        xo.x = move_one(x.x, v.x, pb.x, gb.x, lb.x, ub.x, rg.x, rp.x, w, phi_p_v, phi_g_v);
        xo.y = move_one(x.y, v.y, pb.y, gb.y, lb.y, ub.y, rg.y, rp.y, w, phi_p_v, phi_g_v);
        xo.z = move_one(x.z, v.z, pb.z, gb.z, lb.z, ub.z, rg.z, rp.z, w, phi_p_v, phi_g_v);
        xo.w = move_one(x.w, v.w, pb.w, gb.w, lb.w, ub.w, rg.w, rp.w, w, phi_p_v, phi_g_v);
        if (BETTER) __stcs(pb4 + c, x);  // pso.py:90 — own position becomes the personal best
        __stcs(pop4 + c, xo);
        __stcs(vel4 + c, v);
        acc.add4(xo, a.fp);
      }
      };
      if (better) chunks(std::true_type{});
      else chunks(std::false_type{});
    } else {
      const uint64_t q0 = (uint64_t)(a.row_offset + row) * (uint64_t)n_call;
      for (int e = lane; e < d; e += 32) {
        const float x = a.pop[base + e];
        float v = a.vel[base + e];
        const float pb = better ? x : a.pbest_loc[base + e];
        float rg, rp;
        if constexpr (PHILOX) {
          rg = pick(pso_uniform4(q0 + (e >> 2), a.generation, 0u, a.rk), e & 3);
          rp = pick(pso_uniform4(q0 + (e >> 2), a.generation, 1u, a.rk), e & 3);
        } else {
          rg = a.rg[base + e];
          rp = a.rp[base + e];
        }
        const float xo = move_one(x, v, pb, gbest_row[e], a.lb[e], a.ub[e], rg, rp, w, phi_p, phi_g);
        if (better) a.pbest_loc[base + e] = x;
        a.pop[base + e] = xo;
        a.vel[base + e] = v;
        acc.add(xo, a.fp);
      }
    }
    acc.reduce();
    if (lane == 0) {
      const float f_new = acc.finish(d, a.fp);
      a.fit[row] = f_new;                    // pso.py:106
      if (better) a.pbest_fit[row] = f_old;  // pso.py:91
      if constexpr (FUSED) {
        // a warp meets its rows in ascending order: a strict comparison keeps the first minimum
        MinIdx* mine = &s_warp_min[threadIdx.x >> 5];
        if (mine->i == kNoRow || key_less(f_new, mine->v)) *mine = MinIdx{f_new, row};
      }
    }
  }
  if constexpr (FUSED) {
    __shared__ MinIdx s_red[32];
    __shared__ bool s_last;
    __syncthreads();
    if (threadIdx.x < 32) {
      MinIdx t = (lane < kMoveWarps) ? s_warp_min[lane] : MinIdx{INFINITY, kNoRow};
      t = warp_min_idx(t);
      if (lane == 0) {
        a.partials[blockIdx.x] = t;
        __threadfence();
        s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
      }
    }
    __syncthreads();
    if (!s_last) return;
    // Every other block has finished its rows: nobody reads the records or the global best any more.
    __threadfence();
    MinIdx f{INFINITY, kNoRow};
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
      const volatile MinIdx* p = a.partials + i;
      f = min_idx_combine(f, MinIdx{p->v, p->i});
    }
    f = block_min_idx(f, s_red);
    // store the global best this generation moved towards (pso.py:92-95) ...
    bool take;
    float best;
    const float* src = fold_candidates(a, lane, &take, &best);
    if (take) {
      for (int e = threadIdx.x; e < d; e += blockDim.x) a.gbest_loc_out[e] = src[e];
    }
    __syncthreads();  // ... before its record may be overwritten
    if (threadIdx.x == 0) {
      if (take) *a.gbest_fit = best;
      *a.ticket = 0u;  // ready for the next launch
    }
    const long long g = f.i + a.row_offset;
    const float* row = a.pop + (size_t)f.i * (size_t)d;  // written by another block of this launch: read past L1
    if (a.n_peers == 0) {
      if (threadIdx.x == 0) {
        a.cand_out[0] = __float_as_uint(f.v);
        a.cand_out[1] = (uint32_t)((unsigned long long)g & 0xffffffffull);
        a.cand_out[2] = (uint32_t)((unsigned long long)g >> 32);
        a.cand_out[3] = 0u;
      }
      for (int e = threadIdx.x; e < d; e += blockDim.x) a.cand_out[4 + e] = __float_as_uint(__ldcg(row + e));
    } else {
      // this shard's record goes straight into every rank's exchange buffer (peer stores), then the flags
      const int words = 4 + d;
      const unsigned tag_out = a.tag_in + 1u == 0u ? 1u : a.tag_in + 1u;  // never 0: a cleared buffer holds no tag
      const size_t slot = ((size_t)(tag_out & 1u) * a.n_peers + a.my_rank) * words;
      for (int e = threadIdx.x; e < words; e += blockDim.x) {
        uint32_t v;
        if (e == 0) v = __float_as_uint(f.v);
        else if (e == 1) v = (uint32_t)((unsigned long long)g & 0xffffffffull);
        else if (e == 2) v = (uint32_t)((unsigned long long)g >> 32);
        else if (e == 3) v = 0u;
        else v = __float_as_uint(__ldcg(row + (e - 4)));
        for (int p = 0; p < a.n_peers; ++p) reinterpret_cast<uint32_t*>(a.peer_base[p])[slot + e] = v;
      }
      __threadfence_system();
      __syncthreads();
      if ((int)threadIdx.x < a.n_peers) {
        unsigned int* flags = reinterpret_cast<uint32_t*>(a.peer_base[threadIdx.x]) + (size_t)2 * a.n_peers * words;
        store_release_sys(flags + (size_t)(tag_out & 1u) * a.n_peers + a.my_rank, tag_out);
      }
    }
  }
}

template <int VEC, int FIT>
__global__ void __launch_bounds__(kThreads)
    eval_fitness_kernel(const float* __restrict__ pop, long long P, int d, FitParams fp, float* __restrict__ fit) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const long long n_warps = (long long)gridDim.x * kWarpsPerBlock;
  for (long long row = warp0; row < P; row += n_warps) {
    const size_t base = (size_t)row * (size_t)d;
    Fitness<FIT> acc;
    if constexpr (VEC == 4) {
      const float4* p4 = reinterpret_cast<const float4*>(pop + base);
      const int n4 = d >> 2;
#pragma unroll 4
      for (int c = lane; c < n4; c += 32) {
        const float4 x = __ldg(p4 + c);
        acc.add4(x, fp);
      }
    } else {
      for (int e = lane; e < d; e += 32) acc.add(pop[base + e], fp);
    }
    acc.reduce();
    if (lane == 0) fit[row] = acc.finish(d, fp);
  }
}

// --------------------------------------------------------------------------------------------
// argmin over the shard + optional fold into the running global best.
// Workspace layout: [0] uint32 ticket | [64 ..) MinIdx partials[kMaxPartials].
// --------------------------------------------------------------------------------------------
struct BestArgs {
  const float* fit;
  const float* pop;
  long long P;
  int d;
  long long row_offset;
  uint32_t* candidate;  // record out, or nullptr when folding directly
  float* gbest_loc;     // used when candidate == nullptr
  float* gbest_fit;
  int have_previous;
  unsigned int* ticket;
  MinIdx* partials;
};

__global__ void __launch_bounds__(kThreads) pso_local_best_kernel(const BestArgs a) {
  __shared__ MinIdx smem[32];
  __shared__ bool is_last;
  // +inf with the largest index loses against every real entry (an all-+inf shard still
  // reports index 0 because equal keys resolve to the lower index).
  MinIdx m{INFINITY, kNoRow};
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.P; i += (long long)gridDim.x * blockDim.x) {
    m = min_idx_combine(m, MinIdx{a.fit[i], i});
  }
  m = block_min_idx(m, smem);
  if (threadIdx.x == 0) {
    a.partials[blockIdx.x] = m;
    __threadfence();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    is_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  MinIdx f{INFINITY, kNoRow};
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
    const volatile MinIdx* p = a.partials + i;
    f = min_idx_combine(f, MinIdx{p->v, p->i});
  }
  f = block_min_idx(f, smem);
  if (threadIdx.x == 0) *a.ticket = 0u;  // ready for the next launch
  const float* row = a.pop + (size_t)f.i * (size_t)a.d;
  if (a.candidate != nullptr) {
    if (threadIdx.x == 0) {
      const long long g = f.i + a.row_offset;
      a.candidate[0] = __float_as_uint(f.v);
      a.candidate[1] = (uint32_t)((unsigned long long)g & 0xffffffffull);
      a.candidate[2] = (uint32_t)((unsigned long long)g >> 32);
      a.candidate[3] = 0u;
    }
    for (int e = threadIdx.x; e < a.d; e += blockDim.x) a.candidate[4 + e] = __float_as_uint(row[e]);
  } else {
    // torch.argmin over cat([old best, fit]): the old best sits at index 0 and wins ties.
    const bool take = !a.have_previous || key_less(f.v, *a.gbest_fit);
    if (take) {
      for (int e = threadIdx.x; e < a.d; e += blockDim.x) a.gbest_loc[e] = row[e];
      __syncthreads();
      if (threadIdx.x == 0) *a.gbest_fit = f.v;
    }
  }
}

__global__ void __launch_bounds__(kThreads)
    pso_merge_best_kernel(const uint32_t* __restrict__ cands, int n, int d, int have_previous,
                          float* gbest_loc, float* gbest_fit) {
  __shared__ int winner;
  const int words = 4 + d;
  if (threadIdx.x == 0) {
    MinIdx best{INFINITY, kNoRow};
    int bi = 0;
    for (int r = 0; r < n; ++r) {
      const uint32_t* c = cands + (size_t)r * words;
      const MinIdx m{__uint_as_float(c[0]), (long long)(((unsigned long long)c[2] << 32) | c[1])};
      const bool wins = r == 0 || key_less(m.v, best.v) || (!key_less(best.v, m.v) && m.i < best.i);
      if (wins) {
        best = m;
        bi = r;
      }
    }
    const bool take = !have_previous || key_less(best.v, *gbest_fit);
    winner = take ? bi : -1;
    if (take) *gbest_fit = best.v;
  }
  __syncthreads();
  if (winner < 0) return;
  const uint32_t* c = cands + (size_t)winner * words + 4;
  for (int e = threadIdx.x; e < d; e += blockDim.x) gbest_loc[e] = __uint_as_float(c[e]);
}

template <int VEC>
__global__ void __launch_bounds__(kThreads)
    pso_fill_uniform_kernel(float* __restrict__ out, long long P, int d, const RoundKeys rk, uint64_t generation,
                            uint32_t which, long long row_offset) {
  const int n_call = (d + 3) >> 2;
  const long long total = P * (long long)n_call;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / n_call;
    const int c = (int)(t - row * n_call);
    const uint64_t q = (uint64_t)(row_offset + row) * (uint64_t)n_call + (uint64_t)c;
    const float4 u = pso_uniform4(q, generation, which, rk);
    float* o = out + (size_t)row * (size_t)d + 4 * (size_t)c;
    if constexpr (VEC == 4) {
      *reinterpret_cast<float4*>(o) = u;
    } else {
      const int rem = d - 4 * c;
      o[0] = u.x;
      if (rem > 1) o[1] = u.y;
      if (rem > 2) o[2] = u.z;
      if (rem > 3) o[3] = u.w;
    }
  }
}

// --------------------------------------------------------------------------------------------
// Host-side helpers
// --------------------------------------------------------------------------------------------
struct Workspace {
  unsigned int* ticket;
  MinIdx* partials;
};

constexpr size_t kWsBytes = 64 + sizeof(MinIdx) * kMaxPartials;

int carve(void* ws, size_t bytes, Workspace* out) {
  EVOX_REQUIRE(ws != nullptr, EVOX_ERR_WORKSPACE, "pso: workspace is NULL");
  EVOX_REQUIRE(bytes >= kWsBytes, EVOX_ERR_WORKSPACE, "pso: workspace of %zu bytes is smaller than %zu", bytes, kWsBytes);
  EVOX_REQUIRE(aligned16(ws), EVOX_ERR_INVALID, "pso: workspace must be 16-byte aligned");
  out->ticket = reinterpret_cast<unsigned int*>(ws);
  out->partials = reinterpret_cast<MinIdx*>(reinterpret_cast<char*>(ws) + 64);
  return EVOX_OK;
}

int row_grid(long long P, int blocks_per_sm = 8, int warps_per_block = kWarpsPerBlock) {
  // persistent grid of exactly the resident blocks (one wave), never more rows than exist
  const long long want = (P + warps_per_block - 1) / warps_per_block;
  const long long cap = (long long)sm_count() * blocks_per_sm;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

int check_fit(int fitness_id, const float* params, FitParams* fp) {
  EVOX_REQUIRE(fitness_id >= EVOX_FIT_ACKLEY && fitness_id <= EVOX_FIT_SPHERE, EVOX_ERR_INVALID,
               "unknown fitness_id %d", fitness_id);
  fp->a = fp->b = fp->c = 0.f;
  if (fitness_id == EVOX_FIT_ACKLEY) {
    EVOX_REQUIRE(params != nullptr, EVOX_ERR_INVALID, "Ackley needs params {a, b, c}");
    fp->a = params[0];
    fp->b = params[1];
    fp->c = params[2];
  }
  return EVOX_OK;
}

template <int VEC, bool PHILOX, bool FUSED>
void launch_move(int fitness_id, int grid, cudaStream_t s, const MoveArgs& a) {
  switch (fitness_id) {
    case EVOX_FIT_ACKLEY:
      pso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_ACKLEY, FUSED><<<grid, kMoveThreads, 0, s>>>(a);
      break;
    case EVOX_FIT_RASTRIGIN:
      pso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_RASTRIGIN, FUSED><<<grid, kMoveThreads, 0, s>>>(a);
      break;
    default:
      pso_move_eval_kernel<VEC, PHILOX, EVOX_FIT_SPHERE, FUSED><<<grid, kMoveThreads, 0, s>>>(a);
      break;
  }
}

template <bool FUSED>
void launch_move_any(bool vec, bool philox, int fitness_id, int grid, cudaStream_t s, const MoveArgs& a) {
  if (vec) {
    if (philox) launch_move<4, true, FUSED>(fitness_id, grid, s, a);
    else launch_move<4, false, FUSED>(fitness_id, grid, s, a);
  } else {
    if (philox) launch_move<1, true, FUSED>(fitness_id, grid, s, a);
    else launch_move<1, false, FUSED>(fitness_id, grid, s, a);
  }
}

int launch_local_best(const float* fit, const float* pop, long long P, int d, long long row_offset,
                      uint32_t* candidate, float* gbest_loc, float* gbest_fit, int have_previous,
                      const Workspace& ws, cudaStream_t s) {
  BestArgs b;
  b.fit = fit;
  b.pop = pop;
  b.P = P;
  b.d = d;
  b.row_offset = row_offset;
  b.candidate = candidate;
  b.gbest_loc = gbest_loc;
  b.gbest_fit = gbest_fit;
  b.have_previous = have_previous;
  b.ticket = ws.ticket;
  b.partials = ws.partials;
  long long want = (P + (long long)kThreads * 8 - 1) / ((long long)kThreads * 8);
  long long cap = (long long)sm_count() * 2;
  if (cap > kMaxPartials) cap = kMaxPartials;
  int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
  pso_local_best_kernel<<<grid, kThreads, 0, s>>>(b);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

int check_shape(long long P, int d) {
  EVOX_REQUIRE(P > 0, EVOX_ERR_INVALID, "pop_size must be positive, got %lld", P);
  EVOX_REQUIRE(d > 0, EVOX_ERR_INVALID, "dim must be positive, got %d", d);
  return EVOX_OK;
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_pso_workspace_bytes(int64_t, int32_t) { return kWsBytes; }

extern "C" int32_t evox_pso_candidate_words(int32_t dim) { return 4 + dim; }

extern "C" int evox_eval_fitness(const float* pop, int64_t pop_size, int32_t dim, int32_t fitness_id,
                                 const float* params, float* fit, void* stream) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(pop && fit, EVOX_ERR_INVALID, "eval_fitness: NULL pointer");
  FitParams fp;
  if (int rc = check_fit(fitness_id, params, &fp)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = row_grid(pop_size);
  const bool vec = (dim % 4 == 0) && aligned16(pop);
#define EVOX_EVAL(V, F) eval_fitness_kernel<V, F><<<grid, kThreads, 0, s>>>(pop, pop_size, dim, fp, fit)
  const int fid = fitness_id;
  if (vec) {
    if (fid == EVOX_FIT_ACKLEY) EVOX_EVAL(4, EVOX_FIT_ACKLEY);
    else if (fid == EVOX_FIT_RASTRIGIN) EVOX_EVAL(4, EVOX_FIT_RASTRIGIN);
    else EVOX_EVAL(4, EVOX_FIT_SPHERE);
  } else {
    if (fid == EVOX_FIT_ACKLEY) EVOX_EVAL(1, EVOX_FIT_ACKLEY);
    else if (fid == EVOX_FIT_RASTRIGIN) EVOX_EVAL(1, EVOX_FIT_RASTRIGIN);
    else EVOX_EVAL(1, EVOX_FIT_SPHERE);
  }
#undef EVOX_EVAL
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_pso_local_best(const float* fit, const float* pop, int64_t pop_size, int32_t dim,
                                   int64_t row_offset, uint32_t* candidate, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(fit && pop && candidate, EVOX_ERR_INVALID, "pso_local_best: NULL pointer");
  Workspace ws;
  if (int rc = carve(workspace, workspace_bytes, &ws)) return rc;
  return launch_local_best(fit, pop, pop_size, dim, row_offset, candidate, nullptr, nullptr, 0, ws,
                           reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int evox_pso_merge_best(const uint32_t* candidates, int32_t n_candidates, int32_t dim,
                                   int32_t have_previous, float* global_best_location,
                                   float* global_best_fit, void* stream) {
  EVOX_REQUIRE(candidates && global_best_location && global_best_fit, EVOX_ERR_INVALID, "pso_merge_best: NULL pointer");
  EVOX_REQUIRE(n_candidates > 0 && dim > 0, EVOX_ERR_INVALID, "pso_merge_best: n_candidates and dim must be positive");
  pso_merge_best_kernel<<<1, kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      candidates, n_candidates, dim, have_previous, global_best_location, global_best_fit);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

namespace {

// Argument checks and packing shared by the two forms of the update kernel.
int fill_move_args(MoveArgs* a, bool* vec, float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                   float* fit, const float* global_best_location, const float* lb, const float* ub, const float* w,
                   const float* phi_p, const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                   int32_t dim, int32_t fitness_id, const float* params, uint64_t seed, uint64_t generation,
                   int64_t row_offset) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(pop && velocity && local_best_location && local_best_fit && fit && global_best_location && lb &&
                   ub && w && phi_p && phi_g,
               EVOX_ERR_INVALID, "pso_move_eval: NULL pointer");
  EVOX_REQUIRE((rg == nullptr) == (rp == nullptr), EVOX_ERR_INVALID,
               "pso_move_eval: rg and rp must both be given or both be NULL");
  if (int rc = check_fit(fitness_id, params, &a->fp)) return rc;
  a->pop = pop;
  a->vel = velocity;
  a->pbest_loc = local_best_location;
  a->pbest_fit = local_best_fit;
  a->fit = fit;
  a->gbest_loc = global_best_location;
  a->lb = lb;
  a->ub = ub;
  a->w = w;
  a->phi_p = phi_p;
  a->phi_g = phi_g;
  a->rg = rg;
  a->rp = rp;
  a->P = pop_size;
  a->d = dim;
  a->rk = make_round_keys(seed);
  a->generation = generation;
  a->row_offset = row_offset;
  a->cands = nullptr;
  a->n_cands = 0;
  a->gbest_fit = nullptr;
  a->gbest_loc_out = nullptr;
  a->cand_out = nullptr;
  a->ticket = nullptr;
  a->partials = nullptr;
  a->n_peers = 0;
  a->my_rank = 0;
  a->tag_in = 0u;
  a->status = nullptr;
  for (int p = 0; p < 16; ++p) a->peer_base[p] = 0ull;
  *vec = (dim % 4 == 0) && aligned16(pop) && aligned16(velocity) && aligned16(local_best_location) &&
         aligned16(global_best_location) && aligned16(lb) && aligned16(ub);
  if (rg != nullptr) *vec = *vec && aligned16(rg) && aligned16(rp);
  return EVOX_OK;
}

}  // namespace

extern "C" int evox_pso_move_eval(float* pop, float* velocity, float* local_best_location,
                                  float* local_best_fit, float* fit, const float* global_best_location,
                                  const float* lb, const float* ub, const float* w, const float* phi_p,
                                  const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                                  int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                                  uint64_t generation, int64_t row_offset, void* stream) {
  MoveArgs a;
  bool vec;
  if (int rc = fill_move_args(&a, &vec, pop, velocity, local_best_location, local_best_fit, fit, global_best_location,
                              lb, ub, w, phi_p, phi_g, rg, rp, pop_size, dim, fitness_id, params, seed, generation,
                              row_offset))
    return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  launch_move_any<false>(vec, rg == nullptr, fitness_id, row_grid(pop_size, MOVE_BLOCKS_PER_SM, kMoveWarps), s, a);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_pso_generation(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                                   float* fit, float* global_best_location, float* global_best_fit, const float* lb,
                                   const float* ub, const float* w, const float* phi_p, const float* phi_g,
                                   const float* rg, const float* rp, int64_t pop_size, int32_t dim,
                                   int32_t fitness_id, const float* params, uint64_t seed, uint64_t generation,
                                   int64_t row_offset, const uint32_t* candidates, int32_t n_candidates,
                                   uint32_t* candidate_out, void* workspace, size_t workspace_bytes, void* stream) {
  MoveArgs a;
  bool vec;
  if (int rc = fill_move_args(&a, &vec, pop, velocity, local_best_location, local_best_fit, fit, global_best_location,
                              lb, ub, w, phi_p, phi_g, rg, rp, pop_size, dim, fitness_id, params, seed, generation,
                              row_offset))
    return rc;
  EVOX_REQUIRE(global_best_fit && candidates && candidate_out, EVOX_ERR_INVALID, "pso_generation: NULL pointer");
  EVOX_REQUIRE(n_candidates > 0, EVOX_ERR_INVALID, "pso_generation: n_candidates must be positive, got %d", n_candidates);
  {
    const uintptr_t c0 = reinterpret_cast<uintptr_t>(candidates), o0 = reinterpret_cast<uintptr_t>(candidate_out);
    const uintptr_t rec = sizeof(uint32_t) * (size_t)(4 + dim);
    EVOX_REQUIRE(o0 + rec <= c0 || c0 + rec * (size_t)n_candidates <= o0, EVOX_ERR_INVALID,
                 "pso_generation: candidates and candidate_out overlap");
  }
  Workspace ws;
  if (int rc = carve(workspace, workspace_bytes, &ws)) return rc;
  // the attractor row is read with 16-byte loads straight out of a record: row start = record + 16 bytes
  vec = vec && aligned16(candidates);
  a.cands = candidates;
  a.n_cands = n_candidates;
  a.gbest_fit = global_best_fit;
  a.gbest_loc_out = global_best_location;
  a.cand_out = candidate_out;
  a.ticket = ws.ticket;
  a.partials = ws.partials;
  const int grid = row_grid(pop_size, MOVE_BLOCKS_PER_SM, kMoveWarps);
  EVOX_REQUIRE(grid <= kMaxPartials, EVOX_ERR_INVALID, "pso_generation: grid of %d blocks exceeds %d partials", grid, kMaxPartials);
  launch_move_any<true>(vec, rg == nullptr, fitness_id, grid, reinterpret_cast<cudaStream_t>(stream), a);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" size_t evox_pso_exchange_words(int32_t dim, int32_t n_ranks) {
  if (dim <= 0 || n_ranks <= 0) return 0;
  return (size_t)2 * n_ranks * (4 + (size_t)dim) + (size_t)2 * n_ranks;
}

extern "C" int evox_pso_generation_peer(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                                        float* fit, float* global_best_location, float* global_best_fit, const float* lb,
                                        const float* ub, const float* w, const float* phi_p, const float* phi_g,
                                        const float* rg, const float* rp, int64_t pop_size, int32_t dim,
                                        int32_t fitness_id, const float* params, uint64_t seed, uint64_t generation,
                                        int64_t row_offset, const uint64_t* peer_buffers, int32_t n_ranks, int32_t my_rank,
                                        uint32_t tag, int32_t* status, void* workspace, size_t workspace_bytes,
                                        void* stream) {
  MoveArgs a;
  bool vec;
  if (int rc = fill_move_args(&a, &vec, pop, velocity, local_best_location, local_best_fit, fit, global_best_location,
                              lb, ub, w, phi_p, phi_g, rg, rp, pop_size, dim, fitness_id, params, seed, generation,
                              row_offset))
    return rc;
  EVOX_REQUIRE(global_best_fit && peer_buffers && status, EVOX_ERR_INVALID, "pso_generation_peer: NULL pointer");
  EVOX_REQUIRE(n_ranks >= 1 && n_ranks <= 16, EVOX_ERR_INVALID, "pso_generation_peer: 1 to 16 ranks, got %d", n_ranks);
  EVOX_REQUIRE(my_rank >= 0 && my_rank < n_ranks, EVOX_ERR_INVALID, "pso_generation_peer: rank %d outside [0, %d)", my_rank, n_ranks);
  EVOX_REQUIRE(tag != 0u, EVOX_ERR_INVALID, "pso_generation_peer: tag 0 is reserved for a cleared buffer");
  Workspace ws;
  if (int rc = carve(workspace, workspace_bytes, &ws)) return rc;
  for (int p = 0; p < n_ranks; ++p) {
    EVOX_REQUIRE(peer_buffers[p] != 0 && (peer_buffers[p] & 15u) == 0, EVOX_ERR_INVALID,
                 "pso_generation_peer: exchange buffer of rank %d is NULL or not 16-byte aligned", p);
    a.peer_base[p] = peer_buffers[p];
  }
  // the attractor row is read with 16-byte loads out of a record: records are (4 + dim) words, dim % 4 == 0 here
  a.n_peers = n_ranks;
  a.my_rank = my_rank;
  a.tag_in = tag;
  a.status = status;
  a.gbest_fit = global_best_fit;
  a.gbest_loc_out = global_best_location;
  a.ticket = ws.ticket;
  a.partials = ws.partials;
  const int grid = row_grid(pop_size, MOVE_BLOCKS_PER_SM, kMoveWarps);
  EVOX_REQUIRE(grid <= kMaxPartials, EVOX_ERR_INVALID, "pso_generation_peer: grid of %d blocks exceeds %d partials", grid, kMaxPartials);
  launch_move_any<true>(vec, rg == nullptr, fitness_id, grid, reinterpret_cast<cudaStream_t>(stream), a);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_pso_step(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                             float* fit, float* global_best_location, float* global_best_fit,
                             const float* lb, const float* ub, const float* w, const float* phi_p,
                             const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                             int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                             uint64_t generation, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(fit && pop && global_best_location && global_best_fit, EVOX_ERR_INVALID, "pso_step: NULL pointer");
  Workspace ws;
  if (int rc = carve(workspace, workspace_bytes, &ws)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (int rc = launch_local_best(fit, pop, pop_size, dim, 0, nullptr, global_best_location, global_best_fit, 1, ws, s))
    return rc;
  return evox_pso_move_eval(pop, velocity, local_best_location, local_best_fit, fit, global_best_location, lb, ub,
                            w, phi_p, phi_g, rg, rp, pop_size, dim, fitness_id, params, seed, generation, 0, stream);
}

extern "C" int evox_pso_init_step(const float* pop, float* fit, float* local_best_fit,
                                  float* global_best_location, float* global_best_fit, int64_t pop_size,
                                  int32_t dim, int32_t fitness_id, const float* params, void* workspace,
                                  size_t workspace_bytes, void* stream) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(pop && fit && local_best_fit && global_best_location && global_best_fit, EVOX_ERR_INVALID,
               "pso_init_step: NULL pointer");
  Workspace ws;
  if (int rc = carve(workspace, workspace_bytes, &ws)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (int rc = evox_eval_fitness(pop, pop_size, dim, fitness_id, params, fit, stream)) return rc;
  EVOX_CUDA(cudaMemcpyAsync(local_best_fit, fit, sizeof(float) * (size_t)pop_size, cudaMemcpyDeviceToDevice, s));
  return launch_local_best(fit, pop, pop_size, dim, 0, nullptr, global_best_location, global_best_fit, 0, ws, s);
}

extern "C" int evox_pso_fill_uniform(float* out, int64_t pop_size, int32_t dim, uint64_t seed,
                                     uint64_t generation, int32_t which, int64_t row_offset, void* stream) {
  if (int rc = check_shape(pop_size, dim)) return rc;
  EVOX_REQUIRE(out != nullptr, EVOX_ERR_INVALID, "pso_fill_uniform: NULL pointer");
  EVOX_REQUIRE(which == 0 || which == 1, EVOX_ERR_INVALID, "pso_fill_uniform: which must be 0 (rg) or 1 (rp)");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long total = pop_size * (long long)((dim + 3) / 4);
  long long want = (total + kThreads - 1) / kThreads;
  const long long cap = (long long)sm_count() * 16;
  const int grid = (int)(want < cap ? want : cap);
  if (dim % 4 == 0 && aligned16(out))
    pso_fill_uniform_kernel<4><<<grid, kThreads, 0, s>>>(out, pop_size, dim, make_round_keys(seed), generation, (uint32_t)which, row_offset);
  else
    pso_fill_uniform_kernel<1><<<grid, kThreads, 0, s>>>(out, pop_size, dim, make_round_keys(seed), generation, (uint32_t)which, row_offset);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
