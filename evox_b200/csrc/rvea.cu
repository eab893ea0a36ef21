// P3: RVEA reference-vector-guided selection as one association + APD pass.
//
// Reference semantics: ref_vec_guided and apd_fn (evox/operators/selection/rvea_selection.py:7-99)
// with the relu-form helpers nanmin / maximum / clamp_float (evox/utils/jit_fix_operator.py).
// The reference materialises an (n, nv, m) product and about ten (n, nv) temporaries; here each
// objective row is read once:
//   1. rvea_ideal_kernel   column minima ignoring NaN (ordered-integer atomicMin).
//   2. rvea_vectors_kernel, rvea_gamma_kernel  unit reference vectors and gamma_j = min over k of the
//                          angle between v_j and v_k, the diagonal counted as cosine 0
//                          (rvea_selection.py:63-71).
//   3. rvea_assign_kernel  4 lanes per individual: translate, normalise, cosine against every
//                          vector from shared memory, first-minimum association by angle, APD, and
//                          a 64-bit atomicMin of (APD bits, row) per vector — APD is positive, so
//                          its bit pattern orders like the value and the lowest row wins ties, as
//                          torch.argmin does. The arccosine is taken only where it can matter: the
//                          sweep keeps the largest and the second largest cosine, and a row whose
//                          two largest cosines differ by more than 2e-6 is associated with the
//                          largest one (arccos falls at least as fast as its argument rises, and
//                          the device routine is accurate to 4e-7, so no other vector can have the
//                          smaller computed angle); the few other rows repeat the sweep with the
//                          arccosine of every cosine, exactly as the reference orders them.
//   4. rvea_gather_kernel  rows of x and f for every vector, NaN for vectors nobody joined.
// The unit vectors and gamma stay in the workspace: a caller that passes the same vectors again
// says so and steps 2 are skipped.
// Bytes that must move: n*m*4 (objectives) + nv*(dx+m)*4 (outputs); the pass is latency-bound at
// the benchmark's 2 MB input.
#include <math.h>

#include "common.cuh"

namespace evox {
namespace {

constexpr int kThreads = 256;
constexpr int kLanesPerRow = 4;
constexpr float kEps = 1e-8f;  // torch.nn.functional.cosine_similarity's eps

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// 0xffffffff (the byte pattern a memset leaves) stands for "no number seen": +inf, as nanmin reports it
__device__ __forceinline__ float order_key_inv(uint32_t k) {
  if (k == 0xffffffffu) return INFINITY;
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ float relu_clamp01(float a) {
  const float lo = fmaxf(__fsub_rn(0.0f, a), 0.0f);
  const float hi = fmaxf(__fsub_rn(a, 1.0f), 0.0f);
  return __fsub_rn(__fadd_rn(a, lo), hi);
}

__global__ void rvea_decode_ideal_kernel(const uint32_t* zmin_key, int m, float* zmin) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < m) zmin[t] = order_key_inv(zmin_key[t]);
}
__global__ void rvea_encode_ideal_kernel(const float* zmin, int m, uint32_t* zmin_key) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < m) zmin_key[t] = order_key(zmin[t]);
}

// nanmin over rows (jit_fix_operator.py:289-292): NaN counts as +inf.
__global__ void __launch_bounds__(kThreads)
    rvea_ideal_kernel(const float* __restrict__ f, long long n, int m, uint32_t* zmin_key) {
  // thread t handles column t % m of rows t / m, t / m + stride, ... (coalesced over the row-major matrix)
  const long long total = n * (long long)m;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long step = stride - (stride % m);  // keep each thread on one column
  long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // the block's threads meet in shared memory first (m <= 32): one global atomic per column and block
  __shared__ uint32_t s_key[32];
  if (threadIdx.x < 32) s_key[threadIdx.x] = 0xffffffffu;
  __syncthreads();
  if (t < step) {
    const int col = (int)(t % m);
    float mn = INFINITY;
    for (; t < total; t += step) {
      const float v = f[t];
      if (v == v) mn = fminf(mn, v);
    }
    atomicMin(s_key + col, order_key(mn));
  }
  __syncthreads();
  if (threadIdx.x < m && s_key[threadIdx.x] != 0xffffffffu) atomicMin(zmin_key + threadIdx.x, s_key[threadIdx.x]);
}

// vn = v / max(|v|, eps), one thread per vector.
__global__ void __launch_bounds__(kThreads)
    rvea_vectors_kernel(const float* __restrict__ v, int nv, int m, float* __restrict__ vn) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= nv) return;
  float s = 0.f;
  for (int k = 0; k < m; ++k) s = __fmaf_rn(v[j * m + k], v[j * m + k], s);
  const float nrm = fmaxf(sqrtf(s), kEps);
  for (int k = 0; k < m; ++k) vn[j * m + k] = __fdiv_rn(v[j * m + k], nrm);
}

// gamma_j = min_k acos(clamp01(cos(v_j, v_k))) with cos_jj := 0. One block per j, its threads over k; a
// minimum does not depend on the order it is taken in. (One thread per j walking all k took 194 us for
// 275 vectors: three quarters of the whole selection at 50,000 x 10.)
__global__ void __launch_bounds__(kThreads)
    rvea_gamma_kernel(const float* __restrict__ vn, int nv, int m, float* __restrict__ gamma) {
  __shared__ float s_min[kThreads / 32];
  const int j = blockIdx.x;
  float g = acosf(0.0f);  // the diagonal entry, set to cosine 0 by the reference
  for (int k = threadIdx.x; k < nv; k += blockDim.x) {
    if (k == j) continue;
    float c = 0.f;
    for (int q = 0; q < m; ++q) c = __fmaf_rn(vn[j * m + q], vn[k * m + q], c);
    g = fminf(g, acosf(relu_clamp01(c)));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) g = fminf(g, __shfl_xor_sync(0xffffffffu, g, off));
  if ((threadIdx.x & 31) == 0) s_min[threadIdx.x >> 5] = g;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kThreads / 32; ++w) g = fminf(g, s_min[w]);
    gamma[j] = g;
  }
}

// One output element of the gather: rows of x and f for every vector, NaN for vectors nobody joined.
// sharded: x and f hold rows [row_begin, row_begin + row_count); rows of other shards and empty vectors
// contribute 0 so that a sum over the shards reproduces the gathered row.
__device__ __forceinline__ void gather_element(long long t, unsigned long long key, const float* __restrict__ x, long long dx,
                                               const float* __restrict__ f, int m, float* __restrict__ next_x,
                                               float* __restrict__ next_f, long long* __restrict__ next_index,
                                               long long row_begin, long long row_count, int sharded) {
  const long long per = dx + m;
  const int j = (int)(t / per);
  const long long c = t - (long long)j * per;
  const bool empty = key == 0xffffffffffffffffull;
  // a vector whose members all have APD = +inf: argmin over an all-inf column is row 0
  const bool all_inf = !empty && (uint32_t)(key >> 32) == 0x7f800000u;
  const long long src = all_inf ? 0 : (long long)(uint32_t)key;
  const float nanv = __int_as_float(0x7fc00000);
  const long long loc = src - row_begin;
  const bool mine = !empty && loc >= 0 && loc < row_count;
  if (c < dx) next_x[(long long)j * dx + c] = sharded ? (mine ? x[loc * dx + c] : 0.0f) : (empty ? nanv : x[src * dx + c]);
  else next_f[(long long)j * m + (c - dx)] = sharded ? (mine ? f[loc * m + (c - dx)] : 0.0f) : (empty ? nanv : f[src * m + (c - dx)]);
  if (c == 0 && next_index) next_index[j] = empty ? -1 : src;
}

// key -> *slot = min(*slot, key). The slots only ever fall, so a key that is not below the value this SM last saw
// (an ordinary, possibly stale, cached load) cannot change the slot and is dropped without an atomic: after the
// first rows almost every offer ends here, and the few hundred slots stop being a point of serialisation
// (five million atomics on 275 addresses cost a seventh of the association's time at 5,000,000 rows).
__device__ __forceinline__ void offer_min(unsigned long long* slot, unsigned long long key) {
  if (key < *reinterpret_cast<volatile unsigned long long*>(slot)) atomicMin(slot, key);
}

constexpr float kCosMargin = 2e-6f;

constexpr int kRowsPerGroup = 4;  // rows a group of kLanesPerRow lanes carries through one sweep of the vectors

static_assert(kRowsPerGroup == kLanesPerRow, "lane r of a group prepares and finishes row r of the group");

// Floats between two vectors in shared memory: the next multiple of four, so that every vector starts on a
// 16-byte boundary (ten objectives: two 16-byte loads and one 8-byte load instead of five 8-byte loads).
template <int MP>
constexpr int kVecStride = (MP + 3) / 4 * 4;

template <int MP>
__device__ __forceinline__ void load_vector(const float* __restrict__ row, float (&vj)[MP]) {
  static_assert(MP % 2 == 0, "vector rows are read with 8- or 16-byte loads");
#pragma unroll
  for (int k = 0; k + 4 <= MP; k += 4) {
    const float4 q = *reinterpret_cast<const float4*>(row + k);
    vj[k] = q.x;
    vj[k + 1] = q.y;
    vj[k + 2] = q.z;
    vj[k + 3] = q.w;
  }
  if constexpr (MP % 4 == 2) {
    const float2 q = *reinterpret_cast<const float2*>(row + MP - 2);
    vj[MP - 2] = q.x;
    vj[MP - 1] = q.y;
  }
}

// A group of four lanes owns four consecutive rows. Lane r translates and normalises row r once and hands it to
// the group by shuffles; in the sweep the vectors are dealt among the lanes and every vector a lane reads from
// shared memory is used for all four rows (with one row per group the sweep was bound by shared-memory
// bandwidth: 48 bytes per row-vector pair, 2.1 ms at 5,000,000 rows); lane r then finishes row r (arccosine,
// angle-penalised distance, the atomic minimum of its vector).
template <int MP>
__global__ void __launch_bounds__(kThreads)
    rvea_assign_kernel(const float* __restrict__ f, long long n, int m, const uint32_t* __restrict__ zmin_key,
                       const float* __restrict__ vn, const float* __restrict__ gamma, int nv,
                       const float* __restrict__ theta_p, unsigned long long* best, int* __restrict__ associate,
                       long long row_offset) {
  constexpr int R = kRowsPerGroup;
  constexpr int VS = kVecStride<MP>;
  extern __shared__ __align__(16) float s_vn[];  // nv x VS, zero padded
  __shared__ float s_zmin[MP];
  for (int t = threadIdx.x; t < nv * VS; t += blockDim.x) {
    const int j = t / VS, k = t - j * VS;
    s_vn[t] = (k < m) ? vn[j * m + k] : 0.0f;
  }
  if (threadIdx.x < MP) s_zmin[threadIdx.x] = threadIdx.x < m ? order_key_inv(zmin_key[threadIdx.x]) : 0.0f;
  __syncthreads();
  const float m_theta = __fmul_rn((float)m, *theta_p);  // rvea_selection.py:26: obj.size(1) * theta
  const int sub = threadIdx.x & (kLanesPerRow - 1);
  // only the four lanes of a group meet in the shuffles below (the groups of a warp run different numbers of trips)
  const unsigned group_lanes = ((1u << kLanesPerRow) - 1u) << (threadIdx.x & 31 & ~(kLanesPerRow - 1));
  const long long groups_per_pass = (long long)gridDim.x * (kThreads / kLanesPerRow);
  const long long n_groups = (n + R - 1) / R;
  for (long long grp = (long long)blockIdx.x * (kThreads / kLanesPerRow) + (threadIdx.x / kLanesPerRow); grp < n_groups;
       grp += groups_per_pass) {
    // this lane's row: translate by the ideal point, floor at 1e-32, normalise
    const long long my_row = grp * R + sub;
    const bool my_live = my_row < n;
    float mine[MP];
    bool my_nan = false;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < MP; ++k) {
      float o = 0.f;
      if (my_live && k < m) {
        o = __fsub_rn(f[my_row * m + k], s_zmin[k]);
        o = __fadd_rn(o, fmaxf(__fsub_rn(1e-32f, o), 0.0f));  // maximum(obj, 1e-32), relu form
        my_nan = my_nan || (o != o);
        sq = __fmaf_rn(o, o, sq);
      }
      mine[k] = o;
    }
    const float my_norm = sqrtf(sq);
    const float den = fmaxf(my_norm, kEps);
#pragma unroll
    for (int k = 0; k < MP; ++k) mine[k] = __fdiv_rn(mine[k], den);
    float obj[R][MP];
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int k = 0; k < MP; ++k) obj[r][k] = __shfl_sync(group_lanes, mine[k], r, kLanesPerRow);
    }
    // the sweep: per row the largest cosine (first index among equals) and the largest cosine of all the others
    float c1[R], c2[R];
    int j1[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      c1[r] = -INFINITY;
      c2[r] = -INFINITY;
      j1[r] = 0x7fffffff;
    }
#pragma unroll 4
    for (int j = sub; j < nv; j += kLanesPerRow) {
      float vj[MP];
      load_vector<MP>(s_vn + j * VS, vj);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float c = 0.f;
#pragma unroll
        for (int k = 0; k < MP; ++k) c = __fmaf_rn(obj[r][k], vj[k], c);
        c2[r] = fmaxf(c2[r], fminf(c, c1[r]));  // a NaN cosine leaves both untouched
        if (c > c1[r]) {
          c1[r] = c;
          j1[r] = j;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int off = 1; off < kLanesPerRow; off <<= 1) {
        const float o1 = __shfl_xor_sync(group_lanes, c1[r], off);
        const float o2 = __shfl_xor_sync(group_lanes, c2[r], off);
        const int oj = __shfl_xor_sync(group_lanes, j1[r], off);
        c2[r] = fmaxf(fmaxf(c2[r], o2), fminf(c1[r], o1));
        if (o1 > c1[r] || (o1 == c1[r] && oj < j1[r])) {
          c1[r] = o1;
          j1[r] = oj;
        }
      }
    }
    // Every lane now holds the same c1 / c2 / j1 of the four rows. Lane r keeps row r's; a row whose two largest
    // cosines are close is first settled by the whole group in the reference's own order.
    float my_c1 = c1[0];
    int my_j = j1[0];
    float my_angle = 0.f;
    bool my_slow = false;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r > 0 && sub == r) {
        my_c1 = c1[r];
        my_j = j1[r];
      }
      // compared after the clamp to [0, 1] the angle is taken of: all cosines below 0 share the angle pi / 2
      const bool near = !(fminf(fmaxf(c1[r], 0.0f), 1.0f) - fminf(fmaxf(c2[r], 0.0f), 1.0f) > kCosMargin);
      if (near && grp * R + r < n) {  // the same for the group's four lanes
        // near tie (or no usable cosine at all): arccosine of every cosine, first minimum
        float best_angle = INFINITY;
        int best_j = 0x7fffffff;
        for (int j = sub; j < nv; j += kLanesPerRow) {
          const float* vj = s_vn + j * VS;
          float c = 0.f;
#pragma unroll
          for (int k = 0; k < MP; ++k) c = __fmaf_rn(obj[r][k], vj[k], c);
          const float a = acosf(relu_clamp01(c));
          if (a < best_angle) {
            best_angle = a;
            best_j = j;
          }
        }
#pragma unroll
        for (int off = 1; off < kLanesPerRow; off <<= 1) {
          const float oa = __shfl_xor_sync(group_lanes, best_angle, off);
          const int oj = __shfl_xor_sync(group_lanes, best_j, off);
          if (oa < best_angle || (oa == best_angle && oj < best_j)) {
            best_angle = oa;
            best_j = oj;
          }
        }
        if (sub == r) {
          my_slow = true;
          my_angle = best_angle;
          my_j = best_j;
        }
      }
    }
    if (my_live) {
      if (!my_slow) my_angle = acosf(relu_clamp01(my_c1));
      if (my_nan || my_j >= nv) {
        associate[my_row] = -1;  // rvea_selection.py:81-83
      } else {
        associate[my_row] = my_j;
        // rvea_selection.py:25-29: (1 + m * theta * angle) / gamma * |obj|
        const float left = __fdiv_rn(__fadd_rn(1.0f, __fmul_rn(m_theta, my_angle)), gamma[my_j]);
        const float apd = __fmul_rn(left, my_norm);
        // NaN sorts first (torch.argmin); +inf keeps its bit pattern and is resolved at gather time
        const unsigned long long grow = (unsigned long long)(my_row + row_offset);  // row number in the whole population
        const unsigned long long key =
            (apd != apd) ? grow : (((unsigned long long)__float_as_uint(apd) << 32) | (grow & 0xffffffffull));
        offer_min(best + my_j, key);
      }
    }
  }
}

__global__ void rvea_gather_kernel(const unsigned long long* __restrict__ best, int nv, const float* __restrict__ x,
                                   long long dx, const float* __restrict__ f, int m, float* __restrict__ next_x,
                                   float* __restrict__ next_f, long long* __restrict__ next_index, long long row_begin,
                                   long long row_count, int sharded) {
  const long long total = (long long)nv * (dx + m);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x)
    gather_element(t, best[(int)(t / (dx + m))], x, dx, f, m, next_x, next_f, next_index, row_begin, row_count, sharded);
}

struct Layout {
  size_t zmin, best, clear_bytes, vn, gamma, associate, total;
};

Layout make_layout(long long n, int m, int nv) {
  Layout L;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = (off + bytes + 255) / 256 * 256;
    return at;
  };
  // [zmin | best] start every call as all-ones bytes: one memset
  L.zmin = take(sizeof(uint32_t) * (size_t)m);
  L.best = take(sizeof(unsigned long long) * (size_t)nv);
  L.clear_bytes = off;
  L.vn = take(sizeof(float) * (size_t)nv * m);
  L.gamma = take(sizeof(float) * (size_t)nv);
  L.associate = take(sizeof(int) * (size_t)n);
  L.total = off;
  return L;
}

template <int MP>
int launch_assign(const float* f, long long n, int m, const uint32_t* zmin, const float* vn, const float* gamma, int nv,
                  const float* theta, unsigned long long* best, int* associate, long long row_offset, cudaStream_t s) {
  const size_t smem = sizeof(float) * (size_t)nv * kVecStride<MP>;
  EVOX_REQUIRE(smem <= 200 * 1024, EVOX_ERR_INVALID, "ref_vec_guided: %d reference vectors x %d objectives do not fit in shared memory", nv, m);
  if (smem > 48 * 1024) {
    EVOX_CUDA(cudaFuncSetAttribute(rvea_assign_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const long long rows_per_block = (kThreads / kLanesPerRow) * kRowsPerGroup;
  long long blocks = (n + rows_per_block - 1) / rows_per_block;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  rvea_assign_kernel<MP><<<(unsigned)blocks, kThreads, smem, s>>>(f, n, m, zmin, vn, gamma, nv, theta, best, associate, row_offset);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_rvea_workspace_bytes(int64_t n, int32_t m, int32_t nv) {
  if (n <= 0 || m <= 0 || nv <= 0) return 0;
  return make_layout(n, m, nv).total;
}

namespace {

template <class... A>
int dispatch_assign(int m, A... args) {
  if (m <= 2) return launch_assign<2>(args...);
  if (m <= 4) return launch_assign<4>(args...);
  if (m <= 6) return launch_assign<6>(args...);
  if (m <= 8) return launch_assign<8>(args...);
  if (m <= 10) return launch_assign<10>(args...);
  if (m <= 12) return launch_assign<12>(args...);
  if (m <= 16) return launch_assign<16>(args...);
  return launch_assign<32>(args...);
}

}  // namespace

extern "C" int evox_ref_vec_guided(const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                                   const float* v, int32_t nv, const float* theta, int32_t vectors_ready,
                                   float* next_x, float* next_f, int64_t* next_index, void* workspace,
                                   size_t workspace_bytes, void* stream) {
  EVOX_REQUIRE(x && f && v && theta && next_x && next_f, EVOX_ERR_INVALID, "ref_vec_guided: NULL pointer");
  EVOX_REQUIRE(n > 0 && n < (1ll << 32), EVOX_ERR_INVALID, "ref_vec_guided: n must be in [1, 2^32), got %lld", (long long)n);
  EVOX_REQUIRE(m > 0 && m <= 32, EVOX_ERR_INVALID, "ref_vec_guided: number of objectives must be in [1, 32], got %d", m);
  EVOX_REQUIRE(nv > 0 && dx > 0, EVOX_ERR_INVALID, "ref_vec_guided: nv and dx must be positive");
  const Layout L = make_layout(n, m, nv);
  EVOX_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, EVOX_ERR_WORKSPACE,
               "ref_vec_guided: workspace of %zu bytes is smaller than %zu", workspace_bytes, L.total);
  EVOX_REQUIRE(((uintptr_t)workspace & 255u) == 0, EVOX_ERR_INVALID, "ref_vec_guided: workspace must be 256-byte aligned");
  char* ws = reinterpret_cast<char*>(workspace);
  uint32_t* zmin = reinterpret_cast<uint32_t*>(ws + L.zmin);
  unsigned long long* best = reinterpret_cast<unsigned long long*>(ws + L.best);
  float* vn = reinterpret_cast<float*>(ws + L.vn);
  float* gamma = reinterpret_cast<float*>(ws + L.gamma);
  int* associate = reinterpret_cast<int*>(ws + L.associate);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // column minima and the per-vector winners start as all-ones bytes
  EVOX_CUDA(cudaMemsetAsync(ws + L.zmin, 0xff, L.clear_bytes - L.zmin, s));
  {
    long long want = (n * m + kThreads * 8 - 1) / (kThreads * 8);
    const long long cap = (long long)sm_count() * 4;
    const int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    rvea_ideal_kernel<<<grid, kThreads, 0, s>>>(f, n, m, zmin);
    EVOX_LAUNCH_CHECK();
  }
  if (!vectors_ready) {
    rvea_vectors_kernel<<<(nv + kThreads - 1) / kThreads, kThreads, 0, s>>>(v, nv, m, vn);
    rvea_gamma_kernel<<<nv, kThreads, 0, s>>>(vn, nv, m, gamma);
    EVOX_LAUNCH_CHECK();
  }
  if (int rc = dispatch_assign(m, f, (long long)n, (int)m, (const uint32_t*)zmin, (const float*)vn, (const float*)gamma, (int)nv,
                               theta, best, associate, 0ll, s))
    return rc;
  {
    const long long total = (long long)nv * (dx + m);
    const long long cap = (long long)sm_count() * 8;
    long long want = (total + kThreads - 1) / kThreads;
    rvea_gather_kernel<<<(unsigned)(want < cap ? want : cap), kThreads, 0, s>>>(best, nv, x, dx, f, m, next_x, next_f,
                                                                                 (long long*)next_index, 0, n, 0);
    EVOX_LAUNCH_CHECK();
  }
  return EVOX_OK;
}

// ---------------------------------------------------------------------------------------------
// Row-sharded selection: the same kernels in three phases with one small exchange after each of
// the first two (ideal point: minimum over shards; per-vector winners: minimum over shards of the
// packed (APD, global row) keys) and a sum of the gathered rows at the end.
// ---------------------------------------------------------------------------------------------
extern "C" int evox_ref_vec_guided_phase(int32_t phase, const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                                         const float* v, int32_t nv, const float* theta, int64_t row_offset,
                                         float* ideal, int64_t* best_keys, float* next_x, float* next_f,
                                         int64_t* next_index, void* workspace, size_t workspace_bytes, void* stream) {
  EVOX_REQUIRE(phase >= 1 && phase <= 3, EVOX_ERR_INVALID, "ref_vec_guided_phase: phase must be 1, 2 or 3");
  EVOX_REQUIRE(f && ideal && best_keys, EVOX_ERR_INVALID, "ref_vec_guided_phase: NULL pointer");
  EVOX_REQUIRE(n > 0 && row_offset >= 0 && row_offset + n < (1ll << 32), EVOX_ERR_INVALID, "ref_vec_guided_phase: rows out of range");
  EVOX_REQUIRE(m > 0 && m <= 32 && nv > 0, EVOX_ERR_INVALID, "ref_vec_guided_phase: bad m or nv");
  const Layout L = make_layout(n, m, nv);
  EVOX_REQUIRE(workspace != nullptr && workspace_bytes >= L.total && ((uintptr_t)workspace & 255u) == 0, EVOX_ERR_WORKSPACE,
               "ref_vec_guided_phase: workspace missing, misaligned or smaller than %zu bytes", L.total);
  char* ws = reinterpret_cast<char*>(workspace);
  uint32_t* zmin = reinterpret_cast<uint32_t*>(ws + L.zmin);
  unsigned long long* best = reinterpret_cast<unsigned long long*>(best_keys);
  float* vn = reinterpret_cast<float*>(ws + L.vn);
  float* gamma = reinterpret_cast<float*>(ws + L.gamma);
  int* associate = reinterpret_cast<int*>(ws + L.associate);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (phase == 1) {  // this shard's column minima -> ideal (m floats)
    EVOX_CUDA(cudaMemsetAsync(zmin, 0xff, sizeof(uint32_t) * (size_t)m, s));
    EVOX_CUDA(cudaMemsetAsync(best, 0xff, sizeof(unsigned long long) * (size_t)nv, s));
    long long want = (n * m + kThreads * 8 - 1) / (kThreads * 8);
    const long long cap = (long long)sm_count() * 4;
    rvea_ideal_kernel<<<(int)(want < 1 ? 1 : (want < cap ? want : cap)), kThreads, 0, s>>>(f, n, m, zmin);
    rvea_decode_ideal_kernel<<<1, 32, 0, s>>>(zmin, m, ideal);
    EVOX_LAUNCH_CHECK();
    return EVOX_OK;
  }
  if (phase == 2) {  // ideal = minimum over all shards -> packed winners of this shard (nv keys)
    EVOX_REQUIRE(v && theta, EVOX_ERR_INVALID, "ref_vec_guided_phase: NULL pointer");
    rvea_encode_ideal_kernel<<<1, 32, 0, s>>>(ideal, m, zmin);
    rvea_vectors_kernel<<<(nv + kThreads - 1) / kThreads, kThreads, 0, s>>>(v, nv, m, vn);
    rvea_gamma_kernel<<<nv, kThreads, 0, s>>>(vn, nv, m, gamma);
    EVOX_LAUNCH_CHECK();
    return dispatch_assign(m, f, (long long)n, (int)m, (const uint32_t*)zmin, (const float*)vn, (const float*)gamma, (int)nv, theta,
                           best, associate, (long long)row_offset, s);
  }
  // phase 3: best_keys = minimum over all shards -> this shard's rows of the winners (others 0)
  EVOX_REQUIRE(x && next_x && next_f && dx > 0, EVOX_ERR_INVALID, "ref_vec_guided_phase: NULL pointer");
  const long long total = (long long)nv * (dx + m);
  const long long cap = (long long)sm_count() * 8;
  long long want = (total + kThreads - 1) / kThreads;
  rvea_gather_kernel<<<(unsigned)(want < cap ? want : cap), kThreads, 0, s>>>(best, nv, x, dx, f, m, next_x, next_f,
                                                                               (long long*)next_index, row_offset, n, 1);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
