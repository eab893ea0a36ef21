// P2: NSGA-II environmental selection — non-dominated rank, crowding distance, truncation.
//
// Reference semantics: dominate_relation, the front-peeling loop of non_dominate_rank,
// crowding_distance and nd_environmental_selection
// (evox/operators/selection/non_dominate.py:6-26, 151-195, 198-231, 234-254) and the stable
// lexsort they use (evox/utils/jit_fix_operator.py:216-252).
//
// Rank:
//   1. nds_transpose_kernel    objectives to structure-of-arrays, padded with NaN (a NaN never
//                              dominates and is never dominated, as in the reference's comparisons).
//   2. nds_dominance_kernel    bit-packed dominance matrix Dt: bit i of row j is set iff i
//                              dominates j. A warp holds 32 dominators per word in registers,
//                              walks the columns of a shared-memory tile and turns 32 comparisons
//                              into one word with a ballot; tiles leave through shared memory as
//                              128-byte rows. Tiles above the diagonal band get both directions of a
//                              pair from the same 2 m comparisons and also write the mirrored bits,
//                              so tiles below the band are skipped. n^2 / 8 bytes are written once.
//   3. nds_peel_kernel         persistent cooperative kernel. Front k = the unranked columns whose
//                              row of Dt has no bit left in the unranked mask. Every column keeps a
//                              witness position: the scan of its row resumes where it last found an
//                              unranked dominator and never goes back, so each row of Dt is read
//                              once in total (n^2 / 8 bytes), not once per front as the reference
//                              does. A warp owns 32 columns; a lane whose witness left probes the
//                              next 32 words of its row itself, the columns that need a longer scan
//                              are queued per block and scanned by whichever warp is free; the mask
//                              is double buffered so one bounded grid barrier separates two fronts.
//   For 8192 rows or more the rows are first dealt into bands of descending first objective and, inside a band,
//   into bins of descending second objective (nds_range / bin_count / group / key_count / bin_scan / bin_scatter
//   kernels): ranks do not depend on the row order, a tile of the matrix is then narrow in both objectives, most
//   tiles above the diagonal need m - 1, m - 2 or no comparisons per pair instead of 2 m, and a column's
//   dominators all lie after its bin's first row.
// Selection: histogram of ranks -> last admitted front -> per-objective stable radix sort of that
// front -> neighbour gaps / range -> stable sorts by (rank) and (-crowding) -> gather.
#include <cooperative_groups.h>
#include <math.h>

#include <mutex>

#include "common.cuh"

namespace evox {
namespace {

constexpr int kThreads = 256;
constexpr int kSortThreads = 1024;
// threads per block of the grid peeling kernel: 512, or 1024 when that lets every warp own ONE word of 32 columns
// per front (earlier measurements with one size for every population: 256: 2.37 / 0.435 ms per rank at 1e5 / 2e4
// rows, 512: 2.34 / 0.426, 1024: 2.32 / 0.460)
constexpr int kPeelThreadsSmall = 512, kPeelThreadsLarge = 1024;
constexpr int kTileJ = 128;      // columns (dominated candidates) per dominance tile
constexpr int kPad = 1024;       // population padded to a multiple of this (32 words = 128 B rows)
constexpr unsigned kSpinLimit = 1u << 22;  // grid-barrier polls before giving up (~ seconds)
// The last fronts of a large population, and every front of a small one, are peeled by ONE thread-block
// cluster (nds_peel_tail_kernel): its barrier is a hardware cluster barrier instead of a grid barrier
// through memory.
constexpr int kTailCtas = 8;                      // thread blocks of the cluster (the portable maximum)
constexpr int kTailThreads = 1024;
constexpr int kTailMaxWords = 256;                // mask words (of 32 columns) of the cluster kernel: one per warp
constexpr long long kTailDirectMaxN = 32 * kTailMaxWords;  // up to here the cluster peels the whole matrix itself
// Larger populations are handed over when this many rows are left. Measured on a B200 (DTLZ2-shaped, m = 3): with
// 4,096 the rank takes 2.20 ms at 100,000 rows and 0.394 ms at 20,000 (2.29 / 0.406 without a hand-over,
// 2.20 / 0.427 when handing over at 8,192: the grid kernel's many warps beat one cluster while fronts are large).
constexpr int kTailCompactRows = 4096;
static_assert(kTailMaxWords == kTailCtas * (kTailThreads / 32), "one word of 32 columns per warp of the cluster");
constexpr int kRankBuckets = 1024;   // selection: populations with at most this many fronts take the counting path
constexpr int kRankWarps = 512;      // warps (contiguous row ranges) of the counting path
constexpr int kBins = 4096;      // value bins of the first objective (row ordering for large populations)
constexpr long long kOrderMinN = 8192;  // smaller populations have too few separated tiles to pay for the ordering

// ---------------------------------------------------------------------------------------------
// Workspace
// ---------------------------------------------------------------------------------------------
struct Ctrl {
  unsigned long long bar_word;      // arrivals of the current barrier (low half) + rows they ranked (high half)
  unsigned long long release_word;  // (barrier number << 32) | rows ranked before it; bit 63: a wait gave up
  unsigned spare[2];
  int status;        // 0 ok, 1 barrier timed out, 2 no progress
  int n_fronts;
  int worst_rank;    // last admitted front
  int n_before;      // rows with rank < worst_rank
  int n_last;        // rows with rank == worst_rank
  int tail_rows;     // rows the cluster kernel still has to rank (0: nothing to do)
  int tail_k0;       // number of the first front it assigns
  int tail_buf;      // which of the two mask buffers holds the unranked rows at the hand-over
  int pad[2];
};

struct Layout {
  size_t fs, dt, unranked, newfront, ptr, ctrl, perm, bins, hist, idx_a, key_a, idx_l, sortbuf, contrib, boundary, crowd, order, rank, tail_ids,
      tail_sub, whist, rank_off, tile_stats, total;
  long long npad;
  int wp;
};

size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// `selection` = false: only what the rank needs (the allocation-free entry point's fixed array holds exactly that).
Layout make_layout(long long n, int m, bool with_matrix, bool selection = true) {
  Layout L;
  L.npad = (n + kPad - 1) / kPad * kPad;
  L.wp = (int)(L.npad / 32);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes);
    return at;
  };
  L.ctrl = take(sizeof(Ctrl));
  L.fs = take(sizeof(float) * (size_t)m * L.npad);
  L.unranked = take(sizeof(uint32_t) * L.wp);
  L.newfront = take(sizeof(uint32_t) * L.wp);
  L.ptr = take(sizeof(int) * (size_t)n);
  L.perm = take(sizeof(uint32_t) * (size_t)n);
  L.tile_stats = take(sizeof(float) * 5 * (size_t)(L.npad / kTileJ));
  L.bins = take(sizeof(int) * (size_t)(3 * (kBins + 2) + 4));  // range keys, band of each value bin, counts / offsets, cursors
  L.hist = take(sizeof(int) * (size_t)(n + 1));
  L.idx_a = take(sizeof(uint32_t) * (size_t)n);
  L.key_a = take(sizeof(uint32_t) * (size_t)n);
  L.idx_l = take(sizeof(uint32_t) * (size_t)n);
  L.sortbuf = take(sizeof(uint32_t) * 4 * (size_t)n * (size_t)(m + 2));  // per sort: keys, vals, 2 x temp
  L.contrib = take(sizeof(float) * (size_t)m * (size_t)n);
  L.boundary = take(sizeof(uint32_t) * (size_t)n);
  L.crowd = take(sizeof(float) * (size_t)n);
  L.order = take(sizeof(uint32_t) * (size_t)n);
  L.rank = take(sizeof(int) * (size_t)n);
  L.whist = selection ? take(sizeof(int) * (size_t)kRankWarps * kRankBuckets) : off;
  L.rank_off = selection ? take(sizeof(int) * (size_t)kRankBuckets * 2) : off;  // offsets, then totals
  // populations too large for the cluster kernel to peel alone: the compacted sub-matrix of the last rows
  const bool compact = with_matrix && n > kTailDirectMaxN;
  L.tail_ids = compact ? take(sizeof(uint32_t) * kTailCompactRows) : off;
  L.tail_sub = compact ? take(sizeof(uint32_t) * (size_t)kTailCompactRows * (kTailCompactRows / 32)) : off;
  L.dt = with_matrix ? take(sizeof(uint32_t) * (size_t)n * (size_t)L.wp) : off;
  L.total = off;
  return L;
}

template <class T>
T* at(void* ws, size_t off) {
  return reinterpret_cast<T*>(reinterpret_cast<char*>(ws) + off);
}

// ---------------------------------------------------------------------------------------------
// Rank
// ---------------------------------------------------------------------------------------------
// `perm` (optional): position p of the structure-of-arrays copy holds row perm[p].
__global__ void nds_transpose_kernel(const float* __restrict__ f, long long n, int m, long long npad,
                                     const uint32_t* __restrict__ perm, float* __restrict__ fs) {
  const long long total = (long long)m * npad;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int k = (int)(t / npad);
    const long long i = t - (long long)k * npad;
    fs[t] = (i < n) ? f[(perm ? (long long)perm[i] : i) * m + k] : __int_as_float(0x7fc00000);
  }
}

// ---------------------------------------------------------------------------------------------
// Row ordering for large populations. Ranks do not depend on the order of the rows, so the rows are
// dealt into kBins value bins of the first objective (a counting sort: range, counts, offsets,
// scatter, largest values first) and the matrix is built over that order. A row can only be dominated by
// rows whose first objective is not larger, so most tiles above the diagonal then hold rows i whose
// first objective lies strictly above that of every column j: there "i dominates j" is impossible and
// "j dominates i" needs only the remaining m - 1 comparisons (nds_dominance_kernel tests this per tile, so any
// order, also a poor one, gives the same bits). The order inside a bin is whatever the scatter's
// atomics produce; the ranks, which is all that leaves the computation, do not depend on it.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t range_key(float x) {  // unsigned order = numeric order (finite values)
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float range_value(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

// range[2k] = largest key of a finite objective k, range[2k + 1] = largest inverted key (= smallest value), k = 0, 1
__global__ void nds_range_kernel(const float* __restrict__ f, long long n, int m, unsigned* range) {
  unsigned hi[2] = {0u, 0u}, lo_inv[2] = {0u, 0u};
  const int objs = m >= 2 ? 2 : 1;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    for (int k = 0; k < objs; ++k) {
      const float x = f[i * m + k];
      if (isfinite(x)) {
        const unsigned key = range_key(x);
        hi[k] = max(hi[k], key);
        lo_inv[k] = max(lo_inv[k], ~key);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      hi[k] = max(hi[k], __shfl_xor_sync(0xffffffffu, hi[k], off));
      lo_inv[k] = max(lo_inv[k], __shfl_xor_sync(0xffffffffu, lo_inv[k], off));
    }
    if ((threadIdx.x & 31) == 0) {
      if (hi[k]) atomicMax(range + 2 * k, hi[k]);
      if (lo_inv[k]) atomicMax(range + 2 * k + 1, lo_inv[k]);
    }
  }
}

// Monotone DEcreasing in x: bins 0 .. n_bins - 1 for numbers (+inf in the first, -inf in the last); the caller
// sends NaN elsewhere. Large values come first, so the dominators of a row lie AFTER it.
__device__ __forceinline__ int value_bin(float x, const unsigned* range, int n_bins) {
  const float lo = range_value(~range[1]), hi = range_value(range[0]);
  const float t = (x - lo) * ((float)n_bins / (hi - lo));
  const int up = t >= (float)n_bins ? n_bins - 1 : (t >= 0.f ? (int)t : 0);  // a NaN t (empty or zero range): 0
  return n_bins - 1 - up;
}
__device__ __forceinline__ int f1_bin(float x, const unsigned* range) { return (x != x) ? kBins : value_bin(x, range, kBins); }

// Position of a row in the matrix order: `groups` bands of descending first objective (unions of its kBins value
// bins holding about the same number of rows: group_of_bin), and inside a band kBins / groups bins of descending
// second objective. Rows with a NaN in either go last (bin kBins). With one objective: its value bin.
__device__ __forceinline__ int order_key(const float* __restrict__ row, int m, const unsigned* range, const int* __restrict__ group_of_bin,
                                         int groups) {
  const float x0 = row[0];
  if (x0 != x0) return kBins;
  if (m < 2) return value_bin(x0, range, kBins);
  const float x1 = row[1];
  if (x1 != x1) return kBins;
  const int per = kBins / groups;
  return group_of_bin[value_bin(x0, range, kBins)] * per + value_bin(x1, range + 2, per);
}

__global__ void nds_bin_count_kernel(const float* __restrict__ f, long long n, int m, const unsigned* __restrict__ range,
                                     int* __restrict__ counts) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    atomicAdd(counts + f1_bin(f[i * m], range), 1);
}

// One block of 1024 threads: counts of the first objective's value bins -> the band each bin belongs to
// (bands of about equal row counts, in place).
__global__ void __launch_bounds__(1024) nds_group_kernel(int* __restrict__ counts, int groups) {
  static_assert(kBins == 4096, "four bins per thread");
  __shared__ int s_tot[1024];
  const int t = threadIdx.x;
  int c[4], sum = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    c[q] = counts[t * 4 + q];
    sum += c[q];
  }
  s_tot[t] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int v = t >= off ? s_tot[t - off] : 0;
    __syncthreads();
    s_tot[t] += v;
    __syncthreads();
  }
  const long long total = s_tot[1023];
  long long run = s_tot[t] - sum;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const long long g = total > 0 ? run * groups / total : 0;
    counts[t * 4 + q] = (int)(g < groups ? g : groups - 1);
    run += c[q];
  }
}

__global__ void nds_key_count_kernel(const float* __restrict__ f, long long n, int m, const unsigned* __restrict__ range,
                                     const int* __restrict__ group_of_bin, int groups, int* __restrict__ counts) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    atomicAdd(counts + order_key(f + i * m, m, range, group_of_bin, groups), 1);
}

// One block of 1024 threads: counts[0 .. kBins] -> exclusive offsets, copied to the scatter's cursors.
__global__ void __launch_bounds__(1024) nds_bin_scan_kernel(int* __restrict__ counts, int* __restrict__ cursor) {
  static_assert(kBins == 4096, "four bins per thread");
  __shared__ int s_tot[1024];
  const int t = threadIdx.x;
  int c[4], sum = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    c[q] = counts[t * 4 + q];
    sum += c[q];
  }
  s_tot[t] = sum;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int v = t >= off ? s_tot[t - off] : 0;
    __syncthreads();
    s_tot[t] += v;
    __syncthreads();
  }
  int run = s_tot[t] - sum;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    cursor[t * 4 + q] = run;
    run += c[q];
  }
  if (t == 1023) cursor[kBins] = run;  // the NaN rows come last
}

__global__ void nds_bin_scatter_kernel(const float* __restrict__ f, long long n, int m, const unsigned* __restrict__ range,
                                       const int* __restrict__ group_of_bin, int groups, int* __restrict__ cursor,
                                       uint32_t* __restrict__ perm) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    perm[atomicAdd(cursor + order_key(f + i * m, m, range, group_of_bin, groups), 1)] = (uint32_t)i;
}

// i dominates j: all(f_i <= f_j) and any(f_i < f_j) (non_dominate.py:20-24).
template <int M>
__device__ __forceinline__ bool dominates(const float (&a)[M], const float (&b)[M]) {
  bool le = true, lt = false;
#pragma unroll
  for (int k = 0; k < M; ++k) {
    le = le && (a[k] <= b[k]);
    lt = lt || (a[k] < b[k]);
  }
  return le && lt;
}

// Both directions of one pair from 2 m comparisons: with A = all(a <= b) and B = all(b <= a),
// "a dominates b" = A and not B, "b dominates a" = B and not A. (A and B both true means a == b; a
// NaN in either vector makes both false, so neither dominates, as in the reference.)
template <int M>
__device__ __forceinline__ void dominates_both(const float (&a)[M], const float (&b)[M], bool& a_dom_b, bool& b_dom_a) {
  bool ab = true, ba = true;
#pragma unroll
  for (int k = 0; k < M; ++k) {
    ab = ab && (a[k] <= b[k]);
    ba = ba && (b[k] <= a[k]);
  }
  a_dom_b = ab && !ba;
  b_dom_a = ba && !ab;
}

// Per block of kTileJ consecutive positions of the matrix order: minimum and maximum of the first two objectives
// and whether a NaN (or a padding position) is among them: stats[blk] = {min0, max0, min1, max1, bad}.
__global__ void __launch_bounds__(kTileJ) nds_tile_stats_kernel(const float* __restrict__ fs, long long npad, long long n, int m,
                                                                float* __restrict__ stats) {
  const long long p = (long long)blockIdx.x * kTileJ + threadIdx.x;
  float v[2];
  int bad = 0;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    v[k] = (k < m && p < npad) ? fs[(long long)k * npad + p] : (k < m ? __int_as_float(0x7fc00000) : 0.0f);
    bad |= (v[k] != v[k]);
  }
  bad |= (p >= n);
  float st[4] = {v[0], -v[0], v[1], -v[1]};  // minima of x and of -x; fminf skips the NaNs that `bad` reports
  __shared__ float s_st[kTileJ / 32][4];
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 4; ++q) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) st[q] = fminf(st[q], __shfl_xor_sync(0xffffffffu, st[q], off));
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(&s_bad, 1);
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) s_st[threadIdx.x >> 5][q] = st[q];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float r = s_st[0][q];
      for (int w = 1; w < kTileJ / 32; ++w) r = fminf(r, s_st[w][q]);
      st[q] = r;
    }
    float* o = stats + (size_t)blockIdx.x * 5;
    o[0] = st[0], o[1] = -st[1], o[2] = st[2], o[3] = -st[3], o[4] = s_bad ? 1.0f : 0.0f;
  }
}

// Words of "column j dominates row i" for a tile whose columns lie strictly below its rows in one objective:
// the comparison all(f_j[k] <= f_i[k]) runs over the objectives k in CMP only (a compile-time bit set).
template <int M, int R, unsigned CMP>
__device__ __forceinline__ void separated_words(const float (&fi)[R][M], const float (*sfj)[kTileJ], uint32_t (*sback)[32 * 8 * R + 1],
                                                int warp, int lane) {
#pragma unroll 1
  for (int jw = 0; jw < kTileJ / 32; ++jw) {
    uint32_t back[R];
#pragma unroll
    for (int r = 0; r < R; ++r) back[r] = 0u;
#pragma unroll
    for (int jb = 0; jb < 32; ++jb) {
      float fj[M];
#pragma unroll
      for (int k = 0; k < M; ++k)
        if ((CMP >> k) & 1u) fj[k] = sfj[k][jw * 32 + jb];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        bool le = true;
#pragma unroll
        for (int k = 0; k < M; ++k)
          if ((CMP >> k) & 1u) le = le && (fj[k] <= fi[r][k]);
        if (le) back[r] |= 1u << jb;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) sback[jw][(warp * R + r) * 32 + lane] = back[r];
  }
}

// One block = (32 * 8 * R dominators i) x (128 columns j). Blocks whose columns all lie AFTER their
// dominators compute both directions of every pair at once and also emit the transposed bits
// (row i, bits j); blocks whose columns all lie BEFORE their dominators have nothing left to do;
// the blocks on the diagonal band compute the forward direction only, as every block used to.
// `ordered` != 0 (rows dealt by their first objective, largest first): a block above the band first
// compares the smallest first objective of its rows i with the largest one of its columns j; when the
// latter is strictly smaller (and no NaN is involved) no i can dominate a j — zero words for the forward
// direction — and "j dominates i" is all(f_j[k] <= f_i[k]) over the OTHER objectives: m - 1 comparisons
// per pair instead of 2 m.
template <int M, int R>
__global__ void __launch_bounds__(kThreads)
    nds_dominance_kernel(const float* __restrict__ fs, long long npad, long long n, uint32_t* __restrict__ Dt, int wp,
                         const float* __restrict__ stats, long long s_begin, long long s_end) {
  constexpr int kWords = 8 * R;         // words of dominators per block (8 warps x R)
  constexpr int kRows = 32 * kWords;    // dominators per block
  __shared__ float sfj[M][kTileJ];
  __shared__ uint32_t sout[kTileJ][kWords];
  __shared__ uint32_t sback[kTileJ / 32][kRows + 1];  // transposed direction: [word of j][dominator i]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long i0 = (long long)blockIdx.y * kRows;
  const long long j0 = (long long)blockIdx.x * kTileJ;
  if (j0 + kTileJ <= i0) return;              // covered by the transposed output of the mirrored block
  const bool both = j0 >= i0 + kRows;         // every column index exceeds every dominator index
  // Only rows [s_begin, s_end) of the matrix are kept (all of them unless the matrix is split over several GPUs;
  // the bounds are multiples of the tile sizes): the forward words belong to the rows j, the mirrored ones to the rows i.
  const bool keep_fwd = j0 >= s_begin && j0 < s_end;
  const bool keep_back = both && i0 >= s_begin && i0 < s_end;
  if (!keep_fwd && !keep_back) return;

  // Tile classes (block-uniform), decided from the ranges of the first two objectives over the tile's rows and
  // columns (`stats`, one entry per kTileJ positions; nullptr: every tile is kFull). kFull: every comparison. The
  // others need one of the first two objectives, s, in which every column lies strictly below every row: then no
  // row dominates a column (zero forward words) and column j dominates row i iff f_j <= f_i in every OTHER
  // objective. In the other one of the first two, t: columns all above the rows -> nobody dominates anybody
  // (kZero); columns all at or below -> t needs no comparison either (kSkip01); otherwise t is compared (kSkip0
  // for s = 0, kSkip1 for s = 1). A NaN or a padding position anywhere in the tile: kFull.
  enum { kFull, kZero, kSkip0, kSkip1, kSkip01 };
  int tile_class = kFull;
  if (stats != nullptr && both) {
    constexpr int kObj = M >= 2 ? 2 : 1;
    constexpr int kBlocksI = kRows / kTileJ;
    float imin0 = INFINITY, imax0 = -INFINITY, imin1 = INFINITY, imax1 = -INFINITY, bad = 0.0f;
#pragma unroll
    for (int b = 0; b < kBlocksI; ++b) {
      const float* st = stats + (size_t)(i0 / kTileJ + b) * 5;
      imin0 = fminf(imin0, __ldg(st)), imax0 = fmaxf(imax0, __ldg(st + 1));
      imin1 = fminf(imin1, __ldg(st + 2)), imax1 = fmaxf(imax1, __ldg(st + 3));
      bad += __ldg(st + 4);
    }
    const float* sj = stats + (size_t)(j0 / kTileJ) * 5;
    const float jmin0 = __ldg(sj), jmax0 = __ldg(sj + 1), jmin1 = __ldg(sj + 2), jmax1 = __ldg(sj + 3);
    bad += __ldg(sj + 4);
    if (bad == 0.0f) {
      if (jmax0 < imin0) {
        tile_class = (kObj == 2 && jmin1 > imax1) ? kZero : ((kObj == 2 && jmax1 <= imin1) ? kSkip01 : kSkip0);
      } else if (kObj == 2 && jmax1 < imin1) {
        tile_class = (jmin0 > imax0) ? kZero : ((jmax0 <= imin0) ? kSkip01 : kSkip1);
      }
    }
  }
  const int w0 = (int)(i0 >> 5);
  if (tile_class == kZero) {
    // nothing to compare: the tile's words in both directions are zero
    if (keep_fwd) {
      for (int t = threadIdx.x; t < kTileJ * kWords; t += kThreads) {
        const int jj = t / kWords, w = t - jj * kWords;
        const long long j = j0 + jj;
        if (j < n && w0 + w < wp) Dt[(j - s_begin) * wp + w0 + w] = 0u;
      }
    }
    if (keep_back) {
      const int wj = (int)(j0 >> 5);
      for (int il = threadIdx.x; il < kRows; il += kThreads) {
        const long long i = i0 + il;
        if (i < n && wj + 3 < wp) *reinterpret_cast<uint4*>(Dt + (i - s_begin) * wp + wj) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }

  float fi[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const long long i = i0 + (long long)(warp * R + r) * 32 + lane;
#pragma unroll
    for (int k = 0; k < M; ++k) fi[r][k] = (i < npad) ? fs[(long long)k * npad + i] : __int_as_float(0x7fc00000);
  }
  for (int t = threadIdx.x; t < M * kTileJ; t += kThreads) {
    const int k = t / kTileJ, jj = t - k * kTileJ;
    const long long j = j0 + jj;
    sfj[k][jj] = (j < n) ? fs[(long long)k * npad + j] : __int_as_float(0x7fc00000);
  }
  __syncthreads();
  const bool separated = tile_class != kFull;
  if (separated) {
    // 32 columns per word with the bit position known at compile time: the comparisons of the class and one
    // predicated OR per pair
    if (tile_class == kSkip0) {
      separated_words<M, R, ((1u << M) - 1u) & ~1u>(fi, sfj, sback, warp, lane);
    } else if (tile_class == kSkip1) {
      separated_words<M, R, ((1u << M) - 1u) & ~2u>(fi, sfj, sback, warp, lane);
    } else {
      separated_words<M, R, ((1u << M) - 1u) & ~3u>(fi, sfj, sback, warp, lane);
    }
  } else if (!both) {
#pragma unroll 4
    for (int jj = 0; jj < kTileJ; ++jj) {
      float fj[M];
#pragma unroll
      for (int k = 0; k < M; ++k) fj[k] = sfj[k][jj];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t word = __ballot_sync(0xffffffffu, dominates<M>(fi[r], fj));
        if (lane == 0) sout[jj][warp * R + r] = word;
      }
    }
  } else {
    uint32_t back[R];
#pragma unroll
    for (int r = 0; r < R; ++r) back[r] = 0u;
#pragma unroll 4
    for (int jj = 0; jj < kTileJ; ++jj) {
      float fj[M];
#pragma unroll
      for (int k = 0; k < M; ++k) fj[k] = sfj[k][jj];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        bool fwd, bwd;
        dominates_both<M>(fi[r], fj, fwd, bwd);
        const uint32_t word = __ballot_sync(0xffffffffu, fwd);
        if (lane == 0) sout[jj][warp * R + r] = word;
        back[r] |= (uint32_t)bwd << (jj & 31);
      }
      if ((jj & 31) == 31) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          sback[jj >> 5][(warp * R + r) * 32 + lane] = back[r];
          back[r] = 0u;
        }
      }
    }
  }
  __syncthreads();
  if (keep_fwd) {
    for (int t = threadIdx.x; t < kTileJ * kWords; t += kThreads) {
      const int jj = t / kWords, w = t - jj * kWords;
      const long long j = j0 + jj;
      if (j < n && w0 + w < wp) Dt[(j - s_begin) * wp + w0 + w] = separated ? 0u : sout[jj][w];
    }
  }
  if (keep_back) {
    // row i of Dt, the four words that hold columns j0 .. j0 + 127 (16-byte aligned: j0 is a multiple of 128)
    const int wj = (int)(j0 >> 5);
    for (int il = threadIdx.x; il < kRows; il += kThreads) {
      const long long i = i0 + il;
      if (i < n && wj + 3 < wp) {
        *reinterpret_cast<uint4*>(Dt + (i - s_begin) * wp + wj) = make_uint4(sback[0][il], sback[1][il], sback[2][il], sback[3][il]);
      }
    }
  }
}

// Generic number of objectives (slow path, > 16): one thread per (word, column).
__global__ void __launch_bounds__(kThreads)
    nds_dominance_generic_kernel(const float* __restrict__ fs, long long npad, long long n, int m,
                                 uint32_t* __restrict__ Dt, int wp) {
  const long long total = n * (long long)wp;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long j = t / wp;
    const int w = (int)(t - j * wp);
    uint32_t word = 0;
    for (int b = 0; b < 32; ++b) {
      const long long i = (long long)w * 32 + b;
      bool le = true, lt = false;
      for (int k = 0; k < m; ++k) {
        const float a = fs[(long long)k * npad + i], c = fs[(long long)k * npad + j];
        le = le && (a <= c);
        lt = lt || (a < c);
      }
      word |= (uint32_t)(le && lt) << b;
    }
    Dt[t] = word;
  }
}

// `bin_end` (optional, with `fs` = the objectives in matrix order, structure of arrays with row length npad, and
// the tables of the row order): bin_end[b] is one past the last position of order bin b. Every dominator of a
// column is no larger in the first AND in the second objective, so it lies in the column's own bin or a later
// one: the column's scan starts at its bin's first word.
__global__ void nds_peel_init_kernel(long long n, int wp, uint32_t* unranked, uint32_t* unranked_alt, int* ptr, int* rank,
                                     Ctrl* ctrl, const float* __restrict__ fs, long long npad, int m,
                                     const unsigned* __restrict__ range, const int* __restrict__ group_of_bin, int groups,
                                     const int* __restrict__ bin_end, int tail_rows) {
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = t0; w < wp; w += stride) {
    const long long lo = w * 32;
    uint32_t bits = 0;
    if (lo + 32 <= n) bits = 0xffffffffu;
    else if (lo < n) bits = (1u << (int)(n - lo)) - 1u;
    unranked[w] = bits;
    unranked_alt[w] = bits;
  }
  for (long long j = t0; j < n; j += stride) {
    int start = 0;
    if (bin_end) {
      const float key[2] = {fs[j], m >= 2 ? fs[npad + j] : 0.0f};
      const int b = order_key(key, m, range, group_of_bin, groups);
      start = b ? bin_end[b - 1] : 0;
    }
    ptr[j] = start >> 5;
    rank[j] = -1;
  }
  if (t0 == 0) {
    ctrl->bar_word = 0ull;
    ctrl->release_word = 0ull;
    ctrl->status = 0;
    ctrl->n_fronts = 0;
    ctrl->tail_rows = tail_rows;  // n when the cluster kernel peels everything, 0 until the grid kernel hands over
    ctrl->tail_k0 = 0;
    ctrl->tail_buf = 0;
  }
}

// Grid-wide barrier number `number` (1, 2, ...) of a cooperative (co-resident) launch, which also adds up
// `mine` (the rows this block ranked in the pass) over the grid: the sum comes back in *total. The
// wait is bounded: a block that polls kSpinLimit times records status 1 and every block leaves at its
// next check. Thread 0 makes three dependent trips to memory per barrier (release fence, arrival
// atomic, the poll that sees the release); the barrier number is known to every block, the sum rides
// on the arrival word and comes back with the release word, and a failed wait shows in the same word.
__device__ __forceinline__ bool grid_barrier_sum(Ctrl* ctrl, unsigned n_blocks, unsigned number, unsigned mine, unsigned* total) {
  __shared__ int ok;
  __shared__ unsigned s_total;
  if (threadIdx.x == 0) {
    constexpr unsigned long long kFailed = 1ull << 63;
    volatile unsigned long long* rel_p = &ctrl->release_word;
    __threadfence();
    const unsigned long long old = atomicAdd(&ctrl->bar_word, 1ull | ((unsigned long long)mine << 32));
    bool good = true;
    if ((unsigned)(old & 0xffffffffull) + 1u == n_blocks) {
      const unsigned sum = (unsigned)(old >> 32) + mine;
      ctrl->bar_word = 0ull;
      __threadfence();
      // keeps a failure flag that a block which gave up may have set meanwhile
      const unsigned long long before = atomicMax(&ctrl->release_word, ((unsigned long long)number << 32) | sum);
      good = !(before & kFailed);
      s_total = sum;
    } else {
      unsigned spins = 0;
      for (;;) {
        const unsigned long long w = *rel_p;
        if (w & kFailed) {
          good = false;
          break;
        }
        if ((unsigned)(w >> 32) == number) {
          s_total = (unsigned)w;
          break;
        }
        __nanosleep(32);
        if (++spins > kSpinLimit) {
          atomicExch(&ctrl->status, 1);
          atomicOr(&ctrl->release_word, kFailed);
          good = false;
          break;
        }
      }
    }
    __threadfence();
    ok = good;
  }
  __syncthreads();
  *total = s_total;
  return ok != 0;
}

// The mask snapshot lives in shared memory when it fits; otherwise it is read from L2 (never
// through L1, which may hold the same buffer's contents of two passes ago).
__device__ __forceinline__ uint32_t mask_word(const uint32_t* m, int i, int in_smem) {
  return in_smem ? m[i] : __ldcg(m + i);
}
__device__ __forceinline__ uint4 mask_quad(const uint32_t* m, int i, int in_smem) {
  return in_smem ? *reinterpret_cast<const uint4*>(m + i) : __ldcg(reinterpret_cast<const uint4*>(m + i));
}

__device__ __forceinline__ int first_nonzero(const uint4& v) {
  return v.x ? 0 : (v.y ? 1 : (v.z ? 2 : (v.w ? 3 : -1)));
}

// Front k = unranked columns j whose row of Dt has no bit left under the unranked mask U.
// A warp owns 32 consecutive columns (one word of U). Two copies of U alternate: pass k reads
// U[k & 1] as a snapshot and the owner of a word writes its successor into U[(k + 1) & 1], so one
// grid barrier per front is enough and no atomics touch the masks. Each lane first re-tests its
// column's witness word (where the last scan stopped); only columns whose witness cleared are
// scanned on, and never backwards: over all fronts a row of Dt is read once. Measured per front at
// 100,000 rows: about 1.4 us for the barrier itself, the rest is the slowest block's scans (late fronts:
// few unranked rows are left, so the next unranked dominator of a column is far away).
template <int kPeelThreads, bool kMaskInSmem>
__global__ void __launch_bounds__(kPeelThreads)
    nds_peel_kernel(const uint32_t* __restrict__ Dt, int wp, long long n, uint32_t* U0, uint32_t* U1, int* ptr,
                    int* rank, Ctrl* ctrl, int, const uint32_t* __restrict__ perm, int tail_limit) {
  constexpr int mask_in_smem = kMaskInSmem ? 1 : 0;  // a template argument: the mask is read inside every hot loop
  extern __shared__ __align__(16) uint32_t s_mask[];
  __shared__ unsigned s_cnt[kPeelThreads / 32];
  __shared__ unsigned s_newly[kPeelThreads / 32];  // per owning warp: columns ranked in this trip
  __shared__ long long s_qj[kPeelThreads];         // block queue of columns waiting for a warp-wide scan
  __shared__ int s_qc[kPeelThreads];
  __shared__ unsigned short s_qowner[kPeelThreads];
  __shared__ int s_found[kPeelThreads];            // per owning thread: where its queued column's scan stopped
  __shared__ int s_qn;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // Words of 32 columns are dealt to the blocks first and to a block's warps second (word = block +
  // blocks * (warp + 8 * trip)): with fewer words than warps every block still owns some, and its
  // other warps help with the block's queue of long scans.
  const long long n_warps = ((long long)gridDim.x * kPeelThreads) >> 5;
  const long long n_words = (n + 31) >> 5;
  long long remaining = n;
  const long long trips = (n_words + n_warps - 1) / n_warps;  // the same for every warp: the block synchronises inside
  const bool single_trip = trips == 1;
  int c_reg = 0;
  if (single_trip) {
    const long long j0 = ((long long)blockIdx.x + (long long)gridDim.x * warp) * 32 + lane;
    if (j0 < n) c_reg = ptr[j0];
  }

  for (int k = 0; k <= n; ++k) {
    const uint32_t* R = (k & 1) ? U1 : U0;
    uint32_t* W = (k & 1) ? U0 : U1;
    // this pass's snapshot of the unranked mask, staged in shared memory when it fits
    const uint32_t* Rs = R;
    if (mask_in_smem) {
      for (int w = threadIdx.x * 4; w < wp; w += kPeelThreads * 4)
        *reinterpret_cast<uint4*>(s_mask + w) = __ldcg(reinterpret_cast<const uint4*>(R + w));
      __syncthreads();
      Rs = s_mask;
    }
    unsigned ranked_here = 0;
    for (long long trip = 0; trip < trips; ++trip) {
      const long long wj = (long long)blockIdx.x + (long long)gridDim.x * (warp + (kPeelThreads / 32) * trip);
      const bool have = wj < n_words;
      if (threadIdx.x == 0) s_qn = 0;
      if (lane == 0) s_newly[warp] = 0u;
      __syncthreads();
      const uint32_t own = have ? mask_word(Rs, (int)wj, mask_in_smem) : 0u;
      const long long j = wj * 32 + lane;
      const bool open = (own >> lane) & 1u;  // this lane's column is still unranked
      // One memory round trip settles most columns: a lane reads 32 words of its own row from its
      // witness position on (eight independent 128-bit loads; the witness word is among them) and takes the
      // first word that still holds an unranked dominator as the new witness. When every word of a
      // block's warps is visited once per front (one trip), the witness position lives in a register
      // and is not re-read from memory. Columns with nothing in those 32 words are queued for the block:
      // the warp-wide scans of a front's new members would otherwise pile up in the warps that own them.
      int c = 0;
      bool queued = false;
      if (open) {
        c = single_trip ? c_reg : __ldcg(ptr + j);
        const int c4 = c & ~3;
        const uint4* row4 = reinterpret_cast<const uint4*>(Dt + j * wp);
        uint4 d[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int w = c4 + q * 4;
          d[q] = (w < wp) ? __ldg(row4 + (w >> 2)) : make_uint4(0, 0, 0, 0);
        }
        int hit = -1;
#pragma unroll
        for (int q = 7; q >= 0; --q) {
          const int w = c4 + q * 4;
          if (w < wp) {
            const uint4 u = mask_quad(Rs, w, mask_in_smem);
            const int f = first_nonzero(make_uint4(d[q].x & u.x, d[q].y & u.y, d[q].z & u.z, d[q].w & u.w));
            if (f >= 0) hit = w + f;
          }
        }
        if (hit >= 0) {
          if (hit != c) {
            ptr[j] = hit;
            c_reg = hit;
          }
        } else {
          const int slot = atomicAdd(&s_qn, 1);
          s_qj[slot] = j;
          s_qc[slot] = min(c4 + 32, wp - 1);  // nothing up to here: the scan may skip these words
          s_qowner[slot] = (unsigned short)threadIdx.x;
          queued = true;
        }
      }
      __syncthreads();
      const int qn = s_qn;
      for (int item = warp; item < qn; item += kPeelThreads / 32) {
        const long long jl = s_qj[item];
        const int cl = s_qc[item];
        const uint4* row4 = reinterpret_cast<const uint4*>(Dt + jl * wp);
        int found = -1;
        // 1024 words per step: eight independent 128-bit loads per lane are in flight together. (Issuing the
        // next step's loads before examining this one was measured slower: more registers, same waits.)
        for (int base = (cl & ~1023); base < wp && found < 0; base += 1024) {
          uint4 d[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int w = base + q * 128 + lane * 4;
            d[q] = (w < wp && w + 4 > cl) ? __ldg(row4 + (w >> 2)) : make_uint4(0, 0, 0, 0);  // words before cl are done
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int w = base + q * 128 + lane * 4;
            int f = -1;
            if (w < wp) {
              const uint4 u = mask_quad(Rs, w, mask_in_smem);
              f = first_nonzero(make_uint4(d[q].x & u.x, d[q].y & u.y, d[q].z & u.z, d[q].w & u.w));
            }
            const unsigned m = __ballot_sync(0xffffffffu, f >= 0);
            if (m && found < 0) {
              const int src = __ffs(m) - 1;
              found = base + q * 128 + src * 4 + __shfl_sync(0xffffffffu, f, src);
            }
          }
        }
        if (lane == 0) {
          s_found[s_qowner[item]] = found;
          if (found >= 0) {
            ptr[jl] = found;
          } else {
            const unsigned owner = s_qowner[item];
            atomicOr(&s_newly[owner >> 5], 1u << (owner & 31));
            rank[perm ? (long long)perm[jl] : jl] = k;  // column jl of the matrix is row perm[jl]
          }
        }
      }
      __syncthreads();
      if (queued && s_found[threadIdx.x] >= 0) c_reg = s_found[threadIdx.x];
      const unsigned newly = s_newly[warp];
      if (lane == 0 && have) W[wj] = own & ~newly;
      ranked_here += __popc(newly);
    }
    if (lane == 0) s_cnt[threadIdx.x >> 5] = ranked_here;
    __syncthreads();
    unsigned tot = 0;
    if (threadIdx.x == 0) {
      for (int i = 0; i < kPeelThreads / 32; ++i) tot += s_cnt[i];
    }
    unsigned got = 0;
    if (!grid_barrier_sum(ctrl, gridDim.x, (unsigned)k + 1u, tot, &got)) return;
    remaining -= got;
    if (remaining <= 0) {
      if (blockIdx.x == 0 && threadIdx.x == 0) ctrl->n_fronts = k + 1;
      return;
    }
    if (got == 0) {  // dominance is a strict partial order: every pass must rank someone
      if (blockIdx.x == 0 && threadIdx.x == 0) atomicExch(&ctrl->status, 2);
      return;
    }
    if (remaining <= tail_limit) {  // few rows left: the cluster kernel finishes them without grid barriers
      if (blockIdx.x == 0 && threadIdx.x == 0) {
        ctrl->tail_rows = (int)remaining;
        ctrl->tail_k0 = k + 1;
        ctrl->tail_buf = (k + 1) & 1;
        ctrl->n_fronts = k + 1;
      }
      return;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Hand-over to the cluster kernel: the rows still unranked, in matrix order, and their sub-matrix.
// ---------------------------------------------------------------------------------------------
// One block: ids[a] = position of the a-th set bit of the unranked mask.
__global__ void __launch_bounds__(1024) nds_tail_ids_kernel(const uint32_t* U0, const uint32_t* U1, int wp, const Ctrl* ctrl,
                                                            uint32_t* __restrict__ ids) {
  if (ctrl->tail_rows <= 0 || ctrl->status != 0) return;
  const uint32_t* U = ctrl->tail_buf ? U1 : U0;
  __shared__ int s_scan[1024];
  __shared__ int s_base;
  const int t = threadIdx.x;
  if (t == 0) s_base = 0;
  __syncthreads();
  for (int w0 = 0; w0 < wp; w0 += 1024) {
    const int w = w0 + t;
    uint32_t bits = w < wp ? U[w] : 0u;
    const int cnt = __popc(bits);
    s_scan[t] = cnt;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int v = t >= off ? s_scan[t - off] : 0;
      __syncthreads();
      s_scan[t] += v;
      __syncthreads();
    }
    int at_ = s_base + s_scan[t] - cnt;
    while (bits) {
      const int b = __ffs(bits) - 1;
      bits &= bits - 1;
      if (at_ < kTailCompactRows) ids[at_] = (uint32_t)(w * 32 + b);
      ++at_;
    }
    __syncthreads();
    if (t == 1023) s_base += s_scan[1023];
    __syncthreads();
  }
}

// sub[a][b] = bit ids[b] of row ids[a] of the matrix (does ids[b] dominate ids[a]?), rows of
// kTailCompactRows / 32 words. A warp builds a row: lane l fetches bit b = 32 * i + l, a ballot makes word i,
// lane i keeps it, and every 32 words leave as one 128-byte store.
__global__ void __launch_bounds__(256) nds_tail_gather_kernel(const uint32_t* __restrict__ Dt, int wp, const Ctrl* ctrl,
                                                              const uint32_t* __restrict__ ids, uint32_t* __restrict__ sub) {
  const int T = ctrl->tail_rows;
  if (T <= 0 || ctrl->status != 0) return;
  constexpr int kSubWords = kTailCompactRows / 32;
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  const int words = (T + 31) >> 5;
  for (int a = warp; a < T; a += n_warps) {
    const uint32_t* row = Dt + (size_t)ids[a] * (size_t)wp;
    uint32_t* out = sub + (size_t)a * kSubWords;
    for (int w0 = 0; w0 < words; w0 += 32) {
      uint32_t mine = 0u;
#pragma unroll 4
      for (int i = 0; i < 32; ++i) {
        const int b = (w0 + i) * 32 + lane;
        bool bit = false;
        if (b < T) {
          const uint32_t id = __ldg(ids + b);
          bit = (__ldg(row + (id >> 5)) >> (id & 31u)) & 1u;
        }
        const uint32_t word = __ballot_sync(0xffffffffu, bit);
        if (lane == i) mine = word;
      }
      if (w0 + lane < kSubWords) out[w0 + lane] = mine;  // whole 128-byte groups: the words past `words` are zero
    }
  }
}

__device__ __forceinline__ int tail_first_nonzero(const uint4& v) {
  return v.x ? 0 : (v.y ? 1 : (v.z ? 2 : (v.w ? 3 : -1)));
}
__device__ __forceinline__ uint4 and4(const uint4& a, const uint4& b) { return make_uint4(a.x & b.x, a.y & b.y, a.z & b.z, a.w & b.w); }

// Front peeling by one cluster of kTailCtas blocks over T <= kTailDirectMaxN columns: the whole matrix of a small
// population (ids == nullptr: compact column a is matrix column a, row stride wp) or the compacted sub-matrix of
// the rows a large population still has unranked. Same rule as nds_peel_kernel — a column joins front k when no
// unranked dominator is left in its row, found by re-testing a witness word and scanning the row when the
// witness has left — but every block keeps the whole mask in shared memory, a warp owns one word of 32 columns,
// the successor of that word is stored into every block's copy of the next mask through distributed shared
// memory, and fronts are separated by the cluster's hardware barrier: no polling, so nothing here can wait
// forever. A row is at most 256 words: the warp scans four rows per round trip (two 16-byte loads per lane and row).
// The front loop is bounded by T passes (a strict partial order ranks at least one column per pass).
__global__ void __cluster_dims__(kTailCtas, 1, 1) __launch_bounds__(kTailThreads)
    nds_peel_tail_kernel(const uint32_t* __restrict__ rows, int stride, const uint32_t* __restrict__ ids,
                         const uint32_t* __restrict__ perm, int* __restrict__ rank, Ctrl* ctrl) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ __align__(16) uint32_t s_mask[2][kTailMaxWords];
  const int T = ctrl->tail_rows;
  if (T <= 0 || T > kTailDirectMaxN || ctrl->status != 0) return;  // the same answer in every block of the cluster
  const int k0 = ctrl->tail_k0;
  const int words = (T + 31) >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = (int)cluster.block_rank() * (kTailThreads / 32) + warp;  // the word of 32 columns this warp owns
  for (int i = threadIdx.x; i < kTailMaxWords; i += kTailThreads) {
    uint32_t bits = 0u;
    if (i * 32 + 32 <= T) bits = 0xffffffffu;
    else if (i * 32 < T) bits = (1u << (T - i * 32)) - 1u;
    s_mask[0][i] = bits;
    s_mask[1][i] = 0u;
  }
  cluster.sync();  // every block's masks exist before anyone stores into them
  const int a = w * 32 + lane;                       // this lane's column
  const bool have = w < words;                       // warp-uniform
  const uint32_t* my_row = rows + (size_t)(have ? a : 0) * stride;
  // where this column's rank goes: compact column -> column of the matrix -> row of the caller's table
  uint32_t dst = 0u;
  if (have && a < T) {
    dst = ids ? ids[a] : (uint32_t)a;
    if (perm) dst = perm[dst];
  }
  // which 16-byte groups of a row exist: words [0, 128) and [128, 256), four per lane
  const bool lo_ok = lane * 4 < words, hi_ok = 128 + lane * 4 < words;
  int wit = 0;
  bool done = false;
  int k = 0;
  for (; k < T && !done; ++k) {
    const uint32_t* M = s_mask[k & 1];
    uint32_t* next_local = s_mask[(k + 1) & 1];
    if (have) {
      const uint32_t own = M[w];
      const bool open = (own >> lane) & 1u;
      bool cleared = false;
      if (open) cleared = (__ldg(my_row + wit) & M[wit]) == 0u;
      unsigned todo = __ballot_sync(0xffffffffu, cleared);
      uint32_t newly = 0u;
      if (todo) {
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const uint4 m_lo = lo_ok ? *reinterpret_cast<const uint4*>(M + lane * 4) : zero;
        const uint4 m_hi = hi_ok ? *reinterpret_cast<const uint4*>(M + 128 + lane * 4) : zero;
        while (todo) {
          int src[4];
          uint4 d_lo[4], d_hi[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            src[i] = todo ? __ffs(todo) - 1 : -1;
            if (todo) todo &= todo - 1;
            const uint4* row4 = reinterpret_cast<const uint4*>(rows + (size_t)(w * 32 + (src[i] < 0 ? 0 : src[i])) * stride);
            d_lo[i] = (src[i] >= 0 && lo_ok) ? __ldg(row4 + lane) : zero;
            d_hi[i] = (src[i] >= 0 && hi_ok) ? __ldg(row4 + 32 + lane) : zero;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (src[i] < 0) continue;  // warp-uniform
            const int f_lo = tail_first_nonzero(and4(d_lo[i], m_lo));
            const int f_hi = tail_first_nonzero(and4(d_hi[i], m_hi));
            const int pos = f_lo >= 0 ? lane * 4 + f_lo : (f_hi >= 0 ? 128 + lane * 4 + f_hi : -1);
            const unsigned hit = __ballot_sync(0xffffffffu, pos >= 0);
            if (hit) {
              const int found = __shfl_sync(0xffffffffu, pos, __ffs(hit) - 1);
              if (lane == src[i]) wit = found;
            } else {
              newly |= 1u << src[i];
            }
          }
        }
      }
      const uint32_t next = own & ~newly;
      if (lane < kTailCtas) *cluster.map_shared_rank(next_local + w, lane) = next;
      if ((newly >> lane) & 1u) rank[dst] = k0 + k;
    }
    cluster.sync();  // release / acquire: the next mask is complete in every block
    const int left = __syncthreads_or(threadIdx.x < kTailMaxWords ? (next_local[threadIdx.x] != 0u) : 0);
    done = left == 0;
  }
  if (cluster.block_rank() == 0 && threadIdx.x == 0) {
    ctrl->n_fronts = k0 + k;
    if (!done) atomicExch(&ctrl->status, 2);
  }
}

// ---------------------------------------------------------------------------------------------
// Stable least-significant-digit radix sort of (key, value) pairs by one thread block.
// 8-bit digits; within a tile of blockDim.x elements the order among equal digits is kept with
// match_any + per-warp digit counts, so equal keys stay in input order (what torch.argsort(stable)
// guarantees). Result ends in (keys, vals); (tk, tv) are scratch.
// ---------------------------------------------------------------------------------------------
struct SortSmem {
  unsigned base[256];
  unsigned tile_total[256];
  unsigned wcnt[kSortThreads / 32][256];
};

__device__ void block_radix_sort(uint32_t* keys, uint32_t* vals, uint32_t* tk, uint32_t* tv, int n, int bits,
                                 SortSmem& sm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  uint32_t *src_k = keys, *src_v = vals, *dst_k = tk, *dst_v = tv;
  const int passes = (bits + 7) / 8;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * 8;
    for (int i = tid; i < 256; i += blockDim.x) sm.base[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) atomicAdd(&sm.base[(src_k[i] >> shift) & 255u], 1u);
    __syncthreads();
    if (warp == 0) {  // exclusive scan of 256 counts by one warp, 8 per lane
      unsigned local[8], sum = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        local[q] = sm.base[lane * 8 + q];
        sum += local[q];
      }
      unsigned incl = sum;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      unsigned run = incl - sum;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        sm.base[lane * 8 + q] = run;
        run += local[q];
      }
    }
    __syncthreads();
    for (int s = 0; s < n; s += blockDim.x) {
      const int i = s + tid;
      const bool valid = i < n;
      uint32_t key = 0, val = 0;
      unsigned dg = 256u + (unsigned)lane;  // invalid lanes match nobody
      if (valid) {
        key = src_k[i];
        val = src_v[i];
        dg = (key >> shift) & 255u;
      }
      for (int q = tid; q < n_warps * 256; q += blockDim.x) (&sm.wcnt[0][0])[q] = 0;
      __syncthreads();
      const unsigned peers = __match_any_sync(0xffffffffu, dg);
      const unsigned before = __popc(peers & ((1u << lane) - 1u));
      if (valid && before == 0) sm.wcnt[warp][dg] = __popc(peers);
      __syncthreads();
      if (tid < 256) {
        unsigned run = 0;
        for (int w = 0; w < n_warps; ++w) {
          const unsigned c = sm.wcnt[w][tid];
          sm.wcnt[w][tid] = run;
          run += c;
        }
        sm.tile_total[tid] = run;
      }
      __syncthreads();
      if (valid) {
        const unsigned dest = sm.base[dg] + sm.wcnt[warp][dg] + before;
        dst_k[dest] = key;
        dst_v[dest] = val;
      }
      __syncthreads();
      if (tid < 256) sm.base[tid] += sm.tile_total[tid];
      __syncthreads();
    }
    uint32_t* t = src_k; src_k = dst_k; dst_k = t;
    t = src_v; src_v = dst_v; dst_v = t;
    __threadfence_block();
    __syncthreads();
  }
  if (src_k != keys) {
    for (int i = tid; i < n; i += blockDim.x) {
      keys[i] = src_k[i];
      vals[i] = src_v[i];
    }
    __syncthreads();
  }
}

// float -> uint32 whose unsigned order is torch's ascending sort order: -inf < ... < -0 = +0 < ...
// < +inf < NaN (all NaNs equal, both zeros equal, so a stable sort keeps their input order).
__device__ __forceinline__ uint32_t float_order_key(float x) {
  if (x != x) return 0xffffffffu;
  if (x == 0.0f) x = 0.0f;
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// ---------------------------------------------------------------------------------------------
// Selection
// ---------------------------------------------------------------------------------------------
__global__ void nds_hist_kernel(const int* __restrict__ rank, long long n, int* hist, const Ctrl* ctrl) {
  if (ctrl->n_fronts <= kRankBuckets) return;  // the counting path serves this population
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = rank[i];
    if (r >= 0 && r <= n) atomicAdd(hist + r, 1);
  }
}

// ---------------------------------------------------------------------------------------------
// Selection, counting path (at most kRankBuckets fronts): lexsort([-crowd, rank])[:topk] needs the rows
// before the last admitted front in (rank, index) order and that front's rows in index order. Both are
// stable bucket placements keyed by rank, done by kRankWarps warps that each own a contiguous range of rows:
//   count  per-warp histogram of the ranks of its rows                       (kRankWarps x fronts table)
//   scan   a warp per rank: exclusive prefix over the row ranges and the rank's total; then one block: prefix
//          of the totals over the ranks and from it the last admitted front
//          (torch.topk(rank, k, largest=False)[0][-1], non_dominate.py:250)
//   place  every warp walks its rows in index order again and writes each to its bucket's next slot.
// No atomics on shared addresses and no sort: two passes over the ranks.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void rank_warp_range(long long n, int gw, long long* begin, long long* end) {
  const long long per = ((n + kRankWarps - 1) / kRankWarps + 31) / 32 * 32;
  *begin = (long long)gw * per;
  *end = *begin + per < n ? *begin + per : n;
}

__global__ void __launch_bounds__(256) nds_rank_count_kernel(const int* __restrict__ rank, long long n, const Ctrl* ctrl,
                                                             int* __restrict__ whist) {
  const int fronts = ctrl->n_fronts;
  if (fronts > kRankBuckets || fronts <= 0) return;
  __shared__ int s_cnt[8][kRankBuckets];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = blockIdx.x * 8 + warp;
  for (int r = lane; r < fronts; r += 32) s_cnt[warp][r] = 0;
  __syncwarp();
  long long begin, end;
  rank_warp_range(n, gw, &begin, &end);
  for (long long i0 = begin; i0 < end; i0 += 32) {
    const long long i = i0 + lane;
    const int r = i < end ? rank[i] : -1;
    const bool in = r >= 0 && r < fronts;
    const unsigned peers = __match_any_sync(0xffffffffu, in ? r : -1 - lane);
    if (in && (peers & ((1u << lane) - 1u)) == 0u) s_cnt[warp][r] += __popc(peers);  // one lane per distinct rank
    __syncwarp();
  }
  for (int r = lane; r < fronts; r += 32) whist[(size_t)r * kRankWarps + gw] = s_cnt[warp][r];  // rank-major: the scan reads a rank's row
}

// One warp per rank: exclusive prefix of the rank's counts over the kRankWarps row ranges (in place) and the
// rank's total.
__global__ void __launch_bounds__(256) nds_rank_scan_kernel(const Ctrl* ctrl, int* __restrict__ whist, int* __restrict__ rank_total) {
  const int fronts = ctrl->n_fronts;
  if (fronts > kRankBuckets || fronts <= 0) return;
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= fronts) return;
  constexpr int kPer = kRankWarps / 32;  // consecutive row ranges per lane
  int* row = whist + (size_t)r * kRankWarps + lane * kPer;
  int c[kPer], sum = 0;
#pragma unroll
  for (int q = 0; q < kPer; ++q) {
    c[q] = row[q];
    sum += c[q];
  }
  int incl = sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += t;
  }
  int run = incl - sum;
#pragma unroll
  for (int q = 0; q < kPer; ++q) {
    row[q] = run;  // rows of this rank owned by earlier ranges
    run += c[q];
  }
  if (lane == 31) rank_total[r] = incl;
}

// One block: prefix of the rank totals over the ranks, and from it the last admitted front: the first rank whose
// inclusive count reaches topk.
__global__ void __launch_bounds__(kRankBuckets) nds_rank_offsets_kernel(long long topk, Ctrl* ctrl, const int* __restrict__ rank_total,
                                                                          int* __restrict__ rank_off) {
  const int fronts = ctrl->n_fronts;
  if (fronts > kRankBuckets || fronts <= 0) return;
  __shared__ int s_scan[kRankBuckets];
  const int r = threadIdx.x;
  if (r == 0) {  // what the selection sees if the ranks are incomplete (a failed rank leaves rows at -1)
    ctrl->worst_rank = 0;
    ctrl->n_before = 0;
    ctrl->n_last = 0;
  }
  const int total = r < fronts ? rank_total[r] : 0;
  s_scan[r] = total;
  __syncthreads();
  for (int off = 1; off < kRankBuckets; off <<= 1) {
    const int v = r >= off ? s_scan[r - off] : 0;
    __syncthreads();
    s_scan[r] += v;
    __syncthreads();
  }
  const int before = s_scan[r] - total;  // rows of better ranks
  if (r < fronts) {
    rank_off[r] = before;
    if ((long long)before < topk && (long long)before + total >= topk) {
      ctrl->worst_rank = r;
      ctrl->n_before = before;
      ctrl->n_last = total;
    }
  }
}

__global__ void __launch_bounds__(256) nds_rank_place_kernel(const int* __restrict__ rank, long long n, const Ctrl* ctrl,
                                                             const int* __restrict__ whist, const int* __restrict__ rank_off,
                                                             uint32_t* __restrict__ order, uint32_t* __restrict__ idx_l) {
  const int fronts = ctrl->n_fronts;
  if (fronts > kRankBuckets || fronts <= 0) return;
  __shared__ int s_cur[8][kRankBuckets];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = blockIdx.x * 8 + warp;
  const int worst = ctrl->worst_rank;
  for (int r = lane; r <= worst; r += 32)
    s_cur[warp][r] = whist[(size_t)r * kRankWarps + gw] + (r < worst ? rank_off[r] : 0);
  __syncwarp();
  long long begin, end;
  rank_warp_range(n, gw, &begin, &end);
  for (long long i0 = begin; i0 < end; i0 += 32) {
    const long long i = i0 + lane;
    const int r = i < end ? rank[i] : -1;
    const bool in = r >= 0 && r <= worst;
    const unsigned peers = __match_any_sync(0xffffffffu, in ? r : -1 - lane);
    const unsigned earlier = __popc(peers & ((1u << lane) - 1u));
    int slot = 0;
    if (in) slot = s_cur[warp][r] + (int)earlier;
    __syncwarp();
    if (in && earlier == 0u) s_cur[warp][r] += __popc(peers);
    __syncwarp();
    if (in) {
      if (r < worst) order[slot] = (uint32_t)i;  // (rank, index) order: these rows are all kept, n_before < topk
      else idx_l[slot] = (uint32_t)i;
    }
  }
}

// One block: k-th smallest rank (torch.topk(rank, k, largest=False)[0][-1], non_dominate.py:250),
// then index-ordered lists of the rows before the last admitted front and of that front.
__global__ void __launch_bounds__(kSortThreads)
    nds_partition_kernel(const int* __restrict__ rank, const int* __restrict__ hist, long long n, long long topk,
                         Ctrl* ctrl, uint32_t* idx_a, uint32_t* key_a, uint32_t* idx_l) {
  __shared__ int s_worst;
  __shared__ unsigned s_worst_u;
  __shared__ unsigned s_wsum[kSortThreads / 32][2];
  __shared__ unsigned s_base[2];
  if (ctrl->n_fronts <= kRankBuckets) return;  // the counting path serves this population
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // smallest r with hist[0] + ... + hist[r] >= topk, found a tile of 1024 ranks at a time
  __shared__ unsigned long long s_run;
  __shared__ unsigned s_scan[kSortThreads / 32];
  if (tid == 0) {
    s_worst = -1;
    s_worst_u = 0xffffffffu;
    s_run = 0;
    s_base[0] = s_base[1] = 0;
  }
  __syncthreads();
  for (long long b = 0; b <= n; b += kSortThreads) {
    const long long r = b + tid;
    const unsigned h = (r <= n) ? (unsigned)hist[r] : 0u;
    unsigned incl = h;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    if (lane == 31) s_scan[warp] = incl;
    __syncthreads();
    unsigned long long before = s_run;
    for (int w = 0; w < warp; ++w) before += s_scan[w];
    const bool hit = (r <= n) && (before + incl >= (unsigned long long)topk);
    if (hit) atomicMin(&s_worst_u, (unsigned)r);
    __syncthreads();
    if (tid == 0) {
      unsigned long long t = 0;
      for (int w = 0; w < kSortThreads / 32; ++w) t += s_scan[w];
      s_run += t;
    }
    __syncthreads();
    if (s_worst_u != 0xffffffffu) break;
  }
  if (tid == 0) s_worst = (s_worst_u == 0xffffffffu) ? (int)n : (int)s_worst_u;
  __syncthreads();
  const int worst = s_worst;
  // four consecutive rows per thread and tile: the lists stay in index order (a thread's rows are
  // consecutive, the threads of a warp and the warps of the block follow each other)
  for (long long s = 0; s < n; s += 4 * kSortThreads) {
    const long long i0 = s + (long long)tid * 4;
    int r[4];
    unsigned ca = 0, cl = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      r[q] = (i0 + q < n) ? rank[i0 + q] : 0x7fffffff;
      ca += r[q] < worst;
      cl += r[q] == worst;
    }
    unsigned ia = ca, il = cl;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned ta = __shfl_up_sync(0xffffffffu, ia, off), tl = __shfl_up_sync(0xffffffffu, il, off);
      if (lane >= off) {
        ia += ta;
        il += tl;
      }
    }
    if (lane == 31) {
      s_wsum[warp][0] = ia;
      s_wsum[warp][1] = il;
    }
    __syncthreads();
    unsigned off_a = s_base[0] + (ia - ca), off_l = s_base[1] + (il - cl);
    for (int w = 0; w < warp; ++w) {
      off_a += s_wsum[w][0];
      off_l += s_wsum[w][1];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (r[q] < worst) {
        idx_a[off_a] = (uint32_t)(i0 + q);
        key_a[off_a] = (uint32_t)r[q];
        ++off_a;
      } else if (r[q] == worst) {
        idx_l[off_l++] = (uint32_t)(i0 + q);
      }
    }
    __syncthreads();
    if (tid == 0) {
      unsigned ta = 0, tl = 0;
      for (int w = 0; w < kSortThreads / 32; ++w) {
        ta += s_wsum[w][0];
        tl += s_wsum[w][1];
      }
      s_base[0] += ta;
      s_base[1] += tl;
    }
    __syncthreads();
  }
  if (tid == 0) {
    ctrl->worst_rank = worst;
    ctrl->n_before = (int)s_base[0];
    ctrl->n_last = (int)s_base[1];
  }
}

// Index-ordered list of the rows with mask != 0 (crowding_distance called on its own).
__global__ void __launch_bounds__(kSortThreads)
    nds_mask_list_kernel(const uint8_t* __restrict__ mask, long long n, Ctrl* ctrl, uint32_t* idx_l) {
  __shared__ unsigned s_wsum[kSortThreads / 32];
  __shared__ unsigned s_base;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_base = 0;
  __syncthreads();
  for (long long s = 0; s < n; s += kSortThreads) {
    const long long i = s + tid;
    const bool in = (i < n) && mask[i] != 0;
    const unsigned m = __ballot_sync(0xffffffffu, in);
    if (lane == 0) s_wsum[warp] = __popc(m);
    __syncthreads();
    unsigned off = s_base;
    for (int w = 0; w < warp; ++w) off += s_wsum[w];
    if (in) idx_l[off + __popc(m & ((1u << lane) - 1u))] = (uint32_t)i;
    __syncthreads();
    if (tid == 0) {
      unsigned t = 0;
      for (int w = 0; w < kSortThreads / 32; ++w) t += s_wsum[w];
      s_base += t;
    }
    __syncthreads();
  }
  if (tid == 0) ctrl->n_last = (int)s_base;
}

// Block k sorts the front by objective k (stable) and writes each member's neighbour gap divided
// by the objective's range over the front (non_dominate.py:221-225). Members that come first or
// last in ANY objective are flagged: the reference sets their whole row to +inf (:226-227).
__global__ void __launch_bounds__(kSortThreads)
    nds_crowding_sort_kernel(const float* __restrict__ costs, int m, long long n, const Ctrl* ctrl,
                             const uint32_t* __restrict__ idx_l, uint32_t* sortbuf, float* contrib, uint32_t* boundary) {
  __shared__ SortSmem sm;
  const int k = blockIdx.x;
  const int nl = ctrl->n_last;
  uint32_t* keys = sortbuf + (size_t)k * 4 * n;
  uint32_t* vals = keys + n;
  uint32_t* tk = vals + n;
  uint32_t* tv = tk + n;
  for (int t = threadIdx.x; t < nl; t += blockDim.x) {
    keys[t] = float_order_key(costs[(size_t)idx_l[t] * m + k]);
    vals[t] = (uint32_t)t;
  }
  __syncthreads();
  block_radix_sort(keys, vals, tk, tv, nl, 32, sm);
  if (nl == 0) return;
  const float c_first = costs[(size_t)idx_l[vals[0]] * m + k];
  const float c_last = costs[(size_t)idx_l[vals[nl - 1]] * m + k];
  const float span = __fsub_rn(c_last, c_first);
  for (int p = threadIdx.x; p < nl; p += blockDim.x) {
    const uint32_t t = vals[p];
    if (p == 0 || p == nl - 1) {
      boundary[t] = 1u;
      contrib[(size_t)k * n + t] = INFINITY;
    } else {
      const float hi = costs[(size_t)idx_l[vals[p + 1]] * m + k];
      const float lo = costs[(size_t)idx_l[vals[p - 1]] * m + k];
      contrib[(size_t)k * n + t] = __fdiv_rn(__fsub_rn(hi, lo), span);
    }
  }
}

// Sum of m per-objective terms in the order torch.sum(dim=1) uses on the reference's CPU path
// for a contiguous inner dimension (ATen SumKernel: vectors of 8 floats accumulated lane-wise,
// scalar remainder with 4 interleaved partial sums, lanes added last in index order). For
// m <= 4 and m == 8 this is plain left-to-right order.
__device__ float aten_row_sum(const float* __restrict__ v, int m, size_t stride) {
  auto scalar_sum = [&](int begin, int end) {
    const int size = end - begin, groups = size / 4;
    float ps[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < groups; ++g)
      for (int q = 0; q < 4; ++q) ps[q] = __fadd_rn(ps[q], v[(size_t)(begin + 4 * g + q) * stride]);
    for (int i = begin + groups * 4; i < end; ++i) ps[0] = __fadd_rn(ps[0], v[(size_t)i * stride]);
    ps[0] = __fadd_rn(ps[0], ps[1]);
    ps[0] = __fadd_rn(ps[0], ps[2]);
    ps[0] = __fadd_rn(ps[0], ps[3]);
    return ps[0];
  };
  if (m < 8) return scalar_sum(0, m);
  const int nvec = m / 8, groups = nvec / 4;
  float lanes[8];
  for (int l = 0; l < 8; ++l) {
    float ps[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < groups; ++g)
      for (int q = 0; q < 4; ++q) ps[q] = __fadd_rn(ps[q], v[(size_t)((4 * g + q) * 8 + l) * stride]);
    for (int i = groups * 4; i < nvec; ++i) ps[0] = __fadd_rn(ps[0], v[(size_t)(i * 8 + l) * stride]);
    ps[0] = __fadd_rn(ps[0], ps[1]);
    ps[0] = __fadd_rn(ps[0], ps[2]);
    ps[0] = __fadd_rn(ps[0], ps[3]);
    lanes[l] = ps[0];
  }
  float acc = scalar_sum(nvec * 8, m);
  for (int l = 0; l < 8; ++l) acc = __fadd_rn(acc, lanes[l]);
  return acc;
}

__global__ void nds_crowding_finish_kernel(int m, long long n, const Ctrl* ctrl, const uint32_t* __restrict__ idx_l,
                                           const float* __restrict__ contrib, const uint32_t* __restrict__ boundary,
                                           float* __restrict__ crowd) {
  const int nl = ctrl->n_last;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < nl; t += (long long)gridDim.x * blockDim.x) {
    crowd[idx_l[t]] = boundary[t] ? INFINITY : aten_row_sum(contrib + t, m, (size_t)n);
  }
}

__global__ void nds_fill_kernel(float* p, long long n, float v) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) p[i] = v;
}

// Block 0: rows before the last admitted front by (rank, index). Block 1: the last front by
// (-crowding, index) — together lexsort([-crowd, rank])[:topk] (non_dominate.py:253).
__global__ void __launch_bounds__(kSortThreads)
    nds_order_kernel(long long n, long long topk, const Ctrl* ctrl, uint32_t* idx_a, uint32_t* key_a,
                     const uint32_t* __restrict__ idx_l, const float* __restrict__ crowd, uint32_t* sortbuf, int m,
                     uint32_t* order) {
  __shared__ SortSmem sm;
  const int na = ctrl->n_before, nl = ctrl->n_last;
  uint32_t* scratch = sortbuf + (size_t)(m + blockIdx.x) * 4 * n;
  if (blockIdx.x == 0) {
    if (ctrl->n_fronts <= kRankBuckets) return;  // nds_rank_place_kernel wrote these rows already
    int bits = 1;
    while (bits < 32 && (ctrl->worst_rank >> bits) != 0) ++bits;
    block_radix_sort(key_a, idx_a, scratch, scratch + n, na, bits, sm);
    for (int t = threadIdx.x; t < na && t < topk; t += blockDim.x) order[t] = idx_a[t];
  } else {
    uint32_t* keys = scratch;
    uint32_t* vals = scratch + n;
    for (int t = threadIdx.x; t < nl; t += blockDim.x) {
      keys[t] = float_order_key(-crowd[idx_l[t]]);
      vals[t] = idx_l[t];
    }
    __syncthreads();
    block_radix_sort(keys, vals, scratch + 2 * n, scratch + 3 * n, nl, 32, sm);
    for (long long t = threadIdx.x; t < nl && na + t < topk; t += blockDim.x) order[na + t] = vals[t];
  }
}

__global__ void nds_gather_kernel(const uint32_t* __restrict__ order, long long topk, const float* __restrict__ x,
                                  long long dx, const float* __restrict__ f, int m, const int* __restrict__ rank,
                                  const float* __restrict__ crowd, float* out_x, float* out_f, int* out_rank,
                                  float* out_crowd, long long* out_index) {
  const long long per = dx + m + 1;
  const long long total = topk * per;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / per, c = t - row * per;
    const long long src = order[row];
    if (c < dx) {
      out_x[row * dx + c] = x[src * dx + c];
    } else if (c < dx + m) {
      out_f[row * m + (c - dx)] = f[src * m + (c - dx)];
    } else {
      out_rank[row] = rank[src];
      out_crowd[row] = crowd[src];
      if (out_index) out_index[row] = src;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
template <int M>
void launch_dominance(const float* fs, long long npad, long long n, uint32_t* Dt, int wp, float* stats, cudaStream_t s,
                      long long s_begin = 0, long long s_end = (1ll << 62)) {
  constexpr int R = (M <= 4) ? 4 : ((M <= 8) ? 2 : 1);
  if (stats != nullptr) nds_tile_stats_kernel<<<(unsigned)(npad / kTileJ), kTileJ, 0, s>>>(fs, npad, n, M, stats);
  dim3 grid((unsigned)((n + kTileJ - 1) / kTileJ), (unsigned)((npad + 256 * R - 1) / (256 * R)));
  nds_dominance_kernel<M, R><<<grid, kThreads, 0, s>>>(fs, npad, n, Dt, wp, stats, s_begin, s_end);
}

int grid_1d(long long work, int per_block = kThreads) {
  long long want = (work + per_block - 1) / per_block;
  const long long cap = (long long)sm_count() * 8;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

int run_rank(const float* f, long long n, int m, int* rank, void* ws, const Layout& L, cudaStream_t s) {
  float* fs = at<float>(ws, L.fs);
  uint32_t* Dt = at<uint32_t>(ws, L.dt);
  Ctrl* ctrl = at<Ctrl>(ws, L.ctrl);
  uint32_t* unranked = at<uint32_t>(ws, L.unranked);
  uint32_t* newfront = at<uint32_t>(ws, L.newfront);
  int* ptr = at<int>(ws, L.ptr);
  // large populations: deal the rows into bands of the first objective and, inside a band, by the second one
  // (see order_key): about eight tiles of 1,024 rows per band, so that a tile is narrow in both objectives
  const uint32_t* perm = nullptr;
  unsigned* range = at<unsigned>(ws, L.bins);
  int* group_of_bin = reinterpret_cast<int*>(range + 4);
  int* counts = group_of_bin + (kBins + 2);
  int* cursor = counts + (kBins + 2);
  int groups = (int)(n / 8192);  // measured at 100,000 rows: 1.89 ms per rank with 8 or 12 bands, 1.90 with 4, 1.96 with 16, 2.01 with 2
  groups = groups < 1 ? 1 : (groups > 16 ? 16 : groups);
  while (kBins % groups) --groups;
  if (n >= kOrderMinN && m <= 16) {
    uint32_t* perm_w = at<uint32_t>(ws, L.perm);
    EVOX_CUDA(cudaMemsetAsync(range, 0, sizeof(int) * (size_t)(3 * (kBins + 2) + 4), s));
    nds_range_kernel<<<grid_1d(n), kThreads, 0, s>>>(f, n, m, range);
    if (m >= 2) {
      nds_bin_count_kernel<<<grid_1d(n), kThreads, 0, s>>>(f, n, m, range, group_of_bin);
      nds_group_kernel<<<1, 1024, 0, s>>>(group_of_bin, groups);
    }
    nds_key_count_kernel<<<grid_1d(n), kThreads, 0, s>>>(f, n, m, range, group_of_bin, groups, counts);
    nds_bin_scan_kernel<<<1, 1024, 0, s>>>(counts, cursor);
    nds_bin_scatter_kernel<<<grid_1d(n), kThreads, 0, s>>>(f, n, m, range, group_of_bin, groups, cursor, perm_w);
    EVOX_LAUNCH_CHECK();
    perm = perm_w;
  }
  const int ordered = perm != nullptr;
  nds_transpose_kernel<<<grid_1d((long long)m * L.npad), kThreads, 0, s>>>(f, n, m, L.npad, perm, fs);
  EVOX_LAUNCH_CHECK();
  switch (m) {
#define EVOX_DOM(MM) case MM: launch_dominance<MM>(fs, L.npad, n, Dt, L.wp, ordered ? at<float>(ws, L.tile_stats) : nullptr, s); break;
    EVOX_DOM(1) EVOX_DOM(2) EVOX_DOM(3) EVOX_DOM(4) EVOX_DOM(5) EVOX_DOM(6) EVOX_DOM(7) EVOX_DOM(8)
    EVOX_DOM(9) EVOX_DOM(10) EVOX_DOM(11) EVOX_DOM(12) EVOX_DOM(13) EVOX_DOM(14) EVOX_DOM(15) EVOX_DOM(16)
#undef EVOX_DOM
    default:
      nds_dominance_generic_kernel<<<grid_1d(n * (long long)L.wp), kThreads, 0, s>>>(fs, L.npad, n, m, Dt, L.wp);
  }
  EVOX_LAUNCH_CHECK();
  // the scatter's cursors are now at the bin ends
  nds_peel_init_kernel<<<grid_1d(n), kThreads, 0, s>>>(n, L.wp, unranked, newfront, ptr, rank, ctrl, fs, L.npad, m, range, group_of_bin,
                                                       groups, ordered ? cursor : nullptr, n <= kTailDirectMaxN ? (int)n : 0);
  EVOX_LAUNCH_CHECK();
  if (n <= kTailDirectMaxN) {
    // small population: one cluster peels every front straight from the matrix (measured against the grid kernel:
    // 0.077 / 0.124 / 0.144 / 0.214 ms per rank at 500 / 2,000 / 4,096 / 8,192 rows instead of 0.099 / 0.148 / 0.181 / 0.273)
    nds_peel_tail_kernel<<<kTailCtas, kTailThreads, 0, s>>>(Dt, L.wp, nullptr, perm, rank, ctrl);
    EVOX_LAUNCH_CHECK();
    return EVOX_OK;
  }
  // persistent cooperative grid: every block must be resident for the grid barrier
  int per_sm = 0;
  size_t mask_bytes = sizeof(uint32_t) * (size_t)L.wp;
  int mask_in_smem = mask_bytes <= 64 * 1024 ? 1 : 0;  // larger masks are read through L2
  if (!mask_in_smem) mask_bytes = 0;
  const long long words = (n + 31) / 32;
  // 1024-thread blocks when 512-thread ones would make every warp visit two words per front but 1024-thread ones
  // only one (the witness position then stays in a register and a front has one trip of block barriers, not two:
  // 1.84 against 1.89 ms per rank at 100,000 rows)
  const long long warps512 = (long long)sm_count() * (kPeelThreadsSmall / 32);
  const bool large = words > warps512 && words <= 2 * warps512;
  const int threads = large ? kPeelThreadsLarge : kPeelThreadsSmall;
  const void* kernel = large ? (mask_in_smem ? (const void*)nds_peel_kernel<kPeelThreadsLarge, true> : (const void*)nds_peel_kernel<kPeelThreadsLarge, false>)
                             : (mask_in_smem ? (const void*)nds_peel_kernel<kPeelThreadsSmall, true> : (const void*)nds_peel_kernel<kPeelThreadsSmall, false>);
  if (mask_bytes > 40 * 1024) EVOX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
  EVOX_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, mask_bytes));
  EVOX_REQUIRE(per_sm > 0, EVOX_ERR_CUDA, "nds_peel_kernel cannot be made resident");
  if (per_sm > 4) per_sm = 4;
  {
    // Enough blocks for one word of 32 columns per warp (one trip per front) plus a share of helper
    // warps, but no more: the grid barrier gets slower with every block that takes part (measured at
    // 20,000 rows: 0.47 ms per rank with four blocks per multiprocessor, 0.44 ms with one).
    const long long need = (words + (long long)sm_count() * (threads / 32) - 1) / ((long long)sm_count() * (threads / 32));
    const int want = need <= 1 ? 1 : (int)(need + 1);
    if (want < per_sm) per_sm = want;
  }
  long long blocks = (long long)sm_count() * per_sm;
  const long long useful = (n + 31) / 32;  // at least one word of 32 columns per block
  if (blocks > useful) blocks = useful < 1 ? 1 : useful;
  const uint32_t* Dt_c = Dt;
  int wp = L.wp;
  long long nn = n;
  // the grid kernel peels until kTailCompactRows rows are left, then the cluster kernel takes their sub-matrix
  int tail_limit = kTailCompactRows;
  void* args[] = {(void*)&Dt_c, (void*)&wp, (void*)&nn, (void*)&unranked, (void*)&newfront, (void*)&ptr, (void*)&rank, (void*)&ctrl,
                  (void*)&mask_in_smem, (void*)&perm, (void*)&tail_limit};
  EVOX_CUDA(cudaLaunchCooperativeKernel(kernel, dim3((unsigned)blocks), dim3(threads), args, mask_bytes, s));
  uint32_t* ids = at<uint32_t>(ws, L.tail_ids);
  uint32_t* sub = at<uint32_t>(ws, L.tail_sub);
  nds_tail_ids_kernel<<<1, 1024, 0, s>>>(unranked, newfront, L.wp, ctrl, ids);
  nds_tail_gather_kernel<<<sm_count() * 8, 256, 0, s>>>(Dt, L.wp, ctrl, ids, sub);
  nds_peel_tail_kernel<<<kTailCtas, kTailThreads, 0, s>>>(sub, kTailCompactRows / 32, ids, perm, rank, ctrl);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

int check_ws(const char* who, void* ws, size_t bytes, const Layout& L) {
  EVOX_REQUIRE(ws != nullptr, EVOX_ERR_WORKSPACE, "%s: workspace is NULL", who);
  EVOX_REQUIRE(((uintptr_t)ws & 255u) == 0, EVOX_ERR_INVALID, "%s: workspace must be 256-byte aligned", who);
  EVOX_REQUIRE(bytes >= L.total, EVOX_ERR_WORKSPACE, "%s: workspace of %zu bytes is smaller than %zu", who, bytes, L.total);
  return EVOX_OK;
}

int check_nm(const char* who, long long n, int m) {
  EVOX_REQUIRE(n > 0 && n < (1ll << 31) - kPad, EVOX_ERR_INVALID, "%s: n must be in [1, 2^31), got %lld", who, n);
  EVOX_REQUIRE(m > 0 && m <= 1024, EVOX_ERR_INVALID, "%s: number of objectives must be in [1, 1024], got %d", who, m);
  return EVOX_OK;
}

int run_crowding(const float* costs, long long n, int m, void* ws, const Layout& L, float* crowd, cudaStream_t s) {
  Ctrl* ctrl = at<Ctrl>(ws, L.ctrl);
  uint32_t* idx_l = at<uint32_t>(ws, L.idx_l);
  uint32_t* sortbuf = at<uint32_t>(ws, L.sortbuf);
  float* contrib = at<float>(ws, L.contrib);
  uint32_t* boundary = at<uint32_t>(ws, L.boundary);
  EVOX_CUDA(cudaMemsetAsync(boundary, 0, sizeof(uint32_t) * (size_t)n, s));
  nds_fill_kernel<<<grid_1d(n), kThreads, 0, s>>>(crowd, n, -INFINITY);
  EVOX_LAUNCH_CHECK();
  nds_crowding_sort_kernel<<<m, kSortThreads, 0, s>>>(costs, m, n, ctrl, idx_l, sortbuf, contrib, boundary);
  EVOX_LAUNCH_CHECK();
  nds_crowding_finish_kernel<<<grid_1d(n), kThreads, 0, s>>>(m, n, ctrl, idx_l, contrib, boundary, crowd);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" size_t evox_nds_workspace_bytes(int64_t n, int32_t m) {
  if (n <= 0 || m <= 0) return 0;
  return make_layout(n, m, true).total;
}

extern "C" int evox_nd_rank(const float* f, int64_t n, int32_t m, int32_t* rank, int32_t* status,
                            void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_nm("nd_rank", n, m)) return rc;
  EVOX_REQUIRE(f && rank, EVOX_ERR_INVALID, "nd_rank: NULL pointer");
  const Layout L = make_layout(n, m, true);
  if (int rc = check_ws("nd_rank", workspace, workspace_bytes, L)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (int rc = run_rank(f, n, m, rank, workspace, L, s)) return rc;
  if (status) {
    EVOX_CUDA(cudaMemcpyAsync(status, &at<Ctrl>(workspace, L.ctrl)->status, 2 * sizeof(int), cudaMemcpyDeviceToDevice, s));
  }
  return EVOX_OK;
}

extern "C" int evox_crowding_distance(const float* costs, const uint8_t* mask, int64_t n, int32_t m,
                                      float* distance, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_nm("crowding_distance", n, m)) return rc;
  EVOX_REQUIRE(costs && mask && distance, EVOX_ERR_INVALID, "crowding_distance: NULL pointer");
  const Layout L = make_layout(n, m, true);
  if (int rc = check_ws("crowding_distance", workspace, workspace_bytes, L)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  nds_mask_list_kernel<<<1, kSortThreads, 0, s>>>(mask, n, at<Ctrl>(workspace, L.ctrl), at<uint32_t>(workspace, L.idx_l));
  EVOX_LAUNCH_CHECK();
  return run_crowding(costs, n, m, workspace, L, distance, s);
}

extern "C" int evox_nd_environmental_selection(const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                                               int64_t topk, float* out_x, float* out_f, int32_t* out_rank,
                                               float* out_crowd, int64_t* out_index, int32_t* status,
                                               void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_nm("nd_environmental_selection", n, m)) return rc;
  EVOX_REQUIRE(x && f && out_x && out_f && out_rank && out_crowd, EVOX_ERR_INVALID, "nd_environmental_selection: NULL pointer");
  EVOX_REQUIRE(topk > 0 && topk <= n, EVOX_ERR_INVALID, "nd_environmental_selection: topk must be in [1, n], got %lld", (long long)topk);
  EVOX_REQUIRE(dx > 0, EVOX_ERR_INVALID, "nd_environmental_selection: dx must be positive");
  const Layout L = make_layout(n, m, true);
  if (int rc = check_ws("nd_environmental_selection", workspace, workspace_bytes, L)) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  void* ws = workspace;
  int* rank = at<int>(ws, L.rank);
  Ctrl* ctrl = at<Ctrl>(ws, L.ctrl);
  if (int rc = run_rank(f, n, m, rank, ws, L, s)) return rc;
  uint32_t* idx_a = at<uint32_t>(ws, L.idx_a);
  uint32_t* key_a = at<uint32_t>(ws, L.key_a);
  uint32_t* idx_l = at<uint32_t>(ws, L.idx_l);
  uint32_t* order = at<uint32_t>(ws, L.order);
  // Which of the two paths runs is decided on the device by the number of fronts the rank found (the host does
  // not wait for it): the kernels of the other path return at once.
  {  // at most kRankBuckets fronts: counting placement over kRankWarps row ranges
    int* whist = at<int>(ws, L.whist);
    int* rank_off = at<int>(ws, L.rank_off);
    nds_rank_count_kernel<<<kRankWarps / 8, 256, 0, s>>>(rank, n, ctrl, whist);
    nds_rank_scan_kernel<<<kRankBuckets / 8, 256, 0, s>>>(ctrl, whist, rank_off + kRankBuckets);
    nds_rank_offsets_kernel<<<1, kRankBuckets, 0, s>>>(topk, ctrl, rank_off + kRankBuckets, rank_off);
    nds_rank_place_kernel<<<kRankWarps / 8, 256, 0, s>>>(rank, n, ctrl, whist, rank_off, order, idx_l);
    EVOX_LAUNCH_CHECK();
  }
  {  // more fronts than that: histogram, single-block partition and sort
    int* hist = at<int>(ws, L.hist);
    EVOX_CUDA(cudaMemsetAsync(hist, 0, sizeof(int) * (size_t)(n + 1), s));
    nds_hist_kernel<<<grid_1d(n), kThreads, 0, s>>>(rank, n, hist, ctrl);
    nds_partition_kernel<<<1, kSortThreads, 0, s>>>(rank, hist, n, topk, ctrl, idx_a, key_a, idx_l);
    EVOX_LAUNCH_CHECK();
  }
  float* crowd = at<float>(ws, L.crowd);
  if (int rc = run_crowding(f, n, m, ws, L, crowd, s)) return rc;
  nds_order_kernel<<<2, kSortThreads, 0, s>>>(n, topk, ctrl, idx_a, key_a, idx_l, crowd, at<uint32_t>(ws, L.sortbuf), m, order);
  EVOX_LAUNCH_CHECK();
  nds_gather_kernel<<<grid_1d(topk * (dx + m + 1)), kThreads, 0, s>>>(order, topk, x, dx, f, m, rank, crowd, out_x, out_f,
                                                                      out_rank, out_crowd, (long long*)out_index);
  EVOX_LAUNCH_CHECK();
  if (status) EVOX_CUDA(cudaMemcpyAsync(status, &ctrl->status, 2 * sizeof(int), cudaMemcpyDeviceToDevice, s));
  return EVOX_OK;
}

// ---------------------------------------------------------------------------------------------
// Rank with the dominance matrix split over several GPUs (rows of the matrix = dominated columns).
//
// Every GPU holds all objectives (kilobytes to megabytes) and the rows [shard_begin, shard_begin + shard_rows)
// of the bit matrix, in the row order `perm` all GPUs agree on. One front = one launch of nds_shard_front_kernel
// on every GPU (its columns are tested against the whole unranked mask, exactly as in nds_peel_kernel: witness
// word first, then a forward scan of the row) followed by an allgather of the GPUs' slices of the next mask: the
// one exchange per peeling round, n / 8 bytes in total. The matrix (n^2 / 8 bytes) and the comparisons that
// build it are what is divided; the chain of fronts is not.
// ---------------------------------------------------------------------------------------------
namespace evox {
namespace {

struct ShardLayout {
  size_t fs, dt, ptr, stats, total;
  int wp;
};

ShardLayout make_shard_layout(long long n_cols, int m, long long shard_rows) {
  ShardLayout L;
  L.wp = (int)(n_cols / 32);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes);
    return at;
  };
  L.fs = take(sizeof(float) * (size_t)m * (size_t)n_cols);
  L.ptr = take(sizeof(int) * (size_t)shard_rows);
  L.stats = take(sizeof(float) * 5 * (size_t)(n_cols / kTileJ));
  L.dt = take(sizeof(uint32_t) * (size_t)shard_rows * (size_t)L.wp);
  L.total = off;
  return L;
}

__global__ void nds_shard_init_kernel(long long n, long long shard_begin, long long shard_rows, const int* __restrict__ start_word,
                                      int* __restrict__ ptr, uint32_t* __restrict__ mask_slice, int* __restrict__ rank_local) {
  const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long w = t0; w < shard_rows / 32; w += stride) {
    const long long lo = shard_begin + w * 32;
    uint32_t bits = 0;
    if (lo + 32 <= n) bits = 0xffffffffu;
    else if (lo < n) bits = (1u << (int)(n - lo)) - 1u;
    mask_slice[w] = bits;
  }
  for (long long j = t0; j < shard_rows; j += stride) {
    ptr[j] = start_word ? start_word[j] : 0;
    rank_local[j] = -1;
  }
}

// One front for this GPU's columns, with the steps of nds_peel_kernel's front: a warp owns 32 consecutive columns;
// `mask` is the whole unranked mask (read-only here), the successor of the warp's own word goes to mask_slice_out.
// One memory round trip settles most columns: a lane whose column is still open reads 32 words of its own row from
// its witness position on (eight independent 128-bit loads) and takes the first word that still holds an unranked
// dominator as the new witness; columns with nothing there are queued for the block, whose warps share the long
// scans. (The first version scanned a word's cleared columns one after the other in the owning warp: 26 us per
// front for 50,000 columns of a 100,000-row population, 64 us for 200,000 of 400,000.)
constexpr int kShardThreads = 256;

__global__ void __launch_bounds__(kShardThreads)
    nds_shard_front_kernel(const uint32_t* __restrict__ Dt, int wp, long long shard_rows, const uint32_t* __restrict__ mask,
                           long long shard_begin, int front, int* __restrict__ ptr, uint32_t* __restrict__ mask_slice_out,
                           int* __restrict__ rank_local) {
  constexpr int kWarps = kShardThreads / 32;
  __shared__ unsigned s_newly[kWarps];      // per owning warp: columns ranked in this trip
  __shared__ long long s_qj[kShardThreads];  // block queue of columns waiting for a warp-wide scan
  __shared__ int s_qc[kShardThreads];
  __shared__ unsigned short s_qowner[kShardThreads];
  __shared__ int s_qn;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long n_words = shard_rows / 32, slice0 = shard_begin / 32;
  const long long words_per_pass = (long long)gridDim.x * kWarps;
  const long long trips = (n_words + words_per_pass - 1) / words_per_pass;  // the same for every warp: the block synchronises inside
  for (long long trip = 0; trip < trips; ++trip) {
    const long long w = trip * words_per_pass + (long long)blockIdx.x * kWarps + warp;
    const bool have = w < n_words;
    if (threadIdx.x == 0) s_qn = 0;
    if (lane == 0) s_newly[warp] = 0u;
    __syncthreads();
    const uint32_t own = have ? __ldg(mask + slice0 + w) : 0u;
    const long long jl = w * 32 + lane;  // local row of the matrix
    const bool open = (own >> lane) & 1u;
    if (open) {
      const int c = ptr[jl];
      const int c4 = c & ~3;
      const uint4* row4 = reinterpret_cast<const uint4*>(Dt + jl * wp);
      uint4 d[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int x = c4 + q * 4;
        d[q] = (x < wp) ? __ldg(row4 + (x >> 2)) : make_uint4(0u, 0u, 0u, 0u);
      }
      int hit = -1;
#pragma unroll
      for (int q = 7; q >= 0; --q) {
        const int x = c4 + q * 4;
        if (x < wp) {
          const int f = tail_first_nonzero(and4(d[q], __ldg(reinterpret_cast<const uint4*>(mask + x))));
          if (f >= 0) hit = x + f;
        }
      }
      if (hit >= 0) {
        if (hit != c) ptr[jl] = hit;
      } else {
        const int slot = atomicAdd(&s_qn, 1);
        s_qj[slot] = jl;
        s_qc[slot] = min(c4 + 32, wp - 1);  // nothing up to here: the scan may skip these words
        s_qowner[slot] = (unsigned short)threadIdx.x;
      }
    }
    __syncthreads();
    const int qn = s_qn;
    for (int item = warp; item < qn; item += kWarps) {
      const long long jq = s_qj[item];
      const int cs = s_qc[item];
      const uint4* row4 = reinterpret_cast<const uint4*>(Dt + jq * wp);
      int found = -1;
      for (int base = cs & ~1023; base < wp && found < 0; base += 1024) {
        uint4 d[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int x = base + q * 128 + lane * 4;
          d[q] = (x < wp && x + 4 > cs) ? __ldg(row4 + (x >> 2)) : make_uint4(0u, 0u, 0u, 0u);  // words before cs are done
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int x = base + q * 128 + lane * 4;
          int f = -1;
          if (x < wp) f = tail_first_nonzero(and4(d[q], __ldg(reinterpret_cast<const uint4*>(mask + x))));
          const unsigned hit = __ballot_sync(0xffffffffu, f >= 0);
          if (hit && found < 0) {
            const int l = __ffs(hit) - 1;
            found = base + q * 128 + l * 4 + __shfl_sync(0xffffffffu, f, l);
          }
        }
      }
      if (lane == 0) {
        if (found >= 0) {
          ptr[jq] = found;
        } else {
          const unsigned owner = s_qowner[item];
          atomicOr(&s_newly[owner >> 5], 1u << (owner & 31));
          rank_local[jq] = front;
        }
      }
    }
    __syncthreads();
    if (lane == 0 && have) mask_slice_out[w] = own & ~s_newly[warp];
    __syncthreads();  // the queue and the per-warp words are reused by the next trip
  }
}

}  // namespace
}  // namespace evox

extern "C" size_t evox_nds_shard_workspace_bytes(int64_t n_cols, int32_t m, int64_t shard_rows) {
  if (n_cols <= 0 || m <= 0 || shard_rows <= 0) return 0;
  return make_shard_layout(n_cols, m, shard_rows).total;
}

extern "C" int evox_nd_rank_shard_begin(const float* f, int64_t n, int32_t m, const uint32_t* perm, int64_t n_cols,
                                        int64_t shard_begin, int64_t shard_rows, const int32_t* start_word,
                                        uint32_t* mask_slice, int32_t* rank_local, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  if (int rc = check_nm("nd_rank_shard_begin", n, m)) return rc;
  EVOX_REQUIRE(f && mask_slice && rank_local, EVOX_ERR_INVALID, "nd_rank_shard_begin: NULL pointer");
  EVOX_REQUIRE(m <= 16, EVOX_ERR_INVALID, "nd_rank_shard_begin: at most 16 objectives, got %d", m);
  EVOX_REQUIRE(shard_rows > 0 && shard_rows % kPad == 0 && shard_begin >= 0 && shard_begin % shard_rows == 0 && n_cols % shard_rows == 0 &&
                   n_cols >= n && shard_begin + shard_rows <= n_cols,
               EVOX_ERR_INVALID, "nd_rank_shard_begin: shards must be equal multiples of %d rows that cover the population", kPad);
  const ShardLayout L = make_shard_layout(n_cols, m, shard_rows);
  EVOX_REQUIRE(workspace != nullptr && ((uintptr_t)workspace & 255u) == 0 && workspace_bytes >= L.total, EVOX_ERR_WORKSPACE,
               "nd_rank_shard_begin: workspace missing, misaligned or smaller than %zu bytes", L.total);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* fs = at<float>(workspace, L.fs);
  uint32_t* Dt = at<uint32_t>(workspace, L.dt);
  nds_transpose_kernel<<<grid_1d((long long)m * n_cols), kThreads, 0, s>>>(f, n, m, n_cols, perm, fs);
  EVOX_LAUNCH_CHECK();
  // columns at or beyond n (padding) dominate nothing and are never open: their rows of the matrix are never read
  switch (m) {
#define EVOX_DOM(MM) case MM: launch_dominance<MM>(fs, n_cols, n, Dt, L.wp, at<float>(workspace, L.stats), s, shard_begin, shard_begin + shard_rows); break;
    EVOX_DOM(1) EVOX_DOM(2) EVOX_DOM(3) EVOX_DOM(4) EVOX_DOM(5) EVOX_DOM(6) EVOX_DOM(7) EVOX_DOM(8)
    EVOX_DOM(9) EVOX_DOM(10) EVOX_DOM(11) EVOX_DOM(12) EVOX_DOM(13) EVOX_DOM(14) EVOX_DOM(15) EVOX_DOM(16)
#undef EVOX_DOM
  }
  EVOX_LAUNCH_CHECK();
  nds_shard_init_kernel<<<grid_1d(shard_rows), kThreads, 0, s>>>(n, shard_begin, shard_rows, start_word, at<int>(workspace, L.ptr),
                                                                mask_slice, rank_local);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_nd_rank_shard_front(int64_t n_cols, int32_t m, int64_t shard_begin, int64_t shard_rows, const uint32_t* mask_full,
                                        int32_t front, uint32_t* mask_slice_out, int32_t* rank_local, void* workspace,
                                        size_t workspace_bytes, void* stream) {
  EVOX_REQUIRE(mask_full && mask_slice_out && rank_local, EVOX_ERR_INVALID, "nd_rank_shard_front: NULL pointer");
  EVOX_REQUIRE(n_cols > 0 && m > 0 && shard_rows > 0 && shard_rows % kPad == 0 && n_cols % shard_rows == 0 && shard_begin >= 0 &&
                   shard_begin + shard_rows <= n_cols,
               EVOX_ERR_INVALID, "nd_rank_shard_front: bad shard geometry");
  EVOX_REQUIRE(((uintptr_t)mask_full & 15u) == 0, EVOX_ERR_INVALID, "nd_rank_shard_front: the mask must be 16-byte aligned");
  const ShardLayout L = make_shard_layout(n_cols, m, shard_rows);
  EVOX_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, EVOX_ERR_WORKSPACE, "nd_rank_shard_front: workspace too small");
  const long long warps = shard_rows / 32;
  const long long cap = (long long)sm_count() * 8;
  long long blocks = (warps + kShardThreads / 32 - 1) / (kShardThreads / 32);
  if (blocks > cap) blocks = cap;
  nds_shard_front_kernel<<<(unsigned)blocks, kShardThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      at<uint32_t>(workspace, L.dt), L.wp, shard_rows, mask_full, shard_begin, front, at<int>(workspace, L.ptr), mask_slice_out,
      rank_local);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free rank for small populations.
//
// Some hosts of this library may not allocate device memory at the point where they need a
// rank: code running between fixed-size arenas handed out at start-up, plug-ins that are given
// input and output buffers by their host application and nothing else, and loops that must not
// disturb an allocator's bookkeeping while they run. For them the scratch of evox_nd_rank lives
// in a fixed array inside the library image. Every GPU that loads the library carries those
// kStaticBytes until the process exits, which is why the population is capped.
// ---------------------------------------------------------------------------------------------
namespace evox {
namespace {

constexpr long long kStaticMaxN = 4096;
constexpr int kStaticMaxM = 16;
constexpr size_t kStaticBytes = 4u << 20;  // >= make_layout(kStaticMaxN, kStaticMaxM).total, checked at set-up

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the
// address has to be asked for, once per device, while that device is current.
std::mutex g_static_mutex;
void* g_static_address[64] = {nullptr};
bool g_static_ready[64] = {false};

int static_scratch_address(void** out) {
  int dev = -1;
  EVOX_CUDA(cudaGetDevice(&dev));
  EVOX_REQUIRE(dev >= 0 && dev < 64, EVOX_ERR_INVALID, "nd_rank_static: device ordinal %d is not supported", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ready[dev]) {
    EVOX_REQUIRE(make_layout(kStaticMaxN, kStaticMaxM, true, false).total <= kStaticBytes, EVOX_ERR_INVALID,
                 "nd_rank_static: built-in scratch of %zu bytes cannot hold the maximum problem", kStaticBytes);
    void* p = nullptr;
    EVOX_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    EVOX_REQUIRE(p != nullptr && ((uintptr_t)p & 255u) == 0, EVOX_ERR_CUDA, "nd_rank_static: bad scratch address");
    g_static_address[dev] = p;
    g_static_ready[dev] = true;
  }
  *out = g_static_address[dev];
  return EVOX_OK;
}

}  // namespace
}  // namespace evox

extern "C" int evox_nd_rank_static(const float* f, int64_t n, int32_t m, int32_t* rank, int32_t* status,
                                   void* stream) {
  if (int rc = check_nm("nd_rank_static", n, m)) return rc;
  EVOX_REQUIRE(f && rank, EVOX_ERR_INVALID, "nd_rank_static: NULL pointer");
  EVOX_REQUIRE(n <= kStaticMaxN, EVOX_ERR_INVALID,
               "nd_rank_static: n = %lld exceeds the built-in scratch (at most %lld rows); use evox_nd_rank with a workspace",
               (long long)n, kStaticMaxN);
  EVOX_REQUIRE(m <= kStaticMaxM, EVOX_ERR_INVALID,
               "nd_rank_static: m = %d exceeds the built-in scratch (at most %d objectives); use evox_nd_rank with a workspace",
               m, kStaticMaxM);
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  const Layout L = make_layout(n, m, true, false);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // run_rank rewrites every scratch region it later reads (objectives, matrix rows, masks,
  // witness positions, control block), so what an earlier call left behind is never seen
  if (int rc = run_rank(f, n, m, rank, scratch, L, s)) return rc;
  if (status) {
    EVOX_CUDA(cudaMemcpyAsync(status, &at<Ctrl>(scratch, L.ctrl)->status, 2 * sizeof(int), cudaMemcpyDeviceToDevice, s));
  }
  return EVOX_OK;
}
