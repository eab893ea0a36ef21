// P4 (part 2): one Linear layer of the virtual-LoRA population forward on the 5th-generation
// tensor cores (sm_100a): Y = act(H W^T + bias + sigma * (H A_p^T) B_p^T + sigma * bias_noise_p).
//
// Reference semantics: VirtualLoRAProblem._virtual_forward
// (evox/problems/neuroevolution/virtual_lora_problem.py:160-193) with the factors of
// generate_lora_factors (evox/triton_kernels/kernels/lora_noise.py:86-127); the reference does
// the base product as an fp32 cuBLAS SGEMM and the correction as two batched matmuls over
// materialised factors (lora_noise.py:151-153).
//
// lora_gemm_kernel — persistent, one CTA per SM, warp specialised:
//   warp 0    TMA producer: 128 x 64 tile of H and 256 x 64 tile of W (bf16, 128-byte swizzle)
//             per k-block into a 4-stage shared-memory ring.
//   warp 1    issues tcgen05.mma (M = 128, N = 256, K = 16, bf16 x bf16 -> fp32) from one lane into
//             one of two 256-column TMEM accumulators; tcgen05.commit releases ring stages and
//             hands finished accumulators to the epilogue.
//   warps 2-5 epilogue: regenerate the tile's slice of B_p (and bias noise) from the individuals'
//             Philox streams into shared memory, read the accumulator with tcgen05.ld, add bias,
//             the rank-r correction sigma * t B_p^T (t = H A_p^T from lora_down_bf16_kernel), ReLU,
//             and store bf16 / fp32 — or, for the last layer, reduce (y - target)^2 per row.
//             The second accumulator lets the next tile's products run underneath.
// PAIR variant (rows a multiple of 256): two CTAs of a cluster share one 256 x 256 tile through
// tcgen05.mma.cta_group::2. Each CTA loads its own 128 rows of H and HALF of the W tile (128 rows), so
// a k-block costs 32 KB of shared-memory fill per SM instead of 48 KB and six stages fit; the leader
// CTA (cluster rank 0) issues the products for both, each CTA keeps the accumulator of its own 128
// rows in its own TMEM and runs the same epilogue on it. Both CTAs' copies report to the leader's
// "full" barrier; tcgen05.commit releases the stage in both CTAs and hands the accumulator to both
// epilogues; the epilogues return accumulators to the leader's "empty" barrier by a remote arrive.
// Every mbarrier wait is bounded by a wall-clock limit; on expiry the kernel raises an error flag,
// all roles leave their loops, outstanding copies are drained with the same bound and TMEM is freed.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <mutex>

#include "common.cuh"

namespace evox {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, RANK = 8;
constexpr int kRingBytes = 196608;  // shared-memory ring: 4 stages of 48 KB, or 6 stages of 32 KB for a CTA pair
constexpr int kEpilogueWarps = 8;  // two warps per TMEM lane quarter, 128 columns each
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kGemmThreads = 64 + kEpilogueThreads;
constexpr uint32_t kBytesA = BM * BK * 2;
template <bool PAIR>
struct Ring {
  static constexpr uint32_t kBytesB = (PAIR ? BN / 2 : BN) * BK * 2;  // a CTA of a pair holds half of the W tile
  static constexpr uint32_t kStageBytes = kBytesA + kBytesB;
  static constexpr int STAGES = kRingBytes / kStageBytes;
  static constexpr uint32_t kTxBytes = PAIR ? 2 * kStageBytes : kStageBytes;  // both CTAs report to the leader's barrier
};
constexpr int kMaxStages = 6;
constexpr uint32_t kMaxInd = 2;  // individuals per 128-row tile (batch is a multiple of 64)
constexpr uint32_t kOffBfac = kRingBytes;                             // float [kMaxInd][BN][RANK]
constexpr uint32_t kOffBnoise = kOffBfac + kMaxInd * BN * RANK * 4;  // float [kMaxInd][BN]
constexpr uint32_t kOffAfac = kOffBnoise + kMaxInd * BN * 4;         // float4 [kMaxInd][2][4][BN / 4]: next layer's A_p slice
constexpr uint32_t kOffBars = kOffAfac + kMaxInd * BN * RANK * 4;    // mbarriers + tmem base
constexpr uint32_t kSmemBytes = kOffBars + 256;                      // 231,680 B of the 232,448 B a CTA may use
constexpr unsigned long long kWaitLimitNs = 2000000000ull;           // 2 s per wait

struct GemmArgs {
  long long M, N, K;     // rows = pop * batch, out features, in features
  long long batch;       // rows per individual
  const float* bias;     // [N] or null
  const float* t;        // [M][RANK] = H A_p^T, or null (no LoRA correction)
  const long long* seeds;  // [pop]
  unsigned long long b_counter;      // Philox counter of the B stream of this weight block
  unsigned long long noise_counter;  // Philox counter of the bias-noise block
  int has_bias_noise;
  float sigma;
  int relu;
  __nv_bfloat16* out_bf16;  // [M][N] or null
  float* out_f32;           // [M][N] or null
  const float* target;      // [batch][N] or null: write row_partial instead of the output
  float* row_partial;       // [M][N / BN]
  int* error_flag;
  // K schedule: the product is summed over n_combo passes; pass c reads the K range of length K that
  // starts at column a_piece[c] * K of the first operand and b_piece[c] * K of the second (split-
  // precision products); the plain layer uses one pass over piece 0.
  int n_combo;
  int a_piece[6];
  int b_piece[6];
  float combo_scale[6];        // ACCUM variant: weight of pass c in the sum (pieces may carry a power-of-two scale)
  uint32_t operand_format;     // instruction-descriptor format bits of both operands: bf16 or fp16
  const float* out_scale_dev;  // ACCUM variant: optional device scalar multiplied into out_scale
  float out_scale;
  long long ld_out;         // row stride of out_f32 (elements)
  // Fused down-projection of the NEXT layer: its input is this layer's bf16 output, so each
  // epilogue thread also accumulates y[row][n] * A'_p[q][n] over its 128 columns (A' = the next
  // weight block's factor, counter next_a_counter, row length N) into t_partial[row][2 * n_blk + half][q].
  float* t_partial;
  unsigned long long next_a_counter;
  // The tensor core adds each K = 16 product into the fp32 accumulator with truncation, a bias that
  // grows with the number of accumulations. With chunk_kblocks > 0 an accumulator only collects that
  // many k-blocks; the epilogue (ACCUM variant of the kernel) adds the chunks in round-to-nearest fp32
  // registers and writes out_f32 once.
  int chunk_kblocks;
  // ACCUM variant only: the chunks of a tile are divided among k_split (1 or 2) work items that run on
  // different CTAs; with 2 each adds its sum into the zero-filled out_f32 with an atomic add (two addends:
  // the result does not depend on their order).
  int k_split;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait. Returns false when the limit expired or another role already reported an error.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*((volatile int*)error_flag) != 0) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        atomicCAS(error_flag, 0, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// ---- CTA-pair primitives -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\nbarrier.cluster.wait.acquire;" ::: "memory");
}
// Tile copy issued by either CTA of a pair into its OWN shared memory; the bytes are reported to the
// mbarrier at cluster address `bar` (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"((unsigned long long)map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups
// 1024 bytes apart (descriptor version 1 of sm_100).
__device__ __forceinline__ unsigned long long umma_desc(uint32_t smem_addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3ffffu) >> 4);  // start address
  d |= (unsigned long long)(1024u >> 4) << 32;             // stride byte offset
  d |= 1ull << 46;                                         // version
  d |= 2ull << 61;                                         // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: D = fp32, A = B = bf16, both K-major, N = 256, M = 128
// (M = 256 for a CTA pair: 128 rows in each CTA).
// The operand format bits (A at bit 7, B at bit 10: 0 = fp16, 1 = bf16) are added at run time.
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t kIdescPair = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
constexpr uint32_t kFormatBf16 = (1u << 7) | (1u << 10), kFormatFp16 = 0u;

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, unsigned long long a, unsigned long long b, uint32_t accumulate,
                                          uint32_t format) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(kIdesc | format), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Issued by one thread of the leader CTA: both CTAs' tensor cores multiply their own 128 rows of A by the
// 256-row B tile whose halves sit in the two CTAs' shared memory (same offsets in both).
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, unsigned long long a, unsigned long long b, uint32_t accumulate,
                                               uint32_t format) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(kIdescPair | format), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives, once the products issued so far are complete, on the barrier at offset `bar` in BOTH CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Four standard normals of Philox call `call` of one individual's stream (same arithmetic as
// philox_normal, evox/triton_kernels/kernels/philox.py:87-112).
__device__ __forceinline__ float4 normal4(unsigned long long seed, unsigned long long counter, uint32_t call) {
  const uint4 r = philox4x32_10((uint32_t)counter + call, (uint32_t)(counter >> 32), 0u, 0u, (uint32_t)seed,
                                (uint32_t)(seed >> 32));
  const float u0 = u24_to_unit(r.x), u1 = u24_to_unit(r.y), u2 = u24_to_unit(r.z), u3 = u24_to_unit(r.w);
  // hardware log / sin / cos: the angle is first brought into [-pi, pi), where their absolute
  // error is about 2^-21; the normals agree with philox_normal's to ~1e-6
  const float r0 = sqrtf(-2.0f * __logf(fmaxf(u0, 1e-10f)));
  const float r1 = sqrtf(-2.0f * __logf(fmaxf(u2, 1e-10f)));
  float a0 = 6.283185307179586f * u1, a1 = 6.283185307179586f * u3;
  if (a0 >= 3.14159265358979f) a0 -= 6.283185307179586f;
  if (a1 >= 3.14159265358979f) a1 -= 6.283185307179586f;
  float s0, c0, s1, c1;
  __sincosf(a0, &s0, &c0);
  __sincosf(a1, &s1, &c1);
  return make_float4(r0 * c0, r0 * s0, r1 * c1, r1 * s1);
}

// EPI: what the layer epilogue does, known at compile time so that none of it is a condition inside the
// per-element loops. 0: whatever the arguments say; 1: hidden layer of a virtual-LoRA network (rank-8 correction,
// ReLU, bf16 output, next layer's projection; no bias, no bias noise); 2: its last layer (rank-8 correction, squared
// error against the target; no bias, no bias noise, no ReLU). The accumulate variant ignores it.
template <bool PAIR, bool ACCUM, int EPI = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
    lora_gemm_kernel(const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_w, const GemmArgs a) {
  constexpr int STAGES = Ring<PAIR>::STAGES;
  constexpr uint32_t kStageBytes = Ring<PAIR>::kStageBytes;
  constexpr int TM = PAIR ? 2 * BM : BM;  // rows of one scheduled tile
  static_assert(STAGES <= kMaxStages, "barrier block too small");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const uint32_t smem_base = smem_u32(smem);
  if ((smem_base & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned window: refuse to run otherwise
    if (threadIdx.x == 0) atomicCAS(a.error_flag, 0, 5);
    return;
  }
  float* afac = reinterpret_cast<float*>(smem + kOffAfac);
  float* bfac = reinterpret_cast<float*>(smem + kOffBfac);
  float* bnoise = reinterpret_cast<float*>(smem + kOffBnoise);
  const uint32_t bars = smem_base + kOffBars;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBars + 8 * (2 * STAGES + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long n_tiles_n = a.N / BN;
  const long long n_tiles = (a.M / TM) * n_tiles_n;
  // a CTA pair walks the tile list together; each CTA owns 128 of the tile's 256 rows
  const uint32_t cta_rank = PAIR ? cluster_rank() : 0u;
  const long long tile_first = PAIR ? (long long)(blockIdx.x >> 1) : (long long)blockIdx.x;
  const long long tile_step = PAIR ? (long long)(gridDim.x >> 1) : (long long)gridDim.x;
  const int k_blocks = (int)(a.K / BK);
  const int total_kb = k_blocks * a.n_combo;
  const int chunk_kb = a.chunk_kblocks > 0 ? a.chunk_kblocks : total_kb;
  const int n_chunks = (total_kb + chunk_kb - 1) / chunk_kb;
  // work item w = part * n_tiles + tile: chunks [part * n_chunks / k_split, (part + 1) * n_chunks / k_split) of a tile
  const int k_split = ACCUM ? a.k_split : 1;
  const long long n_work = n_tiles * k_split;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), PAIR ? 2 * kEpilogueThreads : kEpilogueThreads);  // the leader's collects both epilogues
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {  // warp 1 of both CTAs takes part in the pair's allocation
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything is sent to them
  fence_after_sync();
  const uint32_t tmem_base = *((volatile uint32_t*)tmem_slot);

  if (warp == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t issued = 0;  // bit s: a copy into stage s may still be in flight
      bool ok = true;
      const uint32_t leader_full0 = PAIR ? map_to_cta(full_bar(0), 0u) : full_bar(0);
      for (long long work = tile_first; work < n_work && ok; work += tile_step) {
        const long long tile = work % n_tiles;
        const int part = (int)(work / n_tiles);
        const int kb_begin = (part * n_chunks / k_split) * chunk_kb;
        const int kb_end = min(((part + 1) * n_chunks / k_split) * chunk_kb, total_kb);
        const int m0 = (int)((tile / n_tiles_n) * TM) + (int)cta_rank * BM;
        const int n0 = (int)((tile % n_tiles_n) * BN) + (PAIR ? (int)cta_rank * (BN / 2) : 0);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, a.error_flag, 1)) {
            ok = false;
            break;
          }
          const int combo = kb / k_blocks, kk = kb - combo * k_blocks;
          if constexpr (PAIR) {
            if (cta_rank == 0) mbar_expect_tx(full_bar(s), Ring<PAIR>::kTxBytes);
            const uint32_t fb = leader_full0 + 8u * s;
            tma_load_2d_pair(smem_base + s * kStageBytes, &map_h, fb, (int)(a.a_piece[combo] * a.K) + kk * BK, m0);
            tma_load_2d_pair(smem_base + s * kStageBytes + kBytesA, &map_w, fb, (int)(a.b_piece[combo] * a.K) + kk * BK, n0);
          } else {
            mbar_expect_tx(full_bar(s), kStageBytes);
            tma_load_2d(smem_base + s * kStageBytes, &map_h, full_bar(s), (int)(a.a_piece[combo] * a.K) + kk * BK, m0);
            tma_load_2d(smem_base + s * kStageBytes + kBytesA, &map_w, full_bar(s), (int)(a.b_piece[combo] * a.K) + kk * BK, n0);
          }
          issued |= 1u << s;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if constexpr (PAIR) {
        // the leader's releases of this CTA's stages arrive asynchronously: see the last one of every stage
        // land before this CTA may leave
        for (int q = 0; q < STAGES && ok; ++q) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, a.error_flag, 1)) ok = false;
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (!ok) {
        // drain: the last copy issued into each stage must land before shared memory is released
        for (int q = 0; q < STAGES; ++q) {
          if (!(issued & (1u << q))) continue;
          if (PAIR && cta_rank != 0) continue;  // the follower's copies report to the leader: timed wait below
          // stage q was last filled in phase (ph if q < s else ph ^ 1)
          const uint32_t last = (q < s) ? ph : (ph ^ 1u);
          const unsigned long long t0 = global_timer_ns();
          while (!mbar_try(full_bar(q), last) && !mbar_try(full_bar(q), last ^ 1u)) {
            if (global_timer_ns() - t0 > kWaitLimitNs) break;
          }
        }
        if constexpr (PAIR) {
          // nothing in this CTA can observe the follower's copies (or the products the leader still has in
          // flight on this CTA's shared memory): give them a millisecond, far beyond their latency
          const unsigned long long t0 = global_timer_ns();
          while (global_timer_ns() - t0 < 1000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------
    if (lane == 0 && cta_rank == 0) {  // of a pair only the leader issues
      int s = 0;
      uint32_t ph = 0;
      long long it = 0;
      bool ok = true;
      for (long long work = tile_first; work < n_work && ok; work += tile_step) {
        const int part = (int)(work / n_tiles);
        const int ch0 = part * n_chunks / k_split, ch1 = (part + 1) * n_chunks / k_split;
        for (int chunk = ch0; chunk < ch1 && ok; ++chunk, ++it) {
          const int buf = (int)(it & 1);
          const uint32_t acc_ph = (uint32_t)((it >> 1) & 1);
          if (!mbar_wait(tempty_bar(buf), acc_ph ^ 1u, a.error_flag, 2)) {
            ok = false;
            break;
          }
          fence_after_sync();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          const int kb0 = chunk * chunk_kb, kb1 = min(kb0 + chunk_kb, total_kb);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(full_bar(s), ph, a.error_flag, 3)) {
              ok = false;
              break;
            }
            fence_after_sync();
            const uint32_t sa = smem_base + s * kStageBytes, sb = sa + kBytesA;
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              if constexpr (PAIR)
                umma_bf16_pair(d_tmem, umma_desc(sa + k * 32), umma_desc(sb + k * 32), (kb > kb0 || k > 0) ? 1u : 0u, a.operand_format);
              else
                umma_bf16(d_tmem, umma_desc(sa + k * 32), umma_desc(sb + k * 32), (kb > kb0 || k > 0) ? 1u : 0u, a.operand_format);
            }
            // stage reusable (in both CTAs of a pair) once these products have read it
            if constexpr (PAIR) umma_commit_pair(empty_bar(s)); else umma_commit(empty_bar(s));
            if (++s == STAGES) {
              s = 0;
              ph ^= 1u;
            }
          }
          if (ok) {  // accumulator complete
            if constexpr (PAIR) umma_commit_pair(tfull_bar(buf)); else umma_commit(tfull_bar(buf));
          }
        }
      }
    }
  } else {
    // ------------------------------- epilogue (256 threads) --------------------------------
    const int quarter = warp & 3;           // TMEM lanes this warp may read
    const int col_half = (warp - 2) >> 2;   // which 128 of the tile's 256 columns this warp handles
    const int row_in_tile = quarter * 32 + lane;
    const int et = threadIdx.x - 64;        // 0..255 within the epilogue group
    const int inds_per_tile = (a.batch >= BM) ? 1 : (int)(BM / a.batch);
    long long it = 0;
    bool ok = true;
    const uint32_t leader_tempty0 = PAIR ? map_to_cta(tempty_bar(0), 0u) : tempty_bar(0);
    for (long long work = tile_first; work < n_work; work += tile_step) {
      const long long tile = work % n_tiles;
      const int part = (int)(work / n_tiles);
      const int ch0 = part * n_chunks / k_split, ch1 = (part + 1) * n_chunks / k_split;
      const long long m0 = (tile / n_tiles_n) * TM + (long long)cta_rank * BM;
      const int n_blk = (int)(tile % n_tiles_n);
      const long long n0 = (long long)n_blk * BN;
      if constexpr (ACCUM) {
        // plain product summed over the work item's chunks in registers (one row, 128 columns per thread)
        float sum[4][32];
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[ci][j] = 0.f;
        float* o = a.out_f32 + (m0 + row_in_tile) * a.ld_out + n0 + col_half * (BN / 2);
        const float os = a.out_scale_dev ? a.out_scale * __ldg(a.out_scale_dev) : a.out_scale;
        // The chunk sums of a tile always leave as TWO rounded halves, chunks [0, n/2) and [n/2, n), added once:
        // either by two work items (k_split = 2, atomicAdd into the zero-filled output: two addends, any order) or
        // by this one, which stores the first half when it reaches the middle and adds the second at the end.
        // The result then does not depend on how many tiles the launch has (a row shard of a block gives the same
        // bits as the whole block).
        const int mid = (k_split == 1 && n_chunks >= 2) ? n_chunks / 2 : -1;
        for (int chunk = ch0; chunk < ch1; ++chunk, ++it) {
          if (chunk == mid && ok) {
#pragma unroll
            for (int ci = 0; ci < 4; ++ci)
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                *reinterpret_cast<float4*>(o + ci * 32 + j) =
                    make_float4(sum[ci][j] * os, sum[ci][j + 1] * os, sum[ci][j + 2] * os, sum[ci][j + 3] * os);
                sum[ci][j] = sum[ci][j + 1] = sum[ci][j + 2] = sum[ci][j + 3] = 0.f;
              }
          }
          const int buf = (int)(it & 1);
          const uint32_t acc_ph = (uint32_t)((it >> 1) & 1);
          if (ok && !mbar_wait(tfull_bar(buf), acc_ph, a.error_flag, 4)) ok = false;
          if (!ok) continue;
          fence_after_sync();
          const float cs = a.combo_scale[(chunk * chunk_kb) / k_blocks];  // a chunk never straddles two passes
#pragma unroll
          for (int ci = 0; ci < 4; ++ci) {
            uint32_t v[32];
            tmem_ld32(tmem_base + (uint32_t)(buf * BN + col_half * (BN / 2) + ci * 32) + ((uint32_t)(quarter * 32) << 16), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[ci][j] = fmaf(__uint_as_float(v[j]), cs, sum[ci][j]);
          }
          fence_before_sync();
          if constexpr (PAIR) mbar_arrive_cluster(leader_tempty0 + 8u * buf); else mbar_arrive(tempty_bar(buf));
        }
        if (ok) {
#pragma unroll
          for (int ci = 0; ci < 4; ++ci)
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 r = make_float4(sum[ci][j] * os, sum[ci][j + 1] * os, sum[ci][j + 2] * os, sum[ci][j + 3] * os);
              float4* dst = reinterpret_cast<float4*>(o + ci * 32 + j);
              if (k_split > 1) {
                atomicAdd(dst, r);
              } else if (mid >= 0) {
                const float4 first = *dst;  // this thread stored it at the middle chunk
                *dst = make_float4(__fadd_rn(first.x, r.x), __fadd_rn(first.y, r.y), __fadd_rn(first.z, r.z), __fadd_rn(first.w, r.w));
              } else {
                *dst = r;
              }
            }
        }
        continue;
      }
      const long long p_first = m0 / a.batch;
      // what this epilogue does: compile-time constants for the two fixed shapes, the arguments otherwise
      const bool has_t = EPI != 0 ? true : a.t != nullptr;
      const bool has_bias = EPI != 0 ? false : a.bias != nullptr;
      const bool has_noise = EPI != 0 ? false : a.has_bias_noise != 0;
      const bool do_relu = EPI == 1 ? true : (EPI == 2 ? false : a.relu != 0);
      const bool to_target = EPI == 2 ? true : (EPI == 1 ? false : a.target != nullptr);
      const bool to_bf16 = EPI == 1 ? true : (EPI == 2 ? false : a.out_bf16 != nullptr);
      const bool project = EPI == 1 ? true : (EPI == 2 ? false : a.t_partial != nullptr);
      // all epilogue threads are done with the previous tile's factors
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (has_t) {
        // B_p[n][q], q = 0..7: elements n * 8 + q of the stream -> Philox calls 2n and 2n + 1
        for (int idx = et; idx < inds_per_tile * BN * 2; idx += kEpilogueThreads) {
          const int ind = idx / (BN * 2), rest = idx - ind * (BN * 2);
          const int col = rest >> 1, half = rest & 1;
          const unsigned long long seed = (unsigned long long)a.seeds[p_first + ind];
          const float4 z = normal4(seed, a.b_counter, (uint32_t)(((n0 + col) * RANK) / 4 + half));
          *reinterpret_cast<float4*>(bfac + ((size_t)(ind * BN + col) * RANK + half * 4)) = z;
        }
      }
      if (has_noise) {
        for (int idx = et; idx < inds_per_tile * (BN / 4); idx += kEpilogueThreads) {
          const int ind = idx / (BN / 4), c4 = idx - ind * (BN / 4);
          const unsigned long long seed = (unsigned long long)a.seeds[p_first + ind];
          const float4 z = normal4(seed, a.noise_counter, (uint32_t)((n0 >> 2) + c4));
          *reinterpret_cast<float4*>(bnoise + (size_t)ind * BN + c4 * 4) = z;
        }
      }
      if (project) {
        // A'_p[q][n]: element q * N + n of the next block's stream; one call covers 4 columns of one q.
        // A task makes 4 calls (q = 4 half .. 4 half + 3) for columns 4 c4 .. 4 c4 + 3 and stores, per column,
        // the four q values as one float4 at [ind][half][column & 3][column >> 2]: neighbouring threads write
        // neighbouring float4s (the readers all read one address at a time, any layout serves them).
        for (int idx = et; idx < inds_per_tile * 2 * (BN / 4); idx += kEpilogueThreads) {
          const int ind = idx / (2 * (BN / 4)), rest = idx - ind * (2 * (BN / 4));
          const int half = rest / (BN / 4), c4 = rest - half * (BN / 4);
          const unsigned long long seed = (unsigned long long)a.seeds[p_first + ind];
          float4 z[4];
#pragma unroll
          for (int qq = 0; qq < 4; ++qq)
            z[qq] = normal4(seed, a.next_a_counter, (uint32_t)(((long long)(half * 4 + qq) * a.N + n0) / 4 + c4));
          float4* dst = reinterpret_cast<float4*>(afac) + (size_t)ind * (BN * 2) + (size_t)(half * 4) * (BN / 4) + c4;
          dst[0] = make_float4(z[0].x, z[1].x, z[2].x, z[3].x);
          dst[BN / 4] = make_float4(z[0].y, z[1].y, z[2].y, z[3].y);
          dst[2 * (BN / 4)] = make_float4(z[0].z, z[1].z, z[2].z, z[3].z);
          dst[3 * (BN / 4)] = make_float4(z[0].w, z[1].w, z[2].w, z[3].w);
        }
      }
      const long long row = m0 + row_in_tile;
      const int my_ind = (int)(row / a.batch - p_first);
      float tr[RANK];
#pragma unroll
      for (int q = 0; q < RANK; ++q) tr[q] = 0.f;
      if (has_t) {
        const float4 t0 = *reinterpret_cast<const float4*>(a.t + row * RANK);
        const float4 t1 = *reinterpret_cast<const float4*>(a.t + row * RANK + 4);
        tr[0] = t0.x; tr[1] = t0.y; tr[2] = t0.z; tr[3] = t0.w;
        tr[4] = t1.x; tr[5] = t1.y; tr[6] = t1.z; tr[7] = t1.w;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      for (int chunk = ch0; chunk < ch1; ++chunk, ++it) {
      const int buf = (int)(it & 1);
      const uint32_t acc_ph = (uint32_t)((it >> 1) & 1);
      if (ok && !mbar_wait(tfull_bar(buf), acc_ph, a.error_flag, 4)) ok = false;
      if (!ok) continue;  // keep the named barriers balanced, skip the work
      fence_after_sync();
      const float* bf = bfac + (size_t)my_ind * BN * RANK;
      const float* bn = bnoise + (size_t)my_ind * BN;
      const float* af = afac + (size_t)my_ind * BN * RANK;
      float tp[RANK];
#pragma unroll
      for (int q = 0; q < RANK; ++q) tp[q] = 0.f;
      const float* target_row = to_target ? a.target + (row % a.batch) * a.N + n0 : nullptr;
      float sq_sum = 0.f;
      for (int c = col_half * (BN / 2); c < (col_half + 1) * (BN / 2); c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + (uint32_t)(buf * BN + c) + ((uint32_t)(quarter * 32) << 16), v);
        tmem_ld_wait();
        float y[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float acc = __uint_as_float(v[j]) * a.out_scale;
          if (has_bias) acc += __ldg(a.bias + n0 + c + j);
          if (has_t) {
            const float4 b0 = *reinterpret_cast<const float4*>(bf + (size_t)(c + j) * RANK);
            const float4 b1 = *reinterpret_cast<const float4*>(bf + (size_t)(c + j) * RANK + 4);
            float dl = tr[0] * b0.x;
            dl = fmaf(tr[1], b0.y, dl);
            dl = fmaf(tr[2], b0.z, dl);
            dl = fmaf(tr[3], b0.w, dl);
            dl = fmaf(tr[4], b1.x, dl);
            dl = fmaf(tr[5], b1.y, dl);
            dl = fmaf(tr[6], b1.z, dl);
            dl = fmaf(tr[7], b1.w, dl);
            acc = fmaf(a.sigma, dl, acc);
          }
          if (has_noise) acc = fmaf(a.sigma, bn[c + j], acc);
          y[j] = do_relu ? fmaxf(acc, 0.f) : acc;
        }
        if (to_target) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 tg = __ldg(reinterpret_cast<const float4*>(target_row + c + j));
            const float d0 = y[j] - tg.x, d1 = y[j + 1] - tg.y, d2 = y[j + 2] - tg.z, d3 = y[j + 3] - tg.w;
            sq_sum = fmaf(d0, d0, sq_sum);
            sq_sum = fmaf(d1, d1, sq_sum);
            sq_sum = fmaf(d2, d2, sq_sum);
            sq_sum = fmaf(d3, d3, sq_sum);
          }
        } else if (to_bf16) {
          if (project) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float yb = __bfloat162float(__float2bfloat16_rn(y[j]));  // what the next layer will read
              const float4* af4 = reinterpret_cast<const float4*>(af) + (size_t)(j & 3) * (BN / 4) + ((c + j) >> 2);
              const float4 a0 = af4[0];             // q = 0..3 of column c + j
              const float4 a1 = af4[BN];            // q = 4..7: half 1 starts 4 * (BN / 4) float4s further
              tp[0] = fmaf(yb, a0.x, tp[0]);
              tp[1] = fmaf(yb, a0.y, tp[1]);
              tp[2] = fmaf(yb, a0.z, tp[2]);
              tp[3] = fmaf(yb, a0.w, tp[3]);
              tp[4] = fmaf(yb, a1.x, tp[4]);
              tp[5] = fmaf(yb, a1.y, tp[5]);
              tp[6] = fmaf(yb, a1.z, tp[6]);
              tp[7] = fmaf(yb, a1.w, tp[7]);
            }
          }
          __nv_bfloat16* o = a.out_bf16 + row * a.N + n0 + c;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(y[j], y[j + 1]), h1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]), h3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2);
            pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(o + j) = pk;
          }
        } else {
          float* o = a.out_f32 + row * a.ld_out + n0 + c;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            *reinterpret_cast<float4*>(o + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
          }
        }
      }
      if (to_target) a.row_partial[(row * n_tiles_n + n_blk) * 2 + col_half] = sq_sum;
      if (project && to_bf16) {
        float* o = a.t_partial + ((size_t)row * (size_t)(n_tiles_n * 2) + (size_t)(n_blk * 2 + col_half)) * RANK;
        *reinterpret_cast<float4*>(o) = make_float4(tp[0], tp[1], tp[2], tp[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(tp[4], tp[5], tp[6], tp[7]);
      }
      fence_before_sync();
      // this thread no longer reads the accumulator
      if constexpr (PAIR) mbar_arrive_cluster(leader_tempty0 + 8u * buf); else mbar_arrive(tempty_bar(buf));
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  // a pair leaves together: until here the peer may still arrive on this CTA's barriers, and the leader's
  // products read this CTA's shared memory
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 1) {
    fence_after_sync();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// t[p][b][q] = sum_k H[p][b][k] * A_p[q][k] with A_p regenerated from the seed (never stored).
// One block of 256 threads per individual. K is walked in chunks of 128 columns: the chunk of A_p
// (8 x 128 normals, fp32) and of H_p (64 rows x 128, kept in bf16) are staged in shared memory; thread
// (row group g, column slice s) accumulates 4 rows x 8 factors over columns 4s..4s+3 and 64+4s..64+4s+3,
// reading H as 8-byte and A_p as 16-byte words (24 shared-memory loads per 256 multiply-adds, all
// conflict-free); the next chunk of H is already on its way from global memory while one is processed; the
// 16 column slices are folded with shuffles at the end.
__global__ void __launch_bounds__(256)
    lora_down_bf16_kernel(const __nv_bfloat16* __restrict__ h, const long long* __restrict__ seeds, unsigned long long a_counter,
                          long long batch, long long K, float* __restrict__ t) {
  constexpr int KC = 128;
  constexpr int kRowBytes = KC * 2 + 16;  // padded row of the bf16 chunk
  __shared__ __align__(16) float sA[RANK][KC];
  __shared__ __align__(16) uint8_t sH[64 * kRowBytes];
  const long long p = blockIdx.x;
  const unsigned long long seed = (unsigned long long)seeds[p];
  const int tid = threadIdx.x;
  const int slice = tid & 15, group = tid >> 4;     // 16 column slices x 16 row groups
  const int n_pass = (int)((batch + 63) / 64);      // 64 rows (16 groups x 4) per pass
  for (int pass = 0; pass < n_pass; ++pass) {
    const int row0 = pass * 64 + group * 4;
    float acc[4][RANK];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int q = 0; q < RANK; ++q) acc[r][q] = 0.f;
    // this thread's four 16-byte pieces of a chunk: piece i is row (tid + 256 i) / 16, segment (tid + 256 i) % 16
    uint4 stage[4];
    auto fetch = [&](long long k0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = tid + 256 * i, b = idx >> 4, seg = idx & 15;
        const long long row = (long long)pass * 64 + b;
        stage[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row < batch) stage[i] = __ldcs(reinterpret_cast<const uint4*>(h + (p * batch + row) * K + k0 + seg * 8));
      }
    };
    fetch(0);
    for (long long k0 = 0; k0 < K; k0 += KC) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = tid + 256 * i, b = idx >> 4, seg = idx & 15;
        *reinterpret_cast<uint4*>(sH + b * kRowBytes + seg * 16) = stage[i];
      }
      // A_p[q][k]: element q * K + k of the stream -> Philox call (q * K + k) / 4 (K is a multiple of 4)
      {
        const int q = tid >> 5, c4 = tid & 31;  // 8 x 32 calls cover the 8 x 128 chunk
        *reinterpret_cast<float4*>(&sA[q][c4 * 4]) = normal4(seed, a_counter, (uint32_t)(((long long)q * K + k0) / 4 + c4));
      }
      __syncthreads();
      if (k0 + KC < K) fetch(k0 + KC);
#pragma unroll
      for (int set = 0; set < 2; ++set) {
        const int c = set * 64 + slice * 4;
        float4 av[RANK];
#pragma unroll
        for (int q = 0; q < RANK; ++q) av[q] = *reinterpret_cast<const float4*>(&sA[q][c]);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint2 hw = *reinterpret_cast<const uint2*>(sH + (group * 4 + r) * kRowBytes + c * 2);
          const float h0 = __uint_as_float(hw.x << 16), h1 = __uint_as_float(hw.x & 0xffff0000u);
          const float h2 = __uint_as_float(hw.y << 16), h3 = __uint_as_float(hw.y & 0xffff0000u);
#pragma unroll
          for (int q = 0; q < RANK; ++q) {
            float v = acc[r][q];
            v = fmaf(h0, av[q].x, v);
            v = fmaf(h1, av[q].y, v);
            v = fmaf(h2, av[q].z, v);
            v = fmaf(h3, av[q].w, v);
            acc[r][q] = v;
          }
        }
      }
      __syncthreads();
    }
    // fold the 16 column slices (lanes that differ in the low 4 bits)
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int q = 0; q < RANK; ++q) {
        float v = acc[r][q];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        acc[r][q] = v;
      }
    if (slice == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const long long row = row0 + r;
        if (row < batch) {
          float* o = t + (p * batch + row) * RANK;
          *reinterpret_cast<float4*>(o) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
          *reinterpret_cast<float4*>(o + 4) = make_float4(acc[r][4], acc[r][5], acc[r][6], acc[r][7]);
        }
      }
    }
  }
}

// t[row][q] = sum over the 2 * N / 256 column slices of t_partial[row][slice][q], in slice order.
__global__ void t_partial_reduce_kernel(const float* __restrict__ t_partial, long long rows, int slices, float* __restrict__ t) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= rows * RANK) return;
  const long long row = e / RANK;
  const int q = (int)(e - row * RANK);
  float s = 0.f;
  for (int j = 0; j < slices; ++j) s += t_partial[(row * slices + j) * RANK + q];
  t[e] = s;
}

// fitness[p] = -(sum of row partials of individual p) / (batch * N): negative mean squared error.
// One block of 128 threads per individual (fixed summation order: strided per thread, then a tree).
__global__ void __launch_bounds__(128)
    neg_mse_kernel(const float* __restrict__ row_partial, long long batch, long long tiles_n, long long N, long long pop,
                   float* __restrict__ fitness) {
  __shared__ float part[4];
  const long long p = blockIdx.x;
  const long long n = batch * tiles_n * 2;  // two column halves per tile
  const float* rp = row_partial + p * n;
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 128) s += rp[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) fitness[p] = -((part[0] + part[1]) + (part[2] + part[3])) / (float)(batch * N);
}

// Splitting schemes of the gradient's operands (x = sum of the pieces, piece c scaled by kPieceScale^c):
//   kSplitFp16x2  two fp16 pieces, the second one scaled by 2^11: 22 significand bits; the products
//                 hi*hi + (hi*lo + lo*hi) * 2^-11 are exact in the fp32 accumulator and miss x only by 2^-22
//   kSplitBf16x3  three bf16 pieces (24 bits), six products
//   kSplitBf16x1  plain bf16 rounding, one product
enum { kSplitFp16x2 = 0, kSplitBf16x3 = 1, kSplitBf16x1 = 2 };

template <int SCHEME>
struct Pieces {
  static constexpr int N = SCHEME == kSplitFp16x2 ? 2 : (SCHEME == kSplitBf16x3 ? 3 : 1);
  // 16-bit patterns of the pieces of x
  __device__ static __forceinline__ void split(float x, unsigned short (&out)[N]) {
    if constexpr (SCHEME == kSplitFp16x2) {
      const __half hi = __float2half_rn(x);
      const __half lo = __float2half_rn((x - __half2float(hi)) * 2048.0f);
      out[0] = __half_as_ushort(hi);
      out[1] = __half_as_ushort(lo);
    } else {
      float r = x;
#pragma unroll
      for (int c = 0; c < N; ++c) {
        const __nv_bfloat16 pc = __float2bfloat16_rn(r);
        out[c] = __bfloat16_as_ushort(pc);
        r -= __bfloat162float(pc);
      }
    }
  }
};

// scale[0] = 2^-e with 2^(e-1) <= max |fitness| < 2^e (1 if the maximum is zero or not finite), scale[1] = 2^e:
// the fp16 pieces of f_i * B_i then stay in range whatever the magnitude of the fitness.
__global__ void __launch_bounds__(256) fitness_pow2_scale_kernel(const float* __restrict__ fitness, long long pop, float* __restrict__ scale) {
  __shared__ float part[8];
  float m = 0.f;
  for (long long i = threadIdx.x; i < pop; i += 256) {
    const float v = fabsf(fitness[i]);
    if (v == v && v <= 3.0e38f) m = fmaxf(m, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, part[w]);
    int e = 0;
    if (m > 0.f) (void)frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
    e = max(-100, min(100, e));
    scale[0] = ldexpf(1.0f, -e);
    scale[1] = ldexpf(1.0f, e);
  }
}

// Operands of the population gradient sum_i f_i B_i A_i as two K-major matrices over K = pop * 8:
//   bf[j][piece * K + i * 8 + q] = piece of (f_i * B_i[j][q]),   j < d
//   at[l][piece * K + i * 8 + q] = piece of A_i[q][l],            l < k
// with the factors regenerated from the seeds (lora_noise.py:118-125) and split as SCHEME says.
template <int SCHEME>
__global__ void __launch_bounds__(256)
    lora_grad_pack_kernel(const float* __restrict__ fitness, const float* __restrict__ fit_scale, const long long* __restrict__ seeds,
                          unsigned long long a_counter, unsigned long long b_counter, long long pop, long long row_begin,
                          long long d, long long k, unsigned short* __restrict__ bf, unsigned short* __restrict__ at) {
  // d = number of rows of the block computed here, starting at row `row_begin` of the weight
  constexpr int NP = Pieces<SCHEME>::N;
  const long long Kt = pop * RANK;
  const long long n_b = pop * d;          // one task per (i, j): 8 values of B_i[j][:]
  const long long n_a = pop * (k / 4);    // one task per (i, l / 4): 8 x 4 values of A_i[:][l..l+3]
  const float fs = fit_scale ? fit_scale[0] : 1.0f;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n_b + n_a; t += (long long)gridDim.x * blockDim.x) {
    if (t < n_b) {
      // neighbouring threads take neighbouring individuals: their 16-byte pieces are adjacent in a row
      const long long j = t / pop, i = t - j * pop;
      const unsigned long long seed = (unsigned long long)seeds[i];
      const float f = fitness[i] * fs;
      const long long jg = row_begin + j;  // row of the whole weight block
      const float4 z0 = normal4(seed, b_counter, (uint32_t)(2 * jg)), z1 = normal4(seed, b_counter, (uint32_t)(2 * jg + 1));
      const float v[8] = {z0.x * f, z0.y * f, z0.z * f, z0.w * f, z1.x * f, z1.y * f, z1.z * f, z1.w * f};
      __align__(16) unsigned short pc[NP][8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        unsigned short one[NP];
        Pieces<SCHEME>::split(v[q], one);
#pragma unroll
        for (int c = 0; c < NP; ++c) pc[c][q] = one[c];
      }
#pragma unroll
      for (int c = 0; c < NP; ++c)
        *reinterpret_cast<uint4*>(bf + j * (NP * Kt) + c * Kt + i * RANK) = *reinterpret_cast<const uint4*>(pc[c]);
    } else {
      const long long u = t - n_b;
      const long long l4 = u / pop, i = u - l4 * pop;
      const unsigned long long seed = (unsigned long long)seeds[i];
      __align__(16) unsigned short pc[4][NP][8];  // [row l..l+3][piece][q]
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 z = normal4(seed, a_counter, (uint32_t)(((long long)q * k) / 4 + l4));
        const float zz[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          unsigned short one[NP];
          Pieces<SCHEME>::split(zz[r], one);
#pragma unroll
          for (int c = 0; c < NP; ++c) pc[r][c][q] = one[c];
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < NP; ++c)
          *reinterpret_cast<uint4*>(at + (l4 * 4 + r) * (NP * Kt) + c * Kt + i * RANK) = *reinterpret_cast<const uint4*>(pc[r][c]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    EVOX_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    EVOX_REQUIRE(p != nullptr && q == cudaDriverEntryPointSuccess, EVOX_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return EVOX_OK;
}

int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows, bool fp16 = false) {
  EncodeTiledFn fn;
  if (int rc = encode_fn(&fn)) return rc;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  EVOX_REQUIRE(r == CUDA_SUCCESS, EVOX_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return EVOX_OK;
}

// A CTA pair per 256 x 256 tile when the rows allow it, one CTA per 128 x 256 tile otherwise.
template <bool PAIR, bool ACCUM, int EPI = 0>
int launch_variant(cudaLaunchConfig_t& cfg, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& a) {
  EVOX_CUDA(cudaFuncSetAttribute(lora_gemm_kernel<PAIR, ACCUM, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  EVOX_CUDA(cudaLaunchKernelEx(&cfg, lora_gemm_kernel<PAIR, ACCUM, EPI>, map_a, map_b, a));
  return EVOX_OK;
}

// Share of the CTA slots that do work when `items` equal work items are dealt round-robin to `slots`.
double wave_efficiency(long long items, long long slots) {
  const long long waves = (items + slots - 1) / slots;
  return (double)items / (double)(waves * slots);
}

// accumulate = true: plain product summed chunk by chunk in registers into out_f32 (the gradient);
// otherwise the layer epilogue.
int launch_gemm(const void* a_base, long long a_rows, const void* b_base, long long b_rows, long long k_cols, GemmArgs a,
                bool accumulate, cudaStream_t stream) {
  const bool pair = (a.M % (2 * BM) == 0) && sm_count() >= 2;
  CUtensorMap map_a, map_b;
  const bool fp16 = a.operand_format == kFormatFp16;
  if (int rc = make_map(&map_a, a_base, a_rows, k_cols, BM, fp16)) return rc;
  if (int rc = make_map(&map_b, b_base, b_rows, k_cols, pair ? BN / 2 : BN, fp16)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  const long long n_tiles = (a.M / (pair ? 2 * BM : BM)) * (a.N / BN);
  const long long slots = pair ? sm_count() / 2 : sm_count();
  a.k_split = 1;
  if (accumulate) {
    // few tiles and a long K: halve each tile's chunk list when that fills the last wave better
    const long long total_kb = (a.K / BK) * a.n_combo;
    const long long n_chunks = a.chunk_kblocks > 0 ? (total_kb + a.chunk_kblocks - 1) / a.chunk_kblocks : 1;
    if (n_chunks >= 2 && wave_efficiency(2 * n_tiles, slots) > 1.03 * wave_efficiency(n_tiles, slots)) a.k_split = 2;
    if (a.k_split == 2) EVOX_CUDA(cudaMemsetAsync(a.out_f32, 0, sizeof(float) * (size_t)a.M * (size_t)a.ld_out, stream));
  }
  const long long n_work = n_tiles * a.k_split;
  const long long used = slots < n_work ? slots : n_work;
  cfg.gridDim = dim3((unsigned)(pair ? 2 * used : used));
  if (pair) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  // the two layer shapes of a virtual-LoRA network without biases get epilogues with nothing left to decide
  const bool no_bias = a.bias == nullptr && !a.has_bias_noise && a.t != nullptr;
  const bool hidden = no_bias && a.relu && a.out_bf16 != nullptr && a.t_partial != nullptr && a.target == nullptr;
  const bool last = no_bias && !a.relu && a.target != nullptr && a.row_partial != nullptr;
  int rc;
  if (accumulate)
    rc = pair ? launch_variant<true, true>(cfg, map_a, map_b, a) : launch_variant<false, true>(cfg, map_a, map_b, a);
  else if (pair && hidden)
    rc = launch_variant<true, false, 1>(cfg, map_a, map_b, a);
  else if (pair && last)
    rc = launch_variant<true, false, 2>(cfg, map_a, map_b, a);
  else
    rc = pair ? launch_variant<true, false>(cfg, map_a, map_b, a) : launch_variant<false, false>(cfg, map_a, map_b, a);
  if (rc) return rc;
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

}  // namespace
}  // namespace evox

using namespace evox;

extern "C" int evox_lora_gemm_supported(int64_t pop, int64_t batch, int64_t k, int64_t d, int32_t r) {
  return (pop > 0 && batch % 64 == 0 && (batch <= 128 ? 128 % batch == 0 : batch % 128 == 0) && (pop * batch) % BM == 0 &&
          k % BK == 0 && k >= BK && d % BN == 0 && r == RANK && batch * RANK <= 1024)
             ? 1
             : 0;
}

extern "C" int evox_lora_down_bf16(const void* h, const int64_t* seeds, uint64_t a_counter, int64_t pop, int64_t batch,
                                   int64_t k, int32_t r, float* t, void* stream) {
  EVOX_REQUIRE(h && seeds && t, EVOX_ERR_INVALID, "lora_down_bf16: NULL pointer");
  EVOX_REQUIRE(r == RANK && k % 128 == 0 && batch > 0 && pop > 0, EVOX_ERR_INVALID,
               "lora_down_bf16: needs rank 8 and k a multiple of 128");
  EVOX_REQUIRE(((uintptr_t)h & 15u) == 0, EVOX_ERR_INVALID, "lora_down_bf16: h must be 16-byte aligned");
  lora_down_bf16_kernel<<<(unsigned)pop, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)h, (const long long*)seeds, a_counter, batch, k, t);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" int evox_lora_gemm_bf16(const void* h, const void* w, const float* bias, const float* t, const int64_t* seeds,
                                   uint64_t b_counter, int32_t has_bias_noise, uint64_t noise_counter, float sigma,
                                   int64_t pop, int64_t batch, int64_t k, int64_t d, int32_t r, int32_t relu,
                                   void* out_bf16, float* out_f32, const float* target, float* row_partial,
                                   float* t_next_partial, uint64_t next_a_counter, int32_t* error_flag, void* stream) {
  EVOX_REQUIRE(h && w && seeds && error_flag, EVOX_ERR_INVALID, "lora_gemm_bf16: NULL pointer");
  EVOX_REQUIRE(evox_lora_gemm_supported(pop, batch, k, d, r), EVOX_ERR_INVALID,
               "lora_gemm_bf16: shape (pop %lld, batch %lld, k %lld, d %lld, r %d) is not supported by the tensor-core path",
               (long long)pop, (long long)batch, (long long)k, (long long)d, r);
  EVOX_REQUIRE((target != nullptr) ? (row_partial != nullptr) : ((out_bf16 != nullptr) != (out_f32 != nullptr)),
               EVOX_ERR_INVALID, "lora_gemm_bf16: give exactly one of out_bf16 / out_f32, or target + row_partial");
  EVOX_REQUIRE(((uintptr_t)h & 15u) == 0 && ((uintptr_t)w & 15u) == 0, EVOX_ERR_INVALID, "lora_gemm_bf16: operands must be 16-byte aligned");
  GemmArgs a;
  a.M = pop * batch;
  a.N = d;
  a.K = k;
  a.batch = batch;
  a.bias = bias;
  a.t = t;
  a.seeds = (const long long*)seeds;
  a.b_counter = b_counter;
  a.noise_counter = noise_counter;
  a.has_bias_noise = has_bias_noise;
  a.sigma = sigma;
  a.relu = relu;
  a.out_bf16 = (__nv_bfloat16*)out_bf16;
  a.out_f32 = out_f32;
  a.target = target;
  a.row_partial = row_partial;
  a.error_flag = error_flag;
  a.n_combo = 1;
  for (int c = 0; c < 6; ++c) a.a_piece[c] = a.b_piece[c] = 0;
  a.out_scale = 1.0f;
  a.ld_out = d;
  a.chunk_kblocks = 0;
  a.k_split = 1;
  a.operand_format = kFormatBf16;
  a.out_scale_dev = nullptr;
  for (int c = 0; c < 6; ++c) a.combo_scale[c] = 1.0f;
  a.t_partial = t_next_partial;
  a.next_a_counter = next_a_counter;
  EVOX_REQUIRE(t_next_partial == nullptr || out_bf16 != nullptr, EVOX_ERR_INVALID,
               "lora_gemm_bf16: the fused next-layer projection needs the bf16 output sink");
  return launch_gemm(h, a.M, w, d, k, a, false, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int evox_neg_mse_from_partials(const float* row_partial, int64_t pop, int64_t batch, int64_t d, float* fitness,
                                          void* stream) {
  EVOX_REQUIRE(row_partial && fitness, EVOX_ERR_INVALID, "neg_mse_from_partials: NULL pointer");
  EVOX_REQUIRE(pop > 0 && batch > 0 && d > 0 && d % BN == 0, EVOX_ERR_INVALID, "neg_mse_from_partials: bad sizes");
  neg_mse_kernel<<<(unsigned)pop, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(row_partial, batch, d / BN, d, pop, fitness);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}

extern "C" size_t evox_lora_gradient_tc_workspace_bytes(int64_t pop, int64_t d, int64_t k) {
  if (pop <= 0 || d <= 0 || k <= 0) return 0;
  // 256 bytes of scalars, then both operand matrices with up to three 16-bit pieces per value
  return 256 + (size_t)(d + k) * 3 * (size_t)pop * RANK * sizeof(__nv_bfloat16) + 512;
}

extern "C" int evox_lora_gradient_tc_supported(int64_t pop, int64_t d, int64_t k, int32_t r) {
  return (r == RANK && pop > 0 && (pop * RANK) % BK == 0 && d % BM == 0 && k % BN == 0 && 3 * pop * RANK < (1ll << 31)) ? 1 : 0;
}

extern "C" int evox_lora_gradient_tc(const float* fitness, const int64_t* seeds, uint64_t counter, int64_t pop, float sigma,
                                     int64_t row_begin, int64_t d, int64_t k, int32_t r, int32_t passes, float* grad,
                                     void* workspace, size_t workspace_bytes, int32_t* error_flag, void* stream) {
  EVOX_REQUIRE(passes == 1 || passes == 3 || passes == 6, EVOX_ERR_INVALID, "lora_gradient_tc: passes must be 1, 3 or 6");
  EVOX_REQUIRE(row_begin >= 0, EVOX_ERR_INVALID, "lora_gradient_tc: row_begin must be non-negative");
  EVOX_REQUIRE(fitness && seeds && grad && workspace && error_flag, EVOX_ERR_INVALID, "lora_gradient_tc: NULL pointer");
  EVOX_REQUIRE(evox_lora_gradient_tc_supported(pop, d, k, r), EVOX_ERR_INVALID,
               "lora_gradient_tc: shape (pop %lld, d %lld, k %lld, r %d) is not supported", (long long)pop, (long long)d, (long long)k, r);
  EVOX_REQUIRE(workspace_bytes >= evox_lora_gradient_tc_workspace_bytes(pop, d, k), EVOX_ERR_WORKSPACE, "lora_gradient_tc: workspace too small");
  EVOX_REQUIRE(((uintptr_t)workspace & 255u) == 0, EVOX_ERR_INVALID, "lora_gradient_tc: workspace must be 256-byte aligned");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long Kt = pop * RANK;
  // passes: 3 = two fp16 pieces per operand, products hi hi, hi lo, lo hi (fp32-accurate, ~1e-6);
  //         6 = three bf16 pieces, six products (~2e-6, twice the work: kept for comparison);
  //         1 = operands rounded to bf16 (~4e-3)
  const int scheme = passes == 3 ? kSplitFp16x2 : (passes == 6 ? kSplitBf16x3 : kSplitBf16x1);
  const int n_pieces = passes == 3 ? 2 : (passes == 6 ? 3 : 1);
  float* scalars = reinterpret_cast<float*>(workspace);
  unsigned short* bf = reinterpret_cast<unsigned short*>(reinterpret_cast<uint8_t*>(workspace) + 256);
  unsigned short* at = bf + (size_t)d * n_pieces * Kt;  // d * n_pieces * Kt * 2 bytes is a multiple of 256
  const unsigned long long b_counter = counter + (unsigned long long)((RANK * k + 3) / 4 * 4);
  const long long tasks = pop * d + pop * (k / 4);
  long long blocks = (tasks + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  const float* fit_scale = nullptr;
  if (scheme == kSplitFp16x2) {
    fitness_pow2_scale_kernel<<<1, 256, 0, s>>>(fitness, pop, scalars);
    EVOX_LAUNCH_CHECK();
    fit_scale = scalars;
    lora_grad_pack_kernel<kSplitFp16x2><<<grid, 256, 0, s>>>(fitness, fit_scale, (const long long*)seeds, counter, b_counter, pop,
                                                             row_begin, d, k, bf, at);
  } else if (scheme == kSplitBf16x3) {
    lora_grad_pack_kernel<kSplitBf16x3><<<grid, 256, 0, s>>>(fitness, nullptr, (const long long*)seeds, counter, b_counter, pop,
                                                             row_begin, d, k, bf, at);
  } else {
    lora_grad_pack_kernel<kSplitBf16x1><<<grid, 256, 0, s>>>(fitness, nullptr, (const long long*)seeds, counter, b_counter, pop,
                                                             row_begin, d, k, bf, at);
  }
  EVOX_LAUNCH_CHECK();
  GemmArgs a;
  a.M = d;
  a.N = k;
  a.K = Kt;
  a.batch = BM;
  a.bias = nullptr;
  a.t = nullptr;
  a.seeds = (const long long*)seeds;
  a.b_counter = 0;
  a.noise_counter = 0;
  a.has_bias_noise = 0;
  a.sigma = 0.f;
  a.relu = 0;
  a.out_bf16 = nullptr;
  a.out_f32 = grad;
  a.target = nullptr;
  a.row_partial = nullptr;
  a.error_flag = error_flag;
  a.n_combo = passes;
  if (scheme == kSplitFp16x2) {
    static const int pa[3] = {0, 0, 1}, pb[3] = {0, 1, 0};
    static const float sc[3] = {1.0f, 1.0f / 2048.0f, 1.0f / 2048.0f};
    for (int c = 0; c < 6; ++c) {
      a.a_piece[c] = pa[c % 3];
      a.b_piece[c] = pb[c % 3];
      a.combo_scale[c] = sc[c % 3];
    }
    a.operand_format = kFormatFp16;
    a.out_scale_dev = scalars + 1;  // undoes the power-of-two scaling of the fitness
  } else {
    // x = hi + mid + lo for both operands; keep every product down to 2^-24 of the largest one
    static const int pa[6] = {0, 0, 1, 0, 2, 1}, pb[6] = {0, 1, 0, 2, 0, 1};
    for (int c = 0; c < 6; ++c) {
      a.a_piece[c] = pa[c];
      a.b_piece[c] = pb[c];
      a.combo_scale[c] = 1.0f;
    }
    a.operand_format = kFormatBf16;
    a.out_scale_dev = nullptr;
  }
  a.t_partial = nullptr;
  a.next_a_counter = 0;
  a.out_scale = 1.0f / ((float)pop * sigma);
  a.ld_out = k;
  // at most 128 truncating accumulations (32 k-blocks) per accumulator, and no chunk across two passes
  const int k_blocks = (int)(Kt / BK);
  int chunk = k_blocks < 32 ? k_blocks : 32;
  while (k_blocks % chunk != 0) --chunk;
  a.chunk_kblocks = chunk;
  return launch_gemm(bf, d, at, k, (long long)n_pieces * Kt, a, true, s);
}

extern "C" int evox_lora_t_from_partials(const float* t_partial, int64_t rows, int64_t d, float* t, void* stream) {
  EVOX_REQUIRE(t_partial && t, EVOX_ERR_INVALID, "lora_t_from_partials: NULL pointer");
  EVOX_REQUIRE(rows > 0 && d > 0 && d % BN == 0, EVOX_ERR_INVALID, "lora_t_from_partials: bad sizes");
  const long long n = rows * RANK;
  t_partial_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(t_partial, rows,
                                                                                                         (int)(d / BN * 2), t);
  EVOX_LAUNCH_CHECK();
  return EVOX_OK;
}
