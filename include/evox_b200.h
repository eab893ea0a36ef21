/*
 * evox_b200 — C-ABI of the B200 (sm_100a) kernels behind the population-batched
 * generation step of EvoX (PSO step, NSGA-II / RVEA environmental selection,
 * virtual-LoRA ES forward and update) and of the algorithms that share its update shape
 * (CSO, CLPSO, SL-PSO, mating / variation of the multi-objective algorithms, PersistentES).
 *
 * Conventions
 *  - Every pointer named in a signature is a DEVICE pointer unless its comment says
 *    "host". Arrays are dense row-major. Nothing here allocates device memory unless
 *    its comment says so: outputs and scratch ("workspace") are supplied by the caller,
 *    who asks the matching *_workspace_bytes() function for the size.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *    Calls only enqueue work; none of them synchronises the device.
 *  - Return value: 0 on success, a negative EVOX_ERR_* code otherwise;
 *    evox_last_error() returns the message of the calling thread's last failure.
 *  - File and line citations name the function of the reference implementation
 *    (EMI-Group/evox, paths relative to its src/evox/) that the entry point replaces.
 */
#ifndef EVOX_B200_H_
#define EVOX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EVOX_OK 0
#define EVOX_ERR_INVALID (-1)   /* bad argument (shape, alignment, null pointer, unsupported size) */
#define EVOX_ERR_CUDA (-2)      /* a CUDA runtime call or kernel launch failed */
#define EVOX_ERR_WORKSPACE (-3) /* workspace too small */
#define EVOX_ERR_TIMEOUT (-4)   /* a bounded device-side wait gave up (status word reported it) */

/* Fitness functions fused into the PSO step (problems/numerical/basic.py). */
#define EVOX_FIT_ACKLEY 0    /* basic.py:66-69, params = {a, b, c} */
#define EVOX_FIT_RASTRIGIN 1 /* basic.py:115-116, no params */
#define EVOX_FIT_SPHERE 2    /* sum(x^2), no params */

const char* evox_last_error(void);
int evox_version(void);

/* ------------------------------------------------------------------------------------------
 * P1. Particle swarm step fused with the fitness evaluation.
 * ------------------------------------------------------------------------------------------ */

/* Evaluate a numerical test function on every row of `pop` (pop_size x dim, fp32) into
 * `fit` (pop_size). Replaces ShiftAffineNumericalProblem.evaluate with shift = affine = None
 * (problems/numerical/basic.py:52-63) for ackley_func (:66-69) and rastrigin_func (:115-116).
 * `params` is a HOST array of 3 floats (Ackley: a, b, c; ignored otherwise). */
int evox_eval_fitness(const float* pop, int64_t pop_size, int32_t dim, int32_t fitness_id,
                      const float* params, float* fit, void* stream);

/* Bytes of scratch the PSO entry points need for a shard of `pop_size` rows of `dim` columns.
 * The workspace must be zero-filled once before its first use and then left alone. */
size_t evox_pso_workspace_bytes(int64_t pop_size, int32_t dim);

/* Number of 4-byte words of one best-particle candidate record (see evox_pso_local_best). */
int32_t evox_pso_candidate_words(int32_t dim);

/* First half of PSO.step (algorithms/so/pso_variants/pso.py:92-95 with
 * pso_variants/utils.py:18-25): argmin of `fit` over this shard's rows and the row of `pop`
 * it points at, written as one candidate record
 *   word 0: fitness (fp32) | word 1,2: GLOBAL row index (int64 = row_offset + local row)
 *   word 3: 0 | words 4..4+dim-1: the row
 * so that the records of several shards can be exchanged with one allgather. Ties resolve to
 * the lowest index and NaN counts as the minimum, as torch.argmin does. */
int evox_pso_local_best(const float* fit, const float* pop, int64_t pop_size, int32_t dim,
                        int64_t row_offset, uint32_t* candidate, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Second half of min_by: fold `n_candidates` records (n_candidates * evox_pso_candidate_words
 * words, in rank order) into the running global best. The old global best wins ties, then the
 * lowest global row index (torch.cat puts the old best at index 0, pso.py:92-95).
 * With `have_previous` == 0 the old best is ignored (PSO.init_step, pso.py:108-115). */
int evox_pso_merge_best(const uint32_t* candidates, int32_t n_candidates, int32_t dim,
                        int32_t have_previous, float* global_best_location,
                        float* global_best_fit, void* stream);

/* Rest of PSO.step (pso.py:89-91 and :96-106) fused with the fitness evaluation of the moved
 * swarm: personal-best update from (fit, pop), velocity and position update with the relu-form
 * clamp (utils/jit_fix_operator.py:42-44; the velocity is clamped with the POSITION bounds,
 * pso.py:105), then fit = f(pop). pop, velocity, local_best_location, local_best_fit and fit
 * are updated in place. w, phi_p, phi_g are DEVICE scalars (the reference keeps them as 0-d
 * Parameters, pso.py:46-50). rg and rp are either both (pop_size x dim) uniform draws, in the
 * order the reference draws them (pso.py:96-97), or both NULL: then they are generated inside
 * the kernel from Philox4x32-10 with key = seed and counter = (global row, column/4,
 * generation, stream) — exactly the numbers evox_pso_fill_uniform() writes. */
int evox_pso_move_eval(float* pop, float* velocity, float* local_best_location,
                       float* local_best_fit, float* fit, const float* global_best_location,
                       const float* lb, const float* ub, const float* w, const float* phi_p,
                       const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                       int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                       uint64_t generation, int64_t row_offset, void* stream);

/* One whole single-GPU generation as two launches: local_best + merge_best, then move_eval
 * (PSO.step, pso.py:71-106). Needs no record carried from one call to the next. */
int evox_pso_step(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                  float* fit, float* global_best_location, float* global_best_fit,
                  const float* lb, const float* ub, const float* w, const float* phi_p,
                  const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                  int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                  uint64_t generation, void* workspace, size_t workspace_bytes, void* stream);

/* One whole generation of a swarm shard in ONE launch (PSO.step, pso.py:71-106, with min_by of
 * pso_variants/utils.py:6-25 split across two consecutive calls): the kernel of evox_pso_move_eval with
 *  - a head in which every warp folds `candidates` (n_candidates records in rank order, the
 *    fitness minima of the swarm as the PREVIOUS call left it) into the running global best —
 *    the old best wins ties, then the lowest global row index, exactly as evox_pso_merge_best —
 *    and moves towards the winner;
 *  - a tail in which the last block to finish stores that winner in global_best_location /
 *    global_best_fit and writes this shard's record of the NEW fit and pop to `candidate_out`
 *    (the layout of evox_pso_local_best), ready to be gathered and passed to the next call.
 * The records must describe fit and pop as they are when the call starts: after anything else
 * wrote to them, rebuild the record with evox_pso_local_best. `candidates` and `candidate_out`
 * must not overlap (alternate two buffers on a single GPU; with several shards `candidates` is
 * the gathered array). Other arguments as evox_pso_move_eval; workspace as evox_pso_local_best. */
int evox_pso_generation(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                        float* fit, float* global_best_location, float* global_best_fit,
                        const float* lb, const float* ub, const float* w, const float* phi_p,
                        const float* phi_g, const float* rg, const float* rp, int64_t pop_size,
                        int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                        uint64_t generation, int64_t row_offset, const uint32_t* candidates,
                        int32_t n_candidates, uint32_t* candidate_out, void* workspace,
                        size_t workspace_bytes, void* stream);

/* evox_pso_generation for a swarm sharded over the GPUs of one node, with the one exchange of a generation — the
 * allgather of the best-particle records — done by the kernels themselves over peer memory (NVLink), so that a
 * generation is one launch and no library collective. Every rank owns an exchange buffer of
 * evox_pso_exchange_words(dim, n_ranks) 32-bit words, zero-filled once: records[2][n_ranks][4 + dim], then
 * flags[2][n_ranks]. `peer_buffers` is a HOST array of n_ranks device addresses: rank p's buffer as this device
 * addresses it (its own buffer at index my_rank). The head waits until the flags of parity (tag & 1) in its own
 * buffer all read `tag` (the caller writes the records and flags of the first call itself), the tail stores this
 * shard's record of the new swarm into slot ((tag + 1) & 1, my_rank) of EVERY rank's buffer and then the flag
 * tag + 1: pass tag, tag + 1, tag + 2, ... on consecutive calls, never 0. Waits are bounded (about a quarter of a
 * second): a rank whose peer never writes sets *status = 1 and finishes the generation with what it has; the
 * caller reads `status` (device int32) when it synchronises. Replaces the same reference code as
 * evox_pso_generation; the reference's own distributed mode gathers fitness lists with torch.distributed
 * (workflows/std_workflow.py:185-189). */
size_t evox_pso_exchange_words(int32_t dim, int32_t n_ranks);
int evox_pso_generation_peer(float* pop, float* velocity, float* local_best_location, float* local_best_fit,
                             float* fit, float* global_best_location, float* global_best_fit, const float* lb,
                             const float* ub, const float* w, const float* phi_p, const float* phi_g,
                             const float* rg, const float* rp, int64_t pop_size, int32_t dim,
                             int32_t fitness_id, const float* params, uint64_t seed, uint64_t generation,
                             int64_t row_offset, const uint64_t* peer_buffers, int32_t n_ranks, int32_t my_rank,
                             uint32_t tag, int32_t* status, void* workspace, size_t workspace_bytes,
                             void* stream);

/* PSO.init_step (pso.py:108-115): fit = f(pop); local_best_fit = fit; global best = min_by. */
int evox_pso_init_step(const float* pop, float* fit, float* local_best_fit,
                       float* global_best_location, float* global_best_fit, int64_t pop_size,
                       int32_t dim, int32_t fitness_id, const float* params, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Materialise the uniform draws the in-kernel generator of evox_pso_move_eval uses:
 * which = 0 -> rg, 1 -> rp. out is (pop_size x dim) fp32 in [0, 1) with 24 random bits,
 * (u >> 8) * 2^-24 as in triton_kernels/kernels/philox.py:108-110. */
int evox_pso_fill_uniform(float* out, int64_t pop_size, int32_t dim, uint64_t seed,
                          uint64_t generation, int32_t which, int64_t row_offset, void* stream);

/* ------------------------------------------------------------------------------------------
 * Competitive swarm optimiser (a PSO variant with the same memory-bound update shape).
 * ------------------------------------------------------------------------------------------ */

/* Bytes of scratch evox_cso_step needs: the swarm's mean position and per-block column sums. */
size_t evox_cso_workspace_bytes(int64_t pop_size, int32_t dim);

/* CSO.step (algorithms/so/pso_variants/cso.py:71-105) fused with the evaluation of the students.
 * perm (pop_size, int64) is the random permutation of cso.py:81: pair i is (perm[i],
 * perm[i + pop_size / 2]); the one with the smaller fitness teaches (ties and NaN: the second one),
 * the other learns:  v' = l1 * velocity + l2 * (teacher - student) + phi * l3 * (center - student),
 * relu-form clamp to +-(ub - lb), position = clamp(student + v', lb, ub), fit = f(position).
 * pop and fit are updated in place for the students' rows; with store_velocity = 0 velocity is only
 * read (the reference does not store v' either, cso.py:98-105), with 1 the students' rows receive v'
 * (the rule of the original algorithm). phi is a DEVICE scalar. lambdas is the (3, pop_size / 2, dim) uniform
 * draw of cso.py:90, or NULL: then Philox4x32-10 with key = seed and counter = (pair, column / 4,
 * generation, which) supplies it. fitness_id = -1 skips the evaluation (fit is left alone): pass
 * candidates (pop_size / 2, dim) and students (pop_size / 2, int64) to get the new positions and
 * their rows for an evaluation outside.
 * The mean position (cso.py:87) is taken from the workspace when center_ready != 0, otherwise it is
 * computed first. For rows of up to 1,024 floats the update kernel accumulates the NEXT generation's
 * mean while it has every row in hand and *next_center_ready is set to 1: pass that value back as
 * center_ready of the next call if nothing else wrote to pop in between. */
int evox_cso_step(float* pop, float* velocity, int32_t store_velocity, float* fit, const int64_t* perm, const float* lb,
                  const float* ub, const float* phi, const float* lambdas, int64_t pop_size,
                  int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                  uint64_t generation, int32_t center_ready, float* candidates, int64_t* students,
                  void* workspace, size_t workspace_bytes, int32_t* next_center_ready, void* stream);

/* ------------------------------------------------------------------------------------------
 * Comprehensive-learning PSO (algorithms/so/pso_variants/clpso.py).
 * ------------------------------------------------------------------------------------------ */

/* Personal-best update of CLPSO.step (clpso.py:101-103): rows with personal_best_fit > fit copy
 * pop -> personal_best_location and fit -> personal_best_fit, in place. Must complete before
 * evox_clpso_move_eval, which reads OTHER particles' updated personal bests. */
int evox_clpso_update_pbest(const float* pop, const float* fit, float* personal_best_location,
                            float* personal_best_fit, int64_t pop_size, int32_t dim, void* stream);

/* Move of CLPSO.step (clpso.py:110-123) fused with the evaluation: for particle i,
 *   v' = w * v + c * r * (personal_best_location[source_rows[i]] - x),
 * velocity = clamp(v', lb, ub), pop = clamp(x + v', lb, ub) (relu-form clamp), fit = f(pop).
 * source_rows (pop_size, int64) is i itself or the exemplar chosen by clpso.py:95-99 and :110-115
 * (host-side bookkeeping on pop_size scalars). w, c: DEVICE scalars. r: (pop_size x dim) uniform
 * draws (clpso.py:92) or NULL for Philox4x32-10 with key = seed, counter = (row, column / 4,
 * generation). fitness_id = -1 skips the evaluation. pop, velocity (and fit) are updated in place. */
int evox_clpso_move_eval(float* pop, float* velocity, const float* personal_best_location, float* fit,
                         const int64_t* source_rows, const float* lb, const float* ub, const float* w,
                         const float* c, const float* r, int64_t pop_size, int32_t dim,
                         int32_t fitness_id, const float* params, uint64_t seed, uint64_t generation,
                         void* stream);

/* ------------------------------------------------------------------------------------------
 * Social-learning PSO (algorithms/so/pso_variants/sl_pso_gs.py, sl_pso_us.py).
 * ------------------------------------------------------------------------------------------ */

/* Bytes of scratch evox_slpso_step needs (the swarm's mean position and per-block column sums). */
size_t evox_slpso_workspace_bytes(int64_t pop_size, int32_t dim);

/* Update of SLPSOGS.step / SLPSOUS.step (sl_pso_gs.py:90-104, sl_pso_us.py:95-110) fused with the
 * evaluation. For particle i with demonstrator row k = demonstrator_rows[i] (a row of the swarm
 * BEFORE this generation, chosen by the caller as the reference does, sl_pso_gs.py:80-89):
 *   v' = r1 * v + r2 * (pop[k] - pop[i]) + (r3 * social_influence_factor) * (mean(pop) - pop[i]),
 *   pop_new[i] = clamp(pop[i] + v', lb, ub), velocity[i] = clamp(v', lb, ub), fit[i] = f(pop_new[i]).
 * pop is only read; pop_new must be a different buffer (swap the two afterwards). r1, r2, r3 are
 * the three (pop_size x dim) uniform draws or all NULL (Philox4x32-10, key = seed, counter = (row,
 * column / 4, generation, which)). social_influence_factor: DEVICE scalar. fitness_id = -1 skips
 * the evaluation. center_ready / next_center_ready as in evox_cso_step: when set on return, the
 * workspace holds mean(pop_new). */
int evox_slpso_step(const float* pop, float* pop_new, float* velocity, float* fit,
                    const int64_t* demonstrator_rows, const float* lb, const float* ub,
                    const float* social_influence_factor, const float* r1, const float* r2,
                    const float* r3, int64_t pop_size, int32_t dim, int32_t fitness_id,
                    const float* params, uint64_t seed, uint64_t generation, int32_t center_ready,
                    void* workspace, size_t workspace_bytes, int32_t* next_center_ready, void* stream);

/* ------------------------------------------------------------------------------------------
 * Differential evolution, one difference vector (algorithms/so/de_variants/de.py).
 * ------------------------------------------------------------------------------------------ */

/* Mutation, crossover and clamp of DE.step (de.py:105-146) fused with the evaluation of the trials:
 *   mutant_i = base_i + F * (pop[rows_a[i]] - pop[rows_b[i]]),
 *   trial_i  = clamp(where(cross_i < CR or column == forced_column[i], mutant_i, pop_i), lb, ub),
 *   trial_fit_i = f(trial_i).
 * base_i = pop[base_rows[i]] (base vector "rand") or pop[*best_row] for every i (base vector "best":
 * best_row is a DEVICE int64 scalar, e.g. torch.argmin(fit)); exactly one of the two is non-NULL.
 * The row and column indices are int64 device arrays of pop_size elements (de.py:112-113, :137).
 * differential_weight (F) and cross_probability (CR) are DEVICE scalars. cross is the (pop_size x dim)
 * uniform draw of de.py:136 or NULL (Philox4x32-10, key = seed, counter = (row, column / 4,
 * generation)). pop is only read; trial must be a different buffer. fitness_id = -1 skips the
 * evaluation (trial_fit may then be NULL). */
int evox_de_trial(const float* pop, float* trial, float* trial_fit, const int64_t* base_rows,
                  const int64_t* best_row, const int64_t* rows_a, const int64_t* rows_b,
                  const int64_t* forced_column, const float* lb, const float* ub,
                  const float* differential_weight, const float* cross_probability, const float* cross,
                  int64_t pop_size, int32_t dim, int32_t fitness_id, const float* params, uint64_t seed,
                  uint64_t generation, void* stream);

/* Selection of DE.step (de.py:152-157): rows with trial_fit < fit take the trial and its fitness. */
int evox_de_select(const float* trial, const float* trial_fit, float* pop, float* fit, int64_t pop_size,
                   int32_t dim, void* stream);

/* Monte-Carlo hypervolume contributions of HypE: replaces the table-building part of cal_hv
 * (algorithms/mo/hype.py:28-38). fit (n x m) objective rows, samples (n_sample x m) sampling points,
 * alpha (n) the weights of hype.py:14-24, volume a DEVICE scalar = prod(ref - f_min). For every sample s
 * count_s = the number of rows with (fit - sample) <= 0 in every objective (integer, exact); then
 *   hv[i] = (sum over the samples s that row i covers of alpha[count_s - 1]) * volume / n_sample.
 * Nothing of size n x n_sample is stored; the counts are exact and the fp32 sum of one row's weights is
 * taken in a fixed order (four interleaved chains per slice of samples, slices in order).
 * 1 <= m <= 32. workspace: evox_hv_workspace_bytes(n, n_sample) bytes. */
size_t evox_hv_workspace_bytes(int64_t n, int64_t n_sample);
int evox_hv_contribution(const float* fit, const float* samples, const float* alpha, const float* volume,
                         int64_t n, int32_t m, int64_t n_sample, float* hv, void* workspace,
                         size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * P2. NSGA-II environmental selection.
 * ------------------------------------------------------------------------------------------ */

/* Scratch bytes for the three entry points below (dominated by the bit-packed dominance
 * matrix, n * ceil(n / 1024) * 128 bytes). The workspace needs no initialisation and must be
 * 256-byte aligned. */
size_t evox_nds_workspace_bytes(int64_t n, int32_t m);

/* Non-domination rank of every row of f (n x m, fp32): rank 0 = non-dominated, rank r = non-
 * dominated once ranks < r are removed. Replaces non_dominate_rank
 * (operators/selection/non_dominate.py:172-195: dominate_relation :6-26 + the front-peeling
 * loop :151-169); rank is int32 like the reference's. NaN objectives compare false both ways.
 * `status` (optional, device int32[2]) receives {0 = ok | 1 = a bounded grid-barrier wait gave
 * up | 2 = no progress, number of fronts}. */
int evox_nd_rank(const float* f, int64_t n, int32_t m, int32_t* rank, int32_t* status,
                 void* workspace, size_t workspace_bytes, void* stream);

/* Crowding distance of the rows selected by `mask` (n bytes, non-zero = selected), -inf for
 * the others. Replaces crowding_distance (non_dominate.py:198-231) including its stable
 * tie-breaking (utils/jit_fix_operator.py:216-252) and its treatment of rows that are first or
 * last in any objective (+inf). */
int evox_crowding_distance(const float* costs, const uint8_t* mask, int64_t n, int32_t m,
                           float* distance, void* workspace, size_t workspace_bytes, void* stream);

/* rank -> last admitted front -> crowding distance on it -> the first `topk` rows in the order
 * lexsort([-crowding, rank]) -> gathered x (topk x dx), f (topk x m), rank, crowding distance.
 * Replaces nd_environmental_selection (non_dominate.py:234-254). `out_index` (optional, int64)
 * receives the selected row numbers, `status` as in evox_nd_rank. */
int evox_nd_environmental_selection(const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                                    int64_t topk, float* out_x, float* out_f, int32_t* out_rank,
                                    float* out_crowd, int64_t* out_index, int32_t* status,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* Non-dominated rank with the dominance matrix split over several GPUs: the per-front exchange the
 * reference's distributed workflow has no counterpart for (it replicates the whole selection on every rank,
 * workflows/std_workflow.py:167-189); the arithmetic is dominate_relation and the peeling loop of
 * non_dominate_rank (operators/selection/non_dominate.py:6-26, 151-169).
 * All GPUs hold f (n x m) and agree on a row order `perm` (uint32[n], position -> row of f; NULL = identity)
 * and on n_cols = number of shards * shard_rows >= n, shard_rows a multiple of 1,024. A GPU keeps rows
 * [shard_begin, shard_begin + shard_rows) of the bit matrix (shard_rows * n_cols / 8 bytes) in its workspace.
 *   evox_nd_rank_shard_begin  builds them, sets rank_local (int32[shard_rows]) to -1 and writes the shard's
 *       slice of the unranked mask (shard_rows / 32 words). start_word (optional, int32[shard_rows]): first word
 *       of each row that can hold a dominator.
 *   evox_nd_rank_shard_front  peels one front: mask_full (n_cols / 32 words = every shard's slice, gathered)
 *       -> rank_local = `front` for the shard's columns that join it, and the shard's slice of the next mask.
 * The caller gathers the slices after every front and stops when the gathered mask is empty; the ranks in
 * the caller's order are rank[perm[shard_begin + a]] = rank_local[a]. */
size_t evox_nds_shard_workspace_bytes(int64_t n_cols, int32_t m, int64_t shard_rows);
int evox_nd_rank_shard_begin(const float* f, int64_t n, int32_t m, const uint32_t* perm, int64_t n_cols,
                             int64_t shard_begin, int64_t shard_rows, const int32_t* start_word,
                             uint32_t* mask_slice, int32_t* rank_local, void* workspace,
                             size_t workspace_bytes, void* stream);
int evox_nd_rank_shard_front(int64_t n_cols, int32_t m, int64_t shard_begin, int64_t shard_rows,
                             const uint32_t* mask_full, int32_t front, uint32_t* mask_slice_out,
                             int32_t* rank_local, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * P3. RVEA reference-vector-guided selection.
 * ------------------------------------------------------------------------------------------ */

size_t evox_rvea_workspace_bytes(int64_t n, int32_t m, int32_t nv);

/* For every reference vector v_j (nv x m) the individual with the smallest angle-penalised
 * distance among those associated with it; rows of x (n x dx) and f (n x m) are gathered into
 * next_x (nv x dx) and next_f (nv x m), NaN rows for vectors nobody is associated with.
 * Replaces ref_vec_guided (operators/selection/rvea_selection.py:32-99, apd_fn :7-29): ideal
 * point by nanmin, objectives floored at 1e-32, cosine similarity with eps 1e-8, relu-form
 * clamp to [0,1], arccos, first-minimum association (individuals with a NaN objective join no
 * vector), APD = (1 + m * theta * angle) / gamma_j * |f - z|, first-minimum per vector.
 * `theta` is a DEVICE scalar (the reference passes a 0-d tensor). `next_index` (optional,
 * int64[nv]) receives the chosen row numbers, -1 for empty vectors. m <= 32.
 * The unit vectors and gamma_j (rvea_selection.py:63-71) stay in the workspace after a call:
 * `vectors_ready` != 0 says that v, nv, m and the workspace are those of the previous call and
 * that nothing else wrote to the workspace, and the two kernels that derive them are skipped
 * (the reference vectors of RVEA change only every 1 / fr generations, rvea.py:107-133). */
int evox_ref_vec_guided(const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                        const float* v, int32_t nv, const float* theta, int32_t vectors_ready,
                        float* next_x, float* next_f, int64_t* next_index, void* workspace,
                        size_t workspace_bytes, void* stream);

/* evox_ref_vec_guided for a population whose rows are spread over several GPUs. Each shard holds
 * rows [row_offset, row_offset + n) of x and f. phase 1: `ideal` (m floats) = this shard's column
 * minima (the caller takes the minimum over shards). phase 2: with the global `ideal`,
 * `best_keys` (nv int64) = this shard's winners packed as (APD bits << 32 | global row) (the caller
 * takes the minimum over shards; all-ones = nobody). phase 3: with the global `best_keys`, next_x /
 * next_f = the winners' rows this shard owns and zeros elsewhere (the caller sums over shards and
 * writes NaN where next_index is -1); next_index = global row numbers. Same arithmetic as the
 * single-GPU call, so the result does not depend on the sharding. */
int evox_ref_vec_guided_phase(int32_t phase, const float* x, int64_t dx, const float* f, int64_t n, int32_t m,
                              const float* v, int32_t nv, const float* theta, int64_t row_offset,
                              float* ideal, int64_t* best_keys, float* next_x, float* next_f,
                              int64_t* next_index, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Mating and variation around P2 / P3 (NSGA2.step, RVEA.step).
 * ------------------------------------------------------------------------------------------ */

/* selected[r] = the candidate of parents[r][0..tournament_size) that sorts first by the LAST column
 * of fitness (n_candidates x n_keys), ties by the earlier columns, ties by tournament slot.
 * Replaces tournament_selection_multifit (operators/selection/tournament_selection.py:8-29) given
 * its randint draw `parents`. */
int evox_tournament_multifit(const int64_t* parents, int64_t n_round, int32_t tournament_size,
                             const float* fitness, int64_t n_candidates, int32_t n_keys,
                             int64_t* selected, void* stream);

/* offspring (2 * (n / 2) x dim) from parents pop[mating_pool] (or rows 0..n-1 when mating_pool is
 * NULL): simulated binary crossover (operators/crossover/sbx.py:4-39; flags bit 0), polynomial
 * mutation (operators/mutation/pm_mutation.py:6-68; bit 1) and the relu-form clamp that NSGA2.step
 * and RVEA.step apply next (algorithms/mo/nsga2.py:95-97; bit 2) in one pass. The six draw tensors
 * are the reference's torch.rand / randint results in its order (sbx: mu, sign in {0,1} int64,
 * half, pc — each (n/2 x dim); mutation: site, mu — each (2*(n/2) x dim)); all NULL = Philox
 * streams keyed by (seed, generation). */
int evox_offspring(const float* pop, const int64_t* mating_pool, int64_t n, int32_t dim, const float* lb,
                   const float* ub, const float* sbx_mu, const int64_t* sbx_sign, const float* sbx_half,
                   const float* sbx_pc, const float* pm_site, const float* pm_mu, float pro_c, float dis_c,
                   float pro_m, float dis_m, int32_t flags, uint64_t seed, uint64_t generation,
                   float* offspring, void* stream);

/* ------------------------------------------------------------------------------------------
 * P4. Evolution strategies: Philox streams, virtual LoRA population, OpenES.
 * ------------------------------------------------------------------------------------------ */

/* out (pop x n, fp32): per-individual Philox4x32-10 streams, key = int64 seed split low / high,
 * counter low word + call index (no carry into the high word), 24-bit uniforms in [0, 1).
 * Replaces philox_uniform (triton_kernels/kernels/philox.py:52-84, Triton kernel :134-246). */
int evox_philox_uniform(const int64_t* seeds, int64_t pop, int64_t n, uint64_t counter, float* out,
                        void* stream);

/* Standard normals by Box-Muller on consecutive uniform pairs of the same streams.
 * Replaces philox_normal (philox.py:87-112). */
int evox_philox_normal(const int64_t* seeds, int64_t pop, int64_t n, uint64_t counter, float* out,
                       void* stream);

/* t (pop x batch x r) = x A^T per individual; x is (pop x batch x k), or (batch x k) shared by
 * all individuals when x_is_shared != 0; A is (pop x r x k). First half of lora_delta_output
 * (triton_kernels/kernels/lora_noise.py:151). */
int evox_lora_down(const float* x, int32_t x_is_shared, const float* A, int64_t pop, int64_t batch,
                   int64_t k, int32_t r, float* t, void* stream);

/* out (pop x batch x d) = sigma * (x A^T) B^T with B (pop x d x r). Replaces lora_delta_output
 * (lora_noise.py:130-154). t_scratch: pop * batch * r floats. sigma is a host value, as in the
 * reference's signature. */
int evox_lora_delta_output(const float* x, const float* A, const float* B, float sigma, int64_t pop,
                           int64_t batch, int64_t k, int32_t r, int64_t d, float* out,
                           float* t_scratch, void* stream);

/* grad (d x k) = sum_i fitness_i B_i A_i / (pop * sigma); with B == NULL, A is the (pop x k)
 * noise of a 1-D block and grad (k) = fitness A / (pop * sigma). Replaces lora_gradient
 * (lora_noise.py:157-196). */
int evox_lora_gradient(const float* fitness, const float* A, const float* B, int64_t pop, float sigma,
                       int64_t d, int64_t k, int32_t r, float* grad, void* stream);

/* One Linear layer of the virtual-population forward pass, fp32
 * (problems/neuroevolution/virtual_lora_problem.py:160-193):
 *   out = act(h W^T + bias + sigma * t B^T + sigma * bias_noise), act = ReLU if relu != 0.
 * h: (pop x batch x k) or shared (batch x k); W: (d x k); bias, bias_noise (pop x d): optional;
 * t (pop x batch x r) = h A^T from evox_lora_down and B (pop x d x r): both or neither. */
int evox_lora_linear_forward(const float* h, int32_t h_is_shared, const float* W, const float* bias,
                             const float* t, const float* B, const float* bias_noise, float sigma,
                             int64_t pop, int64_t batch, int64_t k, int64_t d, int32_t r, int32_t relu,
                             float* out, void* stream);

/* population (pop x dim) = center + sigma * noise, where noise is (noise_rows x dim) and rows
 * noise_rows.. reuse it negated when noise_rows == pop / 2 (mirrored sampling).
 * First half of OpenES.step (algorithms/so/es_variants/open_es.py:62-68). sigma: device scalar. */
int evox_openes_ask(const float* center, const float* noise, const float* sigma, int64_t pop,
                    int64_t dim, int64_t noise_rows, float* population, void* stream);

/* PersistentES.step, first half (algorithms/so/es_variants/persistent_es.py:76-80): with
 * perts = +-sigma * noise (noise: pop / 2 rows, mirrored), population = center + perts and
 * pert_accum (pop x dim) += perts, in one pass. sigma: device scalar. */
int evox_pes_ask(const float* center, const float* noise, const float* sigma, int64_t pop, int64_t dim,
                 float* pert_accum, float* population, void* stream);

/* population (pop x dim) = center + noise * sigma with one step size PER COORDINATE (sigma: dim
 * floats), the sampling of SNES and DES (es_variants/snes.py:79, des.py:60). */
int evox_es_ask_diag(const float* center, const float* noise, const float* sigma, int64_t pop, int64_t dim,
                     float* population, void* stream);

/* Two row-weighted column sums of x (pop x dim) in one pass over x:
 *   first[l] = sum_i w_i x_il,   second[l] = sum_i w_i ((x_il - shift_l)^2 + offset),
 * row_weights[i] being the weight of row i's fitness rank. SNES (snes.py:83-84): x = noise, shift = NULL,
 * offset = -1 gives grad_mean and grad_sigma; DES (des.py:66-67): x = population, shift = center,
 * offset = 0 gives the weighted mean and the weighted squared deviation. */
int evox_rank_weighted_moments(const float* x, const float* row_weights, const float* shift, float offset,
                               int64_t pop, int64_t dim, float* first, float* second, void* stream);

/* grad (dim) = noise^T fitness / pop / sigma (open_es.py:70), same mirrored convention. */
int evox_openes_gradient(const float* noise, const float* fitness, int64_t pop, int64_t dim,
                         int64_t noise_rows, float sigma, float* grad, void* stream);

/* center -= lr * grad (open_es.py:71-72, virtual_lora_es.py:123-124), or with exp_avg /
 * exp_avg_sq given the reference's Adam (es_variants/adam_step.py:4-26: no bias correction).
 * learning_rate, beta1, beta2 are device scalars; the state is updated in place. */
int evox_es_update(float* center, const float* grad, const float* learning_rate, float* exp_avg,
                   float* exp_avg_sq, const float* beta1, const float* beta2, float eps, int64_t dim,
                   void* stream);

/* 1 if evox_lora_gemm_bf16 / evox_lora_down_bf16 accept this layer shape: batch 64 or 128,
 * pop * batch a multiple of 128, k a multiple of 256, d a multiple of 256, rank 8. */
int evox_lora_gemm_supported(int64_t pop, int64_t batch, int64_t k, int64_t d, int32_t r);

/* t (pop x batch x 8, fp32) = h A_p^T for bf16 activations h (pop x batch x k); A_p (8 x k) is
 * regenerated in the kernel from seeds / a_counter exactly as generate_lora_factors would
 * (lora_noise.py:118-125) and never written to memory. */
int evox_lora_down_bf16(const void* h, const int64_t* seeds, uint64_t a_counter, int64_t pop,
                        int64_t batch, int64_t k, int32_t r, float* t, void* stream);

/* One Linear layer of the virtual-population forward pass on the tensor cores
 * (virtual_lora_problem.py:160-193): bf16 h (pop*batch x k) and W (d x k), fp32 accumulation,
 *   y = act(h W^T + bias + sigma * t B_p^T + sigma * bias_noise_p)
 * with B_p (d x 8) and the bias noise regenerated in the epilogue from the Philox streams
 * (b_counter = block counter + ceil4(8 k); noise_counter = the bias block's counter).
 * t = NULL skips the correction. Exactly one sink: out_bf16 (pop*batch x d), out_f32, or
 * target (batch x d, fp32, shared by all individuals) + row_partial (pop*batch x d/128) which
 * receives per-row sums of (y - target)^2 instead of y. With the bf16 sink, t_next_partial
 * (pop*batch x 2*d/256 x 8, optional) receives the partial down-projection of the NEXT layer,
 * y_bf16 A'_p^T over each 128-column slice, A'_p being the factor at next_a_counter with row
 * length d; evox_lora_t_from_partials sums the slices. error_flag: device int32, zero on entry;
 * non-zero afterwards means a bounded wait expired (1 producer, 2/3 issuer, 4 epilogue) or the
 * shared-memory window was not 1024-byte aligned (5). */
int evox_lora_gemm_bf16(const void* h, const void* w, const float* bias, const float* t,
                        const int64_t* seeds, uint64_t b_counter, int32_t has_bias_noise,
                        uint64_t noise_counter, float sigma, int64_t pop, int64_t batch, int64_t k,
                        int64_t d, int32_t r, int32_t relu, void* out_bf16, float* out_f32,
                        const float* target, float* row_partial, float* t_next_partial,
                        uint64_t next_a_counter, int32_t* error_flag, void* stream);

/* t (rows x 8) = sum of the 2 * d / 256 column slices of t_next_partial, in slice order: the
 * next layer's h A_p^T, accumulated by evox_lora_gemm_bf16 while it still held its output. */
int evox_lora_t_from_partials(const float* t_partial, int64_t rows, int64_t d, float* t, void* stream);

/* Population gradient of a 2-D block on the tensor cores without materialising fp32 factors:
 *   grad (d x k, fp32) = sum_i fitness_i B_i A_i / (pop * sigma)       (lora_noise.py:157-196)
 * with A_i, B_i regenerated from seeds / counter as generate_lora_factors does. With passes = 3
 * the kernel writes f_i B_i (fitness first normalised by a power of two) and A_i as two fp16
 * pieces each, x = hi + lo / 2048, into the workspace and sums the three tcgen05 products hi hi,
 * hi lo, lo hi; every product is exact in the fp32 accumulator, accumulators are drained every 32
 * k-blocks and added in round-to-nearest fp32 registers, so the result stays within about 1e-6 of
 * the reference's fp32 einsum. passes = 6 does the same with three bf16 pieces and six products
 * (twice the work, same accuracy); passes = 1 is a plain bf16 product (about 4e-3), for callers
 * that prefer speed. Needs rank 8, d a multiple of 128, k a multiple of 256, pop a multiple of 8
 * (evox_lora_gradient_tc_supported). error_flag as above.
 * Only the d rows starting at row `row_begin` of the weight are computed (grad points at the
 * first of them): ranks that shard a block by rows each pass their own range. When the tile count
 * is small against the SM count, a tile's K range is halved between two CTA groups that add into
 * the zero-filled grad (two addends, order-independent). */
size_t evox_lora_gradient_tc_workspace_bytes(int64_t pop, int64_t d, int64_t k);
int evox_lora_gradient_tc_supported(int64_t pop, int64_t d, int64_t k, int32_t r);
int evox_lora_gradient_tc(const float* fitness, const int64_t* seeds, uint64_t counter, int64_t pop,
                          float sigma, int64_t row_begin, int64_t d, int64_t k, int32_t r, int32_t passes,
                          float* grad, void* workspace, size_t workspace_bytes, int32_t* error_flag,
                          void* stream);

/* fitness (pop) = -(sum of an individual's row_partial entries) / (batch * d): negative mean
 * squared error of the last layer, summed in a fixed order. */
int evox_neg_mse_from_partials(const float* row_partial, int64_t pop, int64_t batch, int64_t d,
                               float* fitness, void* stream);

/* evox_nd_rank for callers that cannot allocate device memory: no workspace argument, and the
 * call itself allocates nothing (no cudaMalloc / cudaFree, no allocating library routine). It
 * has no counterpart in the reference. It is meant for hosts that only own the buffers they
 * were handed — a plug-in inside another application's memory arena, a loop that must leave
 * the allocator untouched while it runs. The scratch (objectives, dominance bits, masks) is a
 * fixed 4 MiB array inside the library image, present on every GPU that loads the library
 * until the process exits; hence the limits n <= 4096 rows and m <= 16 objectives, beyond which
 * the call fails with EVOX_ERR_INVALID and evox_nd_rank must be used. Same results as
 * evox_nd_rank; `f`, `rank` and the optional `status` are still the caller's buffers.
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture. The address is kept for
 * the life of that device's primary context: after a cudaDeviceReset (or any other teardown of
 * the context) in the same process the entry point must not be called again. All calls on a device
 * share the one array and it keeps the previous call's contents (everything that is read is
 * rewritten first), so two calls must not overlap on the GPU: issue them on one stream, or
 * order them with events. */
int evox_nd_rank_static(const float* f, int64_t n, int32_t m, int32_t* rank, int32_t* status,
                        void* stream);

/* ------------------------------------------------------------------------------------------
 * Measurement support.
 * ------------------------------------------------------------------------------------------ */

/* Issue-rate microbenchmark for the roofline of the dominance phase of non_dominate_rank
 * (operators/selection/non_dominate.py:6-26: m * n^2 fp32 comparisons on kilobytes of input).
 * Every one of evox_bench_compare_rate_threads() threads performs 64 * iterations fp32 "<=" comparisons
 * combined into predicates; `in` holds 1,024 floats (in[1023] is the per-iteration increment of the
 * compared values), `out` receives one word per thread. The caller times the call with CUDA events. */
int64_t evox_bench_compare_rate_threads(void);
int evox_bench_compare_rate(const float* in, uint32_t* out, int32_t iterations, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EVOX_B200_H_ */
