/*
 * lithos_b200.h -- C ABI of the B200 (sm_100a) generation-control library.
 *
 * The library replaces, for NVIDIA B200, the tail of every lithos-metal step program: the dispatches that turn
 * the language-model head's logits into tokens (greedy argmax, or penalties -> temperature -> top-k / top-p / min-p
 * thresholds -> a seeded draw) and the DSpark speculative-verification step (accept prefix + residual resample),
 * plus the scalar step-closing kernels (accept_scan, verify_select, advance) that keep control on the GPU.
 *
 * Conventions
 *   - plain pointers and sizes only; every data pointer is DEVICE memory unless a comment says "host";
 *   - the caller owns every buffer; scratch is sized by lm_workspace_bytes() and passed in; kernels leave the
 *     workspace reusable (a workspace must be zero-filled once before its first use, belongs to the device and the entry points
 *     it was first used with, and must not be written by the caller afterwards: the verify step keeps a launch count in it);
 *   - every call is asynchronous on the CUDA stream given (a cudaStream_t passed as void*; NULL = default stream);
 *   - every entry point returns LM_OK (0) or a negative LM_E_* code; nothing throws across this boundary;
 *   - there is no CPU fallback: without a CUDA device the entry points return LM_E_CUDA.
 *
 * Each declaration cites the lithos-metal interface it stands in for (path within that project : lines).
 */
#ifndef LITHOS_B200_H
#define LITHOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LM_ABI_VERSION 3

#if defined(__GNUC__)
#define LM_API __attribute__((visibility("default")))
#else
#define LM_API
#endif

/* error codes */
#define LM_OK 0
#define LM_E_INVALID (-1)    /* bad argument (null pointer, negative size, unknown enum, temperature < 0, ...) */
#define LM_E_WORKSPACE (-2)  /* workspace missing, misaligned or smaller than lm_workspace_bytes() */
#define LM_E_CUDA (-3)       /* a CUDA runtime call failed (no device, launch error); see lm_last_cuda_error() */
#define LM_E_UNSUPPORTED (-4)/* a size outside the supported range (vocab > LM_MAX_VOCAB, rows > 2^31-1, ...) */

/* logits element types */
#define LM_DTYPE_BF16 0
#define LM_DTYPE_F32 1

/* draw modes */
#define LM_DRAW_GUMBEL 0       /* argmax(z/T + Gumbel noise), noise from the splitmix64 hash of (seed, step, row, index) */
#define LM_DRAW_INVERSE_CDF 1  /* inverse CDF over the kept set ordered by descending logit (equal logits by ascending index: the order of a
                                  sorted top-p pipeline), on integer fixed-point weights, from a caller-supplied uniform */

/* lm_sample_args.flags */
#define LM_FLAG_TOPP_IN_TOPK 1u /* top-p over the top-k set's renormalised mass (the Hugging Face warpers' order) */
#define LM_FLAG_EXACT_ONLY 2u /* skip the one-pass candidate kernel for rows with a top_k: every row takes the histogram path (same results) */
#define LM_FLAG_GRID_LIMIT(n) (((uint32_t)(n) & 0xFFu) << 8) /* at most n thread blocks (0 = one per SM): leaves SMs to other streams */

/* per-row status bits written to lm_sample_args.out_status (optional) */
#define LM_STATUS_GENERIC_PATH 1u /* the row was handled by the generic multi-pass path */
#define LM_STATUS_NAN 2u          /* the row holds a NaN: results for the row are unspecified */
#define LM_STATUS_NEAR_TIE 4u     /* Gumbel draw: best and second-best key closer than 4e-6 (float32 log is library-specific) */
#define LM_STATUS_TOPP_EDGE 8u    /* top-p: cumulative mass within 1e-12 (relative) of the target at the boundary */
#define LM_STATUS_CANDIDATE_PATH 64u /* the row was finished by the one-pass candidate path (informational) */
#define LM_STATUS_SLICED_PATH 256u /* the row was cut into slices over the whole GPU (calls of a few rows; informational) */
#define LM_STATUS_TILE_DECLINED 128u /* lm_tile_finish only: the row was not sampled (token -1); materialise it and call lm_sample */

#define LM_MAX_VOCAB 1048576

/*
 * One sampling step over `rows` independent rows of logits.
 *
 * Stands in for the sampler dispatch chain argmax_partial/argmax_final (kernels/common/argmax.metal:36-99) and
 * sample_hist/sample_select/sample_gumbel/argmax_final (kernels/common/sample.metal:34-198) with the parameter
 * record SampleParams (kernels/common/sample.metal:14-16, monolith/kernels.py:756-768), whose numpy definition is
 * monolith/nn/sampling_ref.py:20-71 and whose module front ends are GreedySampler / StochasticSampler
 * (monolith/nn/sampler.py:15-53). Extensions beyond the reference: per-row knobs, repetition / presence penalties over
 * a token history, FP32 logits, and the inverse-CDF draw from caller-supplied uniforms.
 *
 * Per row r (global row index g = row_offset + r):
 *   z = float32(logits[r, :]); for every distinct history id in [0, vocab): z = (z > 0 ? z / rho : z * rho) - pi;
 *   temperature == 0: token = lowest index of max z (greedy);
 *   otherwise tau = max of the enabled thresholds {k-th largest z (ties kept), the value where the descending
 *   cumulative softmax mass of z/T first reaches top_p * total, vmax + T * ln(min_p)}, kept set = {z >= tau};
 *   draw == LM_DRAW_GUMBEL:      token = argmax over the kept set of z * float32(1/T) + gumbel(seed, step, g, index);
 *   draw == LM_DRAW_INVERSE_CDF: token = first kept index whose cumulative fixed-point weight exceeds
 *                                floor(floor(u * 2^24) * total / 2^24), weights = floor(2^40 * 2^((z - vmax) * log2(e)/T)).
 */
typedef struct lm_sample_args {
  uint32_t struct_size;        /* sizeof(lm_sample_args), for forward compatibility */
  int32_t dtype;               /* LM_DTYPE_* */
  const void* logits;          /* [rows, row_stride] elements; row r starts at logits + r * row_stride */
  int64_t rows;
  int64_t vocab;
  int64_t row_stride;          /* in elements, >= vocab */
  /* knobs: a device array with one entry per row, or NULL to use the scalar next to it for every row */
  const float* temperature;  float temperature_s;   /* 0 = greedy */
  const int32_t* top_k;      int32_t top_k_s;       /* <= 0 = off */
  const float* top_p;        float top_p_s;         /* on iff 0 < p < 1 */
  const float* min_p;        float min_p_s;         /* on iff > 0 */
  uint32_t flags;              /* LM_FLAG_* */
  int32_t draw;                /* LM_DRAW_* */
  /* penalties: off when history == NULL or (rho == 1 and pi == 0) */
  const int32_t* history;      /* [rows, hist_stride] token ids; duplicates allowed; ids outside [0, vocab) ignored */
  int64_t hist_len;
  int64_t hist_stride;
  float repetition_penalty;    /* rho */
  float presence_penalty;      /* pi */
  /* randomness */
  const float* uniforms;       /* [rows] in [0, 1): required for LM_DRAW_INVERSE_CDF */
  uint64_t seed;               /* LM_DRAW_GUMBEL */
  uint32_t step;               /* LM_DRAW_GUMBEL */
  int64_t row_offset;          /* global index of row 0 (row-sharded batches keep results independent of the split) */
  /* outputs (out_tokens required, the rest optional) */
  int32_t* out_tokens;         /* [rows] */
  float* out_tau;              /* [rows] threshold (-inf if none, or greedy) */
  float* out_stats;            /* [rows, 2]: (max logit, FP64 softmax mass of the kept set rounded to float) */
  float* out_probs;            /* [rows, probs_stride]: kept-token probabilities, 0 off the kept set */
  int64_t probs_stride;
  uint32_t* out_status;        /* [rows] LM_STATUS_* bits */
  /* scratch */
  void* workspace;             /* lm_workspace_bytes(rows, vocab) bytes, 256-byte aligned, zero-filled once */
  size_t workspace_bytes;
  void* stream;                /* cudaStream_t */
  /* GPU-resident control (optional): a StepState buffer of layout (t_max, gamma_max). When given, the kernels read on the
   * device what the reference's kernels read there (kernels/common/sample.metal:172-181, argmax.metal:44-46): the noise seed
   * (rng_hi:rng_lo) and step replace `seed` / `step`, only the first t_this_step rows are sampled (the others are left
   * untouched), and nothing is written once the state is done. A captured CUDA graph then draws fresh noise on every replay. */
  const void* step_state;
  int32_t t_max, gamma_max;
  float* out_vmax;             /* [rows] each row's maximum logit (after penalties), or NULL: what the verify step takes as
                                  lm_verify_args.target_vmax when the same rows were sampled without penalties (the reference's
                                  KEPT_STATS carry it from its sampler to its verify kernels) */
  uint64_t* out_mass;          /* [rows] the kept set's mass in the library's fixed point, sum over {z >= tau} of
                                  floor(2^40 * 2^((z - vmax) * log2(e) / T)) (0 for a greedy row), or NULL: lm_verify_args.target_mass */
} lm_sample_args;

LM_API int lm_sample(const lm_sample_args* args);

/*
 * Greedy argmax of every row: token[r] = lowest index of max float32(logits[r, :]); -1 for vocab == 0.
 * Stands in for argmax_partial + argmax_final (kernels/common/argmax.metal:36-99; ArgmaxParams, monolith/kernels.py:509-510)
 * behind GreedySampler.forward (monolith/nn/sampler.py:16-19).
 */
LM_API int lm_argmax(const void* logits, int32_t dtype, int64_t rows, int64_t vocab, int64_t row_stride, int32_t* out_tokens,
              void* workspace, size_t workspace_bytes, void* stream);

/*
 * lm_argmax with its scratch inside the library: for callers that cannot allocate device memory.
 *
 * Has no counterpart in lithos-metal (whose programs size every buffer at compile time). Some hosts of this library
 * are handed tensors and a stream and nothing else: a runtime plug-in called from a frozen decode loop, a step
 * that runs while the engine's allocator is locked or while a memory budget is already spent, code that must not
 * call cudaMalloc because cudaMalloc synchronises the device. They cannot create the workspace lm_argmax needs when it
 * splits rows over several thread blocks, so this entry point keeps that workspace in a fixed device array that is
 * part of the library image: LM_ARGMAX_STATIC_MAX_ROWS entries of 16 bytes (64 KiB), resident on every GPU that
 * loads the library for as long as the process lives.
 *
 *   - same arguments and result as lm_argmax, minus the workspace; rows > LM_ARGMAX_STATIC_MAX_ROWS returns LM_E_UNSUPPORTED;
 *   - it allocates nothing: no cudaMalloc / cudaFree and no allocating library call, on any call;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and remembers it; make that first call before starting a stream capture;
 *   - every call uses the same array and clears the part it needs on the given stream before the kernel runs, so
 *     calls on one stream may follow each other freely, but two calls that can overlap on the GPU (different
 *     streams without an ordering between them, or different host threads) race on it: order them yourself.
 */
#define LM_ARGMAX_STATIC_MAX_ROWS 4096
LM_API int lm_argmax_static(const void* logits, int32_t dtype, int64_t rows, int64_t vocab, int64_t row_stride, int32_t* out_tokens, void* stream);

/*
 * One DSpark verification step: n_draft drafted tokens checked against n_draft + 1 rows of target logits.
 *
 * Stands in for accept_scan's prefix match (kernels/common/spec_ops.metal:162-165) when mode == LM_VERIFY_GREEDY and for
 * spec_q_accept + spec_residual_partial/final (kernels/common/sample.metal:279-347, probabilities per spec_p, :273-276)
 * when mode == LM_VERIFY_STOCHASTIC, with the uniforms supplied by the caller and the drafter's distribution given either
 * as probabilities (draft_probs) or, as the reference keeps it, as the drafter's BF16 logits rows with the row statistics
 * lm_draft_q returned for them (draft_logits + draft_vmax + draft_mass; half the bytes).
 *
 * Row r < n_draft holds the target's distribution for the position draft r fills; row n_draft is the bonus row.
 *   greedy:     pick[r] = argmax row r; accept = longest prefix with pick[r] == draft[r]; final = pick[accept].
 *   stochastic: p_r = kept softmax of row r at `temperature` with threshold tau[r] (NULL = keep everything);
 *               q[r, v] = draft_probs[r, v], or float32(W / draft_mass[r]) with W the fixed-point weight of
 *               draft_logits[r, v] relative to draft_vmax[r] at `temperature` (the drafter's unfiltered softmax);
 *               reject r  <=>  float32(u_accept[r] * q[r, draft[r]]) >= p_r(draft[r]);  accept = first rejected r
 *               (n_draft if none); final = inverse-CDF draw with u_final over max(p - q, 0) of row `accept`
 *               (over p itself on the bonus row, or when the residual is empty).
 * Outputs: out_accept[0] = accept length; out_final[0] = final token; out_tokens (optional, [n_draft + 1]) =
 * drafts[0..accept) followed by the final token, -1 beyond. A launch whose internal waits ran out (see wait_limit) reports -1
 * in all three and leaves its workspace usable for the next call.
 *
 * commit (optional): the fields lm_accept_scan takes (step_state, t_max, gamma_max, ring, ring_cap, eos, eos_list, n_eos, log,
 * log_cap, ctx_cap, lm; `tokens` and `stream` are ignored). The thread that writes out_tokens then runs the accept scan on them
 * (kernels/common/spec_ops.metal:148-195): commit to the token ring, advance the StepState; one launch closes the round. The
 * state must describe this round (verify_len == n_draft, t_this_step == n_draft + 1, unless step_state hands the round to the
 * kernel; a prefill chunk takes the scan's prefill branch); otherwise the state gets error 4 and done = 1. A launch whose
 * internal waits ran out gives error 3 and done = 1.
 */
#define LM_VERIFY_GREEDY 0
#define LM_VERIFY_STOCHASTIC 1

struct lm_step_args;

typedef struct lm_verify_args {
  uint32_t struct_size;
  int32_t mode;                /* LM_VERIFY_* */
  int32_t dtype;               /* dtype of target_logits */
  int32_t n_draft;             /* 1..LM_MAX_DRAFT */
  const void* target_logits;   /* [n_draft + 1, row_stride] */
  int64_t vocab;
  int64_t row_stride;
  const int32_t* draft_ids;    /* [n_draft] */
  const float* draft_probs;    /* [n_draft, probs_stride] float32; stochastic only */
  int64_t probs_stride;
  float temperature;           /* stochastic only, > 0 */
  const float* tau;            /* [n_draft + 1] kept-set thresholds from lm_sample, or NULL */
  const float* u_accept;       /* [n_draft] */
  const float* u_final;        /* [1] */
  int32_t* out_accept;         /* [1] */
  int32_t* out_final;          /* [1] */
  int32_t* out_tokens;         /* [n_draft + 1] or NULL */
  float* out_p_draft;          /* [n_draft] p_r(draft[r]) or NULL (stochastic) */
  void* workspace;             /* lm_verify_workspace_bytes() bytes, 256-byte aligned, zero-filled once */
  size_t workspace_bytes;
  void* stream;
  const void* draft_logits;    /* [n_draft, draft_logits_stride] BF16, used when draft_probs is NULL (stochastic) */
  int64_t draft_logits_stride;
  const float* draft_vmax;     /* [n_draft] row maxima from lm_draft_q */
  const uint64_t* draft_mass;  /* [n_draft] fixed-point row masses from lm_draft_q */
  const struct lm_step_args* commit;  /* NULL, or: close the round in the same launch (see below); needs out_tokens */
  /* randomness on the device: u_accept == NULL takes uniform01(seed, step, 3000 + r, 0) for draft r, the reference's accept
   * stream (kernels/common/sample.metal:291-296); u_final == NULL takes uniform01(seed, step, 4000, 0) */
  uint64_t seed;
  uint32_t step;
  int32_t residual_draw;       /* LM_RESIDUAL_* (stochastic) */
  /* GPU-resident control (optional): a StepState buffer of layout (t_max, gamma_max). When given, the round is read from it on
   * the device (kernels/common/sample.metal:283-296): L = verify_len <= n_draft drafts = pending_tokens[base + 1 ..], rows
   * base .. base + L of target_logits with base = t_this_step - 1 - L, seed = rng_hi:rng_lo, step; out_tokens is indexed by step
   * row; nothing is verified or written when the state is done or the step is a prefill chunk (a commit still runs the scan's
   * prefill branch). A state whose rows do not fit (verify_len > n_draft, t_this_step > n_draft + 1) gets error 4 and done = 1. */
  const void* step_state;
  int32_t t_max, gamma_max;
  uint32_t wait_limit;         /* polls before a wait between thread blocks gives up; 0 = the default (about 0.1 s) */
  uint32_t selftest;           /* LM_VERIFY_SELFTEST_WITHHOLD: block 0 withholds its row maxima, so every wait of the launch runs
                                  out and the error path can be exercised (with a small wait_limit) without hanging anything */
  const float* target_vmax;    /* stochastic mode, optional: [n_draft + 1] (with a step_state: [t_max], indexed like the rows) the exact
                                  maximum of every target row, as the sampler that produced `tau` knows it (the reference's verify
                                  kernels take it from there too: KEPT_STATS, kernels/common/sample.metal:273-303). The launch then
                                  spares the first of its exchanges between thread blocks. A value that is not the row's maximum
                                  gives unspecified tokens (never a hang). NULL: the kernel finds the maxima itself. */
  const uint64_t* target_mass; /* with target_vmax, optional: per row the fixed-point mass of its kept set {z >= tau} at `temperature`, as
                                  lm_sample_args.out_mass gives it for the same rows, thresholds and temperature (the other half of
                                  the reference's KEPT_STATS). Every block then runs the accept test by itself and the launch has a
                                  single exchange left (the draw). Ignored without target_vmax. */
} lm_verify_args;

#define LM_RESIDUAL_INVERSE_CDF 0 /* final token by inverse CDF, in ascending index order, over max(p - q, 0) (over p on the bonus row) from u_final */
#define LM_RESIDUAL_GUMBEL 1      /* the reference's form (kernels/common/sample.metal:322-346): argmax of ln(p - q) + gumbel(seed, step,
                                     4000, i) over the positive residual; with every draft accepted or an empty residual, the row's own
                                     Gumbel-max draw argmax(z/T + gumbel(seed, step, row, i)) over its kept set */
#define LM_VERIFY_SELFTEST_WITHHOLD 1u

#define LM_MAX_DRAFT 15

LM_API int lm_verify(const lm_verify_args* args);

/*
 * Draft-side sampling: the draw of draft k from the drafter's logits row, and the row statistics the verify step needs to
 * evaluate q_k(v) later.
 *
 * Stands in for draft_q_partial + draft_q_final (kernels/common/sample.metal:212-269). Row r of the call is draft
 * position first_position + r:
 *   token[r] = argmax_i ( z_i * float32(1/T) + gumbel(seed, step, 2000 + first_position + r, i) ), ties -> lowest index
 *              (the reference's stream numbering, sample.metal:239): what lm_sample draws for an unfiltered row with
 *              row_offset + row = 2000 + position;
 *   vmax[r]  = max_i z_i;  mass[r] = sum_i floor(2^40 * exp2_fixed((z_i - vmax) * log2(e)/T)), the integer weights every
 *              kernel of this library uses, so q_k(v) = float32(W_v / mass) is the same number on any GPU count or CPU;
 *   lse[r]   = float32(vmax/T + ln(mass * 2^-40)): the reference's q_lse (log sum exp(z/T); it accumulates in FP32 in
 *              an order that depends on its grid, so the two agree to ~1e-6 relative, not bit for bit);
 *   out_q_logits (optional) receives a copy of the rows, as the reference keeps them in its state.
 * BF16 or FP32 rows; 1..LM_MAX_DRAFT + 1 rows per call; temperature > 0. Workspace: lm_verify_workspace_bytes() bytes,
 * 256-byte aligned, zero-filled once (it may be the verify step's workspace: the calls are stream-ordered).
 */
typedef struct lm_draft_q_args {
  uint32_t struct_size;
  int32_t dtype;
  int32_t rows;
  int32_t first_position;
  const void* logits;          /* [rows, row_stride] */
  int64_t vocab;
  int64_t row_stride;
  float temperature;
  uint64_t seed;
  uint32_t step;
  int32_t* out_tokens;         /* [rows] */
  float* out_lse;              /* [rows] or NULL */
  float* out_vmax;             /* [rows] or NULL */
  uint64_t* out_mass;          /* [rows] or NULL */
  uint32_t* out_status;        /* [rows] LM_STATUS_NEAR_TIE / LM_STATUS_NAN bits, or NULL */
  void* out_q_logits;          /* [rows, q_logits_stride] same dtype as logits, or NULL */
  int64_t q_logits_stride;
  void* workspace;
  size_t workspace_bytes;
  void* stream;
  const void* step_state;      /* optional StepState of layout (t_max, gamma_max): seed = rng_hi:rng_lo and step are read from it on the
                                  device (kernels/common/sample.metal:236-239); nothing is written once the state is done */
  int32_t t_max, gamma_max;
} lm_draft_q_args;

LM_API int lm_draft_q(const lm_draft_q_args* args);

/*
 * Vocab-parallel sampling: every row's vocabulary is split into `shards` contiguous pieces, one per GPU.
 *
 * No counterpart in lithos-metal (which is single-device). The result is defined as what lm_sample returns for the
 * whole row, bit for bit. Protocol, per step:
 *   1. every GPU calls lm_vocab_local on its shard: per row it writes one record (lm_vocab_record_bytes(cap) bytes) with
 *      the shard's maximum, its FP64 softmass and every logit at or above the shard's own top_k-th largest value
 *      (ties kept) with global indices;
 *   2. the caller all-gathers the records (the only exchange: rows * record bytes per GPU; NCCL in the Python layer)
 *      into [shards][rows] records, shard order = vocabulary order;
 *   3. every GPU calls lm_vocab_merge on the gathered records and gets the same tokens.
 * Requirements: top_k >= 1 on every row (the kept set must lie inside the top-k candidates), cap =
 * lm_vocab_candidate_cap(largest top_k), at most 64 shards, cap <= (LM_VOCAB_MAX_CANDIDATES / 1024) * (1024 / shards) (integer division: shards * cap <=
 * LM_VOCAB_MAX_CANDIDATES when shards is a power of two), no penalties. A row whose ties overflow
 * a record (or, beyond 1024 logits tied at the top-k boundary, the merge) reports LM_STATUS_OVERFLOW and token -1; a row with a NaN or a
 * maximum that is not finite reports LM_STATUS_NAN and token -1; a row whose per-row temperature is not positive reports status bit 16 and
 * token -1. One exception to "bit for bit": the FP64 softmass is summed per shard and then over the sorted candidates, another
 * order than on one GPU, so a top-p boundary within 1e-12 (relative) of the target may fall on the other side; such rows carry
 * LM_STATUS_TOPP_EDGE here as they do there.
 */
#define LM_VOCAB_MAX_CANDIDATES 8192
#define LM_STATUS_OVERFLOW 32u

typedef struct lm_vocab_args {
  uint32_t struct_size;
  int32_t dtype;
  const void* logits;          /* local step: [rows, row_stride], this GPU's shard */
  int64_t rows;
  int64_t vocab_local;         /* local step: width of the shard */
  int64_t row_stride;
  int64_t shard_start;         /* local step: global index of the shard's first logit */
  int32_t shards;              /* merge step */
  int32_t cap;                 /* candidates per row per shard */
  const float* temperature;  float temperature_s;
  const int32_t* top_k;      int32_t top_k_s;
  const float* top_p;        float top_p_s;      /* merge step */
  const float* min_p;        float min_p_s;      /* merge step */
  uint32_t flags;              /* LM_FLAG_*, merge step */
  int32_t draw;                /* LM_DRAW_*, merge step */
  const float* uniforms;       /* [rows], merge step */
  uint64_t seed; uint32_t step; int64_t row_offset;
  void* records;               /* local step: out [pieces][rows] records; merge step: in [shards][rows] records (every piece of every GPU's shard counts as a shard) */
  int32_t* out_tokens;         /* merge step: [rows] */
  float* out_tau;              /* merge step, optional */
  uint32_t* out_status;        /* merge step, optional */
  void* stream;
  int32_t pieces;              /* local step: records per row that this GPU's shard is cut into, 1 (or 0) or lm_vocab_pieces(...); merge step with record_ptrs: the same */
  int32_t pad_;
  const void* record_ptrs;     /* merge step, optional: device array of shards / pieces addresses (as 64-bit integers), one per GPU in shard order: where that
                                  GPU's [pieces][rows] records lie -- its own memory or a peer's mapping, read in place (plain loads) instead of a gathered
                                  `records` array. The caller orders the GPUs' local steps before this call (a barrier over the GPUs on the stream). */
} lm_vocab_args;

LM_API int lm_vocab_local(const lm_vocab_args* args);
LM_API int lm_vocab_merge(const lm_vocab_args* args);
LM_API size_t lm_vocab_record_bytes(int32_t cap);
LM_API int32_t lm_vocab_candidate_cap(int32_t top_k);
/* How many pieces (records per row) the local step should cut a shard of vocab_local logits into when `shards` GPUs take part and
 * the call has `rows` rows: with one block per piece the local step spreads over the GPU, at the price of more bytes to gather. The
 * merge then sees shards * pieces shards. */
LM_API int32_t lm_vocab_pieces(int32_t shards, int32_t cap, int64_t vocab_local, int64_t rows);

/*
 * The scalar step-closing kernels, on the reference's StepState buffer (monolith/core/step_state.py:38-62: 4-byte fields in the
 * reference's order, for the given t_max / gamma_max; size = lm_step_state_bytes). One thread each, stream-ordered: the
 * host never reads a token to keep the decode loop going.
 *
 * lm_accept_scan stands in for accept_scan (kernels/common/spec_ops.metal:148-195; AcceptParams, monolith/kernels.py:831-835):
 *   greedy prefix match of token[] against pending_tokens, commit of the accepted drafts + bonus token to the token ring
 *   as (sequence << 32) | token, stop at the first stop token / stop_at / context capacity, log entry
 *   (committed << 16) | (L << 8) | accepted, state advance. Errors are device-side status: error 1 = ring overflow,
 *   2 = context capacity reached, with done = 1.
 * lm_verify_select stands in for verify_select (spec_ops.metal:108-146; SelectParams, kernels.py:814-825): stages drafts and
 *   confidences, picks the verify length L (mode 0 confident prefix, 1 cost-aware argmax_l (1 + sum a_i)/cost[l], 2 fixed),
 *   clamps it to t_max - 1 and the context capacity, writes pending_tokens = [anchor, d_0 .. d_{L-1}], t_this_step = 1 + L.
 * lm_advance stands in for advance (kernels/common/advance.metal:15-37; AdvanceParams, kernels.py:748-752): publishes the
 *   last row's token, checks ring / stop / context, advances the state.
 * Stop tokens: `eos` (a single id, -1 for none) and/or a device list of `n_eos` ids (the reference compiles a list into the
 * kernel, kernels.py:729-741).
 */
typedef struct lm_step_args {
  uint32_t struct_size;
  int32_t t_max, gamma_max;    /* the StepState layout */
  void* step_state;            /* device, lm_step_state_bytes(t_max, gamma_max) bytes */
  const int32_t* tokens;       /* accept_scan / advance: the sampler's token[] */
  uint64_t* ring;              /* accept_scan / advance: token ring, ring_cap slots */
  uint32_t ring_cap;
  int32_t eos; const int32_t* eos_list; int32_t n_eos;
  uint32_t* log; uint32_t log_cap;     /* accept_scan: optional accept log */
  uint32_t ctx_cap;            /* 0 = unbounded */
  int32_t lm;                  /* an LM drafter (changes n_inject / drafter_ctx_len bookkeeping) */
  /* verify_select only */
  const int32_t* drafts; const float* conf; uint32_t gamma; float threshold; uint32_t mode; float cost[16];
  float* conf_log; uint32_t conf_log_cap;
  uint32_t t_limit;            /* rows the step program holds (SelectParams.t_max); 0 = the layout's t_max */
  void* stream;
} lm_step_args;

LM_API int lm_accept_scan(const lm_step_args* args);
LM_API int lm_verify_select(const lm_step_args* args);
LM_API int lm_advance(const lm_step_args* args);
LM_API size_t lm_step_state_bytes(int32_t t_max, int32_t gamma_max);

/*
 * The DSpark confidence head that feeds lm_verify_select: conf[k] = sigmoid(bf16(bf16(w . [hidden_k ; emb_k]) + b) / sts[k]) for
 * k < gamma. Stands in for the `confidence` kernel (kernels/common/spec_ops.metal:85-106; parameters as conf_params,
 * monolith/kernels.py:802-808): FP32 FMA accumulation in the same lane order, both BF16 roundings, then the sigmoid (on this
 * library's fixed exp2 instead of the Metal exp: within 2e-7 of it; the reference's own test bar is 2e-3). Positions >= gamma
 * are not written. step_state (optional): nothing is written once the state is done.
 */
typedef struct lm_confidence_args {
  uint32_t struct_size;
  int32_t gamma;               /* positions to score, 0..16 */
  int32_t hidden;              /* width of a hidden row */
  int32_t rank;                /* width of an embedding row (0: no Markov part) */
  const void* hidden_rows;     /* [gamma, hidden] BF16 */
  const void* emb_rows;        /* [gamma, rank] BF16, or NULL when rank == 0 */
  const float* w;              /* [hidden + rank] */
  const float* b;              /* [1] */
  const float* sts;            /* [gamma] positive calibration temperatures, or NULL for 1 */
  float* out_conf;             /* [>= gamma] */
  void* step_state;            /* StepState bytes or NULL */
  int32_t t_max, gamma_max;    /* the layout of step_state */
  void* stream;
} lm_confidence_args;

LM_API int lm_confidence(const lm_confidence_args* args);

/*
 * Sampling from logits that arrive tile by tile: the consumer side of the boundary between the vocabulary projection and the
 * sampler.
 *
 * The reference writes the projection's logits [T, V] to memory in BF16 (lm_head_forward, monolith/nn/lm_head.py:50-60) and the
 * sampler dispatches read them back (monolith/kernels.py:720-775). A projection whose epilogue holds a tile of logits
 * [rows, up to LM_TILE_MAX_COLS columns] hands it to lm_tile_consume instead (or calls the device function of the same name
 * from its epilogue, csrc/sample_tiles.cuh), and [T, V] never has to exist: per row the library keeps the running maximum, the
 * running softmass and the logits that can still be among the row's top_k, in a caller-owned state buffer.
 *
 *   lm_tile_begin    clears the state of `rows` rows and, when a history is given, notes each row's distinct history ids (the
 *                    penalties are then applied to the logits as they arrive); stream-ordered; the tile fields are not read;
 *   lm_tile_consume  takes the columns col0 .. col0 + cols of every row; tiles may come in any column order, each column once;
 *                    FP32 tiles are rounded to BF16 first, as the projection's store would; history / penalties as given to
 *                    lm_tile_begin;
 *   lm_tile_finish   writes what lm_sample would write for the same rows and knobs (tokens, tau, status with
 *                    LM_STATUS_CANDIDATE_PATH; greedy rows: the argmax, status 0), bit-identical; `logits`, `workspace`, the
 *                    history fields, `out_stats` and `out_probs` of the lm_sample_args are not read (out_stats / out_probs must
 *                    be NULL): the penalties are those given to lm_tile_begin.
 *
 * Rows this path does not take get token -1 and LM_STATUS_TILE_DECLINED: stochastic rows without a top_k in 1..1024, rows with a
 * NaN or +inf, rows whose top-k boundary lies at or below zero or whose top-p boundary cannot be decided from the FP32 softmass.
 * The caller materialises those rows and calls lm_sample.
 */
#define LM_TILE_MAX_COLS 2048
typedef struct lm_tile_args {
  uint32_t struct_size;        /* sizeof(lm_tile_args) */
  int32_t dtype;               /* LM_DTYPE_BF16 or LM_DTYPE_F32: the tile's element type */
  const void* tile;            /* [rows, tile_stride]: element (r, j) is the logit of row r, column col0 + j */
  int64_t rows, vocab;
  int64_t tile_stride;         /* elements between rows of the tile (>= cols) */
  int64_t col0, cols;          /* 0 <= col0, col0 + cols <= vocab, 1 <= cols <= LM_TILE_MAX_COLS */
  const float* temperature; float temperature_s;   /* as in lm_sample_args; the same values must be given to lm_tile_finish */
  const int32_t* top_k; int32_t top_k_s;
  void* state;                 /* lm_tile_state_bytes(rows, vocab, history != NULL) bytes, 256-byte aligned, device memory */
  size_t state_bytes;
  void* stream;
  const int32_t* history;      /* [rows, hist_stride] token ids to penalise, or NULL; the same in every call of one step */
  int64_t hist_len, hist_stride;
  float repetition_penalty, presence_penalty;   /* as in lm_sample_args (1 and 0: no penalty) */
} lm_tile_args;

LM_API size_t lm_tile_state_bytes(int64_t rows, int64_t vocab, int32_t with_history);
LM_API int lm_tile_begin(const lm_tile_args* args);
LM_API int lm_tile_consume(const lm_tile_args* args);
LM_API int lm_tile_finish(const lm_sample_args* sample, void* state, size_t state_bytes);

/* Scratch sizes (host calls, no CUDA work). Stand in for sample_workspace (monolith/kernels.py:777-779). */
LM_API size_t lm_workspace_bytes(int64_t rows, int64_t vocab);
LM_API size_t lm_verify_workspace_bytes(int32_t n_draft, int64_t vocab);

/* The counter-based uniform of the reference's hash (kernels/common/sample.metal:26-31; monolith/nn/sampling_ref.py:41-51),
 * computed on the host: lets a caller reproduce the reference's accept-test stream (3000 + r) as injected uniforms. */
LM_API float lm_uniform01(uint64_t seed, uint32_t step, uint32_t t, uint32_t index);

/* Library identification and diagnostics (host calls). */
/*
 * The vocabulary projection of a decode step with the final RMSNorm fused on its input: the reference's `lm_head` op
 * (monolith/nn/lm_head.py:50-60; semantics monolith/nn/oracle.py:20-32): logits[r, v] = bf16(sum_k x[r, k] * weight[v, k]) in
 * FP32, x = the rows of `hidden` as they are (norm_weight NULL: already normalised) or bf16(hidden * rsqrt(mean(hidden^2) + eps) *
 * (one_plus ? 1 + norm_weight : norm_weight)). At most 8 rows (one token, or the rows of a speculative round): a matrix-vector
 * product bound by the weight stream. hidden_dim a multiple of 64, at most 12,736 (the rows sit in shared memory); hidden, weight and their strides 16-byte aligned. The logits
 * are what lm_sample / lm_argmax / lm_verify take next on the same stream (they are still in L2 then). Floating point: the FP32
 * sums are formed in another order than a reference's, so a logit may differ from it by one BF16 unit in the last place.
 */
#define LM_HEAD_MAX_ROWS 8
typedef struct lm_head_args {
  uint32_t struct_size;
  int32_t rows;                /* 1 .. LM_HEAD_MAX_ROWS */
  const void* hidden;          /* [rows, hidden_stride] BF16 */
  int64_t hidden_stride;
  const void* weight;          /* [vocab, weight_stride] BF16: one row of hidden_dim weights per vocabulary entry */
  int64_t weight_stride;
  int64_t hidden_dim;
  int64_t vocab;
  const void* norm_weight;     /* [hidden_dim] BF16 or NULL */
  float eps;
  int32_t one_plus;            /* the norm's scale is 1 + norm_weight (zero-centred weights) */
  void* logits;                /* out [rows, logits_stride] BF16 */
  int64_t logits_stride;
  void* stream;
} lm_head_args;

LM_API int lm_head(const lm_head_args* args);

LM_API int lm_abi_version(void);
LM_API const char* lm_error_string(int code);
LM_API const char* lm_last_cuda_error(void);   /* text of the last CUDA error seen by this thread's calls, "" if none */
LM_API int lm_device_sm_count(void);           /* multiprocessors of the current device, or a negative LM_E_* */

#ifdef __cplusplus
}
#endif
#endif /* LITHOS_B200_H */
