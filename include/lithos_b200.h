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
 *     workspace reusable (a workspace must be zero-filled once before its first use and is kept clean afterwards);
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

#define LM_ABI_VERSION 1

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
#define LM_DRAW_INVERSE_CDF 1  /* inverse CDF over the kept set in ascending index order, from a caller-supplied uniform */

/* lm_sample_args.flags */
#define LM_FLAG_TOPP_IN_TOPK 1u /* top-p over the top-k set's renormalised mass (the Hugging Face warpers' order) */

/* per-row status bits written to lm_sample_args.out_status (optional) */
#define LM_STATUS_GENERIC_PATH 1u /* the row was handled by the generic multi-pass path */
#define LM_STATUS_NAN 2u          /* the row holds a NaN: results for the row are unspecified */
#define LM_STATUS_NEAR_TIE 4u     /* Gumbel draw: best and second-best key closer than 4e-6 (float32 log is library-specific) */
#define LM_STATUS_TOPP_EDGE 8u    /* top-p: cumulative mass within 1e-12 (relative) of the target at the boundary */

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
 * when mode == LM_VERIFY_STOCHASTIC, with the drafter's distribution given as probabilities and the uniforms supplied
 * by the caller.
 *
 * Row r < n_draft holds the target's distribution for the position draft r fills; row n_draft is the bonus row.
 *   greedy:     pick[r] = argmax row r; accept = longest prefix with pick[r] == draft[r]; final = pick[accept].
 *   stochastic: p_r = kept softmax of row r at `temperature` with threshold tau[r] (NULL = keep everything);
 *               reject r  <=>  float32(u_accept[r] * q[r, draft[r]]) >= p_r(draft[r]);  accept = first rejected r
 *               (n_draft if none); final = inverse-CDF draw with u_final over max(p - q, 0) of row `accept`
 *               (over p itself on the bonus row, or when the residual is empty).
 * Outputs: out_accept[0] = accept length; out_final[0] = final token; out_tokens (optional, [n_draft + 1]) =
 * drafts[0..accept) followed by the final token, -1 beyond.
 */
#define LM_VERIFY_GREEDY 0
#define LM_VERIFY_STOCHASTIC 1

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
} lm_verify_args;

#define LM_MAX_DRAFT 15

LM_API int lm_verify(const lm_verify_args* args);

/* Scratch sizes (host calls, no CUDA work). Stand in for sample_workspace (monolith/kernels.py:777-779). */
LM_API size_t lm_workspace_bytes(int64_t rows, int64_t vocab);
LM_API size_t lm_verify_workspace_bytes(int32_t n_draft, int64_t vocab);

/* The counter-based uniform of the reference's hash (kernels/common/sample.metal:26-31; monolith/nn/sampling_ref.py:41-51),
 * computed on the host: lets a caller reproduce the reference's accept-test stream (3000 + r) as injected uniforms. */
LM_API float lm_uniform01(uint64_t seed, uint32_t step, uint32_t t, uint32_t index);

/* Library identification and diagnostics (host calls). */
LM_API int lm_abi_version(void);
LM_API const char* lm_error_string(int code);
LM_API const char* lm_last_cuda_error(void);   /* text of the last CUDA error seen by this thread's calls, "" if none */
LM_API int lm_device_sm_count(void);           /* multiprocessors of the current device, or a negative LM_E_* */

#ifdef __cplusplus
}
#endif
#endif /* LITHOS_B200_H */
