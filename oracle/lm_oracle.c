/*
 * CPU oracle for the generation-control path (sampling thresholds, draws, DSpark verification).
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped package may call this file; it exists so that the CUDA
 * kernels can be checked against an independent CPU restatement of the algorithm, and so that the benchmark can
 * time a CPU baseline next to the GPU.
 *
 * What is restated from the reference (lithos-metal) and where it lives there:
 *   lmo_thresholds        monolith/nn/sampling_ref.py:20-38   (top-k / top-p / min-p logit threshold, FP64 mass)
 *   lmo_uniform01         monolith/nn/sampling_ref.py:41-51, kernels/common/sample.metal:26-31 (splitmix64 hash)
 *   lmo_gumbel            monolith/nn/sampling_ref.py:52, kernels/common/sample.metal:32
 *   lmo_sample_gumbel     monolith/nn/sampling_ref.py:55-62   (masked Gumbel-max draw, ties -> lowest index)
 *   lmo_warped_probs      monolith/nn/sampling_ref.py:65-71   (kept-token probability vector, FP64)
 *   lmo_argmax            monolith/nn/sampler.py:16-19, kernels/common/argmax.metal:22-24
 *   lmo_accept_greedy     kernels/common/spec_ops.metal:162-165 (greedy prefix match + bonus row)
 *   lmo_verify_stochastic kernels/common/sample.metal:273-347 (p/q accept, first reject, residual draw) -- the
 *                         reference has no CPU code and no exact-output test for this part: PARITY UNPINNED; this
 *                         restatement is the frozen definition.
 *   lmo_verify_gumbel     the same step with the reference's own randomness: accept uniforms of stream 3000 + r, Gumbel-max residual
 *                         draw on stream 4000 (sample.metal:291-296, 322-346); PARITY UNPINNED for the same reason
 *   lmo_draft_q           kernels/common/sample.metal:212-269 (the drafter's draw on noise stream 2000 + k; the token is
 *                         pinned by sampling_ref.sample with t = 2000 + k; lse to 2e-6; q from the integer mass: unpinned)
 *   lmo_confidence        kernels/common/spec_ops.metal:85-106 (confidence head; pinned to the reference test's expected
 *                         values, tests/kernels/test_draft_ops.py:228-263, within its own bar of 2e-3)
 * What has no counterpart in the reference (PARITY UNPINNED; this file is the frozen definition):
 *   lmo_apply_penalties   repetition / presence penalties over the distinct ids of a token history
 *   lmo_spec_exp2, lmo_weight_q40, lmo_sample_invcdf   inverse-CDF draw (descending logit order) from a caller-supplied uniform, defined
 *                         on integer fixed-point weights so that CPU and GPU agree bit for bit
 *
 * Everything that feeds an integer decision is built from IEEE-754 binary32/binary64 operations with a fixed
 * order (no contraction: compile with -ffp-contract=off), so a GPU restatement using the same operations gives
 * the same bits.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define LMO_API __attribute__((visibility("default")))

/* ---- small helpers ------------------------------------------------------------------------------------- */

static inline float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

LMO_API float lmo_bf16_to_f32(uint16_t b) { return bits_f((uint32_t)b << 16); }

/* Widen a row of logits to FP32. dtype 0 = BF16 codes, 1 = FP32. (nn/sampler.py:43: logits.to(float32)) */
LMO_API void lmo_widen(const void* logits, int dtype, int64_t n, float* out) {
  if (dtype == 0) { const uint16_t* p = (const uint16_t*)logits; for (int64_t i = 0; i < n; i++) out[i] = lmo_bf16_to_f32(p[i]); }
  else memcpy(out, logits, (size_t)n * 4);
}

/* ---- penalties (no reference counterpart) -------------------------------------------------------------------
 * For every DISTINCT id of the history that lies in [0, V): z <- (z > 0 ? z / rho : z * rho), then z <- z - pi.
 * Both in binary32, in that order. Ids outside [0, V) (for instance -1 padding) are ignored. */
LMO_API void lmo_apply_penalties(float* z, int64_t vocab, const int32_t* history, int64_t hist_len, float rho, float pi) {
  if (hist_len <= 0 || (rho == 1.0f && pi == 0.0f)) return;
  uint8_t* seen = (uint8_t*)calloc((size_t)vocab, 1);
  for (int64_t h = 0; h < hist_len; h++) {
    const int64_t id = history[h];
    if (id < 0 || id >= vocab || seen[id]) continue;
    seen[id] = 1;
    float v = z[id];
    v = (v > 0.0f) ? v / rho : v * rho;
    z[id] = v - pi;
  }
  free(seen);
}

/* ---- argmax (ties -> lowest index; -1 for an empty row) ------------------------------------------------- */
LMO_API int32_t lmo_argmax(const float* z, int64_t vocab) {
  float best = -INFINITY; int64_t bi = -1;
  for (int64_t i = 0; i < vocab; i++) if (bi < 0 || z[i] > best) { best = z[i]; bi = i; }
  return (int32_t)bi;
}

/* ---- thresholds (sampling_ref.py:20-38) --------------------------------------------------------------------- */

static int cmp_desc(const void* a, const void* b) {
  const float x = *(const float*)a, y = *(const float*)b;
  return (x < y) - (x > y);
}

/* Returns tau as a float (-inf when nothing is enabled). temperature/top_p/min_p are the doubles the reference
 * receives (a Python float). Optional outputs: vmax, the FP64 softmax mass of the kept set {z >= tau} relative to
 * vmax, and the size of the kept set. */
LMO_API float lmo_thresholds(const float* z, int64_t vocab, double temperature, int32_t top_k, double top_p, double min_p,
                             int32_t topp_in_topk, float* out_vmax, double* out_kept_mass, int64_t* out_kept_count) {
  float* s = (float*)malloc((size_t)vocab * 4);
  memcpy(s, z, (size_t)vocab * 4);
  qsort(s, (size_t)vocab, 4, cmp_desc);
  const float vmax = s[0];
  double tau = -INFINITY;
  int have = 0;
  float tau_k = -INFINITY;
  if (top_k > 0) {
    const int64_t k = top_k < vocab ? top_k : vocab;
    tau_k = s[k - 1];
    tau = tau_k; have = 1;
  }
  if (top_p > 0.0 && top_p < 1.0) {
    /* distinct values descending with counts; cumulative mass, sequential FP64 sum like np.cumsum */
    double total = 0.0;
    {
      double cum = 0.0;
      int64_t i = 0;
      while (i < vocab) {
        int64_t j = i; while (j < vocab && s[j] == s[i]) j++;
        cum += (double)(j - i) * exp(((double)s[i] - (double)vmax) / temperature);
        if (topp_in_topk && top_k > 0 && s[i] >= tau_k) total = cum;      /* cum[vals >= tau_k][-1] */
        i = j;
      }
      if (!(topp_in_topk && top_k > 0)) total = cum;
    }
    const double target = top_p * total;
    double cum = 0.0; float tau_p = s[0];
    int64_t i = 0; int found = 0;
    while (i < vocab) {
      int64_t j = i; while (j < vocab && s[j] == s[i]) j++;
      cum += (double)(j - i) * exp(((double)s[i] - (double)vmax) / temperature);
      if (cum >= target) { tau_p = s[i]; found = 1; break; }
      i = j;
    }
    if (!found) tau_p = s[0];                                               /* np.argmax of an all-False mask is 0 */
    if (!have || (double)tau_p > tau) tau = tau_p;
    have = 1;
  }
  if (min_p > 0.0) {
    const double tau_m = (double)vmax + temperature * log(min_p);
    if (!have || tau_m > tau) tau = tau_m;
    have = 1;
  }
  /* the reference compares float32 logits with the Python float: the scalar is cast to float32 (NumPy 2 rules) */
  const float tau_f = have ? (float)tau : -INFINITY;
  if (out_vmax) *out_vmax = vmax;
  if (out_kept_mass || out_kept_count) {
    double mass = 0.0; int64_t cnt = 0, i = 0;
    while (i < vocab && s[i] >= tau_f) {
      int64_t j = i; while (j < vocab && s[j] == s[i]) j++;
      mass += (double)(j - i) * exp(((double)s[i] - (double)vmax) / temperature);
      cnt += j - i; i = j;
    }
    if (out_kept_mass) *out_kept_mass = mass;
    if (out_kept_count) *out_kept_count = cnt;
  }
  free(s);
  return tau_f;
}

/* ---- counter-based noise (sampling_ref.py:41-52; sample.metal:26-32) ----------------------------------------- */

LMO_API float lmo_uniform01(uint64_t seed, uint32_t step, uint32_t t, uint32_t i) {
  uint64_t x = seed + (uint64_t)step * 0x9E3779B97F4A7C15ull + (uint64_t)t * 0xC2B2AE3D27D4EB4Full + (uint64_t)i * 0x165667B19E3779F9ull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 27; x *= 0x94D049BB133111EBull; x ^= x >> 31;
  return ((float)((x >> 41) & 0x7FFFFFull) + 0.5f) * (1.0f / 8388608.0f);
}

LMO_API float lmo_gumbel(uint64_t seed, uint32_t step, uint32_t t, uint32_t i) {
  return -logf(-logf(lmo_uniform01(seed, step, t, i)));
}

/* The masked Gumbel-max draw (sampling_ref.py:55-62): argmax over z >= tau of fl32(z * fl32(1/T)) + g, two separate
 * binary32 roundings, ties -> lowest index; -1 if nothing is kept. Also reports the gap between the best and the
 * second-best key so a caller can tell a near-tie (float32 log is not identical across libraries). */
LMO_API int32_t lmo_sample_gumbel(const float* z, int64_t vocab, float tau, double temperature, uint64_t seed, uint32_t step, uint32_t t,
                                  float* out_gap) {
  const float inv_t = (float)(1.0 / temperature);
  float best = -INFINITY, second = -INFINITY; int64_t bi = -1;
  for (int64_t i = 0; i < vocab; i++) {
    if (!(z[i] >= tau)) continue;
    volatile float a = z[i] * inv_t;
    const float key = a + lmo_gumbel(seed, step, t, (uint32_t)i);
    if (key > best) { second = best; best = key; bi = i; } else if (key > second) second = key;
  }
  if (out_gap) *out_gap = best - second;
  return (int32_t)bi;
}

/* The kept-token probability vector (sampling_ref.py:65-71): softmax of (z - vmax)/T over z >= tau, FP64. */
LMO_API void lmo_warped_probs(const float* z, int64_t vocab, float tau, double temperature, double* out) {
  double vmax = -INFINITY;
  for (int64_t i = 0; i < vocab; i++) if ((double)z[i] > vmax) vmax = z[i];
  double sum = 0.0;
  for (int64_t i = 0; i < vocab; i++) { out[i] = (z[i] >= tau) ? exp(((double)z[i] - vmax) / temperature) : 0.0; sum += out[i]; }
  for (int64_t i = 0; i < vocab; i++) out[i] /= sum;
}

/* ---- the integer-exact inverse-CDF draw (no reference counterpart) ----------------------------------------------
 * Weights are binary32 values from a fixed sequence of IEEE operations, turned into 40-bit fixed point; sums,
 * the target and the search are integer arithmetic, so the result does not depend on summation order or on how
 * a row is split between thread blocks or GPUs. */

/* 2^x for x <= 0 by round-to-nearest split and a degree-5 polynomial with fused multiply-adds; 0 below 2^-100. */
LMO_API float lmo_spec_exp2(float x) {
  if (!(x > -100.0f)) return 0.0f;                      /* also NaN and -inf */
  if (x > 0.0f) x = 0.0f;
  const float n = rintf(x);                             /* round half to even */
  const float f = x - n;                                /* exact, in [-0.5, 0.5] */
  float p = 0x1.5bba20p-10f;
  p = fmaf(p, f, 0x1.3cea88p-7f);
  p = fmaf(p, f, 0x1.c6b752p-5f);
  p = fmaf(p, f, 0x1.ebf9bcp-3f);
  p = fmaf(p, f, 0x1.62e42ap-1f);
  p = fmaf(p, f, 1.0f);
  return p * bits_f((uint32_t)((int32_t)n + 127) << 23); /* exact scaling by 2^n, n in [-100, 0] */
}

/* The per-row constant log2(e)/T as a binary32: divided in binary64, rounded once. */
LMO_API float lmo_exp2_scale(float temperature) { return (float)(1.4426950408889634 / (double)temperature); }

/* Fixed-point weight of one kept logit: floor(2^40 * spec_exp2(fl32(fl32(z - vmax) * c))). */
LMO_API uint64_t lmo_weight_q40(float z, float vmax, float c) {
  volatile float d = z - vmax;
  volatile float x = d * c;
  return (uint64_t)(lmo_spec_exp2(x) * 1099511627776.0f);
}

/* target = floor(U24 * S / 2^24), U24 = floor(u * 2^24) clamped to [0, 2^24 - 1] */
LMO_API uint64_t lmo_cdf_target(float u, uint64_t total) {
  int64_t u24 = (u > 0.0f) ? (int64_t)(u * 16777216.0f) : 0;
  if (u24 > 16777215) u24 = 16777215;
  return (uint64_t)(((unsigned __int128)total * (uint64_t)u24) >> 24);
}

/* The kept set in index order: token = the first kept index, ascending, whose inclusive cumulative weight exceeds the target;
 * -1 if the kept set has no weight. The verify step draws this way from a row's own softmax (every block of its kernel owns a
 * contiguous piece of the vocabulary). out_total: the kept set's integer mass. */
LMO_API int32_t lmo_sample_invcdf_index(const float* z, int64_t vocab, float tau, float temperature, float u, uint64_t* out_total) {
  float vmax = -INFINITY;
  for (int64_t i = 0; i < vocab; i++) if (z[i] > vmax) vmax = z[i];
  const float c = lmo_exp2_scale(temperature);
  uint64_t total = 0;
  for (int64_t i = 0; i < vocab; i++) if (z[i] >= tau) total += lmo_weight_q40(z[i], vmax, c);
  if (out_total) *out_total = total;
  if (total == 0) return -1;
  const uint64_t target = lmo_cdf_target(u, total);
  uint64_t cum = 0;
  for (int64_t i = 0; i < vocab; i++) if (z[i] >= tau) { cum += lmo_weight_q40(z[i], vmax, c); if (cum > target) return (int32_t)i; }
  return -1;
}

/* The sampler's inverse-CDF draw: the kept set ordered by descending logit, equal logits by ascending index (the order of a
 * sorted top-p pipeline); token = the first in that order whose inclusive cumulative weight exceeds the target; -1 if the kept
 * set has no weight. Equal logits have equal weights, so this is: the distinct value v at which the cumulative weight of the
 * values above it plus count(v) * w(v) first exceeds the target, then the floor((target - before) / w(v))-th smallest index among
 * the logits equal to v. out_total: the kept set's integer mass. */
typedef struct { float v; int32_t i; uint64_t w; } lmo_kept_t;
static int lmo_kept_cmp(const void* a, const void* b) {
  const lmo_kept_t* x = (const lmo_kept_t*)a; const lmo_kept_t* y = (const lmo_kept_t*)b;
  if (x->v != y->v) return x->v > y->v ? -1 : 1;
  return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}
LMO_API int32_t lmo_sample_invcdf(const float* z, int64_t vocab, float tau, float temperature, float u, uint64_t* out_total) {
  float vmax = -INFINITY;
  for (int64_t i = 0; i < vocab; i++) if (z[i] > vmax) vmax = z[i];
  const float c = lmo_exp2_scale(temperature);
  lmo_kept_t* k = (lmo_kept_t*)malloc((size_t)(vocab > 0 ? vocab : 1) * sizeof(lmo_kept_t));
  int64_t n = 0;
  uint64_t total = 0;
  for (int64_t i = 0; i < vocab; i++) if (z[i] >= tau) {
    const uint64_t w = lmo_weight_q40(z[i], vmax, c);
    if (w) { k[n].v = z[i] == 0.0f ? 0.0f : z[i]; k[n].i = (int32_t)i; k[n].w = w; n++; total += w; }   /* a weightless logit is never drawn */
  }
  if (out_total) *out_total = total;
  int32_t token = -1;
  if (total) {
    qsort(k, (size_t)n, sizeof(lmo_kept_t), lmo_kept_cmp);
    const uint64_t target = lmo_cdf_target(u, total);
    uint64_t cum = 0;
    for (int64_t j = 0; j < n; j++) { cum += k[j].w; if (cum > target) { token = k[j].i; break; } }
  }
  free(k);
  return token;
}

/* ---- draft-side sampling (kernels/common/sample.metal:212-269) -------------------------------------------------------
 * The drafter's draw of draft k from its logits row z (widened) at temperature T, unfiltered, on noise stream 2000 + k
 * (sample.metal:239): the masked Gumbel-max draw with tau = -inf. Alongside, the row statistics the verify step evaluates
 * q_k(v) from: vmax, the integer mass sum_i W(z_i) of the fixed-point weights, and lse = fl32(vmax/T + ln(mass * 2^-40))
 * (the reference's q_lse is an FP32 running sum in grid order: equal to ~1e-6 relative, not bit for bit). */
LMO_API int32_t lmo_draft_q(const float* z, int64_t vocab, float temperature, uint64_t seed, uint32_t step, uint32_t position,
                            float* out_vmax, uint64_t* out_mass, float* out_lse, float* out_gap) {
  float vmax = -INFINITY;
  for (int64_t i = 0; i < vocab; i++) if (z[i] > vmax) vmax = z[i];
  const float c = lmo_exp2_scale(temperature);
  uint64_t mass = 0;
  for (int64_t i = 0; i < vocab; i++) mass += lmo_weight_q40(z[i], vmax, c);
  if (out_vmax) *out_vmax = vmax;
  if (out_mass) *out_mass = mass;
  if (out_lse) *out_lse = mass ? (float)((double)vmax / (double)temperature + log((double)mass * 9.094947017729282e-13)) : -INFINITY;
  return lmo_sample_gumbel(z, vocab, -INFINITY, (double)temperature, seed, step, 2000u + position, out_gap);
}

/* q_k(v) from the drafter's logits row and its statistics: fl32(W(z_v) / mass), 0 for an empty row. */
LMO_API void lmo_draft_probs(const float* z, int64_t vocab, float temperature, float vmax, uint64_t mass, float* out_q) {
  const float c = lmo_exp2_scale(temperature);
  for (int64_t i = 0; i < vocab; i++) out_q[i] = mass ? (float)((double)lmo_weight_q40(z[i], vmax, c) / (double)mass) : 0.0f;
}

/* ---- the confidence head (kernels/common/spec_ops.metal:85-106) ---------------------------------------------------------
 * conf[k] = sigmoid(bf16(bf16(w . [hidden_k ; emb_k]) + b) / sts[k]). The dot product is the reference kernel's: 32 lanes,
 * lane l takes elements l, l + 32, ... of the hidden row and then of the embedding row, one binary32 FMA each; the lanes are
 * summed pairwise at distances 16, 8, 4, 2, 1. The two BF16 roundings are round-to-nearest-even on the bit pattern. The
 * sigmoid uses lmo_spec_exp2 (the reference calls the Metal exp). */
static inline float round_bf16(float x) {
  uint32_t u; memcpy(&u, &x, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  float r; memcpy(&r, &u, 4);
  return r;
}

LMO_API void lmo_confidence(const uint16_t* hidden, const uint16_t* emb, const float* w, float b, const float* sts, int32_t gamma, int32_t n_hidden,
                            int32_t rank, float* out) {
  for (int32_t k = 0; k < gamma; k++) {
    float lane[32];
    for (int l = 0; l < 32; l++) {
      float acc = 0.0f;
      for (int32_t i = l; i < n_hidden; i += 32) acc = fmaf(bits_f((uint32_t)hidden[(int64_t)k * n_hidden + i] << 16), w[i], acc);
      for (int32_t i = l; i < rank; i += 32) acc = fmaf(bits_f((uint32_t)emb[(int64_t)k * rank + i] << 16), w[n_hidden + i], acc);
      lane[l] = acc;
    }
    for (int o = 16; o > 0; o >>= 1) {
      float next[32];
      for (int l = 0; l < 32; l++) { volatile float t = lane[l] + lane[l ^ o]; next[l] = t; }
      memcpy(lane, next, sizeof(lane));
    }
    volatile float zb = round_bf16(lane[0]) + b;
    const float z = round_bf16(zb);
    volatile float x = z / (sts ? sts[k] : 1.0f);
    volatile float arg = -fabsf(x) * 1.44269502f;
    const float e = lmo_spec_exp2(arg);
    volatile float den = 1.0f + e;
    out[k] = x >= 0.0f ? 1.0f / den : e / den;
  }
}

/* ---- DSpark verification ------------------------------------------------------------------------------------- */

/* Greedy (spec_ops.metal:162-165 with base = 0): acc = longest prefix with token[r] == draft[r]; final = token[acc]. */
LMO_API int32_t lmo_accept_greedy(const int32_t* tokens, const int32_t* drafts, int32_t n_draft, int32_t* out_final) {
  int32_t acc = 0;
  while (acc < n_draft && tokens[acc] == drafts[acc]) acc++;
  if (out_final) *out_final = tokens[acc];
  return acc;
}

/* binary32 probability of one token under the kept softmax: fl32(double(W) / double(K)), W and K the integer weights */
static inline float prob_q40(uint64_t w, uint64_t k) { return (float)((double)w / (double)k); }

/* Stochastic verification with caller-supplied uniforms (restates sample.metal:273-347 on the integer weights).
 *   z        [n_draft + 1][vocab]  target logits, widened (row r verifies draft r; row n_draft is the bonus row)
 *   tau      [n_draft + 1]         the target's kept-set threshold per row (-inf for none)
 *   q        [n_draft][vocab]      the drafter's probabilities (binary32)
 *   u_accept [n_draft], u_final    uniforms in [0, 1)
 * p_r(v) = fl32(W_r(v) / K_r) for z >= tau_r, else 0.  reject_r  <=>  fl32(u_r * q_r(d_r)) >= p_r(d_r).
 * j = first rejected r, or n_draft.  Row j: residual weights R(v) = floor(2^40 * fl32(p_j(v) - q_j(v))) where
 * positive (q = 0 on the bonus row); the final token is the inverse-CDF draw over R with u_final; if R sums to 0
 * the draw is over the row's own weights W_j.  Returns j; out_final gets the token. */
LMO_API int32_t lmo_verify_stochastic(const float* z, int64_t vocab, int32_t n_draft, const float* tau, float temperature, const int32_t* drafts,
                                      const float* q, const float* u_accept, float u_final, int32_t* out_final, float* out_p_draft) {
  const float c = lmo_exp2_scale(temperature);
  int32_t j = n_draft;
  float* vmaxs = (float*)malloc(sizeof(float) * (size_t)(n_draft + 1));
  uint64_t* ks = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n_draft + 1));
  for (int32_t r = 0; r <= n_draft; r++) {
    const float* zr = z + (int64_t)r * vocab;
    float vmax = -INFINITY;
    for (int64_t i = 0; i < vocab; i++) if (zr[i] > vmax) vmax = zr[i];
    uint64_t k = 0;
    for (int64_t i = 0; i < vocab; i++) if (zr[i] >= tau[r]) k += lmo_weight_q40(zr[i], vmax, c);
    vmaxs[r] = vmax; ks[r] = k;
  }
  for (int32_t r = 0; r < n_draft; r++) {
    const float* zr = z + (int64_t)r * vocab;
    const int32_t d = drafts[r];
    float pd = 0.0f;
    if (d >= 0 && d < vocab && zr[d] >= tau[r] && ks[r] > 0) pd = prob_q40(lmo_weight_q40(zr[d], vmaxs[r], c), ks[r]);
    const float qd = (d >= 0 && d < vocab) ? q[(int64_t)r * vocab + d] : 0.0f;
    volatile float uq = u_accept[r] * qd;
    if (out_p_draft) out_p_draft[r] = pd;
    if (uq >= pd && r < j) j = r;
  }
  const float* zj = z + (int64_t)j * vocab;
  const float* qj = (j < n_draft) ? q + (int64_t)j * vocab : NULL;
  uint64_t total = 0;
  if (ks[j] > 0) for (int64_t i = 0; i < vocab; i++) {
    if (!(zj[i] >= tau[j])) continue;
    const float p = prob_q40(lmo_weight_q40(zj[i], vmaxs[j], c), ks[j]);
    volatile float res = qj ? p - qj[i] : p;
    if (res > 0.0f) total += (uint64_t)(res * 1099511627776.0f);
  }
  int32_t token = -1;
  if (total > 0) {
    const uint64_t target = lmo_cdf_target(u_final, total);
    uint64_t cum = 0;
    for (int64_t i = 0; i < vocab; i++) {
      if (!(zj[i] >= tau[j])) continue;
      const float p = prob_q40(lmo_weight_q40(zj[i], vmaxs[j], c), ks[j]);
      volatile float res = qj ? p - qj[i] : p;
      if (res > 0.0f) { cum += (uint64_t)(res * 1099511627776.0f); if (cum > target) { token = (int32_t)i; break; } }
    }
  } else {
    token = lmo_sample_invcdf_index(zj, vocab, tau[j], temperature, u_final, NULL);
  }
  if (out_final) *out_final = token;
  free(vmaxs); free(ks);
  return j;
}

/* Stochastic verification with the reference's own randomness (sample.metal:279-347): the accept uniform of draft r is
 * uniform01(seed, step, 3000 + r, 0) unless u_accept is given; the rejected row's token is
 * argmax_i { logf(res_i) + gumbel(seed, step, 4000, i) : res_i > 0 } with res as in lmo_verify_stochastic; with every draft accepted,
 * or an empty residual, the row keeps the ordinary sampler's token argmax_i { fl32(z_i * fl32(1/T)) + gumbel(seed, step, row0 + j, i) :
 * z_i >= tau_j }. Ties -> lowest index. out_gap: best key minus second-best key of the draw that decided (logf is library-specific).
 * PARITY UNPINNED like lmo_verify_stochastic: the reference only checks this path's distribution. */
LMO_API int32_t lmo_verify_gumbel(const float* z, int64_t vocab, int32_t n_draft, const float* tau, float temperature, const int32_t* drafts,
                                  const float* q, const float* u_accept, uint64_t seed, uint32_t step, uint32_t row0, int32_t* out_final, float* out_gap) {
  const float c = lmo_exp2_scale(temperature);
  int32_t j = n_draft;
  float* vmaxs = (float*)malloc(sizeof(float) * (size_t)(n_draft + 1));
  uint64_t* ks = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n_draft + 1));
  for (int32_t r = 0; r <= n_draft; r++) {
    const float* zr = z + (int64_t)r * vocab;
    float vmax = -INFINITY;
    for (int64_t i = 0; i < vocab; i++) if (zr[i] > vmax) vmax = zr[i];
    uint64_t k = 0;
    for (int64_t i = 0; i < vocab; i++) if (zr[i] >= tau[r]) k += lmo_weight_q40(zr[i], vmax, c);
    vmaxs[r] = vmax; ks[r] = k;
  }
  for (int32_t r = 0; r < n_draft; r++) {
    const float* zr = z + (int64_t)r * vocab;
    const int32_t d = drafts[r];
    float pd = 0.0f;
    if (d >= 0 && d < vocab && zr[d] >= tau[r] && ks[r] > 0) pd = prob_q40(lmo_weight_q40(zr[d], vmaxs[r], c), ks[r]);
    const float qd = (d >= 0 && d < vocab) ? q[(int64_t)r * vocab + d] : 0.0f;
    const float u = u_accept ? u_accept[r] : lmo_uniform01(seed, step, 3000u + (uint32_t)r, 0u);
    volatile float uq = u * qd;
    if (uq >= pd && r < j) j = r;
  }
  const float* zj = z + (int64_t)j * vocab;
  const float* qj = (j < n_draft) ? q + (int64_t)j * vocab : NULL;
  float best = -INFINITY, second = -INFINITY; int64_t bi = -1;
  if (qj && ks[j] > 0) for (int64_t i = 0; i < vocab; i++) {
    if (!(zj[i] >= tau[j])) continue;
    const float p = prob_q40(lmo_weight_q40(zj[i], vmaxs[j], c), ks[j]);
    volatile float res = p - qj[i];
    if (!(res > 0.0f)) continue;
    volatile float lr = logf(res);
    const float key = lr + lmo_gumbel(seed, step, 4000u, (uint32_t)i);
    if (key > best) { second = best; best = key; bi = i; } else if (key > second) second = key;
  }
  int32_t token = (int32_t)bi;
  if (bi < 0) {
    float gap = 0.0f;
    token = ks[j] > 0 ? lmo_sample_gumbel(zj, vocab, tau[j], (double)temperature, seed, step, row0 + (uint32_t)j, &gap) : -1;
    if (out_gap) *out_gap = gap;
  } else if (out_gap) *out_gap = best - second;
  if (out_final) *out_final = token;
  free(vmaxs); free(ks);
  return j;
}

/* ---- one full row of the sampler, as the GPU entry point defines it ----------------------------------------- */

/* draw: 0 = Gumbel-max with the counter-based hash (the reference's draw), 1 = inverse CDF from `u`.
 * temperature == 0 selects greedy. Penalties are applied to a private copy. Returns the token. */
LMO_API int32_t lmo_sample_row(const void* logits, int dtype, int64_t vocab, float temperature, int32_t top_k, float top_p, float min_p,
                               int32_t topp_in_topk, const int32_t* history, int64_t hist_len, float rho, float pi, int32_t draw,
                               float u, uint64_t seed, uint32_t step, uint32_t t, float* out_tau, float* out_vmax, float* out_kept,
                               float* out_gap) {
  float* z = (float*)malloc((size_t)vocab * 4);
  lmo_widen(logits, dtype, vocab, z);
  lmo_apply_penalties(z, vocab, history, hist_len, rho, pi);
  int32_t token;
  if (temperature == 0.0f) {
    token = lmo_argmax(z, vocab);
    if (out_tau) *out_tau = -INFINITY;
  } else {
    float vmax; double kept;
    const float tau = lmo_thresholds(z, vocab, (double)temperature, top_k, (double)top_p, (double)min_p, topp_in_topk, &vmax, &kept, NULL);
    if (out_tau) *out_tau = tau;
    if (out_vmax) *out_vmax = vmax;
    if (out_kept) *out_kept = (float)kept;
    token = draw == 0 ? lmo_sample_gumbel(z, vocab, tau, (double)temperature, seed, step, t, out_gap)
                      : lmo_sample_invcdf(z, vocab, tau, temperature, u, NULL);
  }
  free(z);
  return token;
}

/* A batch of rows with per-row knobs (NULL arrays fall back to the scalars); rows are handed out to n_threads
 * POSIX threads through a shared counter. */
#include <pthread.h>
typedef struct {
  const void* logits; int dtype; int64_t rows, vocab, row_stride; const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  const float* top_p; float top_p_s; const float* min_p; float min_p_s; int32_t topp_in_topk; const int32_t* history; int64_t hist_len, hist_stride;
  float rho, pi; int32_t draw; const float* uniforms; uint64_t seed; uint32_t step; int64_t row_offset; int32_t* out_tokens; float* out_tau;
  float* out_stats; int64_t next;
} lmo_batch_t;

static void* lmo_batch_worker(void* arg) {
  lmo_batch_t* b = (lmo_batch_t*)arg;
  const size_t esz = b->dtype == 0 ? 2 : 4;
  for (;;) {
    const int64_t r = __atomic_fetch_add(&b->next, 1, __ATOMIC_RELAXED);
    if (r >= b->rows) break;
    float tau = -INFINITY, vmax = 0.0f, kept = 0.0f;
    b->out_tokens[r] = lmo_sample_row((const char*)b->logits + (size_t)r * (size_t)b->row_stride * esz, b->dtype, b->vocab,
                                      b->temperature ? b->temperature[r] : b->temperature_s, b->top_k ? b->top_k[r] : b->top_k_s,
                                      b->top_p ? b->top_p[r] : b->top_p_s, b->min_p ? b->min_p[r] : b->min_p_s, b->topp_in_topk,
                                      b->history ? b->history + r * b->hist_stride : NULL, b->history ? b->hist_len : 0, b->rho, b->pi, b->draw,
                                      b->uniforms ? b->uniforms[r] : 0.0f, b->seed, b->step, (uint32_t)(b->row_offset + r), &tau, &vmax, &kept, NULL);
    if (b->out_tau) b->out_tau[r] = tau;
    if (b->out_stats) { b->out_stats[2 * r] = vmax; b->out_stats[2 * r + 1] = kept; }
  }
  return NULL;
}

LMO_API void lmo_sample_batch(const void* logits, int dtype, int64_t rows, int64_t vocab, int64_t row_stride, const float* temperature, float temperature_s,
                              const int32_t* top_k, int32_t top_k_s, const float* top_p, float top_p_s, const float* min_p, float min_p_s,
                              int32_t topp_in_topk, const int32_t* history, int64_t hist_len, int64_t hist_stride, float rho, float pi, int32_t draw,
                              const float* uniforms, uint64_t seed, uint32_t step, int64_t row_offset, int32_t* out_tokens, float* out_tau,
                              float* out_stats, int32_t n_threads) {
  lmo_batch_t b = {logits, dtype, rows, vocab, row_stride, temperature, temperature_s, top_k, top_k_s, top_p, top_p_s, min_p, min_p_s, topp_in_topk,
                   history, hist_len, hist_stride, rho, pi, draw, uniforms, seed, step, row_offset, out_tokens, out_tau, out_stats, 0};
  if (n_threads <= 1) { lmo_batch_worker(&b); return; }
  if (n_threads > 256) n_threads = 256;
  pthread_t th[256];
  int started = 0;
  for (int i = 0; i < n_threads; i++) { if (pthread_create(&th[started], NULL, lmo_batch_worker, &b) == 0) started++; }
  if (started == 0) lmo_batch_worker(&b);
  for (int i = 0; i < started; i++) pthread_join(th[i], NULL);
}
