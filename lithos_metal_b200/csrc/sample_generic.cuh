// The generic row sampler: one thread block per row, several passes over the row (the first from HBM, the rest from
// L2), any element type, any values. It is the reference-exact path every other sampler kernel is checked
// against on the GPU, the path for FP32 logits, and the path rows fall back to when the streaming BF16 kernel cannot
// take them.
//
// Thresholds follow the reference's numpy definition (monolith/nn/sampling_ref.py:20-38) in exact arithmetic where it is
// integer (top-k: a 4 x 8-bit radix select on the monotone 32-bit key, ties kept) and in FP64 where it is
// floating point (top-p: the same radix descent on per-bin FP64 softmass, one distinct value per final bin; the
// reference's sample.metal:87-162 does this walk on BF16 buckets in FP32).
#pragma once
#include "common.cuh"
#include "draw.cuh"
#include "spec_ops.cuh"

namespace lm {

struct SampleDev {              // lm_sample_args without the host-only fields
  const void* logits; int dtype; int rows; int vocab; int64_t row_stride;
  const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  const float* top_p; float top_p_s; const float* min_p; float min_p_s;
  uint32_t flags; int draw;
  const int32_t* history; int hist_len; int64_t hist_stride; float rho, pi;
  const float* uniforms; uint64_t seed; uint32_t step; int64_t row_offset;
  int32_t* out_tokens; float* out_tau; float* out_stats; float* out_probs; int64_t probs_stride; uint32_t* out_status;
  float* out_vmax;                                      // optional: the row's maximum (penalised) logit, for the verify step
  unsigned long long* out_mass;                         // optional: the kept set's fixed-point mass, for the verify step
  const uint32_t* state; int t_max, g;                  // optional StepState: seed, step and the active rows come from it
};

// With a StepState, the sampler kernels take from it what the reference's kernels take from theirs (kernels/common/sample.metal:
// 172-181, argmax.metal:44-46): the noise seed and step, and the number of active rows; a finished generation has none. Every
// kernel calls this on its copy of the parameters before anything else.
__device__ __forceinline__ void apply_step_state(SampleDev& P) {
  if (!P.state) return;
  StepStateView st{const_cast<uint32_t*>(P.state), P.t_max, P.g};
  const int active = st.done() ? 0 : static_cast<int>(st.t_this_step());
  P.rows = active < P.rows ? active : P.rows;
  P.seed = st.seed(); P.step = st.step();
}

constexpr uint32_t kStatusBadParam = 16u;
constexpr int kBins = 256;
constexpr int kReplicas = 32;         // per-bin FP64 accumulators, one per lane, so a warp never collides on an address

struct GenericSmem {
  double mass[kBins * kReplicas];     // 64 KB
  double mass0[kBins];                // level-0 bin masses, kept for the top-p descent
  double cum_m[8];
  uint64_t scratch[32];
  DrawSmem draw;
  uint32_t cnt[kBins];
  uint32_t cnt0[kBins];
  uint32_t cum_c[8];
  int sel_pos, last_pos;
  double sel_base_m, sel_incl_m;
  uint32_t sel_base_c;
};

__device__ __forceinline__ double softmass(float z, float vmax, double inv_t) {
  return exp((static_cast<double>(z) - static_cast<double>(vmax)) * inv_t);
}

// Histogram pass over the elements whose key matches `prefix` in the bits above this level's digit.
template <bool MASS>
__device__ void hist_pass(const RowView& rv, int level, uint32_t prefix, float vmax, double inv_t, GenericSmem& s) {
  const int tid = threadIdx.x, lane = tid & 31;
  for (int i = tid; i < kBins; i += kBlock) s.cnt[i] = 0;
  if (MASS) for (int i = tid; i < kBins * kReplicas; i += kBlock) s.mass[i] = 0.0;
  __syncthreads();
  const int shift = 24 - 8 * level;
  const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  for (int c = tid; c < n_chunks; c += kBlock) {
    float z[kChunk];
    const int n = load_chunk(rv, c, z);
#pragma unroll
    for (int e = 0; e < kChunk; e++) {
      if (e >= n) break;
      const uint32_t key = fkey(z[e]);
      if ((key & hi_mask) != prefix) continue;
      const uint32_t bin = (key >> shift) & 0xFFu;
      atomicAdd(&s.cnt[bin], 1u);
      if (MASS) atomicAdd(&s.mass[bin * kReplicas + lane], softmass(z[e], vmax, inv_t));
    }
  }
  __syncthreads();
}

// Threads 0..255 walk the bins from the top (pos 0 = bin 255). Selects the first position where the running
// count reaches `k_target` (BY_MASS = false) or the running mass reaches `m_target` (BY_MASS = true), starting
// from the running totals in s.sel_base_*. Leaves the selected bin in the return value and the running totals
// strictly above it in s.sel_base_c / s.sel_base_m. `cnt`/`mass` are per-bin arrays of kBins entries.
template <bool BY_MASS>
__device__ int select_bin(const uint32_t* cnt, const double* mass, uint32_t k_target, double m_target, GenericSmem& s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) { s.sel_pos = kBins; s.last_pos = -1; }
  __syncthreads();
  uint32_t c = 0, ci = 0; double m = 0.0, mi = 0.0;
  if (tid < kBins) {
    const int bin = kBins - 1 - tid;
    c = cnt[bin]; ci = c;
    if (BY_MASS) { m = mass[bin]; mi = m; }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, ci, o);
      const double tm = BY_MASS ? __shfl_up_sync(kFull, mi, o) : 0.0;
      if (lane >= o) { ci += tc; if (BY_MASS) mi += tm; }
    }
    if (lane == 31) { s.cum_c[warp] = ci; s.cum_m[warp] = mi; }
  }
  __syncthreads();
  if (tid < kBins) {
    uint32_t wc = 0; double wm = 0.0;
    for (int w = 0; w < warp; w++) { wc += s.cum_c[w]; if (BY_MASS) wm += s.cum_m[w]; }
    ci += wc; mi += wm;                                                  // inclusive prefix from the top bin down
    const bool hit = BY_MASS ? (c > 0 && s.sel_base_m + mi >= m_target) : (s.sel_base_c + ci >= k_target);
    if (hit) atomicMin(&s.sel_pos, tid);
    if (c > 0) atomicMax(&s.last_pos, tid);
  }
  __syncthreads();
  const int pos = (s.sel_pos < kBins) ? s.sel_pos : s.last_pos;          // mass never reached (rounding): lowest occupied bin
  __syncthreads();
  if (tid == pos) {
    s.sel_base_c += ci - c;
    if (BY_MASS) { s.sel_incl_m = s.sel_base_m + mi; s.sel_base_m += mi - m; }
  }
  __syncthreads();
  return kBins - 1 - pos;
}

// Fold the 32 per-lane accumulators of every bin (fixed order) into s.mass[bin].
__device__ __forceinline__ void fold_mass(GenericSmem& s) {
  double m = 0.0;
  if (threadIdx.x < kBins) for (int r = 0; r < kReplicas; r++) m += s.mass[threadIdx.x * kReplicas + r];
  __syncthreads();
  if (threadIdx.x < kBins) s.mass[threadIdx.x] = m;
  __syncthreads();
}

// One row, start to finish. All threads of the block call it with the same arguments.
__device__ void sample_row_generic(const SampleDev& P, int row, GenericSmem& s, uint32_t* pen_bits) {
  const int tid = threadIdx.x;
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  uint32_t status = LM_STATUS_GENERIC_PATH;

  RowView rv;
  rv.dtype = P.dtype; rv.vocab = V; rv.rho = P.rho; rv.pi = P.pi; rv.pen = nullptr;
  rv.row = static_cast<const char*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride) * (P.dtype == LM_DTYPE_BF16 ? 2 : 4);
  rv.aligned = (reinterpret_cast<uintptr_t>(rv.row) & 15u) == 0;
  const int n_chunks = (V + kChunk - 1) / kChunk;

  if (V <= 0 || !(T >= 0.0f)) {                                          // empty row or a bad temperature: no token
    if (tid == 0) {
      P.out_tokens[row] = -1;
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_stats) { P.out_stats[2 * row] = 0.0f; P.out_stats[2 * row + 1] = 0.0f; }
      if (P.out_vmax) P.out_vmax[row] = -INFINITY;
      if (P.out_mass) P.out_mass[row] = 0ull;
      if (P.out_status) P.out_status[row] = status | (V > 0 ? kStatusBadParam : 0u);
    }
    return;
  }

  // ---- the row's distinct history ids as a bitmap ----------------------------------------------------------
  if (P.history != nullptr && P.hist_len > 0 && !(P.rho == 1.0f && P.pi == 0.0f)) {
    const int words = (V + 31) / 32;
    for (int i = tid; i < words; i += kBlock) pen_bits[i] = 0u;
    __syncthreads();
    const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
    for (int i = tid; i < P.hist_len; i += kBlock) {
      const int id = __ldg(h + i);
      if (id >= 0 && id < V) atomicOr(&pen_bits[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
    rv.pen = pen_bits;
  }

  // ---- pass A: the maximum and its lowest index --------------------------------------------------------------
  uint64_t best = 0ull;
  bool nan = false;
  for (int c = tid; c < n_chunks; c += kBlock) {
    float z[kChunk];
    const int n = load_chunk(rv, c, z);
#pragma unroll
    for (int e = 0; e < kChunk; e++) if (e < n) {
      nan |= (z[e] != z[e]);
      const uint64_t p = pack_best(z[e], static_cast<uint32_t>(c * kChunk + e));
      best = p > best ? p : best;
    }
  }
  best = block_max_u64(best, s.scratch);
  if (__syncthreads_or(nan)) status |= LM_STATUS_NAN;
  const float vmax = best_value(best);
  const int arg = static_cast<int>(best_index(best));

  if (T == 0.0f) {                                                       // greedy
    if (P.out_probs) {
      float* pr = P.out_probs + static_cast<int64_t>(row) * P.probs_stride;
      for (int i = tid; i < V; i += kBlock) pr[i] = (i == arg) ? 1.0f : 0.0f;
    }
    if (tid == 0) {
      P.out_tokens[row] = arg;
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_stats) { P.out_stats[2 * row] = vmax; P.out_stats[2 * row + 1] = 1.0f; }
      if (P.out_vmax) P.out_vmax[row] = vmax;
      if (P.out_mass) P.out_mass[row] = 0ull;                              // (greedy: no distribution)
      if (P.out_status) P.out_status[row] = status;
    }
    return;
  }

  // ---- thresholds ------------------------------------------------------------------------------------------
  const double T64 = static_cast<double>(T);
  const double inv_t = 1.0 / T64;
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k;
  if (top_k > V) top_k = V;
  double tau64 = -INFINITY;
  bool have_tau = false;
  float tau_k = -INFINITY;

  if (has_k || has_p) {
    if (has_p) hist_pass<true>(rv, 0, 0u, vmax, inv_t, s); else hist_pass<false>(rv, 0, 0u, vmax, inv_t, s);
    if (has_p) fold_mass(s);
    if (tid < kBins) { s.cnt0[tid] = s.cnt[tid]; if (has_p) s.mass0[tid] = s.mass[tid]; }
    __syncthreads();
  }
  if (has_k) {
    if (tid == 0) { s.sel_base_c = 0; s.sel_base_m = 0.0; }
    __syncthreads();
    uint32_t prefix = static_cast<uint32_t>(select_bin<false>(s.cnt0, nullptr, static_cast<uint32_t>(top_k), 0.0, s)) << 24;
    for (int level = 1; level < 4; level++) {
      hist_pass<false>(rv, level, prefix, vmax, inv_t, s);
      prefix |= static_cast<uint32_t>(select_bin<false>(s.cnt, nullptr, static_cast<uint32_t>(top_k), 0.0, s)) << (24 - 8 * level);
    }
    tau_k = fkey_inv(prefix);
    tau64 = tau_k; have_tau = true;
  }
  if (has_p) {
    double total = 0.0;
    if (in_topk) {                                                       // the mass of the top-k set
      double m = 0.0;
      for (int c = tid; c < n_chunks; c += kBlock) {
        float z[kChunk];
        const int n = load_chunk(rv, c, z);
#pragma unroll
        for (int e = 0; e < kChunk; e++) if (e < n && z[e] >= tau_k) m += softmass(z[e], vmax, inv_t);
      }
      total = block_sum_f64(m, s.scratch);
    } else {
      if (tid < 32) {                                                    // sum of the level-0 bins, fixed order
        double m = 0.0;
        for (int b = kBins - 1 - tid; b >= 0; b -= 32) m += s.mass0[b];
        m = warp_sum_f64(m);
        if (tid == 0) s.sel_incl_m = m;
      }
      __syncthreads();
      total = s.sel_incl_m;
      __syncthreads();
    }
    const double target = static_cast<double>(top_p) * total;
    if (tid == 0) { s.sel_base_c = 0; s.sel_base_m = 0.0; }
    __syncthreads();
    uint32_t prefix = static_cast<uint32_t>(select_bin<true>(s.cnt0, s.mass0, 0u, target, s)) << 24;
    for (int level = 1; level < 4; level++) {
      hist_pass<true>(rv, level, prefix, vmax, inv_t, s);
      fold_mass(s);
      prefix |= static_cast<uint32_t>(select_bin<true>(s.cnt, s.mass, 0u, target, s)) << (24 - 8 * level);
    }
    const float tau_p = fkey_inv(prefix);
    const double eps = 1e-12 * total;
    if (fabs(s.sel_incl_m - target) <= eps || fabs(s.sel_base_m - target) <= eps) status |= LM_STATUS_TOPP_EDGE;
    if (!have_tau || static_cast<double>(tau_p) > tau64) tau64 = tau_p;
    have_tau = true;
  }
  if (has_m) {
    const double tau_m = static_cast<double>(vmax) + T64 * log(static_cast<double>(min_p));
    if (!have_tau || tau_m > tau64) tau64 = tau_m;
    have_tau = true;
  }
  // A +inf logit makes every mass NaN: the reference's top-p search then finds nothing and falls back to the largest value, and
  // its min-p threshold is +inf itself (sampling_ref.py:33-37 with numpy's argmax of an all-false mask): only the +inf logits stay.
  if (vmax == INFINITY && (has_p || has_m)) { tau64 = INFINITY; have_tau = true; }
  const float tau = have_tau ? __double2float_rn(tau64) : -INFINITY;

  // ---- kept-set statistics (only when asked for) ----------------------------------------------------------------
  const bool need_mass = (P.out_stats != nullptr) || (P.out_probs != nullptr);
  double kept_mass = 0.0;
  if (need_mass) {
    double m = 0.0;
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if (e < n && z[e] >= tau) m += softmass(z[e], vmax, inv_t);
    }
    kept_mass = block_sum_f64(m, s.scratch);
  }

  // ---- the draw --------------------------------------------------------------------------------------------------
  int token;
  uint64_t kept_weight = 0ull;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    token = draw_inverse_cdf(rv, tau, vmax, T, P.uniforms ? P.uniforms[row] : 0.0f, s.draw, &kept_weight);
  } else {
    bool tie = false;
    token = draw_gumbel(rv, tau, T, P.seed, P.step, static_cast<uint32_t>(P.row_offset + row), s.draw, &tie);
    if (tie) status |= LM_STATUS_NEAR_TIE;
    if (P.out_mass) kept_weight = kept_weight_total(rv, tau, vmax, T, s.draw);
  }

  // ---- outputs ----------------------------------------------------------------------------------------------------
  if (P.out_probs) {
    float* pr = P.out_probs + static_cast<int64_t>(row) * P.probs_stride;
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
      for (int e = 0; e < n; e++) pr[c * kChunk + e] = (z[e] >= tau) ? static_cast<float>(softmass(z[e], vmax, inv_t) / kept_mass) : 0.0f;
    }
  }
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_stats) { P.out_stats[2 * row] = vmax; P.out_stats[2 * row + 1] = static_cast<float>(kept_mass); }
    if (P.out_vmax) P.out_vmax[row] = vmax;
    if (P.out_mass) P.out_mass[row] = kept_weight;
    if (P.out_status) P.out_status[row] = status;
  }
}

}  // namespace lm
