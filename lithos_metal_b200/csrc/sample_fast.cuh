// The streaming BF16 row sampler: one thread block per row, ONE pass over the row from HBM.
//
// A BF16 logit has at most 65536 codes, so a histogram of the row by code (shared memory, 16-bit counters packed in
// pairs, one 32-bit shared-memory reduction per logit) holds everything the thresholds need: the k-th largest value is a
// walk over counts, the top-p boundary a walk over count x exp(value) in FP64, exactly as the reference's numpy
// definition forms them per distinct value (monolith/nn/sampling_ref.py:26-35; the reference's Metal kernels build
// the same histogram in device memory with 256 KB per row, kernels/common/sample.metal:34-162). Logits changed by
// the penalties are arbitrary FP32 values: they are counted in the bin of the largest BF16 value below them
// and kept aside in a short list, so the walk stays exact by refining inside the one bin where it lands.
// The draw then takes a second pass that finds the row in L2 (the next row is prefetched into L2 meanwhile).
//
// Rows this kernel cannot take (a counter overflow: more than 65535 equal logits; more than kSideCap penalised
// logits; more than kBinSideCap of them in the bin a threshold lands in; vocabularies that are not a multiple of
// 8 or exceed kFastMaxVocab; misaligned rows) are marked in `punt` and handled by the generic kernel launched
// behind this one.
#pragma once
#include "common.cuh"
#include "draw.cuh"
#include "sample_generic.cuh"

namespace lm {

constexpr int kFastMaxVocab = 262144;
constexpr int kCodes = 65536;
constexpr int kGroups = kCodes / 32;        // 2048 groups of 32 consecutive positions (descending value order)
constexpr int kSideCap = 4096;              // penalised logits per row the kernel keeps aside
constexpr int kBinSideCap = 32;             // of those, how many may share the BF16 bin a threshold lands in

struct FastSmem {
  uint32_t hist[kCodes / 2];                // 128 KB: 16-bit counters, code c in half (c & 1) of word c >> 1
  double gmass[kGroups];                    // 16 KB
  uint32_t gcnt[kGroups];                   // 8 KB
  float side_val[kSideCap];                 // 16 KB
  float bin_side[32][kBinSideCap];          // 4 KB: side values of the 32 bins of the group being refined
  DrawSmem draw;
  double warp_m[32];
  uint32_t warp_c[32];
  uint32_t side_n, bin_side_n[32];
  uint32_t side_max_key;
  int sel_group;
  uint32_t sel_base_c;
  double sel_base_m;
  float res_tau; double res_cum_m; uint32_t res_cum_c; int res_fail;
  uint32_t pen[kFastMaxVocab / 32];         // 32 KB bitmap of the row's distinct history ids
};

// position in descending value order <-> BF16 code (+inf first ... +0, -0 ... -inf; NaN codes at both ends)
__device__ __forceinline__ uint32_t pos_to_code(uint32_t pos) { return pos < 0x8000u ? 0x7FFFu - pos : pos; }
__device__ __forceinline__ uint32_t code_to_pos(uint32_t code) { return code < 0x8000u ? 0x7FFFu - code : code; }
__device__ __forceinline__ float code_val(uint32_t code) { return __uint_as_float(code << 16); }
// code of the largest BF16 value <= v
__device__ __forceinline__ uint32_t floor_code(float v) {
  const uint32_t u = __float_as_uint(v);
  uint32_t code = u >> 16;
  if ((u & 0x80000000u) && (u & 0xFFFFu)) code += 1u;
  return code;
}
__device__ __forceinline__ uint32_t hist_get(const uint32_t* hist, uint32_t code) { return (hist[code >> 1] >> ((code & 1u) * 16u)) & 0xFFFFu; }
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t code) { atomicAdd(&hist[code >> 1], (code & 1u) ? 0x10000u : 1u); }

// two logits of one 32-bit word into the histogram: address = code / 2 words, increment = 1 << (16 * (code & 1))
__device__ __forceinline__ void hist_add_word(uint32_t* hist, uint32_t w) {
  char* base = reinterpret_cast<char*>(hist);
  atomicAdd(reinterpret_cast<uint32_t*>(base + ((w << 1) & 0x1FFFCu)), (w & 1u) * 0xFFFFu + 1u);
  atomicAdd(reinterpret_cast<uint32_t*>(base + ((w >> 15) & 0x1FFFCu)), ((w >> 16) & 1u) * 0xFFFFu + 1u);
}

__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Exact walk inside one group of 32 positions (warp 0; the other warps wait at the barriers around the call).
// Finds the first distinct value, descending, at which the running count reaches k_target (BY_MASS false) or the
// running mass reaches m_target (BY_MASS true), starting from (base_c, base_m) = totals strictly above the group.
// Results in s.res_*; s.res_fail = 1 if too many side values share one bin.
template <bool BY_MASS, bool NEED_MASS>
__device__ void refine_group(FastSmem& s, int group, uint32_t base_c, double base_m, uint32_t k_target, double m_target, float vmax, double inv_t) {
  const int tid = threadIdx.x, lane = tid & 31;
  // every thread: the side values whose floor position falls in this group go to the list of their bin
  if (tid < 32) s.bin_side_n[tid] = 0u;
  if (tid == 0) s.res_fail = 0;
  __syncthreads();
  const uint32_t n_side = min(s.side_n, static_cast<uint32_t>(kSideCap));
  for (uint32_t i = tid; i < n_side; i += kBlock) {
    const float v = s.side_val[i];
    const uint32_t pos = code_to_pos(floor_code(v));
    if (static_cast<int>(pos >> 5) == group) {
      const uint32_t slot = atomicAdd(&s.bin_side_n[pos & 31u], 1u);
      if (slot < kBinSideCap) s.bin_side[pos & 31u][slot] = v; else s.res_fail = 1;
    }
  }
  __syncthreads();
  if (s.res_fail) return;
  if (tid < 32) {
    const uint32_t pos = static_cast<uint32_t>(group) * 32u + lane;
    const uint32_t code = pos_to_code(pos);
    const float bval = code_val(code);
    const uint32_t cnt = hist_get(s.hist, code);
    const uint32_t mine = s.bin_side_n[lane];                            // side values living in this lane's bin
    const float* sv = s.bin_side[lane];
    const uint32_t pure = cnt - mine;
    double m = 0.0;
    if (NEED_MASS && cnt) {
      if (pure) m = static_cast<double>(pure) * softmass(bval, vmax, inv_t);
      for (uint32_t i = 0; i < mine; i++) m += softmass(sv[i], vmax, inv_t);
    }
    uint32_t ci = cnt; double mi = m;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, ci, o);
      const double tm = __shfl_up_sync(kFull, mi, o);
      if (lane >= o) { ci += tc; mi += tm; }
    }
    const bool hit = BY_MASS ? (cnt > 0 && base_m + mi >= m_target) : (base_c + ci >= k_target);
    const uint32_t hits = __ballot_sync(kFull, hit);
    const uint32_t occ = __ballot_sync(kFull, cnt > 0);
    const int sel = hits ? (__ffs(hits) - 1) : (31 - __clz(occ));        // mass never reached (rounding): the lowest occupied bin
    if (lane == sel) {
      // inside the bin: side values above the BF16 value, descending, equal values as one step, then the BF16 value itself
      uint32_t run_c = base_c + ci - cnt; double run_m = base_m + mi - m;
      float tau = bval; bool done = false;
      float prev = INFINITY;
      for (uint32_t step = 0; step < mine && !done; step++) {
        float best = -INFINITY;                                          // the next distinct side value below `prev` and above bval
        for (uint32_t i = 0; i < mine; i++) { const float v = sv[i]; if (v < prev && v > bval && v > best) best = v; }
        if (best == -INFINITY) break;
        uint32_t n_eq = 0;
        for (uint32_t i = 0; i < mine; i++) if (sv[i] == best) n_eq++;
        run_c += n_eq; if (NEED_MASS) run_m += static_cast<double>(n_eq) * softmass(best, vmax, inv_t);
        if (BY_MASS ? (run_m >= m_target) : (run_c >= k_target)) { tau = best; done = true; }
        prev = best;
      }
      if (!done) {                                                        // the BF16 value's own tie group (pure elements + side values equal to it)
        run_c = base_c + ci; run_m = base_m + mi; tau = bval;
      }
      s.res_tau = tau; s.res_cum_c = run_c; s.res_cum_m = run_m;
    }
  }
  __syncthreads();
}

// Block-wide search over the groups, descending: the first group at which the running count / mass reaches the target.
// Leaves the group in s.sel_group and the totals strictly above it in s.sel_base_c / s.sel_base_m.
template <bool BY_MASS>
__device__ void find_group(FastSmem& s, uint32_t k_target, double m_target) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // thread t owns groups 2t and 2t + 1
  const uint32_t c0 = s.gcnt[2 * tid], c1 = s.gcnt[2 * tid + 1];
  const double m0 = BY_MASS ? s.gmass[2 * tid] : 0.0, m1 = BY_MASS ? s.gmass[2 * tid + 1] : 0.0;
  uint32_t ci = c0 + c1; double mi = m0 + m1;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t tc = __shfl_up_sync(kFull, ci, o);
    const double tm = BY_MASS ? __shfl_up_sync(kFull, mi, o) : 0.0;
    if (lane >= o) { ci += tc; mi += tm; }
  }
  if (tid == 0) s.sel_group = kGroups;
  if (lane == 31) { s.warp_c[warp] = ci; s.warp_m[warp] = mi; }
  __syncthreads();
  uint32_t wc = 0; double wm = 0.0;
  for (int w = 0; w < warp; w++) { wc += s.warp_c[w]; if (BY_MASS) wm += s.warp_m[w]; }
  const uint32_t excl_c = wc + ci - (c0 + c1); const double excl_m = wm + mi - (m0 + m1);
  // first of this thread's two groups that reaches the target
  int g = kGroups;
  if (BY_MASS) {
    if (c0 > 0 && excl_m + m0 >= m_target) g = 2 * tid; else if (c1 > 0 && excl_m + m0 + m1 >= m_target) g = 2 * tid + 1;
  } else {
    if (excl_c + c0 >= k_target) g = 2 * tid; else if (excl_c + c0 + c1 >= k_target) g = 2 * tid + 1;
  }
  if (g < kGroups) atomicMin(&s.sel_group, g);
  __syncthreads();
  int sel = s.sel_group;
  if (sel == kGroups) {                                                   // mass never reached (rounding): the last occupied group
    __syncthreads();
    if (tid == 0) s.sel_group = -1;
    __syncthreads();
    if (c1 > 0) atomicMax(&s.sel_group, 2 * tid + 1); else if (c0 > 0) atomicMax(&s.sel_group, 2 * tid);
    __syncthreads();
    sel = s.sel_group;
  }
  if ((sel >> 1) == tid) {
    s.sel_base_c = excl_c + ((sel & 1) ? c0 : 0u);
    s.sel_base_m = excl_m + ((sel & 1) ? m0 : 0.0);
  }
  __syncthreads();
}

__device__ void sample_row_fast(const SampleDev& P, int row, FastSmem& s, uint32_t* punt) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const uint16_t* rowp = reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride);
  const bool pen_on = P.history != nullptr;
  const bool takeable = (V % kChunk) == 0 && V <= kFastMaxVocab && (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0 && (T >= 0.0f) && V > 0;
  if (!takeable) { if (tid == 0) punt[row] = 1u; return; }

  RowView rv;
  rv.dtype = LM_DTYPE_BF16; rv.vocab = V; rv.rho = P.rho; rv.pi = P.pi; rv.row = rowp; rv.aligned = true; rv.pen = nullptr;
  const int n_chunks = V / kChunk;

  // ---- clear the histogram; the history's distinct ids as a bitmap ---------------------------------------------
  {
    uint4* h4 = reinterpret_cast<uint4*>(s.hist);
    for (int i = tid; i < kCodes / 8; i += kBlock) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) { s.side_n = 0u; s.side_max_key = 0u; }
    if (pen_on) {
      const int words = (V + 31) / 32;
      for (int i = tid; i < words; i += kBlock) s.pen[i] = 0u;
      __syncthreads();
      const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
      for (int i = tid; i < P.hist_len; i += kBlock) {
        const int id = __ldg(h + i);
        if (id >= 0 && id < V) atomicOr(&s.pen[id >> 5], 1u << (id & 31));
      }
      rv.pen = s.pen;
    }
    __syncthreads();
  }

  if (T == 0.0f) {                                                        // greedy: a streaming argmax, no histogram
    uint64_t best = 0ull;
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) { const uint64_t p = pack_best(z[e], static_cast<uint32_t>(c * kChunk + e)); best = p > best ? p : best; }
    }
    best = block_max_u64(best, s.draw.scratch);
    if (tid == 0) {
      P.out_tokens[row] = static_cast<int>(best_index(best));
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_status) P.out_status[row] = (best_value(best) != best_value(best)) ? LM_STATUS_NAN : 0u;
      punt[row] = 0u;
    }
    return;
  }

  // ---- pass 1: the histogram, straight from HBM; penalised logits also go to the side list -------------------------
  {
    const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
    constexpr int kUnroll = 4;
    for (int c0 = tid; c0 < n_chunks; c0 += kBlock * kUnroll) {
      uint4 q[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; j++) { const int c = c0 + j * kBlock; if (c < n_chunks) q[j] = __ldg(p4 + c); }
#pragma unroll
      for (int j = 0; j < kUnroll; j++) {
        const int c = c0 + j * kBlock;
        if (c >= n_chunks) break;
        const uint32_t bits = pen_on ? ((s.pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu) : 0u;
        if (bits == 0u) {
          hist_add_word(s.hist, q[j].x); hist_add_word(s.hist, q[j].y); hist_add_word(s.hist, q[j].z); hist_add_word(s.hist, q[j].w);
        } else {
          const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
          for (int e = 0; e < kChunk; e++) {
            const uint32_t code = (e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xFFFFu);
            if ((bits >> e) & 1u) {
              const float v = penalise(code_val(code), P.rho, P.pi);
              hist_add(s.hist, floor_code(v));
              const uint32_t slot = atomicAdd(&s.side_n, 1u);
              if (slot < kSideCap) s.side_val[slot] = v;
              atomicMax(&s.side_max_key, fkey(v));
            } else {
              hist_add(s.hist, code);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  // the next row of this block: start pulling it into L2 while this one is selected and drawn
  {
    const int next = row + gridDim.x;
    const char* np = reinterpret_cast<const char*>(rowp) + static_cast<size_t>(gridDim.x) * static_cast<size_t>(P.row_stride) * 2;
    if (next < P.rows && tid < 32 && (reinterpret_cast<uintptr_t>(np) & 15u) == 0) {
      const uint32_t bytes = static_cast<uint32_t>(V) * 2u;
      const uint32_t piece = ((bytes / 32u) + 15u) & ~15u;
      const uint32_t off = piece * lane;
      if (off < bytes) prefetch_l2(np + off, min(piece, bytes - off));
    }
  }

  // ---- group counts, the overflow check, the maximum ---------------------------------------------------------------
  uint32_t total_c = 0; uint32_t top_pos = 0xFFFFFFFFu;
  for (int g = warp; g < kGroups; g += 32) {
    const uint32_t pos = static_cast<uint32_t>(g) * 32u + lane;
    const uint32_t cnt = hist_get(s.hist, pos_to_code(pos));
    const uint32_t occ = __ballot_sync(kFull, cnt > 0);
    uint32_t c = cnt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(kFull, c, o);
    if (lane == 0) s.gcnt[g] = c;
    total_c += c;
    if (occ && top_pos == 0xFFFFFFFFu) top_pos = static_cast<uint32_t>(g) * 32u + (__ffs(occ) - 1);
  }
  // total over the warps; the lowest occupied position
  if (lane == 0) { s.warp_c[warp] = total_c; s.draw.scratch[warp] = top_pos; }
  __syncthreads();
  {
    uint32_t t = 0, tp = 0xFFFFFFFFu;
    for (int w = 0; w < 32; w++) { t += s.warp_c[w]; tp = min(tp, static_cast<uint32_t>(s.draw.scratch[w])); }
    total_c = t; top_pos = tp;
  }
  __syncthreads();
  if (total_c != static_cast<uint32_t>(V) || s.side_n > kSideCap) {       // a 16-bit counter wrapped, or too many penalised logits
    if (tid == 0) punt[row] = 1u;
    return;
  }
  uint32_t status = 0u;
  {                                                                       // NaN codes: 0x7F81..0x7FFF and 0xFF81..0xFFFF
    uint32_t nan_c = 0;
    if (tid < 127) nan_c = hist_get(s.hist, 0x7F81u + tid) + hist_get(s.hist, 0xFF81u + tid);
    if (__syncthreads_or(nan_c != 0u)) status |= LM_STATUS_NAN;
  }
  const float top_val = code_val(pos_to_code(top_pos));
  const float side_max = s.side_max_key ? fkey_inv(s.side_max_key) : -INFINITY;
  const float vmax = (s.side_n > 0 && side_max > top_val) ? side_max : top_val;

  // ---- thresholds ----------------------------------------------------------------------------------------------------
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k && has_p;
  if (top_k > V) top_k = V;
  double tau64 = -INFINITY; bool have_tau = false;
  double topk_mass = 0.0;
  if (has_p) {
    // group masses: every bin as if all its logits sat at the bin's BF16 value, then the side values' excess
    for (int g = warp; g < kGroups; g += 32) {
      if (s.gcnt[g] == 0u) { if (lane == 0) s.gmass[g] = 0.0; continue; }
      const uint32_t code = pos_to_code(static_cast<uint32_t>(g) * 32u + lane);
      const uint32_t cnt = hist_get(s.hist, code);
      double m = cnt ? static_cast<double>(cnt) * softmass(code_val(code), vmax, inv_t) : 0.0;
      m = warp_sum_f64(m);
      if (lane == 0) s.gmass[g] = m;
    }
    __syncthreads();
    const uint32_t n_side = s.side_n;
    for (uint32_t i = tid; i < n_side; i += kBlock) {
      const float v = s.side_val[i];
      const uint32_t code = floor_code(v);
      const double d = softmass(v, vmax, inv_t) - softmass(code_val(code), vmax, inv_t);
      if (d != 0.0) atomicAdd(&s.gmass[code_to_pos(code) >> 5], d);
    }
    __syncthreads();
  }
  if (has_k) {
    find_group<false>(s, static_cast<uint32_t>(top_k), 0.0);
    double base_m = 0.0;
    if (in_topk) {                                                        // the mass strictly above the group: needed for the top-k set's mass
      double m = 0.0;
      for (int g = tid; g < s.sel_group; g += kBlock) m += s.gmass[g];
      base_m = block_sum_f64(m, s.draw.scratch);
    }
    if (in_topk) refine_group<false, true>(s, s.sel_group, s.sel_base_c, base_m, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    else refine_group<false, false>(s, s.sel_group, s.sel_base_c, 0.0, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    if (s.res_fail) { if (tid == 0) punt[row] = 1u; return; }
    tau64 = s.res_tau; have_tau = true;
    topk_mass = s.res_cum_m;
    __syncthreads();
  }
  if (has_p) {
    double total;
    if (in_topk) total = topk_mass;
    else {
      double m = 0.0;
      for (int g = tid; g < kGroups; g += kBlock) m += s.gmass[g];
      total = block_sum_f64(m, s.draw.scratch);
    }
    const double target = static_cast<double>(top_p) * total;
    find_group<true>(s, 0u, target);
    refine_group<true, true>(s, s.sel_group, s.sel_base_c, s.sel_base_m, 0u, target, vmax, inv_t);
    if (s.res_fail) { if (tid == 0) punt[row] = 1u; return; }
    const double eps = 1e-12 * total;
    if (fabs(s.res_cum_m - target) <= eps) status |= LM_STATUS_TOPP_EDGE;
    if (!have_tau || static_cast<double>(s.res_tau) > tau64) tau64 = s.res_tau;
    have_tau = true;
    __syncthreads();
  }
  if (has_m) {
    const double tau_m = static_cast<double>(vmax) + T64 * log(static_cast<double>(min_p));
    if (!have_tau || tau_m > tau64) tau64 = tau_m;
    have_tau = true;
  }
  const float tau = have_tau ? __double2float_rn(tau64) : -INFINITY;

  // ---- pass 2: the draw over the kept set (the row is in L2) ---------------------------------------------------------
  int token;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    token = draw_inverse_cdf(rv, tau, vmax, T, P.uniforms ? P.uniforms[row] : 0.0f, s.draw);
  } else {
    bool tie = false;
    token = draw_gumbel(rv, tau, T, P.seed, P.step, static_cast<uint32_t>(P.row_offset + row), s.draw, &tie);
    if (tie) status |= LM_STATUS_NEAR_TIE;
  }
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
    punt[row] = 0u;
  }
}

}  // namespace lm
