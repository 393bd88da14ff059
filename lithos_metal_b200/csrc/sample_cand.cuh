// The candidate path of the streaming BF16 sampler: rows with 1 <= top_k <= kCandMaxK in ONE pass and no histogram.
//
// With top-k on, the kept set lies inside the row's top-k logits. So the single pass over the row only has to (a) collect the
// few logits at or above a cutoff value carried over from the previous row of the block (about 1 % of the row), and
// (b) accumulate the softmass of the whole row in FP32 (the top-p target needs it). Everything exact then happens on the
// candidates alone: the k-th largest value, FP64 masses, the top-p boundary, integer weights, the draw. The FP32 mass is
// only used to decide on which side of top_p * Z a cumulative mass lies; if that is closer than the FP32 error bound, or
// the candidates do not cover the top-k set, the row is redone by the histogram path, which is exact on its own.
// No counterpart in the reference (its sampler always builds the full histogram, kernels/common/sample.metal:34-162).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "draw.cuh"
#include "sample_generic.cuh"

namespace lm {

#ifdef LM_PROFILE_PHASES
__device__ unsigned long long g_phase_cycles[16];    // clock64 totals per phase of block 0 (profiling builds only)
#define LM_CPHASE(i) do { __syncthreads(); if (threadIdx.x == 0 && blockIdx.x == 0) { const long long _t = clock64(); atomicAdd(&g_phase_cycles[i], (unsigned long long)(_t - _t0)); _t0 = _t; } } while (0)
#else
#define LM_CPHASE(i) do {} while (0)
#endif

constexpr int kCandCap = 2048;            // candidates per row (logits at or above the cutoff)
constexpr int kCandBins = 512;            // BF16 codes above the cutoff that the coarse count covers
constexpr int kCandMaxK = 1024;           // largest top_k this path takes
constexpr int kHitSlots = 12288 / kBlock;  // chunks with a candidate one thread may meet in a row (expected 1.4 at 1024 threads)
constexpr int kCandHigh = 1800, kCandLow = 1200;   // the cutoff moves one BF16 step when the candidate count leaves this band

struct CandSmem {                          // lives in the histogram's shared memory: the two paths never run at the same time
  unsigned long long key[kCandCap];        // candidates as (monotone value key << 32) | ~index, in arrival order
  unsigned long long sel[kCandCap];        // those at or above the coarse top-k crossing, sorted: value descending, index ascending
  double cum[kCandCap];                    // inclusive FP64 softmass prefix over sel
  unsigned long long w[kCandCap];          // fixed-point weights / index-sort keys of the kept prefix
  uint32_t bins[kCandBins];                // candidates per BF16 code, relative to the cutoff code
  uint32_t hits[kHitSlots * kBlock];       // per thread: (chunk << 8 | 8-bit mask) of its chunks that hold a candidate; slot-major
  double warp_d[32];
  float warp_f[32];
  uint32_t n, n_sel, wide, cross_bin;
  int hit, token;
  float amb;
};

__device__ __forceinline__ float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// bitonic sort of a[0 .. n_pow2) in shared memory, descending; every thread of the block calls. One compare-exchange
// per thread and step: thread t takes the t-th pair (i, i ^ j) with i's bit j clear.
__device__ __forceinline__ void bitonic_desc(unsigned long long* a, int n_pow2) {
  for (int k = 2; k <= n_pow2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = threadIdx.x; t < (n_pow2 >> 1); t += kBlock) {
        const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
        const int partner = i | j;
        const unsigned long long x = a[i], y = a[partner];
        const bool desc = (i & k) == 0;
        if (desc ? (x < y) : (x > y)) { a[i] = y; a[partner] = x; }
      }
      __syncthreads();
    }
  }
}

__device__ __forceinline__ int next_pow2(int n) { int p = 32; while (p < n) p <<= 1; return p; }

// Inclusive FP64 prefix sum over v[0 .. n) (n <= kCandCap) in place, index order; every thread calls.
__device__ __forceinline__ void scan_f64(double* v, int n, double* warp_d) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double carry = 0.0;
  for (int base = 0; base < n; base += kBlock) {
    const int i = base + tid;
    double x = (i < n) ? v[i] : 0.0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const double t = __shfl_up_sync(kFull, x, o); if (lane >= o) x += t; }
    __syncthreads();
    if (lane == 31) warp_d[warp] = x;
    __syncthreads();
    double wsum = 0.0;
    for (int w = 0; w < warp; w++) wsum += warp_d[w];
    if (i < n) v[i] = carry + wsum + x;
    double tot = 0.0;
    for (int w = 0; w < kWarps; w++) tot += warp_d[w];
    carry += tot;
  }
  __syncthreads();
}

struct CutoffState { uint32_t code; uint32_t valid; };   // the BF16 code (positive, finite) of the cutoff value; per block

// Inclusive u64 prefix sum over v[0 .. n) in place, index order; every thread calls. Returns the total.
__device__ __forceinline__ uint64_t scan_u64(unsigned long long* v, int n, uint64_t* scratch) {
  uint64_t carry = 0ull;
  for (int base = 0; base < n; base += kBlock) {
    const int i = base + threadIdx.x;
    const uint64_t x = (i < n) ? v[i] : 0ull;
    uint64_t tot = 0ull;
    const uint64_t excl = block_exclusive_scan_u64(x, scratch, &tot);
    if (i < n) v[i] = carry + excl + x;
    carry += tot;
    __syncthreads();
  }
  return carry;
}

__device__ __forceinline__ void cand_append(CandSmem& c, float value, uint32_t index, uint32_t cut_code) {
  const uint32_t slot = atomicAdd(&c.n, 1u);
  if (slot < kCandCap) c.key[slot] = (static_cast<unsigned long long>(fkey(value)) << 32) | (0xFFFFFFFFu - index);
  const uint32_t u = __float_as_uint(value);
  const uint32_t rel = (u >> 16) - cut_code;                               // value >= cutoff > 0: the truncated code is its floor code
  if (rel >= kCandBins) c.wide = 1u; else atomicAdd(&c.bins[rel], 1u);
}

// One row through the candidate path. Every thread of the block calls with the same arguments; returns true when
// the row is finished, false when the histogram path has to take it (nothing has been written then).
__device__ bool sample_row_candidates(const SampleDev& P, int row, const uint16_t* rowp, int V, float T, int top_k, float top_p, float min_p,
                                      CandSmem& c, CutoffState& cut, const int* side_idx, float* side_val, uint32_t n_side,
                                      const uint32_t* pen, uint64_t* scratch) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_chunks = V / kChunk;
  const uint32_t cut_code = cut.code;
  const float cut_val = __uint_as_float(cut_code << 16);
  const bool has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_p;
  const bool need_z = has_p && !in_topk;
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const float c2a = static_cast<float>(1.4426950408889634 * inv_t);          // the FP32 softmass only: approximate on purpose

#ifdef LM_PROFILE_PHASES
  long long _t0 = clock64();
#endif
  for (int i = tid; i < kCandBins; i += kBlock) c.bins[i] = 0u;
  if (tid == 0) { c.n = 0u; c.n_sel = 0u; c.wide = 0u; c.hit = kCandCap; c.token = -1; c.amb = 0.0f; c.cross_bin = 0u; }
  __syncthreads();

  // ---- the one pass: candidates at or above the cutoff; FP32 softmass with a per-thread running maximum ---------------
  float m = -INFINITY, sacc = 0.0f;
  int n_hits = 0;
  {
    const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
    const uint32_t cut2 = cut_code | (cut_code << 16);
    const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&cut2);
    constexpr int kUnroll = 4;
    for (int c0 = tid; c0 < n_chunks; c0 += kBlock * kUnroll) {
      uint4 q[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; j++) { const int cc = c0 + j * kBlock; q[j] = (cc < n_chunks) ? __ldg(p4 + cc) : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u); }
#pragma unroll
      for (int j = 0; j < kUnroll; j++) {
        const int cc = c0 + j * kBlock;
        if (cc >= n_chunks) break;
        const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
        const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[0]), t2), m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[1]), t2);
        const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[2]), t2), m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[3]), t2);
        if (m0 | m1 | m2 | m3) {                                           // rare per thread (7 % of its chunks): just note the chunk
          const uint32_t mask = (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) |
                                ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
          if (n_hits < kHitSlots) c.hits[n_hits * kBlock + tid] = (static_cast<uint32_t>(cc) << 8) | mask;
          n_hits++;
        }
        if (need_z) {
          const __nv_bfloat162 a = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&w[0]), *reinterpret_cast<const __nv_bfloat162*>(&w[1]));
          const __nv_bfloat162 b = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&w[2]), *reinterpret_cast<const __nv_bfloat162*>(&w[3]));
          const __nv_bfloat162 ab = __hmax2(a, b);
          const float mx = fmaxf(__low2float(ab), __high2float(ab));
          if (mx > m) { sacc = (m > -INFINITY) ? sacc * ex2_approx((m - mx) * c2a) : 0.0f; m = mx; }
          if (m > -INFINITY) {
            const float nb = -m * c2a;
#pragma unroll
            for (int k = 0; k < 4; k++) sacc += ex2_approx(fmaf(bf16_lo(w[k]), c2a, nb)) + ex2_approx(fmaf(bf16_hi(w[k]), c2a, nb));
          }
        }
      }
    }
  }
  LM_CPHASE(9);
  // ---- the noted chunks, expanded with every lane active: their logits come back from L2, the candidates are written
  // in thread order (a block-wide prefix of the per-thread counts), so the list is the same on every run
  {
    uint32_t my[kHitSlots];
    const int nh = n_hits < kHitSlots ? n_hits : kHitSlots;
    uint32_t ne = 0;
#pragma unroll
    for (int h = 0; h < kHitSlots; h++) {
      my[h] = 0u;
      if (h < nh) {
        const uint32_t ent = c.hits[h * kBlock + tid];
        const int cc = static_cast<int>(ent >> 8);
        uint32_t mask = ent & 0xFFu;
        if (pen) mask &= ~((pen[cc >> 2] >> ((cc & 3) * 8)) & 0xFFu);       // penalised positions come from the side list
        my[h] = (ent & ~0xFFu) | mask;
        ne += __popc(mask);
      }
    }
    if (n_hits > kHitSlots) c.wide = 1u;
    uint64_t tot = 0ull;
    uint32_t slot = static_cast<uint32_t>(block_exclusive_scan_u64(ne, scratch, &tot));
    if (tid == 0) c.n = static_cast<uint32_t>(tot);
    for (int h0 = 0; h0 < kHitSlots; h0 += 4) {                            // four reloads in flight; most threads need one round or none
      if (__syncthreads_or(h0 < nh) == 0) break;
      uint4 qq[4];
#pragma unroll
      for (int h = 0; h < 4; h++) if (h0 + h < nh) qq[h] = __ldg(reinterpret_cast<const uint4*>(rowp) + (my[h0 + h] >> 8));
#pragma unroll
      for (int h = 0; h < 4; h++) {
        if (h0 + h < nh) {
          const uint32_t w[4] = {qq[h].x, qq[h].y, qq[h].z, qq[h].w};
          const uint32_t ent = my[h0 + h];
          const int cc = static_cast<int>(ent >> 8);
#pragma unroll
          for (int e = 0; e < kChunk; e++) {
            if ((ent >> e) & 1u) {
              const float value = (e & 1) ? bf16_hi(w[e >> 1]) : bf16_lo(w[e >> 1]);
              if (slot < kCandCap) c.key[slot] = (static_cast<unsigned long long>(fkey(value)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(cc * kChunk + e));
              slot++;
              const uint32_t rel = (__float_as_uint(value) >> 16) - cut_code;
              if (rel >= kCandBins) c.wide = 1u; else atomicAdd(&c.bins[rel], 1u);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  // the penalised logits: gathers issued before the barrier that ends the pass
  constexpr int kSideSlots = 4096 / kBlock;                                // the side list holds up to 4096 entries
  uint32_t sd_code[kSideSlots]; int sd_idx[kSideSlots];
#pragma unroll
  for (int j = 0; j < kSideSlots; j++) {
    const uint32_t i = tid + j * kBlock;
    sd_idx[j] = (i < n_side) ? side_idx[i] : 0;
    sd_code[j] = (i < n_side) ? __ldg(rowp + sd_idx[j]) : 0u;
  }
  // block maximum of the running maxima
  float M = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(kFull, M, o));
  if (lane == 0) c.warp_f[warp] = M;
  __syncthreads();
  M = lane < kWarps ? c.warp_f[lane] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(kFull, M, o));
  double zsum = (need_z && m > -INFINITY) ? static_cast<double>(sacc * ex2_approx((m - M) * c2a)) : 0.0;
#pragma unroll
  for (int j = 0; j < kSideSlots; j++) {
    if (tid + j * kBlock < n_side) {
      const float raw = __uint_as_float(sd_code[j] << 16);
      const float v = penalise(raw, P.rho, P.pi);
      side_val[tid + j * kBlock] = v;
      if (v >= cut_val) cand_append(c, v, static_cast<uint32_t>(sd_idx[j]), cut_code);
      if (need_z) zsum += static_cast<double>(ex2_approx((v - M) * c2a)) - static_cast<double>(ex2_approx((raw - M) * c2a));
    }
  }
  const double z_tilde = need_z ? block_sum_f64(zsum, scratch) : 0.0;       // relative to M
  __syncthreads();
  const int n = static_cast<int>(c.n);
  // the cutoff follows the candidate count, one BF16 step at a time
  if (tid == 0) {
    if (n > kCandHigh) cut.code = cut_code + 1u; else if (n < kCandLow && cut_code > 0x0081u) cut.code = cut_code - 1u;
    if (n > kCandCap || n < top_k || c.wide) cut.valid = 0u;                // out of range: the histogram path rebuilds the cutoff
  }
  if (n > kCandCap || n < top_k || c.wide) { __syncthreads(); return false; }

  LM_CPHASE(10);
  // ---- the coarse top-k crossing: the highest code bin b with at least top_k candidates in bins >= b ---------------------
  {
    uint32_t cnt = (tid < kCandBins) ? c.bins[kCandBins - 1 - tid] : 0u, incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
    if (lane == 31) c.warp_f[warp] = __uint_as_float(incl);
    __syncthreads();
    uint32_t wsum = 0u;
    for (int w = 0; w < warp; w++) wsum += __float_as_uint(c.warp_f[w]);
    incl += wsum;
    if (tid < kCandBins && incl >= static_cast<uint32_t>(top_k)) atomicMin(&c.hit, tid);
    __syncthreads();
    if (tid == 0) { c.cross_bin = static_cast<uint32_t>(kCandBins - 1 - c.hit); c.hit = kCandCap; }
    __syncthreads();
  }
  const uint32_t cross = c.cross_bin;
  for (int i = tid; i < n; i += kBlock) {
    const unsigned long long k = c.key[i];
    const uint32_t rel = (__float_as_uint(fkey_inv(static_cast<uint32_t>(k >> 32))) >> 16) - cut_code;
    if (rel >= cross) c.sel[atomicAdd(&c.n_sel, 1u)] = k;
  }
  __syncthreads();
  const int n_sel = static_cast<int>(c.n_sel);
  const int p2 = next_pow2(n_sel);
  for (int i = n_sel + tid; i < p2; i += kBlock) c.sel[i] = 0ull;
  __syncthreads();
  LM_CPHASE(11);
  bitonic_desc(c.sel, p2);
  LM_CPHASE(12);

  // ---- exact thresholds on the sorted candidates ------------------------------------------------------------------------
  const float vmax = fkey_inv(static_cast<uint32_t>(c.sel[0] >> 32));
  const float tau_k = fkey_inv(static_cast<uint32_t>(c.sel[top_k - 1] >> 32));
  double tau64 = tau_k;
  uint32_t status = LM_STATUS_CANDIDATE_PATH;
  if (has_p) {
    for (int i = tid; i < n_sel; i += kBlock) c.cum[i] = softmass(fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)), vmax, inv_t);
    __syncthreads();
    scan_f64(c.cum, n_sel, c.warp_d);
    uint64_t cnt_k = 0ull;
    for (int i = tid; i < n_sel; i += kBlock) cnt_k += fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) >= tau_k ? 1ull : 0ull;
    const int n_topk = static_cast<int>(block_sum_u64(cnt_k, scratch));
    double total, err = 0.0;
    if (in_topk) total = c.cum[n_topk - 1];
    else {                                                                 // the FP32 mass of the whole row, moved to the exact maximum
      total = z_tilde * exp2((static_cast<double>(M) - static_cast<double>(vmax)) * 1.4426950408889634 * inv_t);
      err = 2e-6 * total;
    }
    const double target = static_cast<double>(top_p) * total;
    bool amb = false;
    for (int i = tid; i < n_sel; i += kBlock) {
      const bool run_end = (i == n_sel - 1) || ((c.sel[i + 1] >> 32) != (c.sel[i] >> 32));
      if (!run_end) continue;
      const double cm = c.cum[i];
      if (cm >= target) atomicMin(&c.hit, i);
      if (i < n_topk - 1 && fabs(cm - target) <= err && fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) > tau_k) amb = true;
    }
    if (__syncthreads_or(amb)) return false;                               // too close to call in FP32: the exact path decides
    if (c.hit < kCandCap) {
      const float tau_p = fkey_inv(static_cast<uint32_t>(c.sel[c.hit] >> 32));
      if (static_cast<double>(tau_p) > tau64) tau64 = tau_p;
      if (fabs(c.cum[c.hit] - target) <= 1e-12 * total) status |= LM_STATUS_TOPP_EDGE;
    }
  }
  if (has_m) {
    const double tau_m = static_cast<double>(vmax) + T64 * log(static_cast<double>(min_p));
    if (tau_m > tau64) tau64 = tau_m;
  }
  const float tau = __double2float_rn(tau64);
  uint64_t cnt_kept = 0ull;
  for (int i = tid; i < n_sel; i += kBlock) cnt_kept += fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) >= tau ? 1ull : 0ull;
  const int n_kept = static_cast<int>(block_sum_u64(cnt_kept, scratch));     // the kept set is the first n_kept sorted candidates

  LM_CPHASE(13);
  // ---- the draw ----------------------------------------------------------------------------------------------------------
  int token = -1;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    const float c2 = exp2_scale(T);
    const int q2 = next_pow2(n_kept);
    // order the kept candidates by index: keys (~index << 32 | position), descending = index ascending
    for (int i = tid; i < q2; i += kBlock)
      c.key[i] = (i < n_kept) ? ((c.sel[i] & 0xFFFFFFFFull) << 32) | static_cast<unsigned long long>(i) : 0ull;
    __syncthreads();
    bitonic_desc(c.key, q2);
    for (int i = tid; i < n_kept; i += kBlock) {
      const unsigned long long k = c.sel[static_cast<uint32_t>(c.key[i])];
      c.w[i] = weight_q40(fkey_inv(static_cast<uint32_t>(k >> 32)), vmax, c2);
    }
    __syncthreads();
    const uint64_t total = scan_u64(c.w, n_kept, scratch);
    if (total > 0ull) {
      const uint64_t target = cdf_target(P.uniforms ? P.uniforms[row] : 0.0f, total);
      for (int i = tid; i < n_kept; i += kBlock) {
        const uint64_t incl = c.w[i], before = i ? c.w[i - 1] : 0ull;
        if (before <= target && target < incl) c.token = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(c.key[i] >> 32));
      }
    }
    __syncthreads();
    token = c.token;
  } else {
    const float inv_t32 = __double2float_rn(1.0 / T64);
    const uint32_t t_id = static_cast<uint32_t>(P.row_offset + row);
    uint64_t b1 = 0ull; float second = -INFINITY;
    for (int i = tid; i < n_kept; i += kBlock) {
      const unsigned long long k = c.sel[i];
      const uint32_t idx = 0xFFFFFFFFu - static_cast<uint32_t>(k);
      const float key = __fadd_rn(__fmul_rn(fkey_inv(static_cast<uint32_t>(k >> 32)), inv_t32), gumbel(P.seed, P.step, t_id, idx));
      const uint64_t pk = pack_best(key, idx);
      if (pk > b1) { if (b1) second = fmaxf(second, best_value(b1)); b1 = pk; } else second = fmaxf(second, key);
    }
    const uint64_t win = block_max_u64(b1, scratch);
    if (win) {
      const float rival = (b1 == win) ? second : (b1 ? best_value(b1) : -INFINITY);
      if (__syncthreads_or(rival >= best_value(win) - 4e-6f)) status |= LM_STATUS_NEAR_TIE;
      token = static_cast<int>(best_index(win));
    }
  }
  LM_CPHASE(14);
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
  }
  __syncthreads();
  return true;
}

}  // namespace lm
