// The histogram row sampler for BF16 logits: any top_k, top-p, min-p, penalties, both draws; ONE pass over the row from HBM.
//
// A BF16 logit has at most 65536 codes, and the logits of a language model use a small part of them. The block keeps a
// histogram of the row over a WINDOW of codes (magnitudes 2^-39 .. 2^25, both signs: 16384 counters of 16 bits, 32 KB of
// shared memory, plus counters for exact zeros and for -inf), so that two blocks fit one SM and the short serial phases of
// one row hide behind the streaming pass of another. The histogram holds everything the thresholds need: the k-th largest
// value is a walk over counts, the top-p boundary a walk over count x exp(value) in FP64, per distinct value, as the
// reference's numpy definition forms them (monolith/nn/sampling_ref.py:26-35; the reference's Metal kernels build a
// 65536-bucket histogram in device memory, 256 KB per row, kernels/common/sample.metal:34-162).
//
// A penalised logit is a function of its raw code alone, f(code) = (z > 0 ? z / rho : z * rho) - pi, and f is monotone. The
// penalised positions therefore get a second, 8-bit histogram over the same window; compacted, it is a list of distinct
// penalised values that is already in descending order, and the threshold walks merge it with the main histogram without
// sorting anything.
//
// The walks are two-level: 258 groups of 64 window positions (block scan), then one warp inside the group where the target
// falls. The inverse-CDF draw (descending value order, equal values by ascending index) is decided by the same walks on integer
// weights, down to the value; its second look at the row (from L2) only counts the logits equal to that value, in 256-logit
// segments from the nearer end of the row, and stops at the segment that holds the one it wants.
//
// Rows this kernel cannot take go to the generic kernel through the `redo` list: a logit outside the window other than 0
// and -inf (NaN, +inf, |z| >= 2^25, 0 < |z| < 2^-39), more than 65535 equal logits, more than kPenCap distinct penalised ids
// or more than 255 of them on one raw code, vocabularies that are not a multiple of 8 or exceed kHistMaxVocab, misaligned rows.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "sample_generic.cuh"

namespace lm {

constexpr int kHB = 512;                          // threads per block
constexpr int kHW = kHB / 32;
constexpr int kHistMaxVocab = 262144;
constexpr uint32_t kWinLo = 0x2C00u;              // first magnitude code of the window: 2^-39
constexpr uint32_t kWinCodes = 8192u;             // codes per sign: 64 binades
constexpr uint32_t kSlots = 2u * kWinCodes;       // counters: slot = code - kWinLo (positive), 8192 + (|code| - kWinLo) (negative)
constexpr int kGrpSlots = 64;                     // window positions per group of the walks
constexpr int kSignGroups = static_cast<int>(kWinCodes) / kGrpSlots;   // 128
constexpr int kZeroGroup = kSignGroups;           // the group holding the single position of the value 0
constexpr int kNinfGroup = 2 * kSignGroups + 1;   // ... of -inf
constexpr int kGroupsH = 2 * kSignGroups + 2;     // 258
constexpr uint32_t kPosZero = kWinCodes;          // positions run in descending value order: 0..8191 positive, 8192 zero,
constexpr uint32_t kPosNinf = 2u * kWinCodes + 1u;//   8193..16384 negative, 16385 -inf
constexpr int kPenCap = 2048;                     // distinct penalised ids per row
constexpr int kSegChunks = 32;                    // the draw's segments: 32 chunks = 256 logits, one warp-wide load
constexpr int kMaxSegs = kHistMaxVocab / (kSegChunks * kChunk);
constexpr int kDrawIters = 4;                     // segments per warp and batch of the draw
constexpr int kBatchSegs = kDrawIters * kHW;

struct HistSmem {
  uint32_t hist[kSlots / 2];                      // 32 KB: 16-bit counters of the unpenalised logits, slot s in half (s & 1) of word s >> 1
  union {
    uint32_t pen_hist[kSlots / 4];                // 16 KB: 8-bit counters of the penalised logits by raw code, until they are compacted
    double b_mass[kPenCap];                       // then: running sum (inclusive) of count x softmass over the distinct penalised values
  };
  uint32_t ids[kPenCap];                          // the row's distinct history ids
  uint16_t side_raw[kPenCap];                     // their raw codes
  float b_val[kPenCap];                           // distinct penalised values, descending
  uint16_t b_ins[kPenCap];                        // the window position each is inserted before: the smallest p with value(p) <= b_val
  uint16_t b_cnt[kPenCap];                        // how many logits carry each value; from phase 4 on the running sum (inclusive)
  unsigned long long seg_fix[kMaxSegs];           // draw: per segment (as 32-bit counters), its penalised logits equal to the drawn value
  unsigned long long batch_sum[2][kBatchSegs];    // draw: (as 32-bit counters) segment counts of the batch in hand, double-buffered
  double g_mass[kGroupsH + 2];
  uint32_t g_cnt[kGroupsH + 2];
  uint64_t scratch[32];
  double warp_m[kHW];
  uint32_t warp_c[kHW];
  uint32_t n_side, n_b, cz, cninf, pz, pninf, oob, top_pos;    // cz / cninf: unpenalised zeros and -inf; pz / pninf: penalised ones
  int sel_g, last_g;
  uint32_t base_c; double base_m;
  float res_tau; uint32_t res_cum_c; double res_cum_m, res_excl_m;
  int token;
  // followed by the bitmap of the row's distinct history ids: (vocab + 127) / 128 * 16 bytes
};

// ---- codes, slots, positions ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float hcode_val(uint32_t code) { return __uint_as_float(code << 16); }
// code of the largest BF16 value <= v
__device__ __forceinline__ uint32_t hfloor_code(float v) {
  const uint32_t u = __float_as_uint(v);
  uint32_t code = u >> 16;
  if ((u & 0x80000000u) && (u & 0xFFFFu)) code += 1u;
  return code;
}
// smallest BF16 code whose value is >= t: for BF16-valued z, (z >= t) <=> (z >= that value)
__device__ __forceinline__ uint32_t hceil_code(float t) {
  const uint32_t u = __float_as_uint(t);
  uint32_t code = u >> 16;
  if ((u & 0xFFFFu) && !(u & 0x80000000u)) code += 1u;
  return code;
}
// slot of a code inside the window, or 0xFFFFFFFF
__device__ __forceinline__ uint32_t slot_of_code(uint32_t code) {
  const uint32_t r = (code & 0x7FFFu) - kWinLo;
  return r < kWinCodes ? r + ((code >> 15) << 13) : 0xFFFFFFFFu;
}
__device__ __forceinline__ uint32_t code_of_slot(uint32_t slot) { return ((slot >> 13) << 15) | (kWinLo + (slot & (kWinCodes - 1u))); }
__device__ __forceinline__ uint32_t pos_of_slot(uint32_t slot) { return slot < kWinCodes ? kWinCodes - 1u - slot : slot + 1u; }
__device__ __forceinline__ uint32_t slot_of_pos(uint32_t p) { return p < kPosZero ? kWinCodes - 1u - p : p - 1u; }   // p not the zero / -inf position
__device__ __forceinline__ float val_of_pos(uint32_t p) {
  if (p == kPosZero) return 0.0f;
  if (p >= kPosNinf) return -INFINITY;
  return hcode_val(code_of_slot(slot_of_pos(p)));
}
__device__ __forceinline__ int group_of_pos(uint32_t p) {
  if (p < kPosZero) return static_cast<int>(p >> 6);
  if (p == kPosZero) return kZeroGroup;
  if (p >= kPosNinf) return kNinfGroup;
  return kZeroGroup + 1 + static_cast<int>((p - kPosZero - 1u) >> 6);
}
__device__ __forceinline__ uint32_t first_pos_of_group(int g) {
  if (g < kZeroGroup) return static_cast<uint32_t>(g) << 6;
  if (g == kZeroGroup) return kPosZero;
  if (g == kNinfGroup) return kPosNinf;
  return kPosZero + 1u + (static_cast<uint32_t>(g - kZeroGroup - 1) << 6);
}
// the window position a value is inserted before: the smallest p with value(p) <= v (v not NaN, -0 folded into +0)
__device__ __forceinline__ uint32_t ins_pos(float v) {
  const uint32_t fc = hfloor_code(v), mag = fc & 0x7FFFu;
  if (!(fc & 0x8000u)) {
    if (mag >= kWinLo + kWinCodes) return 0u;
    return mag >= kWinLo ? kWinCodes - 1u - (mag - kWinLo) : kPosZero;
  }
  if (mag >= kWinLo + kWinCodes) return kPosNinf;
  return mag >= kWinLo ? kPosZero + 1u + (mag - kWinLo) : kPosZero + 1u;
}
__device__ __forceinline__ uint32_t hcount(const uint32_t* hist, uint32_t slot) { return (hist[slot >> 1] >> ((slot & 1u) * 16u)) & 0xFFFFu; }
__device__ __forceinline__ uint32_t cnt_of_pos(const HistSmem& s, uint32_t p) {
  if (p == kPosZero) return s.cz;
  if (p >= kPosNinf) return s.cninf;
  return hcount(s.hist, slot_of_pos(p));
}
__device__ __forceinline__ float penalised_value(uint32_t code, float rho, float pi) { return canon_zero(penalise(hcode_val(code), rho, pi)); }

// One logit that the fast path of the pass does not take: an exact zero, -inf, or a code outside the window.
__device__ __noinline__ void hist_add_slow(HistSmem& s, uint32_t code) {
  const uint32_t slot = slot_of_code(code);
  if (slot != 0xFFFFFFFFu) atomicAdd(&s.hist[slot >> 1], (slot & 1u) ? 0x10000u : 1u);
  else if ((code & 0x7FFFu) == 0u) atomicAdd(&s.cz, 1u);
  else if (code == 0xFF80u) atomicAdd(&s.cninf, 1u);
  else s.oob = 1u;
}
// Two logits of one 32-bit word into the histogram. Adding 0x4000 - kWinLo to a code moves the window to the codes whose bits
// 14:13 are 10 (0x4000..0x5FFF and 0xC000..0xDFFF), so one mask tests both halves; the slot is bits 12:0 with the sign moved to
// bit 13. (A low half that carries into the high half is a code outside the window: the row is handed on anyway.)
__device__ __forceinline__ void hist_add_word(HistSmem& s, uint32_t w) {
  constexpr uint32_t kShift = 0x4000u - kWinLo;
  const uint32_t y = w + (kShift | (kShift << 16));
  if ((y & 0x60006000u) == 0x40004000u) {
    const uint32_t sl = (y & 0x1FFF1FFFu) | ((y >> 2) & 0x20002000u);
    char* base = reinterpret_cast<char*>(s.hist);
    atomicAdd(reinterpret_cast<uint32_t*>(base + ((sl << 1) & 0x7FFCu)), (sl & 1u) * 0xFFFFu + 1u);
    atomicAdd(reinterpret_cast<uint32_t*>(base + ((sl >> 15) & 0x7FFCu)), ((sl >> 16) & 1u) * 0xFFFFu + 1u);
  } else {
    hist_add_slow(s, w & 0xFFFFu);
    hist_add_slow(s, w >> 16);
  }
}

__device__ __forceinline__ void hprefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Exclusive prefix sum of one u32 per thread over the block (kHB threads), thread order; *total gets the block sum.
__device__ __forceinline__ uint32_t hblock_scan_u32(uint32_t v, uint32_t* warp_c, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
  __syncthreads();
  if (lane == 31) warp_c[warp] = incl;
  __syncthreads();
  uint32_t w = lane < kHW ? warp_c[lane] : 0u, winc = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, winc, o); if (lane >= o) winc += t; }
  if (total) *total = __shfl_sync(kFull, winc, kHW - 1);
  return __shfl_sync(kFull, winc - w, warp) + incl - v;
}

// first index j in [0, n) with a[j] >= key (a ascending)
__device__ __forceinline__ uint32_t lower_bound_u16(const uint16_t* a, uint32_t n, uint32_t key) {
  uint32_t lo = 0u, hi = n;
  while (lo < hi) { const uint32_t mid = (lo + hi) >> 1; if (a[mid] < key) lo = mid + 1u; else hi = mid; }
  return lo;
}

// Totals of the penalised values [j0, j1) from the running sums (valid from phase 4 on).
__device__ __forceinline__ uint32_t b_count_range(const HistSmem& s, uint32_t j0, uint32_t j1) {
  return j1 > j0 ? static_cast<uint32_t>(s.b_cnt[j1 - 1u]) - (j0 ? static_cast<uint32_t>(s.b_cnt[j0 - 1u]) : 0u) : 0u;
}
__device__ __forceinline__ double b_mass_range(const HistSmem& s, uint32_t j0, uint32_t j1) {
  return j1 > j0 ? s.b_mass[j1 - 1u] - (j0 ? s.b_mass[j0 - 1u] : 0.0) : 0.0;
}

// ---- the threshold walk ------------------------------------------------------------------------------------------------------
// Finds the first distinct value, descending, at which the running count reaches k_target (BY_MASS false) or the running
// softmass reaches m_target (BY_MASS true). The row is the merge of two descending sequences: the window positions with their
// counts, and the distinct penalised values b_val[0 .. n_b) with b_ins[j] = the position each is inserted before. Group
// totals (counts, and masses when MASS) are in s.g_cnt / s.g_mass. Every thread calls. Results: s.res_tau, and the running
// totals s.res_cum_c / s.res_cum_m including every logit equal to res_tau, s.res_excl_m excluding them.
template <bool BY_MASS, bool MASS>
__device__ void hist_walk(HistSmem& s, uint32_t k_target, double m_target, float vmax, double inv_t) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // -- level 1: the group. One group per thread, inclusive scan in walk order.
  uint32_t c = 0u, ci = 0u; double m = 0.0, mi = 0.0;
  if (tid == 0) { s.sel_g = kGroupsH; s.last_g = -1; }
  if (tid < kGroupsH) { c = s.g_cnt[tid]; ci = c; if (MASS) { m = s.g_mass[tid]; mi = m; } }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t tc = __shfl_up_sync(kFull, ci, o);
    const double tm = MASS ? __shfl_up_sync(kFull, mi, o) : 0.0;
    if (lane >= o) { ci += tc; if (MASS) mi += tm; }
  }
  if (lane == 31) { s.warp_c[warp] = ci; if (MASS) s.warp_m[warp] = mi; }
  __syncthreads();
  if (tid < kGroupsH) {
    uint32_t wc = 0u; double wm = 0.0;
    for (int w = 0; w < warp; w++) { wc += s.warp_c[w]; if (MASS) wm += s.warp_m[w]; }
    ci += wc; mi += wm;
    const bool hit = BY_MASS ? (c > 0u && mi >= m_target) : (ci >= k_target);
    if (hit) atomicMin(&s.sel_g, tid);
    if (c > 0u) atomicMax(&s.last_g, tid);
  }
  __syncthreads();
  const int g = s.sel_g < kGroupsH ? s.sel_g : s.last_g;                  // target never reached (rounding): the last occupied group
  if (tid == g) { s.base_c = ci - c; s.base_m = mi - m; }
  __syncthreads();
  if (g < 0) { if (tid == 0) { s.res_tau = -INFINITY; s.res_cum_c = 0u; s.res_cum_m = 0.0; s.res_excl_m = 0.0; } __syncthreads(); return; }
  // -- level 2: one warp inside the group. Lane l owns the positions p0 + 2l and p0 + 2l + 1 and the penalised values
  // inserted before each; its items in descending order: B[ja, jb), A(q0), B[jb, jc), A(q1).
  if (warp == 0) {
    const uint32_t p0 = first_pos_of_group(g);
    const bool single = g == kZeroGroup || g == kNinfGroup;
    const uint32_t q0 = p0 + 2u * lane, q1 = q0 + 1u;
    const bool own = !single || lane == 0;
    const uint32_t nb = s.n_b;
    uint32_t ja = 0u, jb = 0u, jc = 0u;
    if (own) {
      ja = lower_bound_u16(s.b_ins, nb, q0); jb = lower_bound_u16(s.b_ins, nb, q0 + 1u);
      jc = single ? jb : lower_bound_u16(s.b_ins, nb, q0 + 2u);
    }
    const uint32_t ca0 = own ? cnt_of_pos(s, q0) : 0u, ca1 = (own && !single) ? cnt_of_pos(s, q1) : 0u;
    const float va0 = val_of_pos(q0), va1 = val_of_pos(q1);
    const double ma0 = (MASS && ca0) ? static_cast<double>(ca0) * softmass(va0, vmax, inv_t) : 0.0;
    const double ma1 = (MASS && ca1) ? static_cast<double>(ca1) * softmass(va1, vmax, inv_t) : 0.0;
    const uint32_t n_items = (jc - ja) + 2u;
    // item t of this lane: value, count, mass
    auto item = [&](uint32_t t, float& v, uint32_t& n, double& mm) {
      const uint32_t nb0 = jb - ja;
      if (t < nb0) { const uint32_t j = ja + t; v = s.b_val[j]; n = b_count_range(s, j, j + 1u); mm = MASS ? b_mass_range(s, j, j + 1u) : 0.0; }
      else if (t == nb0) { v = va0; n = ca0; mm = ma0; }
      else if (t < n_items - 1u) { const uint32_t j = jb + (t - nb0 - 1u); v = s.b_val[j]; n = b_count_range(s, j, j + 1u); mm = MASS ? b_mass_range(s, j, j + 1u) : 0.0; }
      else { v = va1; n = ca1; mm = ma1; }
    };
    const uint32_t c_l = ca0 + ca1 + b_count_range(s, ja, jc);
    const double m_l = MASS ? ma0 + ma1 + b_mass_range(s, ja, jc) : 0.0;
    uint32_t cs = c_l; double ms = m_l;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, cs, o);
      const double tm = MASS ? __shfl_up_sync(kFull, ms, o) : 0.0;
      if (lane >= o) { cs += tc; if (MASS) ms += tm; }
    }
    const uint32_t base_c = s.base_c; const double base_m = s.base_m;
    const bool hit = BY_MASS ? (c_l > 0u && base_m + ms >= m_target) : (base_c + cs >= k_target);
    const uint32_t hits = __ballot_sync(kFull, hit), occ = __ballot_sync(kFull, c_l > 0u);
    const int sel = hits ? (__ffs(hits) - 1) : (occ ? 31 - __clz(occ) : 0);
    if (lane == sel) {
      uint32_t run_c = base_c + cs - c_l; double run_m = base_m + ms - m_l;
      int found = -1, last_occ = -1;
      for (uint32_t t = 0; t < n_items && found < 0; t++) {
        float v; uint32_t n; double mm; item(t, v, n, mm);
        if (n == 0u) continue;
        last_occ = static_cast<int>(t);
        if (BY_MASS ? (run_m + mm >= m_target) : (run_c + n >= k_target)) { found = static_cast<int>(t); break; }
        run_c += n; run_m += mm;
      }
      if (found < 0) {                                                     // not reached after all (rounding): the lane's last occupied item
        found = last_occ;
        run_c = base_c + cs - c_l; run_m = base_m + ms - m_l;
        for (int t = 0; t < found; t++) { float v; uint32_t n; double mm; item(static_cast<uint32_t>(t), v, n, mm); run_c += n; run_m += mm; }
      }
      float tau = -INFINITY; double excl = run_m;
      if (found >= 0) {
        float v; uint32_t n; double mm; item(static_cast<uint32_t>(found), v, n, mm);
        tau = v;
        // items of the same value before this one (equal penalised values, or a penalised value equal to the code it precedes)
        // cannot exist: the walk would have stopped there or they lie above. Those after it join the totals.
        run_c += n; run_m += mm;
        for (uint32_t t = static_cast<uint32_t>(found) + 1u; t < n_items; t++) {
          float v2; uint32_t n2; double mm2; item(t, v2, n2, mm2);
          if (n2 == 0u) continue;
          if (v2 != tau) break;
          run_c += n2; run_m += mm2;
        }
      }
      s.res_tau = tau; s.res_cum_c = run_c; s.res_cum_m = run_m; s.res_excl_m = excl;
    }
  }
  __syncthreads();
}

// ---- the draws -----------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t kept_mask8(const uint4 q, uint32_t tau_code2) {
  const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&tau_code2);
  const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.x), t2), m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.y), t2);
  const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.z), t2), m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.w), t2);
  if ((m0 | m1 | m2 | m3) == 0u) return 0u;
  return (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) | ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
}

// 8-bit mask of the logits of a chunk whose BF16 code equals `code` (zero = true: whose value is zero, either sign).
__device__ __forceinline__ uint32_t equal_mask8(const uint4 q, uint32_t code2, bool zero) {
  const uint32_t strip = zero ? 0x7FFF7FFFu : 0xFFFFFFFFu;
  const uint32_t m0 = __vcmpeq2(q.x & strip, code2), m1 = __vcmpeq2(q.y & strip, code2), m2 = __vcmpeq2(q.z & strip, code2), m3 = __vcmpeq2(q.w & strip, code2);
  if ((m0 | m1 | m2 | m3) == 0u) return 0u;
  return (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) | ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
}

// The inverse-CDF draw: the kept set in descending value order, equal values by ascending index. Equal values have equal
// weights, so the histograms decide almost everything: the total weight S, hence the target; the group of 64 window positions
// where the cumulative weight crosses it (a block scan over the groups' weights); inside the group one warp walks the merged
// sequence of window positions and distinct penalised values down to the value v where the crossing lies. What is left is the
// floor((target - weight above v) / w(v))-th smallest index among the logits equal to v: the row is looked at again (L2) only to
// COUNT them -- segments of 256 logits from whichever end is nearer, a batch of kBatchSegs per barrier, packed 16-bit compares
// against v's raw code, the penalised logits equal to v as per-segment corrections (s.seg_fix) -- and the warp that holds the
// segment locates the token. Every thread calls; every thread gets the token (-1: the kept set has no weight).
__device__ int hist_draw_inverse_cdf(const SampleDev& P, HistSmem& s, const uint32_t* pen, const uint16_t* rowp, int n_chunks, float tau, float vmax, float T, float u,
                                     uint64_t* out_total, bool total_only = false) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float c2 = exp2_scale(T);
  const uint32_t n_side = s.n_side, n_b = s.n_b;
  unsigned long long* g_w = reinterpret_cast<unsigned long long*>(s.g_mass);   // the groups' weights take the place of their masses
  auto kept_weight = [&](float v, uint32_t n) -> uint64_t { return (n && v >= tau) ? static_cast<uint64_t>(n) * weight_q40(v, vmax, c2) : 0ull; };
  // ---- the weight of every group: window positions ...
  for (int sg = warp; sg < static_cast<int>(kSlots) / kGrpSlots; sg += kHW) {
    const int g = sg < kSignGroups ? kSignGroups - 1 - sg : sg + 1;
    uint64_t w = 0ull;
    if (s.g_cnt[g] != 0u) {                                                // (warp-uniform)
      const uint32_t h = s.hist[sg * 32 + lane];
      if (h) {
        const uint32_t slot = static_cast<uint32_t>(sg) * kGrpSlots + 2u * lane;
        const uint32_t n0 = h & 0xFFFFu, n1 = h >> 16;
        const float v0 = hcode_val(code_of_slot(slot)), v1 = hcode_val(code_of_slot(slot + 1u));
        if ((n0 && v0 >= tau) || (n1 && v1 >= tau)) {
          uint64_t w0, w1;
          weight_q40_x2(v0, v1, vmax, c2, w0, w1);
          if (n0 && v0 >= tau) w += static_cast<uint64_t>(n0) * w0;
          if (n1 && v1 >= tau) w += static_cast<uint64_t>(n1) * w1;
        }
      }
      w = warp_sum_u64(w);
    }
    if (lane == 0) g_w[g] = w;
  }
  if (tid == 0) { g_w[kZeroGroup] = kept_weight(0.0f, s.cz); g_w[kNinfGroup] = 0ull; s.sel_g = kGroupsH; s.token = -1; }
  __syncthreads();
  // ... and the distinct penalised values, each into the group of the position it is inserted before
  for (uint32_t j = tid; j < n_b; j += kHB) {
    const uint64_t w = kept_weight(s.b_val[j], b_count_range(s, j, j + 1u));
    if (w) atomicAdd(&g_w[group_of_pos(s.b_ins[j])], static_cast<unsigned long long>(w));
  }
  __syncthreads();
  // ---- the target and the group where the cumulative weight crosses it
  const uint64_t gw = tid < kGroupsH ? g_w[tid] : 0ull;
  uint64_t total = 0ull;
  const uint64_t g_before = block_exclusive_scan_u64(gw, s.scratch, &total);
  *out_total = total;
  if (total == 0ull || total_only) { __syncthreads(); return -1; }        // (total_only: the Gumbel draw picks the token; only the mass is wanted)
  const uint64_t target = cdf_target(u, total);
  if (gw && g_before <= target && target < g_before + gw) { s.sel_g = tid; *reinterpret_cast<unsigned long long*>(&s.base_m) = g_before; }
  __syncthreads();
  const int g = s.sel_g;
  // ---- inside the group: lane l owns the positions p0 + 2l, p0 + 2l + 1 and the penalised values inserted before each; its items in
  // descending order: B[ja, jb), A(q0), B[jb, jc), A(q1). Results in shared memory: the value, the weight above it, how many logits
  // carry it, and whether a window position (a raw code) does.
  if (warp == 0) {
    const uint64_t base = *reinterpret_cast<const unsigned long long*>(&s.base_m);
    const uint32_t p0 = first_pos_of_group(g);
    const bool single = g == kZeroGroup || g == kNinfGroup;
    const uint32_t q0 = p0 + 2u * lane, q1 = q0 + 1u;
    const bool own = !single || lane == 0;
    uint32_t ja = 0u, jb = 0u, jc = 0u;
    if (own) {
      ja = lower_bound_u16(s.b_ins, n_b, q0); jb = lower_bound_u16(s.b_ins, n_b, q0 + 1u);
      jc = single ? jb : lower_bound_u16(s.b_ins, n_b, q0 + 2u);
    }
    const uint32_t ca0 = own ? cnt_of_pos(s, q0) : 0u, ca1 = (own && !single) ? cnt_of_pos(s, q1) : 0u;
    const float va0 = val_of_pos(q0), va1 = val_of_pos(q1);
    const uint32_t n_items = (jc - ja) + 2u;
    auto item = [&](uint32_t t, float& v, uint32_t& n, bool& is_a) {
      const uint32_t nb0 = jb - ja;
      if (t < nb0) { const uint32_t j = ja + t; v = s.b_val[j]; n = b_count_range(s, j, j + 1u); is_a = false; }
      else if (t == nb0) { v = va0; n = ca0; is_a = true; }
      else if (t < n_items - 1u) { const uint32_t j = jb + (t - nb0 - 1u); v = s.b_val[j]; n = b_count_range(s, j, j + 1u); is_a = false; }
      else { v = va1; n = ca1; is_a = true; }
    };
    uint64_t w_l = 0ull;
    for (uint32_t t = 0; t < n_items; t++) { float v; uint32_t n; bool a; item(t, v, n, a); w_l += kept_weight(v, n); }
    uint64_t ws = w_l;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint64_t t = __shfl_up_sync(kFull, ws, o); if (lane >= o) ws += t; }
    const uint64_t l_before = base + ws - w_l;
    if (w_l && l_before <= target && target < l_before + w_l) {
      uint64_t run = l_before;
      for (uint32_t t = 0; t < n_items; t++) {
        float v; uint32_t n; bool a; item(t, v, n, a);
        const uint64_t w = kept_weight(v, n);
        if (w && target < run + w) {
          // the items of one value are adjacent: a penalised value right before the window position it equals
          uint64_t before = run; uint32_t n_raw = a ? n : 0u, n_pen = a ? 0u : n;
          if (a && t > 0u) {
            float vp; uint32_t np; bool ap; item(t - 1u, vp, np, ap);
            if (!ap && np && vp == v) { before -= kept_weight(vp, np); n_pen = np; }
          } else if (!a && t + 1u < n_items) {
            float vn; uint32_t nn; bool an; item(t + 1u, vn, nn, an);
            if (an && nn && vn == v) n_raw = nn;
          }
          s.res_tau = v; s.res_cum_c = n_raw; s.base_c = n_pen;
          *reinterpret_cast<unsigned long long*>(&s.res_cum_m) = before;
          break;
        }
        run += w;
      }
    }
  }
  __syncthreads();
  const float v_star = s.res_tau;
  const uint32_t n_raw = s.res_cum_c, n_pen = s.base_c, members = n_raw + n_pen;
  const uint64_t each = weight_q40(v_star, vmax, c2);
  const uint32_t want = static_cast<uint32_t>((target - *reinterpret_cast<const unsigned long long*>(&s.res_cum_m)) / each);   // < members
  // ---- the penalised logits equal to the value, per segment
  unsigned int* seg_cnt = reinterpret_cast<unsigned int*>(s.seg_fix);      // (cleared with seg_fix at the start of the row)
  if (n_pen) {
    for (uint32_t i = tid; i < n_side; i += kHB) if (penalised_value(s.side_raw[i], P.rho, P.pi) == v_star) atomicAdd(&seg_cnt[s.ids[i] >> 8], 1u);
  }
  // the raw code of the value, if a window position carries it (0xFFFFFFFF: none -- every member is a penalised logit)
  const bool zero = v_star == 0.0f;
  const uint32_t code = n_raw ? (zero ? 0u : (__float_as_uint(v_star) >> 16)) : 0xFFFFFFFFu;
  const uint32_t code2 = code | (code << 16);
  const bool forward = want < members - want;
  const uint32_t tt = forward ? want : members - 1u - want;               // the first segment, in scan order, whose running count exceeds tt
  __syncthreads();                                                        // seg_cnt is complete
  // ---- the segments, a batch at a time, from the nearer end
  const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
  const int n_seg = (n_chunks + kSegChunks - 1) / kSegChunks;
  uint32_t run = 0u, before_cnt = 0u, found_total = 0u;
  int found = -1, found_b0 = 0, buf = 0;
  unsigned int* batch_cnt = reinterpret_cast<unsigned int*>(s.batch_sum);  // [2][kBatchSegs]
  for (int b0 = 0; b0 < n_seg && found < 0; b0 += kBatchSegs, buf ^= 1) {
    uint4 q[kDrawIters];                                                  // the warp's chunks of this batch, all in flight at once
#pragma unroll
    for (int it = 0; it < kDrawIters; it++) {
      const int k = b0 + it * kHW + warp, seg = forward ? k : n_seg - 1 - k, cc = seg * kSegChunks + lane;
      q[it] = (n_raw && k < n_seg && cc < n_chunks) ? __ldg(p4 + cc) : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
    }
#pragma unroll
    for (int it = 0; it < kDrawIters; it++) {
      const int k = b0 + it * kHW + warp, seg = forward ? k : n_seg - 1 - k, cc = seg * kSegChunks + lane;
      uint32_t mask = (n_raw && k < n_seg && cc < n_chunks) ? equal_mask8(q[it], code2, zero) : 0u;
      if (mask && pen != nullptr) mask &= ~((pen[cc >> 2] >> ((cc & 3) * 8)) & 0xFFu);
      const uint32_t cnt = warp_sum_u32(__popc(mask));
      if (lane == 0) batch_cnt[buf * kBatchSegs + it * kHW + warp] = k < n_seg ? cnt + seg_cnt[seg] : 0u;
    }
    __syncthreads();
    // every warp scans the batch's counts for itself: no second barrier (the next batch writes the other buffer)
    const uint32_t a = batch_cnt[buf * kBatchSegs + 2 * lane], b = batch_cnt[buf * kBatchSegs + 2 * lane + 1];
    uint32_t incl = a + b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
    const uint32_t excl = run + incl - a - b;
    const bool hit_a = excl + a > tt, hit_b = excl + a + b > tt;
    const uint32_t hits = __ballot_sync(kFull, hit_b);
    if (hits) {
      const int src = __ffs(hits) - 1;
      const int idx = __shfl_sync(kFull, hit_a ? 2 * lane : 2 * lane + 1, src);
      before_cnt = __shfl_sync(kFull, hit_a ? excl : excl + a, src);
      found_total = __shfl_sync(kFull, hit_a ? a : b, src);
      found = b0 + idx; found_b0 = b0;
    }
    run += __shfl_sync(kFull, incl, 31);
  }
  if (found < 0) return -1;                                               // cannot happen: the segments hold `members` logits
  // ---- inside the segment: the (local)-th logit equal to the value, in index order, by the warp that counted the segment (its
  // chunk comes back from L2: keeping a batch of chunks alive across the loop would cost the kernel registers it does not have)
  {
    const int idx = found - found_b0;                                     // position of the segment in its batch: it * kHW + warp
    if (warp == idx % kHW) {
      const int seg = forward ? found : n_seg - 1 - found;
      const uint32_t prefix = forward ? before_cnt : members - before_cnt - found_total;   // members before the segment
      const uint32_t local = want - prefix;
      const int cc = seg * kSegChunks + lane;
      const uint4 qf = cc < n_chunks ? __ldg(p4 + cc) : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
      const uint32_t bits = (pen != nullptr && cc < n_chunks) ? ((pen[cc >> 2] >> ((cc & 3) * 8)) & 0xFFu) : 0u;
      const uint32_t words[4] = {qf.x, qf.y, qf.z, qf.w};
      uint32_t hit = 0u;
#pragma unroll
      for (int e = 0; e < kChunk; e++) {
        const uint32_t cde = (e & 1) ? (words[e >> 1] >> 16) : (words[e >> 1] & 0xFFFFu);
        const bool is_pen = (bits >> e) & 1u;
        const bool m = cc < n_chunks && (is_pen ? (n_pen && penalised_value(cde, P.rho, P.pi) == v_star)
                                               : (n_raw && (zero ? (cde & 0x7FFFu) == 0u : cde == code)));
        hit |= m ? (1u << e) : 0u;
      }
      const uint32_t mine = __popc(hit);
      uint32_t incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
      const uint32_t excl = incl - mine;
      if (excl <= local && local < incl) {
        uint32_t r = excl;
#pragma unroll
        for (int e = 0; e < kChunk; e++) if ((hit >> e) & 1u) { if (r == local) { s.token = cc * kChunk + e; break; } r++; }
      }
    }
  }
  __syncthreads();
  return s.token;
}

// The Gumbel-max draw over the kept set (monolith/nn/sampling_ref.py:55-62; kernels/common/sample.metal:164-198): the sweeps
// skip the penalised positions (bitmap), whose values come from the list afterwards. *near_tie: another key within 4e-6 of the
// winner's. Every thread calls; every thread gets the token.
__device__ int hist_draw_gumbel(const SampleDev& P, HistSmem& s, const uint32_t* pen, const uint16_t* rowp, int n_chunks, float tau, float T, uint32_t t_id, bool* near_tie) {
  const int tid = threadIdx.x;
  const float inv_t32 = __double2float_rn(1.0 / static_cast<double>(T));
  const uint32_t tc = hceil_code(tau), tau2 = tc | (tc << 16);
  const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
  uint64_t b1 = 0ull; float second = -INFINITY;
  auto offer = [&](float z, uint32_t i) {
    const float key = __fadd_rn(__fmul_rn(z, inv_t32), gumbel(P.seed, P.step, t_id, i));
    const uint64_t p = pack_best(key, i);
    if (p > b1) { if (b1) second = fmaxf(second, best_value(b1)); b1 = p; } else second = fmaxf(second, key);
  };
  constexpr int kU = 4;
  for (int c0 = tid; c0 < n_chunks; c0 += kHB * kU) {
    uint4 q[kU];
#pragma unroll
    for (int j = 0; j < kU; j++) { const int c = c0 + j * kHB; if (c < n_chunks) q[j] = __ldg(p4 + c); }
#pragma unroll
    for (int j = 0; j < kU; j++) {
      const int c = c0 + j * kHB;
      if (c >= n_chunks) break;
      uint32_t mask = tc == 0xFF80u ? 0xFFu : kept_mask8(q[j], tau2);
      if (pen != nullptr) mask &= ~((pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu);
      if (!mask) continue;
      const uint32_t words[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u)
        offer(canon_zero((e & 1) ? bf16_hi(words[e >> 1]) : bf16_lo(words[e >> 1])), static_cast<uint32_t>(c * kChunk + e));
    }
  }
  for (uint32_t i = tid; i < s.n_side; i += kHB) {
    const float v = penalised_value(s.side_raw[i], P.rho, P.pi);
    if (v >= tau) offer(v, s.ids[i]);
  }
  const uint64_t win = block_max_u64(b1, s.scratch);
  bool tie = false; int token = -1;
  if (win) {
    const float rival = (b1 == win) ? second : (b1 ? best_value(b1) : -INFINITY);   // this thread's best candidate other than the winner
    tie = __syncthreads_or(rival >= best_value(win) - 4e-6f) != 0;
    token = static_cast<int>(best_index(win));
  }
  *near_tie = tie;
  return token;
}

// ---- one row ---------------------------------------------------------------------------------------------------------------------
// Every thread of the block calls with the same arguments. `pen`: the block's bitmap area. `next`: the row this block takes
// after this one (-1: none), whose history is pulled into L2 meanwhile. A row the kernel cannot take is appended to `redo`.
__device__ void sample_row_hist(const SampleDev& P, int row, int next, HistSmem& s, uint32_t* pen, int* redo, int* n_redo) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const uint16_t* rowp = reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride);
  const bool pen_on = P.history != nullptr;
  const bool takeable = (V % kChunk) == 0 && V <= kHistMaxVocab && (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0 && (T >= 0.0f) && V > 0;
  auto hand_on = [&]() { if (tid == 0) redo[atomicAdd(n_redo, 1)] = row; };
  if (!takeable) { hand_on(); return; }
  const int n_chunks = V / kChunk;
  const uint4* p4 = reinterpret_cast<const uint4*>(rowp);

  // The row starts its way into L2 now: the set-up below runs under its latency, and the pass finds lines instead of opening
  // them a few at a time (a block alone on its SM has nobody else's loads to hide its own behind).
  {
    const char* rb = reinterpret_cast<const char*>(rowp);
    for (int l = tid; l * 128 < V * 2; l += kHB) asm volatile("prefetch.global.L2 [%0];" ::"l"(rb + static_cast<size_t>(l) * 128));
  }
  if (next >= 0 && tid == 0 && pen_on) {
    const char* hp = reinterpret_cast<const char*>(P.history + static_cast<int64_t>(next) * P.hist_stride);
    const uint32_t hb = (static_cast<uint32_t>(P.hist_len) * 4u) & ~15u;
    if ((reinterpret_cast<uintptr_t>(hp) & 15u) == 0 && hb) hprefetch_l2(hp, hb);
  }

  // ---- phase 0: clear; the history's distinct ids as a bitmap and as a list -------------------------------------------------
  const bool stochastic = T > 0.0f;
  if (tid == 0) { s.n_side = 0u; s.n_b = 0u; s.cz = 0u; s.cninf = 0u; s.pz = 0u; s.pninf = 0u; s.oob = 0u; s.top_pos = 0xFFFFFFFFu; s.token = -1; }
  if (stochastic) {
    const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
    uint4* h4 = reinterpret_cast<uint4*>(s.hist);
    for (int i = tid; i < static_cast<int>(kSlots) / 8; i += kHB) h4[i] = z4;
    if (pen_on) {
      uint4* ph4 = reinterpret_cast<uint4*>(s.pen_hist);
      for (int i = tid; i < static_cast<int>(kSlots) / 16; i += kHB) ph4[i] = z4;
    }
    if (P.draw == LM_DRAW_INVERSE_CDF) {
      uint4* f4 = reinterpret_cast<uint4*>(s.seg_fix);
      for (int i = tid; i < (n_chunks / kSegChunks + 2) / 2; i += kHB) f4[i] = z4;
    }
  }
  if (pen_on) {
    uint4* b4 = reinterpret_cast<uint4*>(pen);
    for (int i = tid; i < (V + 127) / 128; i += kHB) b4[i] = make_uint4(0u, 0u, 0u, 0u);
    const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
    constexpr int kAhead = kPenCap / kHB;                                 // the first ids of every thread are in flight across the barrier
    int ahead[kAhead];
#pragma unroll
    for (int j = 0; j < kAhead; j++) { const int i = tid + j * kHB; ahead[j] = (i < P.hist_len) ? __ldg(h + i) : -1; }
    __syncthreads();
    const int n_hist = (P.hist_len + kHB - 1) / kHB * kHB;                // uniform trip count: warp votes inside
    for (int i = tid, j = 0; i < n_hist; i += kHB, j++) {
      int id = -1;
      if (j < kAhead) {
#pragma unroll
        for (int k = 0; k < kAhead; k++) if (k == j) id = ahead[k];
      } else if (i < P.hist_len) id = __ldg(h + i);
      bool fresh = false;
      if (id >= 0 && id < V) {
        const uint32_t bit = 1u << (id & 31);
        fresh = (atomicOr(&pen[id >> 5], bit) & bit) == 0u;               // the thread that sets the bit owns the id
      }
      const uint32_t votes = __ballot_sync(kFull, fresh);
      uint32_t base = 0;
      if (lane == 0 && votes) base = atomicAdd(&s.n_side, __popc(votes));
      base = __shfl_sync(kFull, base, 0);
      if (fresh) {
        const uint32_t slot = base + __popc(votes & ((1u << lane) - 1u));
        if (slot < kPenCap) s.ids[slot] = static_cast<uint32_t>(id);
      }
    }
  }
  __syncthreads();
  const uint32_t n_side = s.n_side;
  if (n_side > kPenCap) { hand_on(); return; }                            // more distinct penalised ids than the lists hold
  const uint32_t* penmap = pen_on ? pen : nullptr;

  if (!stochastic) {                                                      // greedy: a streaming argmax, no histogram
    uint64_t best = 0ull;
    constexpr int kU = 4;
    for (int c0 = tid; c0 < n_chunks; c0 += kHB * kU) {
      uint4 q[kU];
#pragma unroll
      for (int j = 0; j < kU; j++) { const int c = c0 + j * kHB; if (c < n_chunks) q[j] = __ldg(p4 + c); }
#pragma unroll
      for (int j = 0; j < kU; j++) {
        const int c = c0 + j * kHB;
        if (c >= n_chunks) break;
        const uint32_t bits = pen_on ? ((pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu) : 0u;
        const float z[kChunk] = {bf16_lo(q[j].x), bf16_hi(q[j].x), bf16_lo(q[j].y), bf16_hi(q[j].y), bf16_lo(q[j].z), bf16_hi(q[j].z), bf16_lo(q[j].w), bf16_hi(q[j].w)};
#pragma unroll
        for (int e = 0; e < kChunk; e++) {
          const uint64_t p = pack_best(canon_zero(z[e]), static_cast<uint32_t>(c * kChunk + e));
          if (!((bits >> e) & 1u)) best = p > best ? p : best;            // penalised positions come from the list below
        }
      }
    }
    for (uint32_t i = tid; i < n_side; i += kHB) {
      const uint32_t id = s.ids[i];
      const uint64_t p = pack_best(penalised_value(__ldg(rowp + id), P.rho, P.pi), id);
      best = p > best ? p : best;
    }
    best = block_max_u64(best, s.scratch);
    if (tid == 0) {
      P.out_tokens[row] = static_cast<int>(best_index(best));
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_status) P.out_status[row] = (best_value(best) != best_value(best)) ? LM_STATUS_NAN : 0u;
      if (P.out_vmax) P.out_vmax[row] = best_value(best);
      if (P.out_mass) P.out_mass[row] = 0ull;
    }
    return;
  }

  // ---- phase 1: the histogram of the raw row, straight from HBM ---------------------------------------------------------------
  {
    constexpr int kU = 4;
    for (int c0 = tid; c0 < n_chunks; c0 += kHB * kU) {
      uint4 q[kU];
#pragma unroll
      for (int j = 0; j < kU; j++) { const int c = c0 + j * kHB; q[j] = (c < n_chunks) ? __ldg(p4 + c) : make_uint4(0u, 0u, 0u, 0u); }
#pragma unroll
      for (int j = 0; j < kU; j++) {
        if (c0 + j * kHB < n_chunks) { hist_add_word(s, q[j].x); hist_add_word(s, q[j].y); hist_add_word(s, q[j].z); hist_add_word(s, q[j].w); }
      }
    }
  }
  // ---- phase 2: the penalised logits move from the main histogram to their own (by raw code) ----------------------------------
  {
    constexpr int kPer = kPenCap / kHB;
    uint32_t code[kPer];
#pragma unroll
    for (int j = 0; j < kPer; j++) { const uint32_t i = tid + j * kHB; code[j] = i < n_side ? __ldg(rowp + s.ids[i]) : 0u; }
    __syncthreads();                                                      // the pass is complete
#pragma unroll
    for (int j = 0; j < kPer; j++) {
      const uint32_t i = tid + j * kHB;
      if (i >= n_side) continue;
      s.side_raw[i] = static_cast<uint16_t>(code[j]);
      const uint32_t slot = slot_of_code(code[j]);
      if (slot == 0xFFFFFFFFu) {                                           // a penalised 0 or -inf (counted apart), or a code outside the window
        if ((code[j] & 0x7FFFu) == 0u) { atomicSub(&s.cz, 1u); atomicAdd(&s.pz, 1u); }
        else if (code[j] == 0xFF80u) { atomicSub(&s.cninf, 1u); atomicAdd(&s.pninf, 1u); }
        else s.oob = 1u;
        continue;
      }
      atomicSub(&s.hist[slot >> 1], (slot & 1u) ? 0x10000u : 1u);
      atomicAdd(&s.pen_hist[slot >> 2], 1u << ((slot & 3u) * 8u));
    }
    __syncthreads();
  }
  if (s.oob) { hand_on(); return; }
  // ---- phase 3: group counts and the top position of the main histogram; the penalised histogram compacted into a list --------
  for (int sg = warp; sg < static_cast<int>(kSlots) / kGrpSlots; sg += kHW) {
    const uint32_t w = s.hist[sg * 32 + lane];
    const uint32_t tot = warp_sum_u32((w & 0xFFFFu) + (w >> 16));
    const int g = sg < kSignGroups ? kSignGroups - 1 - sg : sg + 1;
    if (lane == 0) s.g_cnt[g] = tot;
    if (tot) {
      const uint32_t slot = static_cast<uint32_t>(sg) * kGrpSlots + 2u * lane;
      uint32_t p = 0xFFFFFFFFu;
      if (w & 0xFFFFu) p = pos_of_slot(slot);
      if (w >> 16) p = min(p, pos_of_slot(slot + 1u));
      p = warp_min_u32(p);
      if (lane == 0) atomicMin(&s.top_pos, p);
    }
  }
  if (tid == 0) {
    s.g_cnt[kZeroGroup] = s.cz; s.g_cnt[kNinfGroup] = s.cninf;
    if (s.cz) atomicMin(&s.top_pos, kPosZero); else if (s.cninf) atomicMin(&s.top_pos, kPosNinf);
  }
  if (pen_on) {
    // thread t reads 32 counters in walk order: slots 8191 - 32 t downwards (positive values), then 8192 + 32 (t - 256) upwards
    const bool posv = tid < kHB / 2;
    const uint32_t first = posv ? kWinCodes - 32u - 32u * tid : kWinCodes + 32u * (tid - kHB / 2);   // lowest slot of the 32
    const uint4 a = reinterpret_cast<const uint4*>(s.pen_hist)[first / 16u], b = reinterpret_cast<const uint4*>(s.pen_hist)[first / 16u + 1u];
    const uint32_t w8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t nz = 0u, sb = 0u;
#pragma unroll
    for (int k = 0; k < 8; k++) if (w8[k]) {
#pragma unroll
      for (int e = 0; e < 4; e++) { const uint32_t c = (w8[k] >> (8 * e)) & 0xFFu; nz += c ? 1u : 0u; sb += c; }
    }
    // the penalised zeros sit between the positive and the negative codes, the penalised -inf at the very end (marker slots)
    const uint32_t zeros = tid == kHB / 2 ? s.pz : 0u, ninfs = tid == kHB - 1 ? s.pninf : 0u;
    nz += (zeros ? 1u : 0u) + (ninfs ? 1u : 0u); sb += zeros + ninfs;
    uint32_t tot = 0u;
    uint32_t off = hblock_scan_u32((sb << 16) | nz, s.warp_c, &tot) & 0xFFFFu;
    if ((tot >> 16) != n_side) s.oob = 1u;                                 // an 8-bit counter wrapped
    if (tid == 0) s.n_b = tot & 0xFFFFu;
    if (zeros) { s.b_ins[off] = 0xFFFFu; s.b_cnt[off] = static_cast<uint16_t>(zeros); off++; }
    if (nz) {                                                             // (slot, count) pairs, descending value order; the values follow below
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int kk = posv ? 7 - k : k;
        const uint32_t w = w8[kk];
        if (!w) continue;
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int ee = posv ? 3 - e : e;
          const uint32_t c = (w >> (8 * ee)) & 0xFFu;
          if (!c) continue;
          s.b_ins[off] = static_cast<uint16_t>(first + static_cast<uint32_t>(4 * kk + ee)); s.b_cnt[off] = static_cast<uint16_t>(c);
          off++;
        }
      }
    }
    if (ninfs) { s.b_ins[off] = 0xFFFEu; s.b_cnt[off] = static_cast<uint16_t>(ninfs); }
  }
  __syncthreads();
  if (s.oob) { hand_on(); return; }
  const uint32_t n_b = s.n_b;
  for (uint32_t j = tid; j < n_b; j += kHB) {                             // spread over all threads: the division of the penalty is the cost here
    const uint32_t slot = s.b_ins[j];
    const float v = penalised_value(slot == 0xFFFFu ? 0x0000u : (slot == 0xFFFEu ? 0xFF80u : code_of_slot(slot)), P.rho, P.pi);
    s.b_val[j] = v; s.b_ins[j] = static_cast<uint16_t>(ins_pos(v));
  }
  __syncthreads();
  const float top_a = s.top_pos != 0xFFFFFFFFu ? val_of_pos(s.top_pos) : -INFINITY;
  const float vmax = (n_b && s.b_val[0] > top_a) ? s.b_val[0] : top_a;
  if (!(vmax > -INFINITY)) { hand_on(); return; }                         // nothing but -inf

  // ---- phase 4: masses per group (only when a threshold needs them); the penalised values join their groups -------------------
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k && has_p;
  if (top_k > V) top_k = V;
  if (has_p) {
    for (int sg = warp; sg < static_cast<int>(kSlots) / kGrpSlots; sg += kHW) {
      const int g = sg < kSignGroups ? kSignGroups - 1 - sg : sg + 1;
      if (s.g_cnt[g] == 0u) { if (lane == 0) s.g_mass[g] = 0.0; continue; }
      const uint32_t w = s.hist[sg * 32 + lane];
      const uint32_t slot = static_cast<uint32_t>(sg) * kGrpSlots + 2u * lane;
      double m = 0.0;
      if (w & 0xFFFFu) m += static_cast<double>(w & 0xFFFFu) * softmass(hcode_val(code_of_slot(slot)), vmax, inv_t);
      if (w >> 16) m += static_cast<double>(w >> 16) * softmass(hcode_val(code_of_slot(slot + 1u)), vmax, inv_t);
      m = warp_sum_f64(m);
      if (lane == 0) s.g_mass[g] = m;
    }
    if (tid == 0) { s.g_mass[kZeroGroup] = s.cz ? static_cast<double>(s.cz) * softmass(0.0f, vmax, inv_t) : 0.0; s.g_mass[kNinfGroup] = 0.0; }
  }
  if (n_b) {
    // counts and masses of the penalised values become running sums over the list (thread t owns a few consecutive entries):
    // any run of the list is then a difference of two entries
    constexpr int kPer = kPenCap / kHB;
    const uint32_t per = (n_b + kHB - 1u) / kHB;
    uint32_t c_run[kPer], csum = 0u; double m_run[kPer], msum = 0.0;
#pragma unroll
    for (int k = 0; k < kPer; k++) {
      const uint32_t jj = tid * per + k;
      const bool live = static_cast<uint32_t>(k) < per && jj < n_b;
      const uint32_t c = live ? s.b_cnt[jj] : 0u;
      if (live && has_p) msum += static_cast<double>(c) * softmass(s.b_val[jj], vmax, inv_t);
      csum += c; c_run[k] = csum; m_run[k] = msum;
    }
    uint32_t ci = csum; double mi = msum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, ci, o);
      const double tm = __shfl_up_sync(kFull, mi, o);
      if (lane >= o) { ci += tc; mi += tm; }
    }
    if (lane == 31) { s.warp_c[warp] = ci; s.warp_m[warp] = mi; }
    __syncthreads();
    uint32_t cbase = ci - csum; double mbase = mi - msum;
    for (int w = 0; w < warp; w++) { cbase += s.warp_c[w]; mbase += s.warp_m[w]; }
#pragma unroll
    for (int k = 0; k < kPer; k++) {
      const uint32_t jj = tid * per + k;
      if (static_cast<uint32_t>(k) < per && jj < n_b) { s.b_cnt[jj] = static_cast<uint16_t>(cbase + c_run[k]); if (has_p) s.b_mass[jj] = mbase + m_run[k]; }
    }
  }
  __syncthreads();
  for (uint32_t j = tid; j < n_b; j += kHB) {                             // the last entry of each group's run adds the run to the group
    const int g = group_of_pos(s.b_ins[j]);
    if (j + 1u < n_b && group_of_pos(s.b_ins[j + 1u]) == g) continue;
    const uint32_t start = lower_bound_u16(s.b_ins, n_b, first_pos_of_group(g));
    s.g_cnt[g] += b_count_range(s, start, j + 1u);
    if (has_p) s.g_mass[g] += b_mass_range(s, start, j + 1u);
  }
  __syncthreads();
  {
    uint32_t tot = 0u;
    hblock_scan_u32(tid < kGroupsH ? s.g_cnt[tid] : 0u, s.warp_c, &tot);
    if (tot != static_cast<uint32_t>(V)) { hand_on(); return; }           // a 16-bit counter wrapped: more than 65535 equal logits
  }

  // ---- phase 5: thresholds -----------------------------------------------------------------------------------------------------
  uint32_t status = 0u;
  double tau64 = -INFINITY; bool have_tau = false;
  double topk_mass = 0.0;
  if (has_k) {
    if (has_p) hist_walk<false, true>(s, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    else hist_walk<false, false>(s, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    tau64 = s.res_tau; have_tau = true; topk_mass = s.res_cum_m;
    __syncthreads();
  }
  if (has_p) {
    double total;
    if (in_topk) total = topk_mass;
    else total = block_sum_f64(tid < kGroupsH ? s.g_mass[tid] : 0.0, s.scratch);
    const double target = static_cast<double>(top_p) * total;
    hist_walk<true, true>(s, 0u, target, vmax, inv_t);
    const double eps = 1e-12 * total;
    if (fabs(s.res_cum_m - target) <= eps || fabs(s.res_excl_m - target) <= eps) status |= LM_STATUS_TOPP_EDGE;
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

  // ---- phase 6: the draw over the kept set (the row is in L2) ------------------------------------------------------------------
  int token;
  uint64_t kept_weight = 0ull;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    token = hist_draw_inverse_cdf(P, s, penmap, rowp, n_chunks, tau, vmax, T, P.uniforms ? P.uniforms[row] : 0.0f, &kept_weight);
  } else {
    bool tie = false;
    token = hist_draw_gumbel(P, s, penmap, rowp, n_chunks, tau, T, static_cast<uint32_t>(P.row_offset + row), &tie);
    if (tie) status |= LM_STATUS_NEAR_TIE;
    if (P.out_mass) { __syncthreads(); hist_draw_inverse_cdf(P, s, penmap, rowp, n_chunks, tau, vmax, T, 0.0f, &kept_weight, true); }   // the histograms give the mass
  }
  // ---- phase 7: outputs ----------------------------------------------------------------------------------------------------------
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
    if (P.out_vmax) P.out_vmax[row] = vmax;
    if (P.out_mass) P.out_mass[row] = kept_weight;
  }
}

// One block per row in hand, two blocks per SM (vocabularies up to ~200k; one above). Rows cost very different amounts (the
// draw scales with the kept set), so blocks take them from a counter (`next_item`, zeroed by the host) instead of a fixed
// stride; a block always holds the item after its current one too, so that it can pull that row's history into L2 while it
// works. With a row list (written by the top-k kernel: the rows it left) the items are entries of the list, without one they
// are the rows themselves.
__global__ void __launch_bounds__(kHB, 2) sample_hist_kernel(SampleDev P, const int* list, const int* n_list, int* next_item, int* redo, int* n_redo) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  HistSmem& s = *reinterpret_cast<HistSmem*>(smem_raw);
  uint32_t* pen = reinterpret_cast<uint32_t*>(smem_raw + ((sizeof(HistSmem) + 15) & ~static_cast<size_t>(15)));
  __shared__ int item[2];
  // A kernel launched behind this one with programmatic stream serialization (the top-k kernel, which works on other rows and
  // reads nothing this kernel writes) may take every SM a block of this grid has left, instead of waiting for the whole grid.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  apply_step_state(P);
  const int n = list ? min(*n_list, P.rows) : P.rows;
  // many items per block: hold the next item too and claim the one after it at the start of a row (the counter's round trip
  // hides behind the row); few items per block: claim an item only when it is needed, so that no block sits on work
  const bool ahead = n >= 4 * static_cast<int>(gridDim.x);
  if (threadIdx.x == 0) { item[0] = atomicAdd(next_item, 1); item[1] = (ahead && item[0] < n) ? atomicAdd(next_item, 1) : n; }
  __syncthreads();
  for (;;) {
    const int i = item[0], in = item[1];
    if (i >= n) break;
    int fetched = n;
    if (threadIdx.x == 0 && in < n) fetched = atomicAdd(next_item, 1);
    const int row = list ? list[i] : i;
    int next = in < n ? (list ? list[in] : in) : -1;
    if (next >= P.rows) next = -1;
    if (row >= 0 && row < P.rows) sample_row_hist(P, row, next, s, pen, redo, n_redo);   // (a list entry is a row index by construction)
    __syncthreads();
    if (threadIdx.x == 0) { item[0] = ahead ? in : atomicAdd(next_item, 1); item[1] = fetched; }
    __syncthreads();
  }
}

__host__ __device__ inline size_t hist_smem_bytes(int vocab) { return ((sizeof(HistSmem) + 15) & ~static_cast<size_t>(15)) + static_cast<size_t>((vocab + 127) / 128) * 16; }

}  // namespace lm
