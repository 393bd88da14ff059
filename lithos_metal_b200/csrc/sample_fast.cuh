// The streaming BF16 row sampler: one thread block per row, ONE pass over the row from HBM.
//
// A BF16 logit has at most 65536 codes, so a histogram of the row by code (shared memory, 16-bit counters packed in
// pairs, one 32-bit shared-memory reduction per logit) holds everything the thresholds need: the k-th largest value is a
// walk over counts, the top-p boundary a walk over count x exp(value) in FP64, exactly as the reference's numpy
// definition forms them per distinct value (monolith/nn/sampling_ref.py:26-35; the reference's Metal kernels build
// the same histogram in device memory with 256 KB per row, kernels/common/sample.metal:34-162). Logits changed by
// the penalties are arbitrary FP32 values: they leave the histogram and are kept aside as a short (index, value)
// list that joins the walk at group level and exactly inside the one group where a threshold lands.
// The draw then takes a second look at the part of the row it needs, usually still in L2.
//
// Rows this kernel cannot take (a counter overflow: more than 65535 equal logits; more than kSideCap penalised
// logits, or more than kSidePool of them in the 256 codes around a threshold; vocabularies that are not a multiple of 8 or exceed
// kFastMaxVocab; misaligned rows) are listed in `redo` and handled by the generic kernel launched behind this one.
#pragma once
#include "common.cuh"
#include "draw.cuh"
#include "sample_generic.cuh"

namespace lm {

#ifdef LM_PROFILE_PHASES
__device__ unsigned long long g_phase_cycles[16];    // clock64 totals per phase of block 0 (profiling builds only)
#define LM_PHASE(i) do { __syncthreads(); if (threadIdx.x == 0 && blockIdx.x == 0) { const long long _t = clock64(); atomicAdd(&g_phase_cycles[i], (unsigned long long)(_t - _t0)); _t0 = _t; } } while (0)
#else
#define LM_PHASE(i) do {} while (0)
#endif

constexpr int kFastMaxVocab = 262144;
constexpr int kCodes = 65536;
constexpr int kGroupBins = 256;             // positions per group: one 512-byte block of counters = one uint4 per lane
constexpr int kGroups = kCodes / kGroupBins;
constexpr int kSideCap = 4096;              // penalised logits per row the kernel keeps aside
constexpr int kSidePool = 1536;              // of those, how many may fall into the group being refined

struct FastSmem {
  uint32_t hist[kCodes / 2];                // 128 KB: 16-bit counters, code c in half (c & 1) of word c >> 1
  float side_val[kSideCap];                 // 16 KB: penalised values ...
  int side_idx[kSideCap];                   // 16 KB: ... and their vocabulary indices
  union {                                   // the threshold walk and the draw never run at the same time
    struct {
      double pool_mass[kSidePool];              // 12 KB: softmass of the side values of the group being refined, sorted by owning lane
      double lane_bin_mass[32][8];              // 2 KB: softmass of each lane's eight bins
      float pool_val[kSidePool];                // 6 KB: the side values themselves; lane L owns [lane_off[L], lane_off[L + 1])
    };
    struct {
      uint64_t sweep_part[kFastMaxVocab / (kBlock * kChunk)][32];   // 8 KB: per-warp fixed-point mass of every sweep of the draw
      uint32_t side_limb[kFastMaxVocab / (kBlock * kChunk)][3];     // 16-bit limbs of the side values' fixed-point mass per sweep
    };
  };
  double gmass[kGroups];
  uint32_t gcnt[kGroups];
  uint32_t goff[kGroups + 1];               // side list sorted by group: group g holds entries [goff[g], goff[g + 1])
  uint32_t gfill[kGroups];
  uint32_t lane_side_n[32];
  uint32_t lane_off[33];
  uint32_t lane_fill[32];
  uint32_t sel_cnt[8];
  DrawSmem draw;
  double warp_m[32];
  uint32_t warp_c[32];
  uint32_t side_n;
  uint32_t side_max_key;
  uint32_t top_group, top_pos;
  int sel_group;
  uint32_t sel_base_c;
  double sel_base_m;
  float res_tau; double res_cum_m, res_above_m; uint32_t res_cum_c; int res_fail;
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

// two logits of one 32-bit word into the histogram: address = code / 2 words, increment = 1 << (16 * (code & 1))
__device__ __forceinline__ void hist_add_word(uint32_t* hist, uint32_t w) {
  char* base = reinterpret_cast<char*>(hist);
  atomicAdd(reinterpret_cast<uint32_t*>(base + ((w << 1) & 0x1FFFCu)), (w & 1u) * 0xFFFFu + 1u);
  atomicAdd(reinterpret_cast<uint32_t*>(base + ((w >> 15) & 0x1FFFCu)), ((w >> 16) & 1u) * 0xFFFFu + 1u);
}

__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// The eight counters a lane owns in group g: positions 256 g + 8 lane + j, j = 0..7, in descending value order.
// Group g is one aligned block of 256 codes (block 127 - g for the positive half, block g for the negative half);
// in the positive half codes run against positions, so the lane takes the mirrored uint4 and reverses it.
__device__ __forceinline__ void lane_counts(const uint32_t* hist, int g, int lane, uint32_t cnt[8]) {
  const bool pos_half = g < kGroups / 2;
  const int block = pos_half ? (kGroups / 2 - 1 - g) : g;
  const int q = pos_half ? (31 - lane) : lane;
  const uint4 v = reinterpret_cast<const uint4*>(hist)[block * 32 + q];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const int jj = pos_half ? 7 - j : j;                                  // code offset inside the uint4
    cnt[j] = (w[jj >> 1] >> ((jj & 1) * 16)) & 0xFFFFu;
  }
}
__device__ __forceinline__ uint32_t sum8(const uint4 v) {
  const uint32_t a = (v.x & 0xFFFFu) + (v.x >> 16), b = (v.y & 0xFFFFu) + (v.y >> 16), c = (v.z & 0xFFFFu) + (v.z >> 16), d = (v.w & 0xFFFFu) + (v.w >> 16);
  return a + b + c + d;
}

// Exact walk inside one group of 256 positions. Finds the first distinct value, descending, at which the running
// count reaches k_target (BY_MASS false) or the running mass reaches m_target (BY_MASS true), starting from
// (base_c, base_m) = totals strictly above the group. Lane L of warp 0 owns positions 8L..8L+7 of the group and
// the side values whose bin lies there; the masses are computed by all warps first (warp w for owner lane w) so
// that no thread runs a long chain of FP64 exponentials. Results in s.res_*; s.res_fail = 1 if the group holds more
// side values than the pool.
template <bool BY_MASS, bool NEED_MASS>
__device__ void refine_group(FastSmem& s, int group, uint32_t base_c, double base_m, uint32_t k_target, double m_target, float vmax, double inv_t) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < 32) { s.lane_side_n[tid] = 0u; s.lane_fill[tid] = 0u; }
  if (tid == 0) s.res_fail = 0;
  __syncthreads();
  const uint32_t s0 = s.goff[group], s1 = s.goff[group + 1];               // this group's side values (the list is sorted by group)
  if (s1 - s0 > static_cast<uint32_t>(kSidePool)) { if (tid == 0) s.res_fail = 1; __syncthreads(); return; }
  for (uint32_t i = s0 + tid; i < s1; i += kBlock)                         // counting sort by owning lane: count, offsets, fill
    atomicAdd(&s.lane_side_n[(code_to_pos(floor_code(s.side_val[i])) % kGroupBins) >> 3], 1u);
  __syncthreads();
  if (tid < 32) {
    const uint32_t n = s.lane_side_n[tid];
    uint32_t incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
    s.lane_off[tid] = incl - n;
    if (tid == 31) s.lane_off[32] = incl;
  }
  __syncthreads();
  for (uint32_t i = s0 + tid; i < s1; i += kBlock) {
    const float v = s.side_val[i];
    const uint32_t owner = (code_to_pos(floor_code(v)) % kGroupBins) >> 3;
    s.pool_val[s.lane_off[owner] + atomicAdd(&s.lane_fill[owner], 1u)] = v;
  }
  __syncthreads();
  if (NEED_MASS) {                                                         // a warp per owner lane: the masses of its bins and side values
    for (int o = warp; o < 32; o += kWarps) {
      const uint32_t pos0 = static_cast<uint32_t>(group) * kGroupBins + o * 8u;
      if (lane < 8) {
        const uint32_t code = pos_to_code(pos0 + lane);
        const uint32_t c = hist_get(s.hist, code);
        s.lane_bin_mass[o][lane] = c ? static_cast<double>(c) * softmass(code_val(code), vmax, inv_t) : 0.0;
      } else {
        for (uint32_t i = s.lane_off[o] + lane - 8; i < s.lane_off[o + 1]; i += 24) s.pool_mass[i] = softmass(s.pool_val[i], vmax, inv_t);
      }
    }
    __syncthreads();
  }
  if (tid < 32) {
    uint32_t cnt[8];
    lane_counts(s.hist, group, lane, cnt);
    const uint32_t m_side = s.lane_side_n[lane];
    const double* sm = s.pool_mass + s.lane_off[lane];
    uint32_t c_lane = m_side; double m_lane = 0.0;
#pragma unroll
    for (int j = 0; j < 8; j++) { c_lane += cnt[j]; if (NEED_MASS) m_lane += s.lane_bin_mass[lane][j]; }
    if (NEED_MASS) for (uint32_t i = 0; i < m_side; i++) m_lane += sm[i];
    uint32_t ci = c_lane; double mi = m_lane;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, ci, o);
      const double tm = __shfl_up_sync(kFull, mi, o);
      if (lane >= o) { ci += tc; mi += tm; }
    }
    const bool hit = BY_MASS ? (c_lane > 0 && base_m + mi >= m_target) : (base_c + ci >= k_target);
    const uint32_t hits = __ballot_sync(kFull, hit);
    const uint32_t occ = __ballot_sync(kFull, c_lane > 0);
    const int sel = hits ? (__ffs(hits) - 1) : (31 - __clz(occ));        // mass never reached (rounding): the lowest occupied lane
    // The selected lane's distinct values, descending: its eight BF16 bins (pure counts) and its side values. The warp ranks
    // them together: lane l takes items l, l + 32, ... and sums, over all items, those at or above its own value; the
    // answer is the largest value whose inclusive total reaches the target (or, if rounding left it unreached, the smallest).
    if (lane == sel) {
#pragma unroll
      for (int j = 0; j < 8; j++) s.sel_cnt[j] = cnt[j];
    }
    __syncwarp();
    const uint32_t n_side_sel = __shfl_sync(kFull, m_side, sel);
    const uint32_t top_c = __shfl_sync(kFull, base_c + ci - c_lane, sel);
    const double top_m = __shfl_sync(kFull, base_m + mi - m_lane, sel);
    const float* ssv = s.pool_val + s.lane_off[sel];
    const double* ssm = s.pool_mass + s.lane_off[sel];
    const uint32_t spos0 = static_cast<uint32_t>(group) * kGroupBins + static_cast<uint32_t>(sel) * 8u;
    const uint32_t n_items = 8u + n_side_sel;
    uint32_t best_key = 0u, low_key = 0xFFFFFFFFu;                          // best: largest qualifying value; low: smallest value present
    uint32_t best_c = 0u, low_c = 0u; double best_m = 0.0, best_above = 0.0, low_m = 0.0, low_above = 0.0;
    for (uint32_t i = lane; i < n_items; i += 32) {
      const float v = i < 8u ? code_val(pos_to_code(spos0 + i)) : ssv[i - 8u];
      if (i < 8u && s.sel_cnt[i] == 0u) continue;
      uint32_t inc_c = top_c; double inc_m = top_m, abv_m = top_m;
      for (uint32_t t = 0; t < n_items; t++) {
        const float vt = t < 8u ? code_val(pos_to_code(spos0 + t)) : ssv[t - 8u];
        const uint32_t ct = t < 8u ? s.sel_cnt[t] : 1u;
        if (ct == 0u || vt < v) continue;
        const double mt = NEED_MASS ? (t < 8u ? s.lane_bin_mass[sel][t] : ssm[t - 8u]) : 0.0;
        inc_c += ct; inc_m += mt;
        if (vt > v) abv_m += mt;
      }
      const uint32_t key = fkey(v);
      if ((BY_MASS ? (inc_m >= m_target) : (inc_c >= k_target)) && key > best_key) { best_key = key; best_c = inc_c; best_m = inc_m; best_above = abv_m; }
      if (key < low_key) { low_key = key; low_c = inc_c; low_m = inc_m; low_above = abv_m; }
    }
    uint32_t win = best_key, lowest = low_key;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { win = max(win, __shfl_xor_sync(kFull, win, o)); lowest = min(lowest, __shfl_xor_sync(kFull, lowest, o)); }
    const bool mine = win ? (best_key == win) : (low_key == lowest);
    const uint32_t owners = __ballot_sync(kFull, mine);
    if (lane == __ffs(owners) - 1) {                                        // equal values carry equal totals: any owner will do
      s.res_tau = fkey_inv(win ? win : lowest);
      s.res_cum_c = win ? best_c : low_c; s.res_cum_m = win ? best_m : low_m; s.res_above_m = win ? best_above : low_above;
    }
  }
  __syncthreads();
}

// Block-wide search over the groups, descending: the first group at which the running count / mass reaches the target.
// Leaves the group in s.sel_group and the totals strictly above it in s.sel_base_c / s.sel_base_m.
template <bool BY_MASS>
__device__ void find_group(FastSmem& s, uint32_t k_target, double m_target) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t c = 0, ci = 0; double m = 0.0, mi = 0.0;
  if (tid == 0) s.sel_group = kGroups;
  if (tid < kGroups) {
    c = s.gcnt[tid]; ci = c;
    if (BY_MASS) { m = s.gmass[tid]; mi = m; }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tc = __shfl_up_sync(kFull, ci, o);
      const double tm = BY_MASS ? __shfl_up_sync(kFull, mi, o) : 0.0;
      if (lane >= o) { ci += tc; mi += tm; }
    }
    if (lane == 31) { s.warp_c[warp] = ci; s.warp_m[warp] = mi; }
  }
  __syncthreads();
  if (tid < kGroups) {
    uint32_t wc = 0; double wm = 0.0;
    for (int w = 0; w < warp; w++) { wc += s.warp_c[w]; if (BY_MASS) wm += s.warp_m[w]; }
    ci += wc; mi += wm;
    const bool hit = BY_MASS ? (c > 0 && mi >= m_target) : (ci >= k_target);
    if (hit) atomicMin(&s.sel_group, tid);
  }
  __syncthreads();
  int sel = s.sel_group;
  if (sel == kGroups) {                                                   // mass never reached (rounding): the last occupied group
    __syncthreads();
    if (tid == 0) s.sel_group = -1;
    __syncthreads();
    if (tid < kGroups && c > 0) atomicMax(&s.sel_group, tid);
    __syncthreads();
    sel = s.sel_group;
  }
  if (tid == sel) { s.sel_base_c = ci - c; s.sel_base_m = mi - m; }
  __syncthreads();
}

// The inverse-CDF draw of the streaming kernel. The total weight S of the kept set comes from the histogram (count x weight
// per code) and the side list, so the target is known before the row is read again. The sweeps over the row then run from
// whichever end is closer to the target (a suffix sum is as exact as a prefix sum in integers) and stop at the sweep that
// holds it: a quarter of the row on average instead of all of it. Every thread calls; every thread gets the token.
__device__ int draw_inverse_cdf_bidir(const RowView& rv, FastSmem& s, const SideList& side, float tau, float vmax, float temperature, float u) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_chunks = rv.vocab / kChunk;
  const int n_sweeps = (n_chunks + kBlock - 1) / kBlock;
  const float c2 = exp2_scale(temperature);
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  DrawSmem& d = s.draw;
  uint32_t* side_limb = &s.side_limb[0][0];
  uint64_t* sweep_part = &s.sweep_part[0][0];
  for (int i = tid; i < n_sweeps * 3; i += kBlock) side_limb[i] = 0u;
  if (tid == 0) { d.token = -1; d.found_sweep = -1; d.found_base = 0ull; }
  __syncthreads();
  // ---- S: every kept BF16 code once, times its count; the kept side values join their sweep's limbs on the way ----------
  uint64_t mine = 0ull;
  {
    const uint32_t pos_last = tc == 0x0000u ? 0x8000u : code_to_pos(tc);   // the last kept position (-0 is kept with +0)
    const uint32_t pos_first = max(0x7Fu, s.top_group * static_cast<uint32_t>(kGroupBins));   // +inf, or the first occupied group
    for (uint32_t pos = pos_first + tid; pos <= pos_last && pos <= 0xFF80u; pos += kBlock) {
      const uint32_t code = pos_to_code(pos);
      const uint32_t cnt = hist_get(s.hist, code);
      if (cnt) mine += static_cast<uint64_t>(cnt) * weight_q40(code_val(code), vmax, c2);
    }
    for (uint32_t i = tid; i < side.n; i += kBlock) {
      const float v = side.val[i];
      if (v >= tau) {
        const uint64_t w = weight_q40(v, vmax, c2);
        if (w) {
          mine += w;
          uint32_t* l = side_limb + 3 * ((side.idx[i] / kChunk) / kBlock);
          atomicAdd(l, static_cast<uint32_t>(w & 0xFFFFull)); atomicAdd(l + 1, static_cast<uint32_t>((w >> 16) & 0xFFFFull));
          atomicAdd(l + 2, static_cast<uint32_t>(w >> 32));
        }
      }
    }
  }
  const uint64_t total = block_sum_u64(mine, d.scratch);
  if (total == 0ull) return -1;
  const uint64_t target = cdf_target(u, total);
  const bool forward = target < total - target;
  const uint64_t tt = forward ? target : total - target - 1ull;             // the first sweep, in scan order, whose running sum exceeds tt
  // ---- the sweeps, four at a time, from the nearer end ----------------------------------------------------------------------
  const uint4* p4 = reinterpret_cast<const uint4*>(rv.row);
  const uint4 neg = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
  uint64_t run = 0ull;
  int found = -1; uint64_t before = 0ull, found_total = 0ull;
  for (int b0 = 0; b0 < n_sweeps && found < 0; b0 += kDrawBatch) {
    uint4 q[kDrawBatch];
#pragma unroll
    for (int j = 0; j < kDrawBatch; j++) {
      const int it = forward ? b0 + j : n_sweeps - 1 - (b0 + j);
      const int cc = it * kBlock + tid;
      q[j] = (b0 + j < n_sweeps && cc < n_chunks) ? __ldg(p4 + cc) : neg;
    }
#pragma unroll
    for (int j = 0; j < kDrawBatch; j++) {
      if (b0 + j >= n_sweeps) break;
      const int it = forward ? b0 + j : n_sweeps - 1 - (b0 + j);
      const int cc = it * kBlock + tid;
      float z[kChunk];
      const uint32_t mask = (cc < n_chunks) ? kept_from_q(rv, cc, q[j], tau2, z) : 0u;
      uint64_t w = 0ull;
      if (mask) {
#pragma unroll
        for (int e = 0; e < kChunk; e += 2) if ((mask >> e) & 3u) {             // two logits per packed evaluation
          uint64_t wa, wb;
          weight_q40_x2(z[e], z[e + 1], vmax, c2, wa, wb);
          w += ((mask >> e) & 1u) ? wa : 0ull;
          w += ((mask >> e) & 2u) ? wb : 0ull;
        }
      }
      if (__any_sync(kFull, w != 0ull)) w = warp_sum_u64(w);
      if (lane == 0) sweep_part[it * 32 + warp] = w;
    }
    __syncthreads();
    if (warp < kDrawBatch && b0 + warp < n_sweeps) {                        // warp j sums sweep j of the batch
      const int it = forward ? b0 + warp : n_sweeps - 1 - (b0 + warp);
      uint64_t t = lane < kWarps ? sweep_part[it * 32 + lane] : 0ull;
      t = warp_sum_u64(t);
      t += static_cast<uint64_t>(side_limb[3 * it]) + (static_cast<uint64_t>(side_limb[3 * it + 1]) << 16) + (static_cast<uint64_t>(side_limb[3 * it + 2]) << 32);
      if (lane == 0) d.sweep_total[it] = t;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kDrawBatch; j++) {
      if (b0 + j >= n_sweeps || found >= 0) break;
      const int it = forward ? b0 + j : n_sweeps - 1 - (b0 + j);
      const uint64_t t = d.sweep_total[it];
      if (run + t > tt) { found = it; before = run; found_total = t; }
      run += t;
    }
  }
  if (found < 0) return -1;                                                 // cannot happen: the sweeps sum to `total`
  // ---- inside the sweep: the first cumulative weight, in index order, that exceeds the target ----------------------------
  const uint64_t prefix = forward ? before : total - before - found_total;  // the weight of everything before the sweep
  const uint64_t local_target = target - prefix;
  {
    const int c = found * kBlock + tid;
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, c, tau, tau2, z);
    uint64_t w[kChunk];
    uint64_t sum = 0ull;
#pragma unroll
    for (int e = 0; e < kChunk; e++) { w[e] = ((mask >> e) & 1u) ? weight_q40(z[e], vmax, c2) : 0ull; sum += w[e]; }
    const uint64_t excl = block_exclusive_scan_u64(sum, d.scratch, nullptr);
    if (excl <= local_target && local_target < excl + sum) {
      uint64_t r = excl;
#pragma unroll
      for (int e = 0; e < kChunk; e++) { r += w[e]; if (w[e] && r > local_target) { d.token = c * kChunk + e; break; } }
    }
  }
  __syncthreads();
  return d.token;
}

// `next` is the row this block takes after this one (-1: none): it is pulled into L2 while this one is worked on.
// A row the kernel cannot take is appended to `redo` (length in *n_redo) for the generic kernel.
__device__ void sample_row_fast(const SampleDev& P, int row, int next, FastSmem& s, int* redo, int* n_redo) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const uint16_t* rowp = reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride);
  const bool pen_on = P.history != nullptr;
  const bool takeable = (V % kChunk) == 0 && V <= kFastMaxVocab && (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0 && (T >= 0.0f) && V > 0;
  if (!takeable) { if (tid == 0) redo[atomicAdd(n_redo, 1)] = row; return; }

#ifdef LM_PROFILE_PHASES
  long long _t0 = clock64();
#endif
  RowView rv;
  rv.dtype = LM_DTYPE_BF16; rv.vocab = V; rv.rho = P.rho; rv.pi = P.pi; rv.row = rowp; rv.aligned = true; rv.pen = nullptr;
  const int n_chunks = V / kChunk;

  // the history of this block's next row: start pulling it into L2 now. (Doing the same for the next row's logits was measured
  // and dropped: the histogram pass is bound by its shared-memory atomics, not by load latency, and the prefetched rows push
  // the current rows out of L2 before the draw looks at them again.)
  if (next >= 0 && tid == 0 && pen_on) {
    const char* hp = reinterpret_cast<const char*>(P.history + static_cast<int64_t>(next) * P.hist_stride);
    const uint32_t hb = (static_cast<uint32_t>(P.hist_len) * 4u) & ~15u;
    if ((reinterpret_cast<uintptr_t>(hp) & 15u) == 0 && hb) prefetch_l2(hp, hb);
  }

  // ---- the history's distinct ids as a bitmap and as a list -------------------------------------
  {
    if (tid == 0) { s.side_n = 0u; s.side_max_key = 0u; s.top_group = kGroups; s.top_pos = 0xFFFFFFFFu; }
    if (tid < kGroups) { s.gfill[tid] = 0u; s.goff[tid] = 0u; }
    if (tid == 0) s.goff[kGroups] = 0u;
    if (pen_on) {
      const int words = (V + 31) / 32;
      for (int i = tid; i < words; i += kBlock) s.pen[i] = 0u;
      __syncthreads();
      const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
      const int n_hist = (P.hist_len + kBlock - 1) / kBlock * kBlock;       // uniform trip count: warp votes inside
      for (int i = tid; i < n_hist; i += kBlock) {
        const int id = (i < P.hist_len) ? __ldg(h + i) : -1;
        bool fresh = false;
        if (id >= 0 && id < V) {
          const uint32_t bit = 1u << (id & 31);
          fresh = (atomicOr(&s.pen[id >> 5], bit) & bit) == 0u;           // the thread that sets the bit owns the id
        }
        const uint32_t votes = __ballot_sync(kFull, fresh);
        uint32_t base = 0;
        if (lane == 0 && votes) base = atomicAdd(&s.side_n, __popc(votes));
        base = __shfl_sync(kFull, base, 0);
        if (fresh) {
          const uint32_t slot = base + __popc(votes & ((1u << lane) - 1u));
          if (slot < kSideCap) s.side_idx[slot] = id;
        }
      }
      rv.pen = s.pen;
    }
    __syncthreads();
  }
  LM_PHASE(0);
  if (s.side_n > kSideCap) { if (tid == 0) redo[atomicAdd(n_redo, 1)] = row; return; }      // more distinct penalised ids than the list holds
  const uint32_t n_side = s.side_n;
  const SideList side{s.side_idx, s.side_val, n_side};

  if (T == 0.0f) {                                                        // greedy: a streaming argmax, no histogram
    uint64_t best = 0ull;
    for (int c = tid; c < n_chunks; c += kBlock) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(rowp) + c);
      const uint32_t bits = pen_on ? ((s.pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu) : 0u;
      const float z[kChunk] = {bf16_lo(q.x), bf16_hi(q.x), bf16_lo(q.y), bf16_hi(q.y), bf16_lo(q.z), bf16_hi(q.z), bf16_lo(q.w), bf16_hi(q.w)};
#pragma unroll
      for (int e = 0; e < kChunk; e++) {
        const uint64_t p = pack_best(canon_zero(z[e]), static_cast<uint32_t>(c * kChunk + e));
        if (!((bits >> e) & 1u)) best = p > best ? p : best;              // penalised positions come from the list below
      }
    }
    for (uint32_t i = tid; i < n_side; i += kBlock) {
      const int id = s.side_idx[i];
      const float v = canon_zero(penalise(code_val(__ldg(rowp + id)), P.rho, P.pi));
      const uint64_t p = pack_best(v, static_cast<uint32_t>(id));
      best = p > best ? p : best;
    }
    best = block_max_u64(best, s.draw.scratch);
    if (tid == 0) {
      P.out_tokens[row] = static_cast<int>(best_index(best));
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_status) P.out_status[row] = (best_value(best) != best_value(best)) ? LM_STATUS_NAN : 0u;
    }
    return;
  }

  LM_PHASE(8);
  {
    uint4* h4 = reinterpret_cast<uint4*>(s.hist);
    for (int i = tid; i < kCodes / 8; i += kBlock) h4[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
  }
  // ---- pass 1: the histogram of the raw row, straight from HBM ----------------------------------------------------------
  {
    const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
    constexpr int kUnroll = 4;
    for (int c0 = tid; c0 < n_chunks; c0 += kBlock * kUnroll) {
      uint4 q[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; j++) { const int c = c0 + j * kBlock; q[j] = (c < n_chunks) ? __ldg(p4 + c) : make_uint4(0u, 0u, 0u, 0u); }
#pragma unroll
      for (int j = 0; j < kUnroll; j++) {
        if (c0 + j * kBlock < n_chunks) {
          hist_add_word(s.hist, q[j].x); hist_add_word(s.hist, q[j].y); hist_add_word(s.hist, q[j].z); hist_add_word(s.hist, q[j].w);
        }
      }
    }
  }
  // ---- the penalised logits leave the histogram (their raw value was counted above) and go to the side list, sorted by
  // group. Each thread keeps its (index, code) in registers: the gathers are issued before the barrier that ends
  // pass 1, and the list is rewritten in place once every thread has read its entries.
  uint32_t sd_code[kSideCap / kBlock]; int sd_idx[kSideCap / kBlock];
#pragma unroll
  for (int j = 0; j < kSideCap / kBlock; j++) {
    const uint32_t i = tid + j * kBlock;
    sd_idx[j] = (i < n_side) ? s.side_idx[i] : 0;
    sd_code[j] = (i < n_side) ? __ldg(rowp + sd_idx[j]) : 0u;
  }
  __syncthreads();
  LM_PHASE(1);
  if (n_side) {
    float sd_val[kSideCap / kBlock]; uint32_t sd_grp[kSideCap / kBlock];
    uint32_t mx = 0u;
#pragma unroll
    for (int j = 0; j < kSideCap / kBlock; j++) {
      if (tid + j * kBlock < n_side) {
        const float v = penalise(code_val(sd_code[j]), P.rho, P.pi);
        sd_val[j] = v; sd_grp[j] = code_to_pos(floor_code(v)) / kGroupBins;
        atomicSub(&s.hist[sd_code[j] >> 1], (sd_code[j] & 1u) ? 0x10000u : 1u);
        atomicAdd(&s.gfill[sd_grp[j]], 1u);
        mx = max(mx, fkey(v));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(kFull, mx, o));
    if (lane == 0 && mx) atomicMax(&s.side_max_key, mx);
    __syncthreads();
    if (tid < kGroups) {                                                  // exclusive prefix of the per-group side counts -> goff
      const uint32_t c = s.gfill[tid];
      uint32_t ci = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, ci, o); if (lane >= o) ci += t; }
      if (lane == 31) s.warp_c[warp] = ci;
      __syncwarp();
      s.gcnt[tid] = ci - c;                                               // parked here until the warp totals are known
    }
    __syncthreads();
    if (tid < kGroups) {
      uint32_t wc = 0;
      for (int w = 0; w < warp; w++) wc += s.warp_c[w];
      s.goff[tid] = s.gcnt[tid] + wc;
      s.gfill[tid] = 0u;
      if (tid == kGroups - 1) s.goff[kGroups] = n_side;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kSideCap / kBlock; j++) {
      if (tid + j * kBlock < n_side) {
        const uint32_t slot = s.goff[sd_grp[j]] + atomicAdd(&s.gfill[sd_grp[j]], 1u);
        s.side_val[slot] = sd_val[j]; s.side_idx[slot] = sd_idx[j];
      }
    }
    __syncthreads();
  }
  LM_PHASE(2);
  // ---- group counts (pure BF16 logits), the overflow check, the maximum ------------------------------------------------
  for (int g = warp; g < kGroups; g += kWarps) {
    const bool pos_half = g < kGroups / 2;
    const int block = pos_half ? (kGroups / 2 - 1 - g) : g;
    uint32_t c = sum8(reinterpret_cast<const uint4*>(s.hist)[block * 32 + lane]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(kFull, c, o);
    if (lane == 0) { s.gcnt[g] = c; if (c) atomicMin(&s.top_group, static_cast<uint32_t>(g)); }
  }
  __syncthreads();
  uint32_t total_c = 0;
  if (tid < kGroups) total_c = s.gcnt[tid];
  total_c = static_cast<uint32_t>(block_sum_u64(total_c, s.draw.scratch));
  if (total_c + n_side != static_cast<uint32_t>(V)) {                     // a 16-bit counter wrapped: more than 65535 equal logits
    if (tid == 0) redo[atomicAdd(n_redo, 1)] = row;
    return;
  }
  uint32_t status = 0u;
  {                                                                       // NaN codes: 0x7F81..0x7FFF and 0xFF81..0xFFFF
    uint32_t nan_c = 0;
    if (tid < 127) nan_c = hist_get(s.hist, 0x7F81u + tid) + hist_get(s.hist, 0xFF81u + tid);
    if (__syncthreads_or(nan_c != 0u)) status |= LM_STATUS_NAN;
  }
  if (tid < 32 && s.top_group < kGroups) {                                // the highest occupied bin of the highest occupied group
    uint32_t cnt[8];
    lane_counts(s.hist, static_cast<int>(s.top_group), lane, cnt);
    uint32_t p = 0xFFFFFFFFu;
#pragma unroll
    for (int j = 7; j >= 0; j--) if (cnt[j]) p = s.top_group * kGroupBins + lane * 8u + j;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) p = min(p, __shfl_xor_sync(kFull, p, o));
    if (lane == 0) s.top_pos = p;
  }
  __syncthreads();
  const float top_val = (s.top_pos != 0xFFFFFFFFu) ? code_val(pos_to_code(s.top_pos)) : -INFINITY;
  const float side_max = s.side_max_key ? fkey_inv(s.side_max_key) : -INFINITY;
  const float vmax = (n_side > 0 && side_max > top_val) ? side_max : top_val;
  LM_PHASE(3);

  // ---- thresholds ----------------------------------------------------------------------------------------------------
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k && has_p;
  if (top_k > V) top_k = V;
  double tau64 = -INFINITY; bool have_tau = false;
  double topk_mass = 0.0;
  if (has_p) {
    // group masses: count x exp64 per occupied bin (eight bins per lane) plus the exact softmass of the group's side values
    for (int g = warp; g < kGroups; g += kWarps) {
      const uint32_t s0 = s.goff[g], s1 = s.goff[g + 1];
      if (s.gcnt[g] == 0u && s0 == s1) { if (lane == 0) s.gmass[g] = 0.0; continue; }
      double m = 0.0;
      if (s.gcnt[g]) {
        uint32_t cnt[8];
        lane_counts(s.hist, g, lane, cnt);
        const uint32_t pos0 = static_cast<uint32_t>(g) * kGroupBins + lane * 8u;
#pragma unroll
        for (int j = 0; j < 8; j++) if (cnt[j]) m += static_cast<double>(cnt[j]) * softmass(code_val(pos_to_code(pos0 + j)), vmax, inv_t);
      }
      for (uint32_t i = s0 + lane; i < s1; i += 32) m += softmass(s.side_val[i], vmax, inv_t);
      m = warp_sum_f64(m);
      if (lane == 0) s.gmass[g] = m;
    }
    __syncthreads();
  }
  if (tid < kGroups) s.gcnt[tid] += s.goff[tid + 1] - s.goff[tid];         // the side values join the group counts
  __syncthreads();
  LM_PHASE(4);
  // The running mass strictly above tau_k (the top-k walk carries masses whenever top-p is on): if it stays below the
  // top-p target, the top-p boundary lies at or below tau_k and tau = tau_k without a second walk.
  double above_k_mass = 0.0;
  if (has_k) {
    find_group<false>(s, static_cast<uint32_t>(top_k), 0.0);
    double base_m = 0.0;
    if (has_p) {                                                          // the mass strictly above the group
      double m = 0.0;
      if (tid < s.sel_group) m = s.gmass[tid];
      base_m = block_sum_f64(m, s.draw.scratch);
    }
    if (has_p) refine_group<false, true>(s, s.sel_group, s.sel_base_c, base_m, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    else refine_group<false, false>(s, s.sel_group, s.sel_base_c, 0.0, static_cast<uint32_t>(top_k), 0.0, vmax, inv_t);
    if (s.res_fail) { if (tid == 0) redo[atomicAdd(n_redo, 1)] = row; return; }
    tau64 = s.res_tau; have_tau = true;
    topk_mass = s.res_cum_m; above_k_mass = s.res_above_m;
    __syncthreads();
  }
  LM_PHASE(5);
  if (has_p) {
    double total;
    if (in_topk) total = topk_mass;
    else {
      double m = 0.0;
      if (tid < kGroups) m = s.gmass[tid];
      total = block_sum_f64(m, s.draw.scratch);
    }
    const double target = static_cast<double>(top_p) * total;
    if (!has_k || above_k_mass >= target) {
      find_group<true>(s, 0u, target);
      refine_group<true, true>(s, s.sel_group, s.sel_base_c, s.sel_base_m, 0u, target, vmax, inv_t);
      if (s.res_fail) { if (tid == 0) redo[atomicAdd(n_redo, 1)] = row; return; }
      const double eps = 1e-12 * total;
      if (fabs(s.res_cum_m - target) <= eps) status |= LM_STATUS_TOPP_EDGE;
      if (!have_tau || static_cast<double>(s.res_tau) > tau64) tau64 = s.res_tau;
      have_tau = true;
      __syncthreads();
    } else if (fabs(above_k_mass - target) <= 1e-12 * total) status |= LM_STATUS_TOPP_EDGE;
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
  LM_PHASE(6);

  // ---- pass 2: the draw over the kept set (the row is in L2) ---------------------------------------------------------
  int token;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    token = draw_inverse_cdf_bidir(rv, s, side, tau, vmax, T, P.uniforms ? P.uniforms[row] : 0.0f);
  } else {
    bool tie = false;
    token = draw_gumbel<true>(rv, tau, T, P.seed, P.step, static_cast<uint32_t>(P.row_offset + row), s.draw, &tie, side);
    if (tie) status |= LM_STATUS_NEAR_TIE;
  }
  LM_PHASE(7);
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
  }
}

}  // namespace lm
