// Vocab-parallel sampling: the vocabulary of every row is split into contiguous shards, one per GPU. No counterpart
// in the reference (which is single-device); the result is defined as the single-GPU sampler's result on the whole
// row, bit for bit.
//
//   local step          (each GPU, its shard): per row the shard's maximum, its FP64 softmass relative to that maximum, and every
//                       logit at or above (a lower bound of) the shard's own k-th largest value, with global indices -> a
//                       fixed-size record per row. vocab_local_kernel: one block and one record per row, any top_k; for a top_k
//                       up to 64 the shard is cut into pieces, one block and one record per piece (slice_local_kernel,
//                       sample_sliced.cuh), so that the step spreads over the GPU;
//   [one all-gather of the records, done by the host layer over NCCL]
//   vocab_merge_kernel  (every GPU, identically): takes the candidates of all records (every piece of every GPU a shard), puts
//                       those at or above the row's top-k bound in order, rebuilds the global maximum and mass, finds
//                       tau_k / tau_p / tau_m exactly as the single-GPU walk does, and draws.
//
// Every logit at or above the global k-th largest value is a candidate of its shard (a shard holds fewer than k logits
// above that value, so its own k-th largest lies at or below it), which is why the merge sees the complete top-k set.
#pragma once
#include "common.cuh"
#include "sample_generic.cuh"

namespace lm {

constexpr int kVpHeader = 32;          // float vmax, float pad, double mass, int32 n, uint32 status, 8 bytes pad
constexpr int kVpMaxCandidates = 1024; // candidates of one row that can reach the sort (those at or above the row's top-k bound); the merge's threads
constexpr int kVpMergeCap = 8192;      // candidates of one row that the merge takes in, all shards together
constexpr int kVpPerThread = kVpMergeCap / kVpMaxCandidates;   // ... of which every thread of the merge holds so many
constexpr int kSelectBins = 2048;
constexpr uint32_t kStatusOverflow = 32u;
constexpr int kVpMaxShards = 64;       // shards (or slices) of one row

struct VpLocalDev {
  const void* logits; int dtype; int rows; int vocab_local; int64_t row_stride; int shard_start;
  const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  int cap; unsigned char* records; int64_t record_bytes;
};

__global__ void __launch_bounds__(kBlock, 1) vocab_local_kernel(VpLocalDev P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  GenericSmem& s = *reinterpret_cast<GenericSmem*>(smem_raw);
  __shared__ uint32_t s_n, s_ninf;
  const int tid = threadIdx.x;
  for (int row = blockIdx.x; row < P.rows; row += gridDim.x) {
    const int V = P.vocab_local;
    const float T = P.temperature ? P.temperature[row] : P.temperature_s;
    int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
    unsigned char* rec = P.records + static_cast<int64_t>(row) * P.record_bytes;
    float* out_val = reinterpret_cast<float*>(rec + kVpHeader);
    int32_t* out_idx = reinterpret_cast<int32_t*>(rec + kVpHeader + 4 * static_cast<size_t>(P.cap));
    RowView rv;
    rv.dtype = P.dtype; rv.vocab = V; rv.rho = 1.0f; rv.pi = 0.0f; rv.pen = nullptr;
    rv.row = static_cast<const char*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride) * (P.dtype == LM_DTYPE_BF16 ? 2 : 4);
    rv.aligned = (reinterpret_cast<uintptr_t>(rv.row) & 15u) == 0;
    const int n_chunks = (V + kChunk - 1) / kChunk;
    if (tid == 0) { s_n = 0u; s_ninf = 0xFFFFFFFFu; }
    // the shard's maximum
    uint64_t best = 0ull;
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if (e < n) { const uint64_t p = pack_best(z[e], static_cast<uint32_t>(c * kChunk + e)); best = p > best ? p : best; }
    }
    best = block_max_u64(best, s.scratch);
    const float vmax = best_value(best);
    // its FP64 softmass relative to that maximum
    const double inv_t = 1.0 / static_cast<double>(T);
    double m = 0.0;
    if (vmax > -INFINITY) {                                                // (a shard of nothing but -inf has no mass)
      for (int c = tid; c < n_chunks; c += kBlock) {
        float z[kChunk];
        const int n = load_chunk(rv, c, z);
#pragma unroll
        for (int e = 0; e < kChunk; e++) if (e < n) m += softmass(z[e], vmax, inv_t);
      }
    }
    const double mass = block_sum_f64(m, s.scratch);
    // its k-th largest value: 4 x 8-bit radix select on the monotone key, ties kept
    if (top_k > V) top_k = V;
    if (top_k < 1) top_k = 1;
    if (tid == 0) { s.sel_base_c = 0; s.sel_base_m = 0.0; }
    __syncthreads();
    uint32_t prefix = 0u;
    for (int level = 0; level < 4; level++) {
      hist_pass<false>(rv, level, prefix, vmax, inv_t, s);
      prefix |= static_cast<uint32_t>(select_bin<false>(s.cnt, nullptr, static_cast<uint32_t>(top_k), 0.0, s)) << (24 - 8 * level);
    }
    const float tau_local = fkey_inv(prefix);
    // every logit at or above it, with its global index. A shard with fewer than top_k logits above -inf (a masked vocabulary)
    // hands over those and ONE -inf logit (its first), which stands for the rest: they weigh nothing, and a row with fewer than
    // top_k logits above -inf still finds its k-th largest at -inf.
    const bool open = !(tau_local > -INFINITY);
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if (e < n) {
        if (open ? z[e] > -INFINITY : z[e] >= tau_local) {
          const uint32_t slot = atomicAdd(&s_n, 1u);
          if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = z[e]; out_idx[slot] = P.shard_start + c * kChunk + e; }
        } else if (open && z[e] == -INFINITY) atomicMin(&s_ninf, static_cast<uint32_t>(c * kChunk + e));
      }
    }
    __syncthreads();
    if (open && tid == 0 && s_ninf != 0xFFFFFFFFu) {
      const uint32_t slot = s_n++;
      if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = -INFINITY; out_idx[slot] = P.shard_start + static_cast<int>(s_ninf); }
    }
    __syncthreads();
    if (tid == 0) {
      const uint32_t n = s_n;
      *reinterpret_cast<float*>(rec) = vmax;
      *reinterpret_cast<float*>(rec + 4) = 0.0f;
      *reinterpret_cast<double*>(rec + 8) = mass;
      *reinterpret_cast<int32_t*>(rec + 16) = static_cast<int32_t>(n < static_cast<uint32_t>(P.cap) ? n : static_cast<uint32_t>(P.cap));
      *reinterpret_cast<uint32_t*>(rec + 20) = (n > static_cast<uint32_t>(P.cap) ? kStatusOverflow : 0u) | ((vmax != vmax) ? LM_STATUS_NAN : 0u);
    }
    __syncthreads();
  }
}

// A lower bound (as a monotone key) of the k-th largest of the keys the block's threads hold in registers (keys[i] == 0: none; at
// least k of them are set), all of them within [lo_key, hi_key]: the 2048 bins divide that span, so one level usually separates the
// keys well. Returns the bound after one level if at most `limit` keys lie at or above it, else the bound after a second level
// inside the k-th key's bin.
// B threads, all of them call; bins: kSelectBins words, scratch: 32 words, pick: 3 words of shared memory.
template <int B, int PER>
__device__ uint32_t kth_key_bound_in_span(const uint32_t (&keys)[PER], uint32_t k, uint32_t lo_key, uint32_t hi_key, uint32_t limit,
                                          uint32_t* bins, uint64_t* scratch, uint32_t* pick) {
  const int tid = threadIdx.x;
  const uint32_t span = hi_key - lo_key;
  int shift = span ? max(0, 32 - __clz(span) - 11) : 0;
  uint32_t base = lo_key, above = 0u, width = 0u;                         // width: keys under consideration lie in [base, base + width); 0: all
#pragma unroll 1
  for (int level = 0; level < 2; level++) {
    for (int i = tid; i < kSelectBins; i += B) bins[i] = 0u;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < PER; i++) {
      const uint32_t key = keys[i];
      if (key && key >= base) {
        const uint32_t d = key - base;
        if (width == 0u || d < width) atomicAdd(&bins[min(d >> shift, static_cast<uint32_t>(kSelectBins - 1))], 1u);
      }
    }
    __syncthreads();
    constexpr int kPer = kSelectBins / B;                  // thread t owns kPer bins, walked downwards from the top
    uint32_t cnt[kPer]; uint64_t sum = 0ull;
#pragma unroll
    for (int j = 0; j < kPer; j++) { cnt[j] = bins[kSelectBins - 1 - (kPer * tid + j)]; sum += cnt[j]; }
    const uint64_t excl = block_exclusive_scan_u64(sum, scratch, nullptr);
    uint32_t run = above + static_cast<uint32_t>(excl);
    if (run < k && run + static_cast<uint32_t>(sum) >= k) {
#pragma unroll
      for (int j = 0; j < kPer; j++) {
        if (run < k && run + cnt[j] >= k) { pick[0] = static_cast<uint32_t>(kSelectBins - 1 - (kPer * tid + j)); pick[1] = run; pick[2] = run + cnt[j]; }
        run += cnt[j];
      }
    }
    __syncthreads();
    base += pick[0] << shift; above = pick[1];
    const uint32_t at_or_above = pick[2];
    __syncthreads();
    if (at_or_above <= limit || shift == 0) break;
    width = 1u << shift; shift = max(0, shift - 11);
  }
  return base;
}

struct VpMergeDev {
  const unsigned char* records;      // [shards][rows] records, as the all-gather leaves them; or, with `bases`, unused
  const unsigned long long* bases;   // per GPU, the address of its [pieces][rows] records (its own memory or a peer's, read in place); or null
  int pieces;                        // with `bases`: records per row and GPU (shard s of the merge = piece s % pieces of GPU s / pieces)
  int shards; int rows; int cap; int64_t record_bytes;
  const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  const float* top_p; float top_p_s; const float* min_p; float min_p_s;
  uint32_t flags; int draw; const float* uniforms; uint64_t seed; uint32_t step; int64_t row_offset;
  int32_t* out_tokens; float* out_tau; uint32_t* out_status; float* out_vmax; unsigned long long* out_mass;
  uint32_t path_status;              // ORed into every row's status (0 in the vocab-parallel mode)
  int hand_on;                       // single-GPU use (sample_sliced.cuh): a row whose records overflowed is left to the caller
  double inv_t_s;                    // 1 / temperature_s in FP64 (the host's division: one per call instead of one per thread)
  int per, per_log2;                 // kVpMaxCandidates / shards, and its base-2 logarithm if it is a power of two (else -1)
  double mass_band;                  // how far (relative) the records' masses may be from the exact ones (0: they are FP64 sums); with hand_on only
};

struct VpMergeSmem {
  unsigned long long key[kVpMaxCandidates];   // (monotone value key << 32) | ~global index: descending = value desc, index asc
  double cum[kVpMaxCandidates];
  unsigned long long w[kVpMaxCandidates];      // the candidates as they arrive (before the sort); later their fixed-point weights
  uint64_t scratch[32];
  double warp_m[32];
  int n_total; int hit; int token; uint32_t status;
  uint32_t n_sel; uint32_t pick[3]; uint32_t lo_key, hi_key; int amb;
  double h_w[kVpMaxShards]; double z_total; float vmax;
};

// The thresholds and the draw of a row with at most 64 ordered candidates (the usual case for a top_k up to ~60): warp 0 alone, lane
// i holding candidate i (E = 1: up to 32) or candidates i and 32 + i (E = 2), with shuffles and votes where the block-wide code below needs barriers. The same arithmetic in
// the same order (the block-wide prefix sums reduce to those of warps 0 and 1). Sets s.amb instead of writing when the row has to be
// handed on.
// Where the record of (shard, row) lies: in the gathered array, or in place in the memory of the GPU that wrote it.
__device__ __forceinline__ const unsigned char* merge_record(const VpMergeDev& P, int shard, int row) {
  if (P.bases) {
    const int gpu = shard / P.pieces, piece = shard - gpu * P.pieces;
    return reinterpret_cast<const unsigned char*>(P.bases[gpu]) + (static_cast<int64_t>(piece) * P.rows + row) * P.record_bytes;
  }
  return P.records + (static_cast<int64_t>(shard) * P.rows + row) * P.record_bytes;
}

template <int E>
__device__ void merge_tail_one_warp(const VpMergeDev& P, int row, VpMergeSmem& s, int N, float T, int top_k, float top_p, float min_p, double inv_t,
                                    uint32_t status0) {
  const int lane = threadIdx.x & 31;
  unsigned long long key[E]; bool valid[E]; float val[E]; int idx[E]; uint32_t hi[E];
#pragma unroll
  for (int e = 0; e < E; e++) {
    key[e] = s.key[lane + 32 * e];
    valid[e] = lane + 32 * e < N;
    hi[e] = static_cast<uint32_t>(key[e] >> 32);
    val[e] = valid[e] ? fkey_inv(hi[e]) : -INFINITY;
    idx[e] = valid[e] ? static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(key[e])) : -1;
  }
  // the value at position i of the order (every lane asks for the same i)
  auto at_f = [&](const float (&v)[E], int i) { const float a = __shfl_sync(kFull, v[0], i & 31), b = __shfl_sync(kFull, v[E - 1], i & 31); return i < 32 ? a : b; };
  auto at_d = [&](const double (&v)[E], int i) { const double a = __shfl_sync(kFull, v[0], i & 31), b = __shfl_sync(kFull, v[E - 1], i & 31); return i < 32 ? a : b; };
  auto at_i = [&](const int (&v)[E], int i) { const int a = __shfl_sync(kFull, v[0], i & 31), b = __shfl_sync(kFull, v[E - 1], i & 31); return i < 32 ? a : b; };
  // position of the first candidate for which `f` holds (-1: none)
  auto first_of = [&](const bool (&f)[E]) { const uint32_t m0 = __ballot_sync(kFull, f[0]), m1 = E > 1 ? __ballot_sync(kFull, f[E - 1]) : 0u; return m0 ? __ffs(static_cast<int>(m0)) - 1 : (m1 ? 31 + __ffs(static_cast<int>(m1)) : -1); };
  const float vmax = s.vmax;
  const double T64 = static_cast<double>(T);
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  double tau64 = -INFINITY; bool have_tau = false;
  float tau_k = -INFINITY;
  uint32_t edge = 0u;
  if (has_k) {
    tau_k = at_f(val, (top_k < N ? top_k : N) - 1);
    tau64 = tau_k; have_tau = true;
  }
  if (has_p) {
    double mi[E];
#pragma unroll
    for (int e = 0; e < E; e++) {
      mi[e] = valid[e] ? softmass(val[e], vmax, inv_t) : 0.0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const double t = __shfl_up_sync(kFull, mi[e], o); if (lane >= o) mi[e] += t; }
    }
    if (E > 1) mi[E - 1] += __shfl_sync(kFull, mi[0], 31);
    const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k;
    double total = s.z_total;
    if (in_topk) {                                                        // the top-k set is a prefix of the order
      int n_topk = 0;
#pragma unroll
      for (int e = 0; e < E; e++) n_topk += __popc(__ballot_sync(kFull, valid[e] && val[e] >= tau_k));
      total = at_d(mi, n_topk - 1);
    }
    const double target = static_cast<double>(top_p) * total;
    bool run_end[E], reached[E];
#pragma unroll
    for (int e = 0; e < E; e++) {                                         // the candidate after this one: the next lane's, or the first of the second set
      const uint32_t down = __shfl_down_sync(kFull, hi[e], 1), wrap = __shfl_sync(kFull, hi[E - 1], 0);
      const bool last = lane + 32 * e == N - 1 || (lane == 31 && e == E - 1);
      run_end[e] = valid[e] && (last || (lane == 31 ? wrap : down) != hi[e]);
      reached[e] = run_end[e] && mi[e] >= target;
    }
    const int hit = first_of(reached);
    bool amb = false;
#pragma unroll
    for (int e = 0; e < E; e++)
      amb |= P.hand_on && P.mass_band > 0.0 && !in_topk && run_end[e] && val[e] > tau_k && fabs(mi[e] - target) <= P.mass_band * total;
    if (__any_sync(kFull, amb)) { if (lane == 0) s.amb = 1; return; }
    if (hit >= 0) {
      const float tau_p = at_f(val, hit);
      if (!have_tau || static_cast<double>(tau_p) > tau64) tau64 = tau_p;
      have_tau = true;
    }
    bool near = false;
#pragma unroll
    for (int e = 0; e < E; e++) near |= run_end[e] && fabs(mi[e] - target) <= 1e-12 * total;
    if (__any_sync(kFull, near)) edge = LM_STATUS_TOPP_EDGE;
  }
  if (has_m) {
    const double tau_m = static_cast<double>(vmax) + T64 * log(static_cast<double>(min_p));
    if (!have_tau || tau_m > tau64) tau64 = tau_m;
    have_tau = true;
  }
  const float tau = have_tau ? __double2float_rn(tau64) : -INFINITY;
  bool kept[E];
#pragma unroll
  for (int e = 0; e < E; e++) kept[e] = valid[e] && val[e] >= tau;
  uint32_t status = status0 | edge | P.path_status;
  uint64_t kept_weight = 0ull;
  int token = -1;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    const float c2 = exp2_scale(T);
    uint64_t w[E], incl[E];
#pragma unroll
    for (int e = 0; e < E; e++) {
      w[e] = kept[e] ? weight_q40(val[e], vmax, c2) : 0ull;
      incl[e] = w[e];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const uint64_t t = __shfl_up_sync(kFull, incl[e], o); if (lane >= o) incl[e] += t; }
    }
    if (E > 1) incl[E - 1] += __shfl_sync(kFull, incl[0], 31);
    const uint64_t total = __shfl_sync(kFull, incl[E - 1], 31);
    kept_weight = total;
    const uint64_t target = cdf_target(P.uniforms ? P.uniforms[row] : 0.0f, total);
    bool mine[E];
#pragma unroll
    for (int e = 0; e < E; e++) { const uint64_t before = incl[e] - w[e]; mine[e] = total > 0ull && w[e] && before <= target && target < before + w[e]; }
    const int who = first_of(mine);
    if (who >= 0) token = at_i(idx, who);
  } else {
    const float inv_t32 = __double2float_rn(1.0 / T64);
    uint64_t mine[E], top = 0ull; float kf[E];
#pragma unroll
    for (int e = 0; e < E; e++) { mine[e] = 0ull; kf[e] = -INFINITY; }
#pragma unroll
    for (int e = 0; e < E; e++) if (kept[e]) {
      kf[e] = __fadd_rn(__fmul_rn(val[e], inv_t32), gumbel(P.seed, P.step, static_cast<uint32_t>(P.row_offset + row), static_cast<uint32_t>(idx[e])));
      mine[e] = pack_best(kf[e], static_cast<uint32_t>(idx[e]));
      top = mine[e] > top ? mine[e] : top;
    }
    const uint64_t win = warp_max_u64(top);
    if (win) {
      const float edge_kf = best_value(win) - 4e-6f;
      bool tie = false;
#pragma unroll
      for (int e = 0; e < E; e++) tie |= kept[e] && mine[e] != win && kf[e] >= edge_kf;
      if (__any_sync(kFull, tie)) status |= LM_STATUS_NEAR_TIE;
      token = static_cast<int>(best_index(win));
    }
    if (P.out_mass) {
      const float c2 = exp2_scale(T);
      uint64_t ws = 0ull;
#pragma unroll
      for (int e = 0; e < E; e++) ws += kept[e] ? weight_q40(val[e], vmax, c2) : 0ull;
      kept_weight = warp_sum_u64(ws);
    }
  }
  if (lane == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
    if (P.out_vmax) P.out_vmax[row] = vmax;
    if (P.out_mass) P.out_mass[row] = kept_weight;
  }
}

// One row of the merge. Every thread of the block (kVpMaxCandidates threads) calls with the same arguments; returns false when
// the row's records overflowed and the caller asked to hand such rows on (P.hand_on): nothing has been written then.
// The host has checked shards <= kVpMaxShards and cap <= kVpPerThread * (kVpMaxCandidates / shards).
__device__ bool vocab_merge_row(const VpMergeDev& P, int row, VpMergeSmem& s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const double T64 = static_cast<double>(T), inv_t = P.temperature ? 1.0 / T64 : P.inv_t_s;
  uint32_t edge = 0u;
  if (!(T > 0.0f)) {                                                     // a per-row temperature the host could not check: no token
    if (tid == 0) { P.out_tokens[row] = -1; if (P.out_tau) P.out_tau[row] = -INFINITY; if (P.out_status) P.out_status[row] = kStatusBadParam; }
    return true;
  }
  // ---- One round of loads. This thread's share of the candidates (a group of threads per shard, slot j of the record to thread
  // j mod group size), asked for before the shard's header says how many slots are filled (every slot of a record is readable);
  // meanwhile warp 0 adds up the shards' counts and warp 1 rebuilds the row's maximum and softmass from the shards' (the masses
  // rescaled to the common maximum and summed in shard order, by one thread).
  if (tid == 0) { s.hit = kVpMaxCandidates; s.token = -1; s.status = 0u; s.n_sel = 0u; s.lo_key = 0xFFFFFFFFu; s.hi_key = 0u; s.amb = 0; }
  const int per = P.per;
  const int g = P.per_log2 >= 0 ? tid >> P.per_log2 : tid / per, r = tid - g * per;
  float pv[kVpPerThread]; int32_t pi[kVpPerThread];
#pragma unroll
  for (int i = 0; i < kVpPerThread; i++) { pv[i] = 0.0f; pi[i] = 0; }
  int cnt = 0;
  if (g < P.shards) {
    const unsigned char* rec = merge_record(P, g, row);
    const float* rv = reinterpret_cast<const float*>(rec + kVpHeader);
    const int32_t* ri = reinterpret_cast<const int32_t*>(rec + kVpHeader + 4 * static_cast<size_t>(P.cap));
    cnt = *reinterpret_cast<const int32_t*>(rec + 16);
#pragma unroll
    for (int i = 0; i < kVpPerThread; i++) {
      const int j = r + i * per;
      if (j < P.cap) { pv[i] = rv[j]; pi[i] = ri[j]; }
    }
  }
  __syncthreads();                                                        // (the shared fields above are set)
  if (warp == 0) {
    int n2 = 0; uint32_t st = 0u;
    for (int q = lane; q < P.shards; q += 32) {
      const unsigned char* rec = merge_record(P, q, row);
      n2 += *reinterpret_cast<const int32_t*>(rec + 16);
      st |= *reinterpret_cast<const uint32_t*>(rec + 20);
    }
    const int total = static_cast<int>(warp_sum_u32(static_cast<uint32_t>(n2)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) st |= __shfl_xor_sync(kFull, st, o);
    if (lane == 0) { s.n_total = total; if (st) atomicOr(&s.status, st); }
  } else if (warp == 1) {
    float hv[2]; double hm[2];
    float m = -INFINITY;
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int q = lane + 32 * e;
      hv[e] = -INFINITY; hm[e] = 0.0;
      if (q < P.shards) {
        const unsigned char* rec = merge_record(P, q, row);
        hv[e] = *reinterpret_cast<const float*>(rec); hm[e] = *reinterpret_cast<const double*>(rec + 8);
      }
      m = fmaxf(m, hv[e]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFull, m, o));
#pragma unroll
    for (int e = 0; e < 2; e++)
      if (lane + 32 * e < P.shards) s.h_w[lane + 32 * e] = hm[e] * exp((static_cast<double>(hv[e]) - static_cast<double>(m)) * inv_t);
    __syncwarp();
    if (lane == 0) {
      double z = 0.0;
      for (int q = 0; q < P.shards; q++) z += s.h_w[q];
      s.z_total = z; s.vmax = m;
    }
  }
  // ---- keys of the filled slots and their span
  uint32_t keys[kVpPerThread];
  {
    uint32_t kmin = 0xFFFFFFFFu, kmax = 0u;
#pragma unroll
    for (int i = 0; i < kVpPerThread; i++) {
      const bool have = r + i * per < cnt;
      keys[i] = have ? fkey(pv[i]) : 0u;
      if (have) { kmin = min(kmin, keys[i]); kmax = max(kmax, keys[i]); }
    }
    kmin = warp_min_u32(kmin); kmax = warp_max_u32(kmax);
    if (lane == 0 && kmax) { atomicMin(&s.lo_key, kmin); atomicMax(&s.hi_key, kmax); }
  }
  __syncthreads();
  const int n_all = s.n_total;
  // A NaN in the row or a maximum that is not finite: the generic row algorithm defines what happens (single GPU); not supported
  // across GPUs, where such a row reports LM_STATUS_NAN and token -1.
  if ((s.status & LM_STATUS_NAN) || !(fabsf(s.vmax) < INFINITY)) {
    if (P.hand_on) return false;
    if (tid == 0) { P.out_tokens[row] = -1; if (P.out_tau) P.out_tau[row] = -INFINITY; if (P.out_status) P.out_status[row] = s.status | LM_STATUS_NAN; }
    __syncthreads();
    return true;
  }
  // ---- the candidates that can matter: those at or above a lower bound of the row's top_k-th largest value (the k-th largest of
  // the candidates is the k-th largest of the row); only they are put in order
  uint32_t bound = 0u;
  if (top_k >= 1 && n_all > top_k)
    bound = kth_key_bound_in_span<kVpMaxCandidates, kVpPerThread>(keys, static_cast<uint32_t>(top_k), s.lo_key, s.hi_key, static_cast<uint32_t>(max(2 * top_k, 128)),
                                  reinterpret_cast<uint32_t*>(s.cum), s.scratch, s.pick);
#pragma unroll
  for (int i = 0; i < kVpPerThread; i++) {
    if (keys[i] && keys[i] >= bound) {
      const uint32_t slot = atomicAdd(&s.n_sel, 1u);
      if (slot < static_cast<uint32_t>(kVpMaxCandidates)) s.w[slot] = (static_cast<unsigned long long>(keys[i]) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(pi[i]));
    }
  }
  __syncthreads();
  const uint32_t n_sel = s.n_sel;
  // ---- descending order by rank: the keys are distinct (they hold the index), so the number of larger keys is the position
  unsigned long long key = 0ull;
  if (n_sel <= static_cast<uint32_t>(kVpMaxCandidates)) {
    const int m = static_cast<int>(n_sel);
    int rank = 0;
    if (tid < m) {
      key = s.w[tid];
      for (int t = 0; t < m; t++) rank += (s.w[t] > key) ? 1 : 0;
      s.key[rank] = key;
    } else s.key[tid] = 0ull;
  } else if (tid == 0) s.status |= kStatusOverflow;                        // more ties at the bound than the sort holds
  __syncthreads();
  const int N = static_cast<int>(n_sel < static_cast<uint32_t>(kVpMaxCandidates) ? n_sel : static_cast<uint32_t>(kVpMaxCandidates));
  const uint32_t status0 = s.status;
  if ((status0 & kStatusOverflow) && P.hand_on) return false;             // single GPU: the caller gives the row to the generic path
  if ((status0 & kStatusOverflow) || N == 0) {
    if (tid == 0) { P.out_tokens[row] = -1; if (P.out_tau) P.out_tau[row] = -INFINITY; if (P.out_status) P.out_status[row] = status0; }
    __syncthreads();
    return true;
  }
  if (N <= 64) {                                                          // few candidates in order: one warp does the rest, no more barriers but the last
    if (warp == 0) { if (N <= 32) merge_tail_one_warp<1>(P, row, s, N, T, top_k, top_p, min_p, inv_t, status0); else merge_tail_one_warp<2>(P, row, s, N, T, top_k, top_p, min_p, inv_t, status0); }
    __syncthreads();
    return s.amb == 0;
  }
  key = s.key[tid];
  const bool valid = tid < N;
  const float val = valid ? fkey_inv(static_cast<uint32_t>(key >> 32)) : -INFINITY;
  const int idx = valid ? static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(key)) : -1;
  const float vmax = s.vmax;
  const double z_total = s.z_total;
  // ---- thresholds
  const bool has_k = top_k > 0, has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  double tau64 = -INFINITY; bool have_tau = false;
  float tau_k = -INFINITY;
  if (has_k) {
    const int kk = (top_k < N ? top_k : N) - 1;
    tau_k = fkey_inv(static_cast<uint32_t>(s.key[kk] >> 32));
    tau64 = tau_k; have_tau = true;
  }
  if (has_p) {
    // inclusive FP64 prefix of the softmass in sorted order
    double m = valid ? softmass(val, vmax, inv_t) : 0.0, mi = m;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const double t = __shfl_up_sync(kFull, mi, o); if (lane >= o) mi += t; }
    if (lane == 31) s.warp_m[warp] = mi;
    __syncthreads();
    double wm = 0.0;
    for (int w = 0; w < warp; w++) wm += s.warp_m[w];
    mi += wm;
    s.cum[tid] = mi;
    __syncthreads();
    double total = z_total;
    if ((P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k) {                     // mass of the top-k set: prefix at the last candidate >= tau_k
      int last = 0;
      for (int t = 0; t < N; t++) if (fkey_inv(static_cast<uint32_t>(s.key[t] >> 32)) >= tau_k) last = t; else break;
      total = s.cum[last];
    }
    const double target = static_cast<double>(top_p) * total;
    const bool run_end = valid && (tid == N - 1 || (s.key[tid + 1] >> 32) != (key >> 32));
    if (run_end && mi >= target) atomicMin(&s.hit, tid);
    // approximate masses: a boundary above the top-k threshold that lies within the band of the target is not decided here
    const bool amb = P.hand_on && P.mass_band > 0.0 && !((P.flags & LM_FLAG_TOPP_IN_TOPK) && has_k) && run_end && val > tau_k &&
                     fabs(mi - target) <= P.mass_band * total;
    if (__syncthreads_or(amb)) return false;
    if (s.hit < kVpMaxCandidates) {
      const float tau_p = fkey_inv(static_cast<uint32_t>(s.key[s.hit] >> 32));
      if (!have_tau || static_cast<double>(tau_p) > tau64) tau64 = tau_p;
      have_tau = true;
    }
    // The masses are summed here in another order than on one GPU (per shard, then over the sorted candidates): a boundary of the
    // cumulative mass within 1e-12 of the target, on either side, may be decided differently and is reported like there.
    const bool near = run_end && fabs(mi - target) <= 1e-12 * total;
    if (__syncthreads_or(near)) edge = LM_STATUS_TOPP_EDGE;
  }
  if (has_m) {
    const double tau_m = static_cast<double>(vmax) + T64 * log(static_cast<double>(min_p));
    if (!have_tau || tau_m > tau64) tau64 = tau_m;
    have_tau = true;
  }
  const float tau = have_tau ? __double2float_rn(tau64) : -INFINITY;
  const bool kept = valid && val >= tau;
  uint32_t status = status0 | edge | P.path_status;
  // ---- the draw
  uint64_t kept_weight = 0ull;
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    // the kept candidates are already in the draw's order (descending logit, equal logits by ascending index): one prefix sum
    const float c2 = exp2_scale(T);
    const uint64_t w = kept ? weight_q40(val, vmax, c2) : 0ull;
    uint64_t total = 0ull;
    const uint64_t before = block_exclusive_scan_u64(w, s.scratch, &total);
    kept_weight = total;
    if (total > 0ull && w) {
      const uint64_t target = cdf_target(P.uniforms ? P.uniforms[row] : 0.0f, total);
      if (before <= target && target < before + w) s.token = idx;
    }
  } else {
    const float inv_t32 = __double2float_rn(1.0 / T64);
    uint64_t mine = 0ull; float kf = -INFINITY;
    if (kept) {
      kf = __fadd_rn(__fmul_rn(val, inv_t32), gumbel(P.seed, P.step, static_cast<uint32_t>(P.row_offset + row), static_cast<uint32_t>(idx)));
      mine = pack_best(kf, static_cast<uint32_t>(idx));
    }
    const uint64_t win = block_max_u64(mine, s.scratch);
    if (win) {
      if (__syncthreads_or(kept && mine != win && kf >= best_value(win) - 4e-6f)) status |= LM_STATUS_NEAR_TIE;
      if (tid == 0) s.token = static_cast<int>(best_index(win));
    }
    if (P.out_mass) kept_weight = block_sum_u64(kept ? weight_q40(val, vmax, exp2_scale(T)) : 0ull, s.scratch);
  }
  __syncthreads();
  if (tid == 0) {
    P.out_tokens[row] = s.token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
    if (P.out_vmax) P.out_vmax[row] = vmax;
    if (P.out_mass) P.out_mass[row] = kept_weight;
  }
  __syncthreads();
  return true;
}

__global__ void __launch_bounds__(kVpMaxCandidates, 1) vocab_merge_kernel(VpMergeDev P) {
  __shared__ VpMergeSmem s;
  for (int row = blockIdx.x; row < P.rows; row += gridDim.x) vocab_merge_row(P, row, s);
}

}  // namespace lm
