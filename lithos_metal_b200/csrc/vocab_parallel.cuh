// Vocab-parallel sampling: the vocabulary of every row is split into contiguous shards, one per GPU. No counterpart
// in the reference (which is single-device); the result is defined as the single-GPU sampler's result on the whole
// row, bit for bit.
//
//   vocab_local_kernel  (each GPU, its shard): per row the shard's maximum, its FP64 softmass relative to that
//                       maximum, and every logit at or above the shard's own k-th largest value (ties kept), with
//                       global indices -> one fixed-size record per row;
//   [one all-gather of the records, done by the host layer over NCCL]
//   vocab_merge_kernel  (every GPU, identically): sorts the gathered candidates, rebuilds the global maximum and
//                       mass, finds tau_k / tau_p / tau_m exactly as the single-GPU walk does, and draws.
//
// Every logit at or above the global k-th largest value is a candidate of its shard (a shard holds fewer than k logits
// above that value, so its own k-th largest lies at or below it), which is why the merge sees the complete top-k set.
#pragma once
#include "common.cuh"
#include "sample_generic.cuh"

namespace lm {

constexpr int kVpHeader = 32;          // float vmax, float pad, double mass, int32 n, uint32 status, 8 bytes pad
constexpr int kVpMaxCandidates = 1024; // all shards together, per row
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
  __shared__ uint32_t s_n;
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
    if (tid == 0) s_n = 0u;
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
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if (e < n) m += softmass(z[e], vmax, inv_t);
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
    // every logit at or above it, with its global index
    for (int c = tid; c < n_chunks; c += kBlock) {
      float z[kChunk];
      const int n = load_chunk(rv, c, z);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if (e < n && z[e] >= tau_local) {
        const uint32_t slot = atomicAdd(&s_n, 1u);
        if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = z[e]; out_idx[slot] = P.shard_start + c * kChunk + e; }
      }
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

struct VpMergeDev {
  const unsigned char* records;      // [shards][rows] records, as the all-gather leaves them
  int shards; int rows; int cap; int64_t record_bytes;
  const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  const float* top_p; float top_p_s; const float* min_p; float min_p_s;
  uint32_t flags; int draw; const float* uniforms; uint64_t seed; uint32_t step; int64_t row_offset;
  int32_t* out_tokens; float* out_tau; uint32_t* out_status; float* out_vmax; unsigned long long* out_mass;
  uint32_t path_status;              // ORed into every row's status (0 in the vocab-parallel mode)
  int hand_on;                       // single-GPU use (sample_sliced.cuh): a row whose records overflowed is left to the caller
};

struct VpMergeSmem {
  unsigned long long key[kVpMaxCandidates];   // (monotone value key << 32) | ~global index: descending = value desc, index asc
  double cum[kVpMaxCandidates];
  unsigned long long w[kVpMaxCandidates];      // the candidates as they arrive (before the sort); later their fixed-point weights
  uint64_t scratch[32];
  double warp_m[32];
  // the record headers of the row, one per shard (at most kVpMaxCandidates / cap of them: cap >= 1)
  float h_vmax[kVpMaxShards]; double h_mass[kVpMaxShards]; int h_n[kVpMaxShards]; int h_base[kVpMaxShards];
  int n_total; int hit; int token; uint32_t status;
};

// One row of the merge. Every thread of the block (kVpMaxCandidates threads) calls with the same arguments; returns false when
// the row's records overflowed and the caller asked to hand such rows on (P.hand_on): nothing has been written then.
__device__ bool vocab_merge_row(const VpMergeDev& P, int row, VpMergeSmem& s) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  uint32_t edge = 0u;
  if (!(T > 0.0f)) {                                                     // a per-row temperature the host could not check: no token
    if (tid == 0) { P.out_tokens[row] = -1; if (P.out_tau) P.out_tau[row] = -INFINITY; if (P.out_status) P.out_status[row] = kStatusBadParam; }
    return true;
  }
  // ---- the record headers, all at once (one thread per shard), then the offsets of the shards in the concatenation
  if (tid == 0) { s.hit = kVpMaxCandidates; s.token = -1; s.status = 0u; }
  __syncthreads();
  if (tid < P.shards) {
    const unsigned char* rec = P.records + (static_cast<int64_t>(tid) * P.rows + row) * P.record_bytes;
    s.h_vmax[tid] = *reinterpret_cast<const float*>(rec);
    s.h_mass[tid] = *reinterpret_cast<const double*>(rec + 8);
    s.h_n[tid] = *reinterpret_cast<const int32_t*>(rec + 16);
    const uint32_t st = *reinterpret_cast<const uint32_t*>(rec + 20);
    if (st) atomicOr(&s.status, st);
  }
  __syncthreads();
  if (warp == 0) {                                                       // exclusive prefix of the counts over the shards (at most 64)
    const int a = lane < P.shards ? s.h_n[lane] : 0, b = lane + 32 < P.shards ? s.h_n[lane + 32] : 0;
    int ia = a, ib = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int ta = __shfl_up_sync(kFull, ia, o), tb = __shfl_up_sync(kFull, ib, o); if (lane >= o) { ia += ta; ib += tb; } }
    const int first = __shfl_sync(kFull, ia, 31);
    if (lane < P.shards) s.h_base[lane] = ia - a;
    if (lane + 32 < P.shards) s.h_base[lane + 32] = first + ib - b;
    if (lane == 31) {
      const int total = first + ib;
      s.n_total = total < kVpMaxCandidates ? total : kVpMaxCandidates;
      if (total > kVpMaxCandidates) s.status |= kStatusOverflow;
    }
  }
  __syncthreads();
  // ---- gather: candidate t of the concatenated shards (one thread per candidate)
  unsigned long long key = 0ull;
  {
    int g = 0;
    for (int q = 1; q < P.shards; q++) g += (s.h_base[q] <= tid) ? 1 : 0;   // the last shard that starts at or before t (bases ascend)
    if (tid < s.n_total && tid - s.h_base[g] < s.h_n[g]) {
      const unsigned char* rec = P.records + (static_cast<int64_t>(g) * P.rows + row) * P.record_bytes;
      const int j = tid - s.h_base[g];
      const float v = reinterpret_cast<const float*>(rec + kVpHeader)[j];
      const int32_t i = reinterpret_cast<const int32_t*>(rec + kVpHeader + 4 * static_cast<size_t>(P.cap))[j];
      key = (static_cast<unsigned long long>(fkey(v)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(i));
    }
  }
  s.w[tid] = key;
  __syncthreads();
  // ---- descending order by rank: the keys are distinct (they hold the index), so the number of larger keys is the position
  {
    const int n_all = s.n_total;
    int rank = 0;
    if (tid < n_all) {
      for (int t = 0; t < n_all; t++) rank += (s.w[t] > key) ? 1 : 0;
      s.key[rank] = key;
    } else s.key[tid] = 0ull;
  }
  __syncthreads();
  const int N = s.n_total;
  const uint32_t status0 = s.status;
  if ((status0 & kStatusOverflow) && P.hand_on) return false;             // single GPU: the caller gives the row to the generic path
  if ((status0 & kStatusOverflow) || N == 0) {
    if (tid == 0) { P.out_tokens[row] = -1; if (P.out_tau) P.out_tau[row] = -INFINITY; if (P.out_status) P.out_status[row] = status0; }
    __syncthreads();
    return true;
  }
  key = s.key[tid];
  const bool valid = tid < N;
  const float val = valid ? fkey_inv(static_cast<uint32_t>(key >> 32)) : -INFINITY;
  const int idx = valid ? static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(key)) : -1;
  // ---- global maximum and mass (shards in order)
  float vmax = -INFINITY;
  for (int g = 0; g < P.shards; g++) vmax = fmaxf(vmax, s.h_vmax[g]);
  if (tid < P.shards) s.cum[tid] = s.h_mass[tid] * exp((static_cast<double>(s.h_vmax[tid]) - static_cast<double>(vmax)) * inv_t);
  __syncthreads();
  double z_total = 0.0;
  for (int g = 0; g < P.shards; g++) z_total += s.cum[g];                // (in shard order, whatever the number of threads)
  __syncthreads();
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
    __syncthreads();
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
