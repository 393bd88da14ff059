// A few rows on the whole GPU: every row is cut into slices, one thread block per slice.
//
// One block per row (the batch kernels) leaves a call of one or a handful of rows on as many SMs, and the row's latency is that of
// one block walking 150k logits several times. The decode step of a single stream is exactly that call (the reference's sampler
// dispatches run on T <= 8 rows per step, monolith/kernels.py:720-775). Here the slices of a row go to different SMs:
//
//   slice_local_kernel  (64 slices x rows blocks)  reads its slice ONCE into shared memory (BF16 or FP32, widened; the penalties of
//                       the history ids that fall into the slice applied), and leaves a record: the slice's maximum, its FP64
//                       softmass relative to that maximum, and every logit at or above a lower bound of the slice's own k-th
//                       largest (the k-th largest of the threads' own maxima, to 22 key bits);
//   sliced_merge_kernel (one block per row) the merge that joins the shards of the vocab-parallel mode (vocab_parallel.cuh):
//                       gathers the candidates of all slices, puts those at or above the row's top-k bound in order, rebuilds
//                       the row's maximum and mass, thresholds, draw.
//
// The record format is the vocab-parallel one, a slice standing for a shard. Rows with a top_k of 1 .. 64 only: a slice's record
// has room for twice the top_k (16 at least), so that only a slice with that many logits at or above its bound (ties at its own
// k-th value) overflows it; the merge's block then runs the generic row algorithm on such a row itself.
#pragma once
#include "common.cuh"
#include "sample_generic.cuh"
#include "sample_topk.cuh"
#include "vocab_parallel.cuh"

namespace lm {

constexpr int kSliceBlockBig = 1024;     // threads per slice when every slice has an SM to itself (latency), else kSliceBlockSmall
constexpr int kSliceBlockSmall = 256;   // ... and kSliceBlockTiny when the top_k leaves its record room (fewer warps: fewer instructions per slice)
constexpr int kSliceBlockTiny = 128;
constexpr int kSliceTinyMaxK = 50;        // largest top_k for kSliceBlockTiny: about 62 of a record's 100 slots filled then
constexpr int kSliceMaxLen = 32768;       // logits of one slice (128 KB of shared memory as binary32)
constexpr int kSlicedMaxRows = 32;        // rows per call on this path
constexpr int kSlicedMinVocab = 16384;
constexpr int kSlices = 64;               // slices per row
constexpr int kSliceMaxCap = 128;         // candidates in one slice's record: twice the largest top_k
constexpr size_t kSlicedWsBytes = static_cast<size_t>(kSlicedMaxRows) * kSlices * (kVpHeader + 8 * kSliceMaxCap);

struct SliceDev {
  const void* logits; int dtype; int rows; int vocab; int64_t row_stride;
  int slices; int slice_len;                          // slice_len: a multiple of 8 (the last slices of a row may be short or empty)
  float temperature; int top_k; int cap; int need_mass;
  const float* temperature_rows; const int32_t* top_k_rows;   // per-row values instead of the two scalars (vocab-parallel callers)
  int exact_mass;                                     // the softmass as an FP64 sum (where no exact path stands behind the merge)
  int index_base;                                     // added to every candidate's index (the shard's first logit)
  const int32_t* history; int hist_len; int64_t hist_stride; float rho, pi;
  unsigned char* records; int64_t record_bytes;       // [slices][rows] records
  const uint32_t* state; int t_max, g;                // optional StepState: rows beyond t_this_step, and a finished state, are left alone
};

// How far (relative) a slice's FP32 softmass can be from the exact one, first order, worst case, with a quarter added (u = 2^-24):
//   - c2a = fl32(c): term j is off by a factor 2^(x_j delta), |delta| <= u, x_j = (z_j - vmax) c <= 0; weighted by the terms that is
//     ln2 u E_w|x| <= u ln(slice_len) (E_w[-x ln2] = H - ln Z <= ln n: H the entropy of the slice's softmax, Z >= 1 relative to its maximum);
//   - the FMA rounds its result: half an ulp of |x| < 32 is at most 2^-20, a factor 1 + 6.6e-7 on the term (the terms with |x| >= 32
//     weigh less than n 2^-32 altogether);
//   - ex2.approx.ftz.f32: 2 ulp = 4 u;
//   - a thread adds ceil(slice_len / threads) terms one after the other in FP32, then the threads meet in FP64.
// The slices' masses are scaled to the row's maximum and added in FP64; the bound holds for the sum as for each of them.
inline double slice_mass_band(int slice_len, int threads) {
  const double u = 5.9604644775390625e-8;
  return 1.25 * (u * (log(static_cast<double>(slice_len)) + 4.0 + static_cast<double>((slice_len + threads - 1) / threads + 1)) + 6.6e-7);
}

__host__ __device__ inline size_t slice_marks_offset(int slice_len) { return static_cast<size_t>(slice_len) * 4; }
__host__ __device__ inline size_t slice_smem_bytes(int slice_len) { return slice_marks_offset(slice_len) + static_cast<size_t>(slice_len / 32 + 1) * 4; }

// A lower bound of the k-th largest of vals[0 .. n) (1 <= k <= n) that shares its upper 22 key bits: a radix descent of 11 + 11
// bits on the monotone keys. (BF16 logits have no key bits below those; for binary32 logits the few values that share the upper
// 22 bits with the k-th largest pass the bound too, which the merge sorts out.)
template <int B>
__device__ uint32_t slice_kth_key(const float* vals, int n, uint32_t k, uint32_t* bins, uint64_t* scratch, uint32_t* pick) {
  const int tid = threadIdx.x;
  uint32_t prefix = 0u, above = 0u;
#pragma unroll 1
  for (int level = 0; level < 2; level++) {
    const int shift = level == 0 ? 21 : 10;
    const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shift + 11));
    for (int i = tid; i < kSelectBins; i += B) bins[i] = 0u;
    __syncthreads();
    for (int j = tid; j < n; j += B) {
      const uint32_t key = fkey(vals[j]);
      if ((key & hi_mask) == prefix) atomicAdd(&bins[(key >> shift) & (kSelectBins - 1)], 1u);
    }
    __syncthreads();
    constexpr int kPer = kSelectBins / B;                                 // thread t owns kPer bins, walked downwards from the top
    uint32_t cnt[kPer]; uint64_t sum = 0ull;
#pragma unroll
    for (int j = 0; j < kPer; j++) { cnt[j] = bins[kSelectBins - 1 - (kPer * tid + j)]; sum += cnt[j]; }
    const uint64_t excl = block_exclusive_scan_u64(sum, scratch, nullptr);
    uint32_t run = above + static_cast<uint32_t>(excl);
    if (run < k && run + static_cast<uint32_t>(sum) >= k) {
#pragma unroll
      for (int j = 0; j < kPer; j++) {
        if (run < k && run + cnt[j] >= k) { pick[0] = static_cast<uint32_t>(kSelectBins - 1 - (kPer * tid + j)); pick[1] = run; }
        run += cnt[j];
      }
    }
    __syncthreads();
    prefix |= pick[0] << shift; above = pick[1];
    __syncthreads();
  }
  return prefix;
}

template <int B>
__global__ void __launch_bounds__(B) slice_local_kernel(SliceDev P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* vals = reinterpret_cast<float*>(smem_raw);
  uint32_t* marks = reinterpret_cast<uint32_t*>(smem_raw + slice_marks_offset(P.slice_len));
  __shared__ uint32_t bins[kSelectBins];
  __shared__ float tmax[B];                                                 // every thread's own largest logit
  __shared__ uint64_t scratch[32];
  __shared__ uint32_t pick[2];
  __shared__ uint32_t s_n, s_flags, s_ninf;
  // the merge may be made resident while the slices are at work; it waits for this grid
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, slice = blockIdx.x, row = blockIdx.y;
  if (tid == 0) { s_n = 0u; s_flags = 0u; s_ninf = 0xFFFFFFFFu; }
  if (P.state) {
    StepStateView st{const_cast<uint32_t*>(P.state), P.t_max, P.g};
    if (st.done() || row >= static_cast<int>(st.t_this_step())) return;
  }
  const int lo = slice * P.slice_len;
  const int n = max(0, min(P.slice_len, P.vocab - lo));
  unsigned char* rec = P.records + (static_cast<int64_t>(slice) * P.rows + row) * P.record_bytes;
  float* out_val = reinterpret_cast<float*>(rec + kVpHeader);
  int32_t* out_idx = reinterpret_cast<int32_t*>(rec + kVpHeader + 4 * static_cast<size_t>(P.cap));
  if (n == 0) {                                                            // nothing of the row falls into this slice
    if (tid == 0) {
      *reinterpret_cast<float*>(rec) = -INFINITY; *reinterpret_cast<float*>(rec + 4) = 0.0f; *reinterpret_cast<double*>(rec + 8) = 0.0;
      *reinterpret_cast<int32_t*>(rec + 16) = 0; *reinterpret_cast<uint32_t*>(rec + 20) = 0u;
    }
    return;
  }
  // ---- the slice, once, into shared memory
  RowView rv;
  rv.dtype = P.dtype; rv.vocab = n; rv.rho = 1.0f; rv.pi = 0.0f; rv.pen = nullptr;
  rv.row = static_cast<const char*>(P.logits) + (static_cast<size_t>(row) * static_cast<size_t>(P.row_stride) + static_cast<size_t>(lo)) * (P.dtype == LM_DTYPE_BF16 ? 2 : 4);
  rv.aligned = (reinterpret_cast<uintptr_t>(rv.row) & 15u) == 0;
  const int n_chunks = (n + kChunk - 1) / kChunk;
  const bool pen_on = P.history != nullptr;
  if (pen_on) for (int i = tid; i < P.slice_len / 32 + 1; i += B) marks[i] = 0u;
  for (int c = tid; c < n_chunks; c += B) {
    float z[kChunk];
    const int m = load_chunk(rv, c, z);
#pragma unroll
    for (int e = 0; e < kChunk; e++) if (e < m) vals[c * kChunk + e] = z[e];
  }
  __syncthreads();
  if (pen_on) {                                                            // every distinct history id inside the slice, once
    const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
    for (int i = tid; i < P.hist_len; i += B) {
      const int id = __ldg(h + i) - lo;
      if (id >= 0 && id < n) {
        const uint32_t bit = 1u << (id & 31);
        if ((atomicOr(&marks[id >> 5], bit) & bit) == 0u) vals[id] = canon_zero(penalise(vals[id], P.rho, P.pi));
      }
    }
    __syncthreads();
  }
  // ---- maximum, softmass relative to it
  uint64_t best = 0ull;
  bool nan = false;
  for (int j = tid; j < n; j += B) {
    const float v = vals[j];
    nan |= v != v;
    const uint64_t p = pack_best(v, static_cast<uint32_t>(j)); best = p > best ? p : best;
  }
  if (nan) s_flags = LM_STATUS_NAN;                                         // (the row goes to the generic algorithm, which defines what a NaN does)
  tmax[tid] = best ? best_value(best) : -INFINITY;
  best = block_max_u64(best, scratch);
  const float vmax = best_value(best);
  const double inv_t = 1.0 / static_cast<double>(P.temperature_rows ? P.temperature_rows[row] : P.temperature);
  double mass = 0.0;
  if (P.need_mass && P.exact_mass && vmax > -INFINITY) {
    double m = 0.0;
    for (int j = tid; j < n; j += B) m += softmass(vals[j], vmax, inv_t);
    mass = block_sum_f64(m, scratch);
  } else if (P.need_mass && vmax > -INFINITY) {                            // (only a top-p over the whole row asks for it)
    // In FP32, one ex2 per logit: sum_j 2^(z_j c2a + nb) with c2a = fl32(log2(e) / T) and nb = fl32(-vmax c2a); the common factor
    // that nb's rounding leaves is taken out exactly afterwards, so the result approximates sum_j 2^((z_j - vmax) c2a). The merge
    // knows how far that can be from the exact mass (slice_mass_band) and hands a row on when its top-p boundary is closer than that.
    const float c2a = static_cast<float>(1.4426950408889634 * inv_t);
    const float nb = __fmul_rn(-vmax, c2a);
    float acc = 0.0f;
    for (int j = tid; j < n; j += B) acc += ex2_approx(__fmaf_rn(vals[j], c2a, nb));
    mass = block_sum_f64(static_cast<double>(acc), scratch) * exp2(-(static_cast<double>(vmax) * static_cast<double>(c2a) + static_cast<double>(nb)));
  }
  // ---- the slice's k-th largest value and everything at or above it
  // The k-th largest of the threads' own maxima is a logit of the slice with at least k logits at or above it: a lower bound of
  // the slice's k-th largest that lets through only a few logits more (two of the slice's largest seldom fall to one thread).
  const uint32_t k = static_cast<uint32_t>(min(max(P.top_k_rows ? P.top_k_rows[row] : P.top_k, 1), min(n, B)));
  const uint32_t bound = slice_kth_key<B>(tmax, min(n, B), k, bins, scratch, pick);
  // Fewer than k threads with a logit above -inf (a masked vocabulary): every logit above -inf is a candidate, and one -inf logit
  // (the first) stands for the rest, so that a row with fewer than top_k logits above -inf still finds its k-th largest at -inf.
  constexpr uint32_t kNinfKey = 0x007FFFFFu;                               // fkey(-inf)
  const bool open = bound <= kNinfKey;
  if (!open) {
    const float tau_local = fkey_inv(bound);
    for (int j = tid; j < n; j += B) {
      if (vals[j] >= tau_local) {
        const uint32_t slot = atomicAdd(&s_n, 1u);
        if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = vals[j]; out_idx[slot] = P.index_base + lo + j; }
      }
    }
  } else {
    for (int j = tid; j < n; j += B) {
      const float v = vals[j];
      if (v > -INFINITY) {
        const uint32_t slot = atomicAdd(&s_n, 1u);
        if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = v; out_idx[slot] = P.index_base + lo + j; }
      } else if (v == -INFINITY) atomicMin(&s_ninf, static_cast<uint32_t>(j));
    }
  }
  __syncthreads();
  if (open && tid == 0 && s_ninf != 0xFFFFFFFFu) {
    const uint32_t slot = s_n++;
    if (slot < static_cast<uint32_t>(P.cap)) { out_val[slot] = -INFINITY; out_idx[slot] = P.index_base + lo + static_cast<int>(s_ninf); }
  }
  if (tid == 0) {
    const uint32_t cnt = s_n;
    *reinterpret_cast<float*>(rec) = vmax;
    *reinterpret_cast<float*>(rec + 4) = 0.0f;
    *reinterpret_cast<double*>(rec + 8) = mass;
    *reinterpret_cast<int32_t*>(rec + 16) = static_cast<int32_t>(cnt < static_cast<uint32_t>(P.cap) ? cnt : static_cast<uint32_t>(P.cap));
    *reinterpret_cast<uint32_t*>(rec + 20) = (cnt > static_cast<uint32_t>(P.cap) ? kStatusOverflow : 0u) | s_flags;
  }
}

// The merge of the sliced path: one block per row. Launched with programmatic stream serialization behind slice_local_kernel.
__global__ void __launch_bounds__(kVpMaxCandidates, 1) sliced_merge_kernel(VpMergeDev M, SampleDev P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ VpMergeSmem s;
  asm volatile("griddepcontrol.wait;" ::: "memory");                      // the records are complete behind this
  SampleDev Q = P;                                                         // with a StepState: the noise seed, the step and the active rows come from it
  apply_step_state(Q);
  VpMergeDev N = M;
  N.seed = Q.seed; N.step = Q.step;
  const int row = blockIdx.x;
  if (row >= Q.rows) return;
  if (!vocab_merge_row(N, row, s)) {                                      // overflowed records: the generic row algorithm, here and now
    GenericSmem& g = *reinterpret_cast<GenericSmem*>(smem_raw);
    sample_row_generic(Q, row, g, reinterpret_cast<uint32_t*>(smem_raw + sizeof(GenericSmem)));
  }
}

}  // namespace lm
