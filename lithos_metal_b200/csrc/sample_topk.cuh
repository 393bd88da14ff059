// The top-k candidate kernel: rows with 1 <= top_k <= kTopkMaxK in ONE pass over the row, no histogram, small blocks.
//
// With top-k on, the kept set lies inside the row's top-k logits. So the pass only has to (a) collect the few logits at or
// above a cutoff (estimated per row from 8192 of its logits: about 1 % of the row ends up above it), and
// (b) accumulate the softmass of the whole row in FP32 (the top-p target needs it). Everything exact then happens on the
// candidates alone: the k-th largest value, FP64 masses, the top-p boundary, integer weights, the draw. The FP32 mass is
// only used to decide on which side of top_p * Z a cumulative mass lies; if that is closer than the FP32 error bound (derived
// where it is applied), or the candidates do not cover the top-k set, or anything else does not fit, the row is handed on and
// the histogram kernel launched behind this one redoes it exactly.
// Two blocks of 512 threads share an SM (~93 KB of shared memory each): the per-row phases after the pass are chains of short
// dependent steps, and only the row in the other block can hide them.
// No counterpart in the reference (its sampler always builds the full histogram, kernels/common/sample.metal:34-162).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "sample_generic.cuh"

namespace lm {

constexpr int kTB = 512;                   // threads per block
constexpr int kTopkPerSM = 2;              // blocks per SM (64 registers per thread, ~92 KB of shared memory each)
constexpr int kTW = kTB / 32;
constexpr int kTopkCap = 2048;             // candidates per row (a power of two: the sorts pad to one)
constexpr int kTopkBins = 512;             // BF16 codes above the cutoff that the coarse count covers
constexpr int kTopkMaxK = 1024;            // largest top_k this kernel takes
constexpr int kTopkHist = 2048;            // longest history it takes
constexpr int kTopkMaxVocab = 1 << 18;
constexpr int kMaxProbes = 30;             // counters of the cutoff search per row: three per round, one round for the bracket + eight for the whole code range
constexpr int kBinSortMax = 256;           // a code bin with more candidates than this must already be in order (all equal)
constexpr int kSampleChunks = 1024 / kTB;   // chunks per thread in the cutoff sample: 1024 chunks = 8192 logits
constexpr int kTopkMinVocab = 32768;

constexpr int kStages = 4;                 // 16-byte asynchronous copies in flight per thread during the pass

struct TopkSmem {
  union {
    struct {
      unsigned long long key[kTopkCap];    // candidates as (monotone value key << 32) | ~index, arrival order; later the draw's index buckets
      unsigned long long sel[kTopkCap];    // those at or above the top-k crossing, in descending value order
    };
    uint4 ring[kStages][kTB];              // during the pass: each thread's own landing slots for its chunks of the row
  };
  union {
    double cum[kTopkCap];                  // FP64 softmass prefix over sel ...
    unsigned long long w[kTopkCap];        // ... then the fixed-point weights of the kept prefix
    uint32_t side_id[kTopkHist];           // before either: the distinct history ids
  };
  uint32_t pen[kTopkMaxVocab / 32];        // bitmap of the row's distinct history ids
  uint32_t hitlist[2048];                  // (chunk << 8 | 8-bit mask) of the chunks that hold a logit >= cutoff
  uint32_t bins[kTopkBins];                // candidates per BF16 code, relative to the cutoff code
  uint32_t off[kTopkBins];                 // candidates in the bins above each bin
  uint64_t scratch[32];
  double warp_d[kTW];
  uint32_t warp_u[kTW];
  uint32_t probe_cnt[kMaxProbes];          // block totals of the cutoff search, one slot per probe
  uint32_t prev_cut[8];                    // the block's last cutoff per size class of the candidate target (0: none yet)
  float warp_f[kTW];
  unsigned long long base;
  uint32_t n_hit, n, n_side, wide, cross_bin, ref_key;
  int hit, token, row;
};

static_assert(kTopkPerSM * (sizeof(TopkSmem) + 1024) <= 233472, "the blocks of the top-k kernel must fit one SM's shared memory");

// What the candidate path knows about the softmass of the whole row when it reaches the exact phases: z_tilde approximates
// sum_i 2^(z_i c + shift'), the exact mass relative to a maximum vmax is z_tilde * 2^(shift - vmax c); z_raw is the part of it
// that was accumulated in FP32 (sequences of acc_terms additions), z_corr what was added and removed term by term (penalties);
// ref is the logit the exponents were taken relative to (a logit of the row at or near its maximum).
struct RowMass { bool need; double z_tilde, z_raw, z_corr, shift, acc_terms; float ref; };

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void prefetch_l2_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
// Inclusive FP64 prefix sum over v[0 .. n) in place, index order; every thread calls. warp_d: one entry per warp.
__device__ __forceinline__ void scan_f64(double* v, int n, double* warp_d) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  double carry = 0.0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    double x = (i < n) ? v[i] : 0.0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const double t = __shfl_up_sync(kFull, x, o); if (lane >= o) x += t; }
    __syncthreads();
    if (lane == 31) warp_d[warp] = x;
    __syncthreads();
    double wsum = 0.0, tot = 0.0;
    for (int w = 0; w < nw; w++) { if (w < warp) wsum += warp_d[w]; tot += warp_d[w]; }
    if (i < n) v[i] = carry + wsum + x;
    carry += tot;
  }
  __syncthreads();
}

// Warp-aggregated append: every lane of the warp calls with its count; returns the lane's first slot.
__device__ __forceinline__ uint32_t warp_reserve(uint32_t* counter, uint32_t mine) {
  const int lane = threadIdx.x & 31;
  uint32_t incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
  const uint32_t total = __shfl_sync(kFull, incl, 31);
  uint32_t base = 0u;
  if (lane == 0 && total) base = atomicAdd(counter, total);
  base = __shfl_sync(kFull, base, 0);
  return base + incl - mine;
}

// Whether a row is this kernel's at all, from its knobs and address alone (no look at the logits).
__device__ __forceinline__ bool topk_row_eligible(const SampleDev& P, int row) {
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  const int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const uint16_t* rowp = reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride);
  return T > 0.0f && top_k >= 1 && top_k <= kTopkMaxK && (V % kChunk) == 0 && V >= kTopkMinVocab && V <= kTopkMaxVocab &&
         (reinterpret_cast<uintptr_t>(rowp) & 15u) == 0 && !(P.history != nullptr && P.hist_len > kTopkHist);
}

// The rows that are not the top-k kernel's, listed for the histogram kernel (one thread per row).
__global__ void sample_classify_kernel(SampleDev P, int* list, int* n_list) {
  apply_step_state(P);
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < P.rows && !topk_row_eligible(P, row)) list[atomicAdd(n_list, 1)] = row;
}

struct TopkSmem;
__device__ bool topk_finish(const SampleDev& P, int row, TopkSmem& c, uint32_t cut_code, const RowMass& zm);

// One row. Every thread of the block calls with the same arguments; returns true when the row is finished, false when the
// histogram kernel has to take it (nothing has been written then).
// `next` is the row this block takes afterwards (-1: none): its sample and history are pulled into L2 meanwhile.
__device__ bool topk_row(const SampleDev& P, int row, int next, TopkSmem& c) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = P.vocab;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  const int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const uint16_t* rowp = reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(row) * static_cast<size_t>(P.row_stride);
  const bool pen_on = P.history != nullptr;
  const int n_chunks = V / kChunk;
  const uint4* p4 = reinterpret_cast<const uint4*>(rowp);
  const bool has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_p;
  const bool need_z = has_p && !in_topk;
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const float c2a = static_cast<float>(1.4426950408889634 * inv_t);          // the FP32 softmass only: approximate on purpose

  // the first chunks of the pass do not depend on the cutoff: they start now and land in this thread's slots
  const int n_it = (n_chunks + kTB - 1) / kTB;
#pragma unroll
  for (int it = 0; it < kStages - 1; it++) {
    if (it * kTB + tid < n_chunks) cp_async16(&c.ring[it][tid], p4 + it * kTB + tid);
    cp_async_commit();
  }
  if (next >= 0) {
    const uint4* np4 = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(P.logits) + static_cast<size_t>(next) * static_cast<size_t>(P.row_stride));
    if ((tid & 7) == 0) {                                                   // one prefetch per 128-byte line of the sample runs
#pragma unroll
      for (int j = 0; j < kSampleChunks; j++) prefetch_l2_line(np4 + tid + j * (n_chunks / kSampleChunks));
    }
    if (pen_on && tid * 32 < P.hist_len) prefetch_l2_line(P.history + static_cast<int64_t>(next) * P.hist_stride + tid * 32);
  }
  // ---- the cutoff sample goes out first; the bitmap and the list of the history's distinct ids are built under its latency ---
  // (runs of chunks spread over the row: token ids are not exchangeable in a real vocabulary)
  uint4 qs[kSampleChunks];
#pragma unroll
  for (int j = 0; j < kSampleChunks; j++) qs[j] = __ldg(p4 + tid + j * (n_chunks / kSampleChunks));
  constexpr int kHistPer = kTopkHist / kTB;
  int hid[kHistPer];                                                        // this thread's share of the history, in flight with the sample
#pragma unroll
  for (int j = 0; j < kHistPer; j++) {
    const int i = tid + j * kTB;
    hid[j] = (pen_on && i < P.hist_len) ? __ldg(P.history + static_cast<int64_t>(row) * P.hist_stride + i) : -1;
  }
  for (int i = tid; i < kTopkBins; i += kTB) c.bins[i] = 0u;
  if (tid < kMaxProbes) c.probe_cnt[tid] = 0u;
  if (pen_on) {
    uint4* p = reinterpret_cast<uint4*>(c.pen);
    for (int i = tid; i < (V + 127) / 128; i += kTB) p[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (tid == 0) { c.n_hit = 0u; c.n = 0u; c.n_side = 0u; c.wide = 0u; c.ref_key = 0u; c.hit = kTopkCap; c.token = -1; c.cross_bin = 0u; }
  __syncthreads();
  // the thread that sets an id's bit owns the id and lists it
#pragma unroll
  for (int j = 0; j < kHistPer; j++) {
    const int id = hid[j];
    bool fresh = false;
    if (id >= 0 && id < V) {
      const uint32_t bit = 1u << (id & 31);
      fresh = (atomicOr(&c.pen[id >> 5], bit) & bit) == 0u;
    }
    const uint32_t slot = warp_reserve(&c.n_side, fresh ? 1u : 0u);
    if (fresh) c.side_id[slot] = static_cast<uint32_t>(id);
  }
  // ---- the cutoff: the largest positive BF16 code with at least `want` of the 8192 sampled logits at or above it ---------
  // (about 1.3 k + 150 candidates expected in the whole row, at most ~1500)
  // A bisection over the codes, one barrier per probe; it starts from a bracket around the cutoff of the block's last
  // row of the same size class, which usually holds (rows of one batch come from one model), and costs ~7 probes then.
  uint32_t cut_code;
  {
    const int n_target = min(1500, top_k + top_k / 3 + 150);
    const uint32_t want = max(8u, static_cast<uint32_t>((static_cast<long long>(n_target) * kSampleChunks * kTB * kChunk + V - 1) / V));
    const int cls = min(31 - __clz(want), 7);
    int probe = 0;
    // sampled logits at or above each of three codes, with one barrier; every thread calls
    auto count3 = [&](uint32_t a, uint32_t b, uint32_t d, uint32_t out[3]) {
      const uint32_t codes[3] = {a, b, d};
      uint32_t cnt[3] = {0u, 0u, 0u};
#pragma unroll
      for (int t = 0; t < 3; t++) {
        const uint32_t m2 = codes[t] | (codes[t] << 16);
        const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&m2);
#pragma unroll
        for (int j = 0; j < kSampleChunks; j++) {
          cnt[t] += __popc(__hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].x), t2)) + __popc(__hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].y), t2)) +
                    __popc(__hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].z), t2)) + __popc(__hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].w), t2));
        }
        cnt[t] = warp_sum_u32(cnt[t] >> 4);                     // 16 mask bits per logit
        if (lane == 0 && cnt[t]) atomicAdd(&c.probe_cnt[probe + t], cnt[t]);
      }
      __syncthreads();
#pragma unroll
      for (int t = 0; t < 3; t++) out[t] = c.probe_cnt[probe + t];
      probe += 3;
    };
    // the largest sampled logit: the reference point of the FP32 softmass (any value near the row maximum will do); it
    // travels with the first probe's barrier
    if (need_z) {
      __nv_bfloat162 mx = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&qs[0].x), *reinterpret_cast<const __nv_bfloat162*>(&qs[0].y));
      mx = __hmax2(mx, __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&qs[0].z), *reinterpret_cast<const __nv_bfloat162*>(&qs[0].w)));
#pragma unroll
      for (int j = 1; j < kSampleChunks; j++) {
        mx = __hmax2(mx, __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].x), *reinterpret_cast<const __nv_bfloat162*>(&qs[j].y)));
        mx = __hmax2(mx, __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&qs[j].z), *reinterpret_cast<const __nv_bfloat162*>(&qs[j].w)));
      }
      const uint32_t key = warp_max_u32(fkey(fmaxf(__low2float(mx), __high2float(mx))));
      if (lane == 0) atomicMax(&c.ref_key, key);
    }
    uint32_t lo = 0x0000u, hi = 0x7F7Fu;                                    // invariant: count(sample >= lo) >= want, or lo is still 0 (handed back below)
    const uint32_t prev = c.prev_cut[cls];
    uint32_t n3[3];
    if (prev >= 0x0080u) {                                                  // both ends of the bracket and its middle in one round
      const uint32_t blo = max(prev, 0x0090u) - 16u, bhi = min(prev + 15u, 0x7F7Eu), mid = (blo + bhi + 1u) >> 1;
      count3(blo, mid, bhi + 1u, n3);
      if (n3[0] < want) hi = blo - 1u;
      else if (n3[2] >= want) lo = bhi + 1u;
      else if (n3[1] >= want) { lo = mid; hi = bhi; }
      else { lo = blo; hi = mid - 1u; }
    }
    while (lo < hi && probe + 3 <= kMaxProbes) {                            // three cuts per round: the range shrinks fourfold
      const uint32_t span = hi - lo;
      const uint32_t q1 = lo + (span + 3u) / 4u, q2 = lo + (2u * span + 3u) / 4u, q3 = lo + (3u * span + 3u) / 4u;   // lo < q1 <= q2 <= q3 <= hi
      count3(q1, q2, q3, n3);
      if (n3[2] >= want) lo = q3;
      else if (n3[1] >= want) { lo = q2; hi = q3 - 1u; }
      else if (n3[0] >= want) { lo = q1; hi = q2 - 1u; }
      else hi = q1 - 1u;
    }
    cut_code = lo;
    if (cut_code < 0x0080u || lo < hi) { cp_async_wait<0>(); return false; }   // fewer positive logits than candidates wanted: not this kernel's row
                                                                            // (the copies in flight must land before the slots are used again)
    if (tid == 0) c.prev_cut[cls] = cut_code;
  }
  const float cut_val = __uint_as_float(cut_code << 16);

  // ---- the one pass: note the chunks that hold a logit >= cutoff; FP32 softmass relative to the sampled maximum ----------
  const float M = need_z ? fkey_inv(c.ref_key) : 0.0f;
  const float nb = -M * c2a;
  float2 sacc = make_float2(0.0f, 0.0f);
  uint32_t nan_seen = 0u;
  {
    const uint32_t cut2 = cut_code | (cut_code << 16);
    const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&cut2);
    const uint4 pad = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);   // -inf
#pragma unroll 4
    for (int it = 0; it < n_it; it++) {                                     // uniform trip count: warp votes inside
      {
        const int ahead = it + kStages - 1, ca = ahead * kTB + tid;         // refill the slot read one step ago
        if (ca < n_chunks) cp_async16(&c.ring[ahead % kStages][tid], p4 + ca);
        cp_async_commit();
      }
      cp_async_wait<kStages - 1>();                                         // this step's chunk has landed
      const int cc = it * kTB + tid;
      const bool live = cc < n_chunks;                                      // warp-uniform control flow below: votes inside
      const uint4 q = live ? c.ring[it % kStages][tid] : pad;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[0]), t2), m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[1]), t2);
      const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[2]), t2), m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&w[3]), t2);
      const bool hit = live && (m0 | m1 | m2 | m3) != 0u;
      const uint32_t votes = __ballot_sync(kFull, hit);
      if (votes) {                                                          // one reservation per warp for all its hit chunks
        uint32_t base = 0u;
        if (lane == 0) base = atomicAdd(&c.n_hit, __popc(votes));
        base = __shfl_sync(kFull, base, 0);
        if (hit) {
          const uint32_t mask = (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) |
                                ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
          const uint32_t slot = base + __popc(votes & ((1u << lane) - 1u));
          if (slot < 2048u) c.hitlist[slot] = (static_cast<uint32_t>(cc) << 8) | mask;
        }
      }
      if (need_z) {                                                         // (the padding is -inf: weight 0; a NaN or +inf logit poisons the sum)
#pragma unroll
        for (int k = 0; k < 4; k++) {                                         // two logits per packed multiply-add and per packed add
          const float2 x = __ffma2_rn(make_float2(bf16_lo(w[k]), bf16_hi(w[k])), make_float2(c2a, c2a), make_float2(nb, nb));
          sacc = __fadd2_rn(sacc, make_float2(ex2_approx(x.x), ex2_approx(x.y)));
        }
      } else {                                                              // no mass wanted: the NaN check on its own
        const __nv_bfloat162 a = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&w[0]), *reinterpret_cast<const __nv_bfloat162*>(&w[1]));
        const __nv_bfloat162 b = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162*>(&w[2]), *reinterpret_cast<const __nv_bfloat162*>(&w[3]));
        const __nv_bfloat162 ab = __hmax2_nan(a, b);
        nan_seen |= ~__heq2_mask(ab, ab);                                   // a NaN anywhere in the chunk survives the maxima
      }
    }
    cp_async_wait<0>();
  }
  // a NaN or +inf logit (or a logit far above the sampled maximum) has made this thread's sum NaN or infinite: the exact path
  // takes such rows and reports them
  double zsum = 0.0, zadd = 0.0, zsub = 0.0;                                // the pass's mass; what the penalised logits add; what their raw values had added
  if (need_z) {
    const float total = sacc.x + sacc.y;
    if (!(total < INFINITY)) nan_seen = 1u;
    zsum = static_cast<double>(total);
  }
  if (__syncthreads_or(nan_seen != 0u)) return false;                       // rows with a NaN go to the exact path, which reports them
  const uint32_t n_hit = c.n_hit;                                           // (complete: every warp is past the pass)
  if (n_hit > 2048u) return false;

  // the raw logits of the penalised positions are fetched now, after the pass (the row has just gone through L2), and used
  // behind the expansion below: both sets of loads are in flight together
  constexpr int kGather = kTopkHist / kTB;
  uint32_t ids[kGather]; uint16_t raws[kGather];
  if (pen_on) {
#pragma unroll
    for (int j = 0; j < kGather; j++) {
      const uint32_t i = j * kTB + tid;
      ids[j] = i < c.n_side ? c.side_id[i] : 0u;
      raws[j] = __ldg(rowp + ids[j]);
    }
  }
  // ---- the noted chunks, expanded: their logits come back from L2; penalised positions are skipped (the hash set knows them)
  constexpr int kExpand = 1024 / kTB;                                       // chunk reloads in flight per thread
  for (uint32_t e0 = 0; e0 < n_hit; e0 += kTB * kExpand) {                  // uniform trip count
    uint32_t ents[kExpand]; uint4 qq[kExpand];
#pragma unroll
    for (int j = 0; j < kExpand; j++) {
      const uint32_t e = e0 + j * kTB + tid;
      ents[j] = (e < n_hit) ? c.hitlist[e] : 0u;
      qq[j] = (e < n_hit) ? __ldg(p4 + (ents[j] >> 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < kExpand; j++) {
      if (e0 + j * kTB >= n_hit) break;                                     // block-uniform
      const uint32_t ent = ents[j];
      uint32_t mask = ent & 0xFFu;
      const uint32_t cc = ent >> 8;
      const uint32_t keep = pen_on ? mask & ~((c.pen[cc >> 2] >> ((cc & 3u) * 8u)) & 0xFFu) : mask;   // penalised positions come from the list
      uint32_t slot = warp_reserve(&c.n, __popc(keep));
      for (uint32_t m = keep; m; m &= m - 1u) {                             // usually one bit
        const uint32_t b = __ffs(m) - 1u;
        const uint32_t word = b < 4u ? (b < 2u ? qq[j].x : qq[j].y) : (b < 6u ? qq[j].z : qq[j].w);
        const float value = (b & 1u) ? bf16_hi(word) : bf16_lo(word);
        if (slot < kTopkCap) c.key[slot] = (static_cast<unsigned long long>(fkey(value)) << 32) | (0xFFFFFFFFu - (cc * kChunk + b));
        slot++;
        const uint32_t rel = (__float_as_uint(value) >> 16) - cut_code;
        if (rel >= kTopkBins) c.wide = 1u; else atomicAdd(&c.bins[rel], 1u);
      }
    }
  }
  // ---- the penalised logits, from the list ---------------------------------------------------------------------------------
  if (pen_on) {
    const uint32_t n_side = c.n_side;
#pragma unroll
    for (int j = 0; j < kGather; j++) {
      const uint32_t i = j * kTB + tid;
      if (j * kTB >= n_side) break;                                         // block-uniform
      float v = -INFINITY;
      if (i < n_side) {
        const float raw = __uint_as_float(static_cast<uint32_t>(raws[j]) << 16);
        v = penalise(raw, P.rho, P.pi);
        if (need_z) { zadd += static_cast<double>(ex2_approx(__fmaf_rn(v, c2a, nb))); zsub += static_cast<double>(ex2_approx(__fmaf_rn(raw, c2a, nb))); }
      }
      const bool cand = v >= cut_val;
      const uint32_t slot = warp_reserve(&c.n, cand ? 1u : 0u);
      if (cand) {
        if (slot < kTopkCap) c.key[slot] = (static_cast<unsigned long long>(fkey(v)) << 32) | (0xFFFFFFFFu - ids[j]);
        const uint32_t rel = (__float_as_uint(v) >> 16) - cut_code;
        if (rel >= kTopkBins) c.wide = 1u; else atomicAdd(&c.bins[rel], 1u);
      }
    }
  }
  double z_raw = 0.0, z_add = 0.0, z_sub = 0.0;                             // block totals, relative to the sampled maximum
  if (need_z) {
    zsum = warp_sum_f64(zsum); zadd = warp_sum_f64(zadd); zsub = warp_sum_f64(zsub);
    double* sd = reinterpret_cast<double*>(c.scratch);
    __syncthreads();
    if (lane == 0) { sd[warp] = zsum; sd[kTW + warp] = zadd; c.warp_d[warp] = zsub; }
    __syncthreads();
    for (int w = 0; w < kTW; w++) { z_raw += sd[w]; z_add += sd[kTW + w]; z_sub += c.warp_d[w]; }
  }
  const double z_tilde = z_raw - z_sub + z_add;
  if (need_z && !(z_tilde > 0.0)) return false;                             // nothing left after the corrections (cancellation): the exact path
  __syncthreads();
  RowMass zm;
  zm.need = need_z; zm.z_tilde = z_tilde; zm.z_raw = z_raw; zm.z_corr = z_sub + z_add; zm.shift = -static_cast<double>(nb);
  zm.ref = M; zm.acc_terms = 4.0 * n_it + 1.0;
  return topk_finish(P, row, c, cut_code, zm);
}

// The exact phases of the candidate path, on what the pass (or a producer of logits tiles, sample_tiles.cuh) has left in shared
// memory: c.key[0 .. c.n) = every logit of the row at or above the cutoff code as (monotone value key << 32) | ~index, c.bins[b] =
// how many of them have BF16 code cut_code + b, c.wide set if one lies beyond the bins. `zm` is what is known about the mass of
// the WHOLE row. Every thread of the block calls with the same arguments; returns true when the row is finished (token, tau
// and status written), false when the exact path has to take it (nothing has been written then).
__device__ bool topk_finish(const SampleDev& P, int row, TopkSmem& c, uint32_t cut_code, const RowMass& zm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float T = P.temperature ? P.temperature[row] : P.temperature_s;
  const int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
  const float top_p = P.top_p ? P.top_p[row] : P.top_p_s;
  const float min_p = P.min_p ? P.min_p[row] : P.min_p_s;
  const bool has_p = top_p > 0.0f && top_p < 1.0f, has_m = min_p > 0.0f;
  const bool in_topk = (P.flags & LM_FLAG_TOPP_IN_TOPK) && has_p;
  const double T64 = static_cast<double>(T), inv_t = 1.0 / T64;
  const int n = static_cast<int>(c.n);
  if (n > kTopkCap || n < top_k || c.wide) return false;

  // ---- the candidates at or above the top-k crossing, in descending value order: a counting sort by code bin ---------------
  // (the bins are the BF16 codes relative to the cutoff; the crossing is the highest bin b with at least top_k
  // candidates in the bins >= b; inside a bin only penalised values can differ, and one thread puts its bin in order)
  {
    constexpr int kPer = kTopkBins / kTB;                                    // bins per thread, walked from the top
    uint32_t run = 0u, cb[kPer], mine = 0u;
#pragma unroll
    for (int j = 0; j < kPer; j++) { cb[j] = c.bins[kTopkBins - 1 - (kPer * tid + j)]; mine += cb[j]; }
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
    if (lane == 31) c.warp_u[warp] = incl;
    __syncthreads();
    for (int w = 0; w < warp; w++) run += c.warp_u[w];
    uint32_t acc = run + incl - mine;
#pragma unroll
    for (int j = 0; j < kPer; j++) {
      c.off[kTopkBins - 1 - (kPer * tid + j)] = acc;
      if (acc < static_cast<uint32_t>(top_k) && acc + cb[j] >= static_cast<uint32_t>(top_k)) c.cross_bin = static_cast<uint32_t>(kTopkBins - 1 - (kPer * tid + j));
      acc += cb[j];
    }
    __syncthreads();
  }
  const uint32_t cross = c.cross_bin;
  const int n_sel = static_cast<int>(c.off[cross] + c.bins[cross]);
  __syncthreads();                                                          // the counts are consumed below
  for (int i = tid; i < n; i += kTB) {
    const unsigned long long k = c.key[i];
    const uint32_t rel = (__float_as_uint(fkey_inv(static_cast<uint32_t>(k >> 32))) >> 16) - cut_code;
    if (rel >= cross) c.sel[c.off[rel] + atomicSub(&c.bins[rel], 1u) - 1u] = k;
  }
  __syncthreads();
  for (uint32_t b = cross + tid; b < kTopkBins; b += kTB) {
    const uint32_t lo = c.off[b], hi = (b == cross) ? static_cast<uint32_t>(n_sel) : c.off[b - 1];
    bool sorted = true;
    for (uint32_t i = lo + 1u; i < hi; i++) sorted = sorted && (c.sel[i - 1u] >> 32) >= (c.sel[i] >> 32);
    if (sorted) continue;
    if (hi - lo > static_cast<uint32_t>(kBinSortMax)) { c.wide = 1u; continue; }
    for (uint32_t i = lo + 1u; i < hi; i++) {                               // insertion sort on the value part: equal values stay put
      const unsigned long long k = c.sel[i];
      uint32_t j = i;
      while (j > lo && (c.sel[j - 1u] >> 32) < (k >> 32)) { c.sel[j] = c.sel[j - 1u]; j--; }
      c.sel[j] = k;
    }
  }
  __syncthreads();
  if (c.wide) return false;                                                 // a large bin of unequal (penalised) values: the exact path takes the row

  // ---- exact thresholds on the sorted candidates ------------------------------------------------------------------------
  const float vmax = fkey_inv(static_cast<uint32_t>(c.sel[0] >> 32));
  const float tau_k = fkey_inv(static_cast<uint32_t>(c.sel[top_k - 1] >> 32));
  double tau64 = tau_k;
  uint32_t status = LM_STATUS_CANDIDATE_PATH;
  if (has_p) {
    for (int i = tid; i < n_sel; i += kTB) c.cum[i] = softmass(fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)), vmax, inv_t);
    __syncthreads();
    scan_f64(c.cum, n_sel, c.warp_d);
    uint64_t cnt_k = 0ull;
    for (int i = tid; i < n_sel; i += kTB) cnt_k += fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) >= tau_k ? 1ull : 0ull;
    const int n_topk = static_cast<int>(block_sum_u64(cnt_k, c.scratch));
    double total, err = 0.0;
    if (in_topk) total = c.cum[n_topk - 1];
    else {
      // The FP32 mass of the whole row, moved to the exact maximum. z_tilde approximates sum_i 2^(z_i c2a + nb); nb's own rounding
      // is a common factor and is taken out exactly here (zm.shift is the true -nb, not M c2a).
      const double c64 = 1.4426950408889634 * inv_t;
      total = zm.z_tilde * exp2(zm.shift - static_cast<double>(vmax) * c64);
      // What separates it from sum_i 2^((z_i - vmax) c), relative, first order, worst case (u = 2^-24, the FP32 unit roundoff):
      //   - c2a = fl32(c): every term is off by a factor 2^(x_i delta), |delta| <= u, x_i = (z_i - M) c; weighted by the terms that is
      //     ln2 u E_w|x| <= u (ln V + 2 ln2 D): E_w[-x ln2] = H - ln Z <= ln V (H the entropy of the softmax, Z >= 1 relative to the
      //     row maximum, V <= 2^18: ln V <= 12.5), and the terms above the sampled maximum have 0 < x <= D = (vmax - M) c;
      //   - the FMA rounds its result: half an ulp of |x| < 32 is at most 2^-20, a factor 2^(2^-20) = 1 + 6.6e-7 on the term; the terms
      //     with |x| >= 32 weigh less than V 2^-32 altogether;
      //   - ex2.approx.ftz.f32: 2 ulp = 4 u;
      //   - each lane accumulates 4 n_it terms one after the other in FP32, then two accumulators and the lanes meet in FP64:
      //     (4 n_it + 1) u (zm.acc_terms);
      // These are relative to the mass the pass summed (z_raw), which holds the penalised positions at their raw values. The penalised
      // logits then enter as z_raw - z_sub + z_add, every term of z_sub and z_add with the per-term errors above (FMA, ex2, c2a on a
      // single term: 1.6e-6 covers them for |x| < 32); when penalised tokens carried most of the raw mass the band grows with them.
      // The band is this bound with a quarter added. A boundary of the cumulative mass inside it is decided by the exact path.
      const double u = 5.9604644775390625e-8;
      const double D = fmax(0.0, (static_cast<double>(vmax) - static_cast<double>(zm.ref)) * c64);
      const double rel = u * (12.5 + 1.3862943611198906 * D) + 6.6e-7 + 4.0 * u + zm.acc_terms * u;
      err = 1.25 * (rel * zm.z_raw + 1.6e-6 * zm.z_corr) * (total / zm.z_tilde);
    }
    const double target = static_cast<double>(top_p) * total;
    bool amb = false;
    for (int i = tid; i < n_sel; i += kTB) {
      const bool run_end = (i == n_sel - 1) || ((c.sel[i + 1] >> 32) != (c.sel[i] >> 32));
      if (!run_end) continue;
      const double cm = c.cum[i];
      if (cm >= target) atomicMin(&c.hit, i);
      if (i < n_topk - 1 && fabs(cm - target) <= err && fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) > tau_k) amb = true;
    }
    if (__syncthreads_or(amb)) return false;                               // too close to call in FP32: the exact path decides
    if (c.hit < kTopkCap) {
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
  for (int i = tid; i < n_sel; i += kTB) cnt_kept += fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)) >= tau ? 1ull : 0ull;
  const int n_kept = static_cast<int>(block_sum_u64(cnt_kept, c.scratch));   // the kept set is the first n_kept sorted candidates

  // ---- the draw ----------------------------------------------------------------------------------------------------------
  int token = -1;
  uint64_t kept_weight = 0ull;                                             // the kept set's fixed-point mass (for out_mass)
  if (P.draw == LM_DRAW_INVERSE_CDF) {
    // The kept candidates are in descending value order, which is the draw's order up to the order inside a run of equal values
    // (equal values have equal weights): an inclusive prefix sum of the weights finds the candidate where the target is crossed,
    // hence the value; the token is the floor((target - before) / w)-th smallest index of that value's run.
    const float c2 = exp2_scale(T);
    constexpr int kPer = kTopkCap / kTB;                                    // consecutive candidates per thread
    uint64_t wv[kPer], sum = 0ull;
#pragma unroll
    for (int j = 0; j < kPer; j++) {
      const int i = tid * kPer + j;
      wv[j] = i < n_kept ? weight_q40(fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)), vmax, c2) : 0ull;
      sum += wv[j];
    }
    uint64_t total = 0ull;
    uint64_t run = block_exclusive_scan_u64(sum, c.scratch, &total);
    kept_weight = total;
    if (tid == 0) { c.hit = kTopkCap; c.cross_bin = 0u; c.n_hit = static_cast<uint32_t>(n_kept); }
    __syncthreads();
    if (total > 0ull) {
      const uint64_t target = cdf_target(P.uniforms ? P.uniforms[row] : 0.0f, total);
#pragma unroll
      for (int j = 0; j < kPer; j++) {
        const int i = tid * kPer + j;
        run += wv[j];
        if (i < n_kept) c.w[i] = run;                                       // inclusive
        if (wv[j] && run > target && run - wv[j] <= target) c.hit = i;      // exactly one candidate
      }
      __syncthreads();
      const int at = c.hit;
      const uint32_t vkey = static_cast<uint32_t>(c.sel[at] >> 32);
      // the run of this value: [first, last)
      for (int i = tid; i < n_kept; i += kTB) {
        if (static_cast<uint32_t>(c.sel[i] >> 32) != vkey) continue;
        if (i == 0 || static_cast<uint32_t>(c.sel[i - 1] >> 32) != vkey) c.cross_bin = static_cast<uint32_t>(i);
        if (i == n_kept - 1 || static_cast<uint32_t>(c.sel[i + 1] >> 32) != vkey) c.n_hit = static_cast<uint32_t>(i + 1);
      }
      __syncthreads();
      const int first = static_cast<int>(c.cross_bin), last = static_cast<int>(c.n_hit);
      const uint64_t before = first > 0 ? c.w[first - 1] : 0ull;
      const uint64_t each = c.w[first] - before;
      const uint32_t want = static_cast<uint32_t>((target - before) / each);   // < last - first: the crossing lies inside the run
      for (int i = first + tid; i < last; i += kTB) {
        const uint32_t idx_i = 0xFFFFFFFFu - static_cast<uint32_t>(c.sel[i]);
        uint32_t smaller = 0u;
        for (int t = first; t < last; t++) smaller += (0xFFFFFFFFu - static_cast<uint32_t>(c.sel[t])) < idx_i ? 1u : 0u;
        if (smaller == want) c.token = static_cast<int>(idx_i);
      }
    }
    __syncthreads();
    token = c.token;
  } else {
    const float inv_t32 = __double2float_rn(1.0 / T64);
    const uint32_t t_id = static_cast<uint32_t>(P.row_offset + row);
    uint64_t b1 = 0ull; float second = -INFINITY;
    for (int i = tid; i < n_kept; i += kTB) {
      const unsigned long long k = c.sel[i];
      const uint32_t idx = 0xFFFFFFFFu - static_cast<uint32_t>(k);
      const float key = __fadd_rn(__fmul_rn(fkey_inv(static_cast<uint32_t>(k >> 32)), inv_t32), gumbel(P.seed, P.step, t_id, idx));
      const uint64_t pk = pack_best(key, idx);
      if (pk > b1) { if (b1) second = fmaxf(second, best_value(b1)); b1 = pk; } else second = fmaxf(second, key);
    }
    const uint64_t win = block_max_u64(b1, c.scratch);
    if (win) {
      const float rival = (b1 == win) ? second : (b1 ? best_value(b1) : -INFINITY);
      if (__syncthreads_or(rival >= best_value(win) - 4e-6f)) status |= LM_STATUS_NEAR_TIE;
      token = static_cast<int>(best_index(win));
    }
    if (P.out_mass) {
      const float c2 = exp2_scale(T);
      uint64_t w = 0ull;
      for (int i = tid; i < n_kept; i += kTB) w += weight_q40(fkey_inv(static_cast<uint32_t>(c.sel[i] >> 32)), vmax, c2);
      kept_weight = block_sum_u64(w, c.scratch);
    }
  }
  if (tid == 0) {
    P.out_tokens[row] = token;
    if (P.out_tau) P.out_tau[row] = tau;
    if (P.out_status) P.out_status[row] = status;
    if (P.out_vmax) P.out_vmax[row] = vmax;
    if (P.out_mass) P.out_mass[row] = kept_weight;
  }
  __syncthreads();
  return true;
}

// Rows are handed out through a counter in the workspace (counters[0], zeroed by the host before the launch): a block takes
// the next row, passes over it if it is not this kernel's (listing it if `list_others`), and else either finishes it or appends it to `list` (length in
// counters[1]) for the histogram kernel. The order of the list varies from run to run; what is computed per row does not.
__global__ void __launch_bounds__(kTB, kTopkPerSM) sample_topk_kernel(SampleDev P, int* list, int* counters, int list_others) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkSmem& c = *reinterpret_cast<TopkSmem*>(smem_raw);
  __shared__ int item[2];                                                   // the row in hand and the one after it
  apply_step_state(P);
  if (threadIdx.x < 8) c.prev_cut[threadIdx.x] = 0u;
  // With many rows per block a block holds the row after its current one too (it pulls that row into L2 while it works) and
  // claims the one after that at the start of a row, so the counter's round trip hides behind the row. With few rows per block
  // claiming ahead would leave blocks without work while others hold two rows: a block then claims a row when it needs one.
  const bool ahead = P.rows >= 4 * static_cast<int>(gridDim.x);
  if (threadIdx.x == 0) { item[0] = atomicAdd(&counters[0], 1); item[1] = (ahead && item[0] < P.rows) ? atomicAdd(&counters[0], 1) : P.rows; }
  __syncthreads();
  for (;;) {
    const int row = item[0], next = item[1];
    if (row >= P.rows) break;
    int fetched = P.rows;
    if (threadIdx.x == 0 && next < P.rows) fetched = atomicAdd(&counters[0], 1);
    if (!topk_row_eligible(P, row)) {                                       // not this kernel's row: listed here, or already by sample_classify_kernel
      if (list_others && threadIdx.x == 0) list[atomicAdd(&counters[1], 1)] = row;
    } else {
      const bool done = topk_row(P, row, next < P.rows ? next : -1, c);
      if (threadIdx.x == 0 && !done) list[atomicAdd(&counters[1], 1)] = row;
    }
    __syncthreads();                                                        // nobody reads item[] any more
    if (threadIdx.x == 0) { item[0] = ahead ? next : atomicAdd(&counters[0], 1); item[1] = fetched; }
    __syncthreads();
  }
  // This grid may have been started before the grid launched ahead of it had finished (programmatic stream serialization). The
  // stream takes the end of this grid for the end of both, so no block leaves before the earlier grid is complete.
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace lm
