// DSpark verification of one speculative step in ONE launch: n_draft drafted tokens against n_draft + 1 rows of
// target logits. Greedy: row-wise argmax and prefix match (kernels/common/spec_ops.metal:162-165). Stochastic:
// accept draft r with probability min(1, p/q), replace the first rejected one by a draw from max(p - q, 0)
// (kernels/common/sample.metal:273-347), on the integer fixed-point weights so the outcome is independent of how the
// vocabulary is split between blocks.
//
// The step is latency-bound (a few MB of input, a chain of three data dependencies), so the kernel is one
// cooperative launch of one block per SM; every block owns the same vocabulary slice of every row in every phase.
// Phase 0 is the only one that touches HBM: it pulls the block's slice of all target rows and all draft-probability
// rows into shared memory (one pass over both inputs, every load in flight at once); the later phases work from
// there. Partial results meet in a small workspace, and the phases are separated by a bounded grid barrier on a
// counter in that workspace.
#pragma once
#include "common.cuh"
#include "spec_ops.cuh"

namespace lm {

#ifndef LM_VERIFY_BLOCK
#define LM_VERIFY_BLOCK 1024
#endif
constexpr int kVerifyBlock = LM_VERIFY_BLOCK;
constexpr int kVerifyMaxRows = LM_MAX_DRAFT + 1;
constexpr unsigned kBarrierSpinLimit = 1u << 22;       // ~ tens of ms: far beyond any legitimate wait

struct VerifyWs {                                       // lives in the caller's workspace, zero-filled once
  unsigned barrier;                                     // arrivals; returns to 0 when the launch ends
  unsigned exits;
  unsigned error;                                       // sticky: 1 = a barrier wait ran out
  unsigned pad;
  unsigned long long row_best[kVerifyMaxRows];          // packed (max logit, lowest index) per row
  unsigned long long row_mass[kVerifyMaxRows];          // fixed-point mass of the kept set per row
  unsigned long long draft_w[kVerifyMaxRows];           // fixed-point weight of draft r in row r (0 if not kept)
  unsigned long long rival[kVerifyMaxRows];             // draft-side sampling: the best Gumbel key that lost (monotone code)
  // followed by: unsigned long long part_w[kVerifyMaxRows][grid], part_r[grid]
};

struct VerifyDev {
  int mode; int dtype; int n_draft; int vocab; int64_t row_stride;
  const void* target; const int32_t* drafts; const float* q; int64_t q_stride; float temperature;
  const uint16_t* q_logits; int64_t q_logits_stride; const float* q_vmax; const unsigned long long* q_mass;   // q from the drafter's BF16 logits when q is null
  const float* tau; const float* u_accept; const float* u_final;
  int32_t* out_accept; int32_t* out_final; int32_t* out_tokens; float* out_p_draft;
  VerifyWs* ws;
  int commit; AcceptDev accept;                          // commit != 0: close the round on the StepState as accept_scan would
};

// The round's bookkeeping, by the thread that has just written out_tokens: the accept scan on those tokens
// (kernels/common/spec_ops.metal:148-195). The verify rows must be the step's rows (a decode round: t_this_step = verify_len + 1
// = n_draft + 1); a prefill chunk takes the scan's prefill branch, which reads no token; anything else is a caller error and
// ends the generation with error code 4.
__device__ __forceinline__ void verify_commit(const VerifyDev& P) {
  if (!P.commit) return;
  StepStateView st{P.accept.state, P.accept.t_max, P.accept.g};
  if (!st.done() && P.ws->error != 0u) { st.error() = 3u; st.done() = 1u; return; }   // a grid barrier of this launch ran out: nothing to commit
  if (!st.done() && st.prefill_left() == 0u && (st.verify_len() != static_cast<uint32_t>(P.n_draft) || st.t_this_step() != static_cast<uint32_t>(P.n_draft) + 1u)) {
    st.error() = 4u; st.done() = 1u;
    return;
  }
  __threadfence();
  accept_scan_body(P.accept);
}

// Every block arrives, then waits until `target` arrivals are visible. Bounded: on time-out the error word is set and
// the block carries on (its results are then meaningless, the host sees the error).
__device__ __forceinline__ void grid_barrier(VerifyWs* ws, unsigned target) {
  __syncthreads();                                                        // the block's writes happen-before thread 0's release below
  if (threadIdx.x == 0) {
    unsigned seen = 0, spins = 0;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&ws->barrier) : "memory");
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&ws->barrier) : "memory");
      if (seen >= target) break;
      if (++spins > kBarrierSpinLimit) { atomicExch(&ws->error, 1u); break; }
    } while (true);
  }
  __syncthreads();
}

__device__ __forceinline__ uint64_t ws_load(const unsigned long long* p) { return __ldcg(p); }

__device__ __forceinline__ float verify_load(const VerifyDev& P, int row, int i) {
  const char* base = static_cast<const char*>(P.target);
  const float z = (P.dtype == LM_DTYPE_BF16)
                      ? __uint_as_float(static_cast<uint32_t>(__ldg(reinterpret_cast<const uint16_t*>(base) + static_cast<int64_t>(row) * P.row_stride + i)) << 16)
                      : __ldg(reinterpret_cast<const float*>(base) + static_cast<int64_t>(row) * P.row_stride + i);
  return canon_zero(z);
}

// q_r(v): the drafter's probability of token v at draft position r, as given or from the drafter's logits and row statistics.
__device__ __forceinline__ float q_from_code(uint32_t code, float vmax, unsigned long long mass, float c2) {
  return mass ? prob_q40(weight_q40(canon_zero(__uint_as_float(code << 16)), vmax, c2), mass) : 0.0f;
}
__device__ __forceinline__ float verify_q(const VerifyDev& P, int r, int i, float c2) {
  if (P.q) return __ldg(P.q + static_cast<int64_t>(r) * P.q_stride + i);
  return q_from_code(__ldg(P.q_logits + static_cast<int64_t>(r) * P.q_logits_stride + i), __ldg(P.q_vmax + r), __ldg(P.q_mass + r), c2);
}

// The block's view of its slice: shared-memory copies when they fit, global memory otherwise.
struct VerifySlice {
  const VerifyDev* P; const float* zs; const float* qs; int per, lo; float c2;
  __device__ __forceinline__ float z(int r, int i) const { return zs ? zs[r * per + i] : verify_load(*P, r, lo + i); }
  __device__ __forceinline__ float q(int r, int i) const { return qs ? qs[r * per + i] : verify_q(*P, r, lo + i, c2); }
};

#ifdef LM_PROFILE_PHASES
__device__ unsigned long long g_verify_times[8];
#define LM_VSTAMP(i) do { if (threadIdx.x == 0 && blockIdx.x == 0) { unsigned long long _t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); g_verify_times[i] = _t; } } while (0)
#else
#define LM_VSTAMP(i) do {} while (0)
#endif

__global__ void __launch_bounds__(kVerifyBlock, 1) verify_kernel(VerifyDev P, int cached) {
  extern __shared__ __align__(16) float v_smem[];
  __shared__ uint64_t scratch[32];
  __shared__ int s_j, s_token;
  __shared__ int s_drafts[kVerifyMaxRows];
  __shared__ unsigned long long s_best[kVerifyMaxRows], s_mass[kVerifyMaxRows];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, G = gridDim.x, b = blockIdx.x;
  constexpr int kWarps = kVerifyBlock / 32;
  const int R = P.n_draft + 1, V = P.vocab;
  const bool stochastic = P.mode == LM_VERIFY_STOCHASTIC;
  VerifyWs* ws = P.ws;
  unsigned long long* part_w = reinterpret_cast<unsigned long long*>(ws + 1);   // [kVerifyMaxRows][G]
  unsigned long long* part_r = part_w + static_cast<size_t>(kVerifyMaxRows) * G; // [G]
  // this block's vocabulary slice, a multiple of 8 elements
  const int per = ((V + G - 1) / G + 7) & ~7;
  const int lo = min(V, b * per), hi = min(V, lo + per);
  const int len = hi - lo;
  LM_VSTAMP(0);
  float* zs = cached ? v_smem : nullptr;
  float* qs = (cached && stochastic) ? v_smem + R * per : nullptr;
  const float c2 = stochastic ? exp2_scale(P.temperature) : 0.0f;
  VerifySlice S{&P, zs, qs, per, lo, c2};

  // ---- phase 0: the only HBM pass. Slices of every target row and every draft-probability row into shared memory,
  // then row maxima with their lowest index (which is also the greedy pick).
  // the scalars the accept test needs later are fetched now, so their latency hides behind the slice loads
  int my_draft = -1; float my_q = 0.0f, my_u = 0.0f;
  if (tid < P.n_draft) { my_draft = P.drafts[tid]; s_drafts[tid] = my_draft; }
  if (stochastic && tid < P.n_draft) {
    my_u = P.u_accept[tid];
    if (my_draft >= 0 && my_draft < V) my_q = verify_q(P, tid, my_draft, c2);
  }
  if (cached) {
    // 8 elements per load item (one 16-byte load of BF16 logits, two of FP32 logits or draft probabilities), every item of
    // a thread issued before the first is used: the whole slice arrives in one memory round trip
    const int n_q = stochastic ? P.n_draft : 0;
    const int chunks = (len + 7) / 8;
    const bool z_vec = (P.dtype == LM_DTYPE_BF16 ? (P.row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(P.target) & 15u) == 0)
                                                 : (P.row_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(P.target) & 15u) == 0));
    const bool q_vec = n_q == 0 || (P.q ? (P.q_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(P.q) & 15u) == 0)
                                        : (P.q_logits_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(P.q_logits) & 15u) == 0));
    const int n_items = (R + n_q) * chunks;
    constexpr int kItems = 3;                                             // items in flight per thread
    for (int i0 = 0; i0 < n_items; i0 += kItems * kVerifyBlock) {
      float4 va[kItems], vb[kItems];
#pragma unroll
      for (int k = 0; k < kItems; k++) {
        const int item = i0 + k * kVerifyBlock + tid;
        va[k] = make_float4(0.f, 0.f, 0.f, 0.f); vb[k] = va[k];
        if (item >= n_items) continue;
        const int r = item / chunks, c8 = (item - r * chunks) * 8;
        const bool full = c8 + 8 <= len;
        if (r < R) {
          if (P.dtype == LM_DTYPE_BF16) {
            const uint16_t* src = reinterpret_cast<const uint16_t*>(P.target) + static_cast<int64_t>(r) * P.row_stride + lo + c8;
            if (full && z_vec) va[k] = __ldg(reinterpret_cast<const float4*>(src));      // eight BF16 codes, widened below
          } else {
            const float* src = reinterpret_cast<const float*>(P.target) + static_cast<int64_t>(r) * P.row_stride + lo + c8;
            if (full && z_vec) { va[k] = __ldg(reinterpret_cast<const float4*>(src)); vb[k] = __ldg(reinterpret_cast<const float4*>(src) + 1); }
          }
        } else if (P.q) {
          const float* src = P.q + static_cast<int64_t>(r - R) * P.q_stride + lo + c8;
          if (full && q_vec) { va[k] = __ldg(reinterpret_cast<const float4*>(src)); vb[k] = __ldg(reinterpret_cast<const float4*>(src) + 1); }
        } else {
          const uint16_t* src = P.q_logits + static_cast<int64_t>(r - R) * P.q_logits_stride + lo + c8;
          if (full && q_vec) va[k] = __ldg(reinterpret_cast<const float4*>(src));          // eight BF16 codes of the drafter's row
        }
      }
#pragma unroll
      for (int k = 0; k < kItems; k++) {
        const int item = i0 + k * kVerifyBlock + tid;
        if (item >= n_items) continue;
        const int r = item / chunks, c8 = (item - r * chunks) * 8;
        const bool full = c8 + 8 <= len;
        float* dst = (r < R ? zs + r * per : qs + (r - R) * per) + c8;
        const bool vec = full && (r < R ? z_vec : q_vec);
        if (!vec) {                                                       // a ragged last chunk or an unaligned tensor: element by element
          for (int e = 0; e < 8 && c8 + e < len; e++)
            dst[e] = r < R ? verify_load(P, r, lo + c8 + e) : verify_q(P, r - R, lo + c8 + e, c2);
          continue;
        }
        float4 x = va[k], y = vb[k];
        if (r >= R && !P.q) {                                             // the drafter's logits: probabilities from the row statistics
          const float qv = __ldg(P.q_vmax + (r - R)); const unsigned long long qm = __ldg(P.q_mass + (r - R));
          const uint32_t w0 = __float_as_uint(va[k].x), w1 = __float_as_uint(va[k].y), w2 = __float_as_uint(va[k].z), w3 = __float_as_uint(va[k].w);
          x = make_float4(q_from_code(w0 & 0xFFFFu, qv, qm, c2), q_from_code(w0 >> 16, qv, qm, c2), q_from_code(w1 & 0xFFFFu, qv, qm, c2), q_from_code(w1 >> 16, qv, qm, c2));
          y = make_float4(q_from_code(w2 & 0xFFFFu, qv, qm, c2), q_from_code(w2 >> 16, qv, qm, c2), q_from_code(w3 & 0xFFFFu, qv, qm, c2), q_from_code(w3 >> 16, qv, qm, c2));
        }
        if (r < R && P.dtype == LM_DTYPE_BF16) {
          const uint32_t w0 = __float_as_uint(va[k].x), w1 = __float_as_uint(va[k].y), w2 = __float_as_uint(va[k].z), w3 = __float_as_uint(va[k].w);
          x = make_float4(bf16_lo(w0), bf16_hi(w0), bf16_lo(w1), bf16_hi(w1));
          y = make_float4(bf16_lo(w2), bf16_hi(w2), bf16_lo(w3), bf16_hi(w3));
        }
        if (r < R) {
          x = make_float4(canon_zero(x.x), canon_zero(x.y), canon_zero(x.z), canon_zero(x.w));
          y = make_float4(canon_zero(y.x), canon_zero(y.y), canon_zero(y.z), canon_zero(y.w));
        }
        reinterpret_cast<float4*>(dst)[0] = x; reinterpret_cast<float4*>(dst)[1] = y;
      }
    }
    __syncthreads();
  }
  LM_VSTAMP(1);
  // every row is shared by `split` warps; their partial results meet in the workspace through atomics
  const int split = max(1, kWarps / R);
  for (int item = warp; item < R * split; item += kWarps) {
    const int r = item / split, part = item - r * split;
    uint64_t best = 0ull;
    for (int i = part * 32 + lane; i < len; i += 32 * split) {
      const uint64_t p = pack_best(S.z(r, i), static_cast<uint32_t>(lo + i));
      best = p > best ? p : best;
    }
    best = warp_max_u64(best);
    if (lane == 0 && best) atomicMax(&ws->row_best[r], static_cast<unsigned long long>(best));
  }
  LM_VSTAMP(2);
  grid_barrier(ws, 1u * G);
  LM_VSTAMP(3);

  if (!stochastic) {
    if (b == 0 && tid < 32) {                                              // one round trip for every row's pick, then a vote
      const int pick = tid < R ? static_cast<int>(best_index(ws_load(&ws->row_best[tid]))) : -1;
      const uint32_t miss = __ballot_sync(kFull, tid < P.n_draft && pick != s_drafts[tid]);
      const int acc = miss ? (__ffs(miss) - 1) : P.n_draft;
      const int fin = __shfl_sync(kFull, pick, acc);
      const bool bad = ws->error != 0;
      if (tid == 0) { P.out_accept[0] = bad ? -1 : acc; P.out_final[0] = bad ? -1 : fin; }
      if (P.out_tokens && tid < R) P.out_tokens[tid] = tid < acc ? s_drafts[tid] : (tid == acc ? fin : -1);
      __syncwarp();
      if (tid == 0) verify_commit(P);
    }
    // the last block to leave puts the workspace back to its clean state
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(&ws->exits, 1u) == static_cast<unsigned>(G) - 1u) {
        for (int r = 0; r < R; r++) ws->row_best[r] = 0ull;
        ws->exits = 0u; __threadfence(); ws->barrier = 0u;
      }
    }
    return;
  }

  // ---- phase 1: fixed-point mass of every row's kept set; the drafts' own weights -----------------------------------
  if (tid < R) part_w[static_cast<size_t>(tid) * G + b] = 0ull;
  __syncthreads();
  for (int item = warp; item < R * split; item += kWarps) {
    const int r = item / split, part = item - r * split;
    const float vmax = best_value(ws_load(&ws->row_best[r]));
    const float tau = P.tau ? P.tau[r] : -INFINITY;
    uint64_t w = 0ull;
    for (int i = part * 32 + lane; i < len; i += 32 * split) {
      const float z = S.z(r, i);
      if (z >= tau) w += weight_q40(z, vmax, c2);
    }
    w = warp_sum_u64(w);
    if (lane == 0) {
      if (w) { atomicAdd(&part_w[static_cast<size_t>(r) * G + b], static_cast<unsigned long long>(w)); atomicAdd(&ws->row_mass[r], static_cast<unsigned long long>(w)); }
      if (part == 0 && r < P.n_draft) {
        const int d = s_drafts[r];
        if (d >= lo && d < hi) {
          const float z = S.z(r, d - lo);
          ws->draft_w[r] = (z >= tau) ? weight_q40(z, vmax, c2) : 0ull;
        }
      }
    }
  }
  LM_VSTAMP(4);
  grid_barrier(ws, 2u * G);
  LM_VSTAMP(5);

  // ---- phase 2: accept tests (every block, identically), then this slice's share of the residual mass -----------
  if (tid < 32) {                                                           // every row's maximum and mass in one round trip
    uint64_t best = 0ull, mass = 0ull, dw = 0ull;
    if (tid < R) { best = ws_load(&ws->row_best[tid]); mass = ws_load(&ws->row_mass[tid]); }
    if (tid < P.n_draft) dw = ws_load(&ws->draft_w[tid]);
    if (tid < R) { s_best[tid] = best; s_mass[tid] = mass; }
    bool reject = false;
    if (tid < P.n_draft) {
      const int r = tid, d = my_draft;
      const float pd = (d >= 0 && d < V && mass > 0ull) ? prob_q40(dw, mass) : 0.0f;
      reject = __fmul_rn(my_u, my_q) >= pd;
      if (b == 0 && P.out_p_draft) P.out_p_draft[r] = pd;
    }
    const uint32_t rejects = __ballot_sync(kFull, reject);
    if (tid == 0) s_j = rejects ? (__ffs(rejects) - 1) : P.n_draft;
  }
  __syncthreads();
  const int j = s_j;
  const float vmax_j = best_value(s_best[j]);
  const float tau_j = P.tau ? P.tau[j] : -INFINITY;
  const uint64_t mass_j = s_mass[j];
  const bool has_q = j < P.n_draft;
  // residual weight of element i of this slice (0 when not kept or not positive)
  auto residual = [&](int i) -> uint64_t {
    const float z = S.z(j, i);
    if (!(z >= tau_j)) return 0ull;
    const float p = prob_q40(weight_q40(z, vmax_j, c2), mass_j);
    const float res = has_q ? __fsub_rn(p, S.q(j, i)) : p;
    return res > 0.0f ? residual_q40(res) : 0ull;
  };
  {
    uint64_t w = 0ull;
    if (mass_j > 0ull) for (int i = tid; i < len; i += kVerifyBlock) w += residual(i);
    w = block_sum_u64(w, scratch);
    if (tid == 0) part_r[b] = w;
  }
  LM_VSTAMP(6);
  grid_barrier(ws, 3u * G);
  LM_VSTAMP(7);

  // ---- phase 3: locate the draw; the block whose slice holds it writes the outputs -------------------------------
  {
    // totals and this block's exclusive prefix over the per-block partials, for the residual and for the row's own mass
    uint64_t tot_r = 0ull, pre_r = 0ull, pre_w = 0ull;
    for (int g = tid; g < G; g += kVerifyBlock) {
      const uint64_t vr = ws_load(&part_r[g]), vw = ws_load(&part_w[static_cast<size_t>(j) * G + g]);
      tot_r += vr;
      if (g < b) { pre_r += vr; pre_w += vw; }
    }
    {                                                                     // three sums, one pair of barriers
      __shared__ uint64_t sums[3][32];
      tot_r = warp_sum_u64(tot_r); pre_r = warp_sum_u64(pre_r); pre_w = warp_sum_u64(pre_w);
      if (lane == 0) { sums[0][warp] = tot_r; sums[1][warp] = pre_r; sums[2][warp] = pre_w; }
      __syncthreads();
      tot_r = warp_sum_u64(lane < kWarps ? sums[0][lane] : 0ull);
      pre_r = warp_sum_u64(lane < kWarps ? sums[1][lane] : 0ull);
      pre_w = warp_sum_u64(lane < kWarps ? sums[2][lane] : 0ull);
    }
    const bool use_res = tot_r > 0ull;                                   // an empty residual: draw from the row's own kept softmax
    const uint64_t total = use_res ? tot_r : mass_j;
    const uint64_t mine = use_res ? ws_load(&part_r[b]) : ws_load(&part_w[static_cast<size_t>(j) * G + b]);
    const uint64_t pre = use_res ? pre_r : pre_w;
    if (tid == 0) s_token = -2;
    __syncthreads();
    if (total > 0ull) {
      const uint64_t target = cdf_target(P.u_final[0], total);
      if (mine > 0ull && pre <= target && target < pre + mine) {           // the crossing lies in this block's slice
        uint64_t base = pre;
        for (int i0 = 0; i0 < len; i0 += kVerifyBlock) {                  // uniform trip count: block-wide scans inside
          const int i = i0 + tid;
          uint64_t w = 0ull;
          if (i < len) {
            if (use_res) w = residual(i);
            else { const float z = S.z(j, i); if (z >= tau_j) w = weight_q40(z, vmax_j, c2); }
          }
          uint64_t sweep = 0ull;
          const uint64_t excl = block_exclusive_scan_u64(w, scratch, &sweep);
          if (w && base + excl <= target && target < base + excl + w) s_token = lo + i;
          base += sweep;
          __syncthreads();
          if (s_token != -2) break;
        }
        if (tid == 0) {
          const bool bad = ws->error != 0;
          P.out_accept[0] = bad ? -1 : j; P.out_final[0] = bad ? -1 : s_token;
          if (P.out_tokens) for (int r = 0; r < R; r++) P.out_tokens[r] = r < j ? P.drafts[r] : (r == j ? s_token : -1);
          verify_commit(P);
        }
      }
    } else if (b == 0 && tid == 0) {                                     // a row with no weight at all (empty or all -inf)
      P.out_accept[0] = ws->error ? -1 : j; P.out_final[0] = -1;
      if (P.out_tokens) for (int r = 0; r < R; r++) P.out_tokens[r] = r < j ? P.drafts[r] : -1;
      verify_commit(P);
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&ws->exits, 1u) == static_cast<unsigned>(G) - 1u) {
      for (int r = 0; r < R; r++) { ws->row_best[r] = 0ull; ws->row_mass[r] = 0ull; ws->draft_w[r] = 0ull; }
      ws->exits = 0u; __threadfence(); ws->barrier = 0u;
    }
  }
}

}  // namespace lm
