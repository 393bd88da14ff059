// Draft-side sampling: the Gumbel-max draw of draft k from the drafter's logits row plus the row statistics (maximum,
// fixed-point mass, log-sum-exp) that let the verify step evaluate q_k(v) later; optionally a copy of the row.
// Follows draft_q_partial / draft_q_final (kernels/common/sample.metal:212-269): same noise stream (2000 + k), same key
// z * float32(1/T) + g; the mass is kept as the integer sum of this library's fixed-point weights instead of an FP32
// running sum, so q_k(v) does not depend on how the row is split.
//
// One or a few rows of ~300 KB: latency-bound, so like the verify kernel this is one cooperative launch of one block per SM,
// every block owning the same vocabulary slice of every row (kept in shared memory between the two phases), one bounded
// grid barrier (the weights need the row maximum), and the last block to leave writes the outputs and cleans the workspace.
#pragma once
#include "common.cuh"
#include "spec_ops.cuh"

namespace lm {

constexpr int kDraftQBlock = 1024;
constexpr int kDraftQMaxRows = LM_MAX_DRAFT + 1;
constexpr unsigned kBarrierSpinLimit = 1u << 17;       // polls of the counter (about a microsecond each) before the wait gives up

struct DraftQWs {                                       // lives in the caller's workspace, zero-filled once, left all zero by every launch
  unsigned barrier;                                     // arrivals; returns to 0 when the launch ends
  unsigned exits;
  unsigned error;                                       // 1 = the barrier wait of this launch ran out
  unsigned nan_rows;                                    // bit r: row r holds a NaN
  unsigned long long row_best[kDraftQMaxRows];          // packed (max logit, lowest index) per row
  unsigned long long row_mass[kDraftQMaxRows];          // fixed-point mass per row
  unsigned long long key_best[kDraftQMaxRows];          // packed best Gumbel key per row
  unsigned long long rival[kDraftQMaxRows];             // the best Gumbel key that lost (monotone code)
};

// Every block arrives, then waits until `target` arrivals are visible. Bounded: on time-out the error word is set and
// the block carries on (its results are then meaningless; the outputs report the error).
__device__ __forceinline__ void grid_barrier(DraftQWs* ws, unsigned target) {
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

struct DraftQDev {
  int dtype; int rows; int first_position; int vocab; int64_t row_stride;
  const void* logits; float temperature; uint64_t seed; uint32_t step;
  int32_t* out_tokens; float* out_lse; float* out_vmax; unsigned long long* out_mass; uint32_t* out_status;
  void* out_q_logits; int64_t q_logits_stride;
  DraftQWs* ws;
  const uint32_t* state; int t_max, g;                   // optional StepState: seed and step come from it; a done state ends the launch
};

__global__ void __launch_bounds__(kDraftQBlock, 1) draft_q_kernel(DraftQDev P) {
  extern __shared__ __align__(16) float dq_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, G = gridDim.x, b = blockIdx.x;
  constexpr int kWarps = kDraftQBlock / 32;
  const int R = P.rows, V = P.vocab;
  DraftQWs* ws = P.ws;
  uint64_t seed = P.seed; uint32_t step = P.step;
  if (P.state) {
    StepStateView st{const_cast<uint32_t*>(P.state), P.t_max, P.g};
    if (st.done()) return;                                                // every block sees the same state: none touches the workspace
    seed = st.seed(); step = st.step();
  }
  unsigned long long* second = ws->rival;                                 // per row: the best key that is not the winner's
  const int per = ((V + G - 1) / G + 7) & ~7;
  const int lo = min(V, b * per), hi = min(V, lo + per);
  const int len = hi - lo;
  float* zs = dq_smem;                                                    // [R][per] widened logits of this block's slice

  // ---- phase 0: the slice of every row into shared memory (and into the copy, if one is wanted) ------------------------
  for (int i = tid; i < R * len; i += kDraftQBlock) {
    const int r = i / len, e = i - r * len;
    float z;
    if (P.dtype == LM_DTYPE_BF16) {
      const uint16_t code = __ldg(reinterpret_cast<const uint16_t*>(P.logits) + static_cast<int64_t>(r) * P.row_stride + lo + e);
      z = __uint_as_float(static_cast<uint32_t>(code) << 16);
      if (P.out_q_logits) reinterpret_cast<uint16_t*>(P.out_q_logits)[static_cast<int64_t>(r) * P.q_logits_stride + lo + e] = code;
    } else {
      z = __ldg(reinterpret_cast<const float*>(P.logits) + static_cast<int64_t>(r) * P.row_stride + lo + e);
      if (P.out_q_logits) reinterpret_cast<float*>(P.out_q_logits)[static_cast<int64_t>(r) * P.q_logits_stride + lo + e] = z;
    }
    zs[r * per + e] = canon_zero(z);
  }
  __syncthreads();
  // every row is shared by `split` warps: row maximum and best Gumbel key (with this thread's runner-up, for the tie flag)
  const int split = max(1, kWarps / R);
  const float inv_t32 = __double2float_rn(1.0 / static_cast<double>(P.temperature));
  uint64_t my_best = 0ull; float my_second = -INFINITY;                       // of the (single) item this warp owns
  for (int item = warp; item < R * split; item += kWarps) {
    const int r = item / split, part = item - r * split;
    const uint32_t t_id = 2000u + static_cast<uint32_t>(P.first_position + r);
    uint64_t vbest = 0ull, kbest = 0ull; float ksecond = -INFINITY; bool nan = false;
    for (int i = part * 32 + lane; i < len; i += 32 * split) {
      const float z = zs[r * per + i];
      const uint32_t idx = static_cast<uint32_t>(lo + i);
      nan = nan || (z != z);
      const uint64_t pv = pack_best(z, idx);
      vbest = pv > vbest ? pv : vbest;
      const float key = __fadd_rn(__fmul_rn(z, inv_t32), gumbel(seed, step, t_id, idx));
      const uint64_t pk = pack_best(key, idx);
      if (pk > kbest) { if (kbest) ksecond = fmaxf(ksecond, best_value(kbest)); kbest = pk; } else ksecond = fmaxf(ksecond, key);
    }
    const uint64_t wv = warp_max_u64(vbest), wk = warp_max_u64(kbest);
    if (lane == 0 && wv) atomicMax(&ws->row_best[r], static_cast<unsigned long long>(wv));
    if (lane == 0 && wk) atomicMax(&ws->key_best[r], static_cast<unsigned long long>(wk));
    if (__any_sync(kFull, nan) && lane == 0) atomicOr(&ws->nan_rows, 1u << r);
    if (item < kWarps) { my_best = kbest; my_second = ksecond; }            // R * split <= kWarps: one item per warp
  }
  grid_barrier(ws, 1u * G);

  // ---- phase 1: the fixed-point mass relative to the row maximum; the best key that lost ----------------------------------
  const float c2 = exp2_scale(P.temperature);
  for (int item = warp; item < R * split; item += kWarps) {
    const int r = item / split, part = item - r * split;
    const float vmax = best_value(ws_load(&ws->row_best[r]));
    const uint64_t winner = ws_load(&ws->key_best[r]);
    uint64_t w = 0ull;
    for (int i = part * 32 + lane; i < len; i += 32 * split) w += weight_q40(zs[r * per + i], vmax, c2);
    w = warp_sum_u64(w);
    if (lane == 0 && w) atomicAdd(&ws->row_mass[r], static_cast<unsigned long long>(w));
    // this thread's best candidate other than the winner, as a packed key (index irrelevant)
    float rival = (my_best == winner) ? my_second : (my_best ? best_value(my_best) : -INFINITY);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rival = fmaxf(rival, __shfl_xor_sync(kFull, rival, o));
    if (lane == 0 && rival > -INFINITY) atomicMax(&second[r], static_cast<unsigned long long>(fkey(rival)));
  }
  __syncthreads();
  __shared__ bool s_last;
  if (tid == 0) {
    __threadfence();
    s_last = atomicAdd(&ws->exits, 1u) == static_cast<unsigned>(G) - 1u;
  }
  __syncthreads();
  if (!s_last) return;
  // ---- the last block to arrive: outputs, and the workspace back to its clean state -----------------------------------------
  __threadfence();
  if (tid < R) {
    const int r = tid;
    const uint64_t vb = ws_load(&ws->row_best[r]), kb = ws_load(&ws->key_best[r]), mass = ws_load(&ws->row_mass[r]);
    const uint64_t sec = ws_load(&second[r]);
    const bool bad = ws->error != 0;
    const float vmax = best_value(vb);
    P.out_tokens[r] = (bad || !kb) ? -1 : static_cast<int>(best_index(kb));
    if (P.out_vmax) P.out_vmax[r] = vmax;
    if (P.out_mass) P.out_mass[r] = mass;
    if (P.out_lse) P.out_lse[r] = mass ? __double2float_rn(static_cast<double>(vmax) / static_cast<double>(P.temperature) + log(static_cast<double>(mass) * 9.094947017729282e-13)) : -INFINITY;
    if (P.out_status) {
      uint32_t st = 0u;
      if (kb && sec && fkey_inv(static_cast<uint32_t>(sec)) >= best_value(kb) - 4e-6f) st |= LM_STATUS_NEAR_TIE;
      if ((__ldcg(&ws->nan_rows) >> r) & 1u) st |= LM_STATUS_NAN;
      P.out_status[r] = st;
    }
    ws->row_best[r] = 0ull; ws->key_best[r] = 0ull; ws->row_mass[r] = 0ull; second[r] = 0ull;
  }
  __syncthreads();
  if (tid == 0) { ws->nan_rows = 0u; ws->error = 0u; ws->exits = 0u; __threadfence(); ws->barrier = 0u; }
}

}  // namespace lm
