// DSpark verification of one speculative step in ONE launch: up to n_draft drafted tokens against n_draft + 1 rows of target
// logits. Greedy: row-wise argmax and prefix match (kernels/common/spec_ops.metal:162-165). Stochastic: accept draft r with
// probability min(1, p/q), replace the first rejected one by a draw from max(p - q, 0) (kernels/common/sample.metal:273-347),
// on the integer fixed-point weights so the outcome is independent of how the vocabulary is split between blocks.
//
// The step is latency-bound (a few MB of input, a chain of three data dependencies: row maxima -> row masses and the accept
// test -> the residual's total -> the token), so the kernel is one cooperative launch of one block per SM; every block owns the
// same vocabulary slice of every row in every phase. Phase 0 is the only one that touches HBM: it pulls the block's slice of
// all target rows and all draft rows into shared memory (every load in flight at once); the later phases work from there.
//
// Blocks exchange their partial results through TAGGED WORDS in a small workspace: every partial is one 64-bit word whose top
// bit says "written". A block publishes with one plain store per word and consumes by polling the words it needs, so a
// dependency costs one trip to L2 and back -- no counter, no fence, no second read. The words live in one of two BANKS. A launch
// uses the bank its number selects, and every block clears its own words of the other bank while its loads are in flight, so
// the next launch finds a clean bank and nobody tidies up at the end. The launch number is the count of blocks that have ever
// left, divided by the grid size: a block adds itself on its way out (no reply awaited), and the quotient cannot change before
// the last block of the launch has read it. The workspace starts all zero and belongs to one device (one grid size). Every poll
// is bounded: when it runs out the launch reports an error through its outputs (and through the StepState when it commits); the
// GPU is never left waiting.
//
// With a StepState given, the kernel takes the round from it on the device, as the reference's kernels do
// (kernels/common/sample.metal:283-296): verify length, drafts (pending_tokens), seed, step, and it leaves at once when the
// state is done. The accept uniforms then come from the reference's stream 3000 + r of the counter-based noise.
#pragma once
#include "common.cuh"
#include "spec_ops.cuh"

namespace lm {

constexpr int kVerifyBlock = 1024;
constexpr int kVerifyWarps = kVerifyBlock / 32;
constexpr int kVerifyMaxRows = LM_MAX_DRAFT + 1;
constexpr int kVerifyMaxGrid = 1024;                    // far above any SM count
constexpr unsigned kVerifyWaitLimit = 1u << 17;         // polls of one word before a wait gives up: about 0.1 s
constexpr unsigned long long kTagged = 1ull << 63;

struct VerifyBank {
  unsigned error;                                       // a wait of the launch that used this bank ran out
  unsigned pad[3];
  unsigned long long draft_w[kVerifyMaxRows];           // tagged: fixed-point weight of draft r in row r (0 if not kept)
  unsigned long long best[kVerifyMaxRows][kVerifyMaxGrid];   // tagged: per row and block, the slice's packed (max logit, lowest index)
  unsigned long long mass[kVerifyMaxRows][kVerifyMaxGrid];   // tagged: per row and block, the slice's fixed-point mass
  unsigned long long resid[2][kVerifyMaxGrid];          // tagged: per block, the slice's residual mass / its best draw keys
};
struct VerifyWs {                                       // lives in the caller's workspace, zero-filled once
  unsigned long long exits;                             // blocks that have ever left: grid size x launches so far
  unsigned long long pad;
  VerifyBank bank[2];
};

struct VerifyDev {
  int mode; int dtype; int n_draft; int vocab; int64_t row_stride; int draw;
  const void* target; const int32_t* drafts; const float* q; int64_t q_stride; float temperature;
  const uint16_t* q_logits; int64_t q_logits_stride; const float* q_vmax; const unsigned long long* q_mass;   // q from the drafter's BF16 logits when q is null
  const float* tau; const float* u_accept; const float* u_final;
  const float* row_max;                                  // stochastic mode, optional: the exact maxima of the step's rows (from the sampler): spares the first exchange
  const unsigned long long* row_mass;                    // ... and their kept sets' fixed-point masses (needs row_max): the accept test needs no exchange at all
  uint64_t seed; uint32_t step;
  int32_t* out_accept; int32_t* out_final; int32_t* out_tokens; float* out_p_draft;
  VerifyWs* ws;
  uint32_t* state; int t_max, g;                          // StepState (optional): the round is read from it
  int commit; AcceptDev accept;                          // commit != 0: close the round on the StepState as accept_scan would
  unsigned wait_limit; unsigned withhold;                // self-test of the bounded waits: block 0 publishes no row maxima
};

// ---- tagged words ------------------------------------------------------------------------------------------------------------
// The 52-bit packed (value, lowest index) of the row maxima: indices stay below 2^20 (LM_MAX_VOCAB).
__device__ __forceinline__ uint64_t pack52(float v, uint32_t idx) { return (static_cast<uint64_t>(fkey(v)) << 20) | (0xFFFFFu - idx); }
__device__ __forceinline__ float pack52_value(uint64_t p) { return fkey_inv(static_cast<uint32_t>(p >> 20)); }
__device__ __forceinline__ uint32_t pack52_index(uint64_t p) { return 0xFFFFFu - static_cast<uint32_t>(p & 0xFFFFFu); }

__device__ __forceinline__ void publish(unsigned long long* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(static_cast<unsigned long long>(v) | kTagged) : "memory");
}
__device__ __forceinline__ unsigned long long peek(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Polls one word until its tag is set; gives up after `limit` polls (then *failed is set and 0 returned). `first`: a value
// already read from the word.
__device__ __forceinline__ uint64_t consume(const unsigned long long* p, unsigned limit, bool* failed, unsigned long long first = 0ull) {
  unsigned long long v = first;
  for (unsigned spins = 0;; spins++) {
    if (v & kTagged) return v & ~kTagged;
    if (spins >= limit) { *failed = true; return 0ull; }
    if (spins > 64u) __nanosleep(100);                                    // a long wait: leave the memory system to the blocks still working
    v = peek(p);
  }
}

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

// The block's view of its slice: shared-memory copies when they fit, global memory otherwise. Target rows are step rows
// (row0 + r), draft rows are draft positions r.
struct VerifySlice {
  const VerifyDev* P; const float* zs; const float* qs; int per, lo, row0; float c2;
  __device__ __forceinline__ float z(int r, int i) const { return zs ? zs[r * per + i] : verify_load(*P, row0 + r, lo + i); }
  __device__ __forceinline__ float q(int r, int i) const { return qs ? qs[r * per + i] : verify_q(*P, r, lo + i, c2); }
};

// The round's bookkeeping, by the warp whose lane 0 has just written out_tokens: the accept scan on those tokens
// (kernels/common/spec_ops.metal:148-195). A prefill chunk takes the scan's prefill branch, which reads no token. All 32 lanes call.
__device__ __forceinline__ void verify_commit(const VerifyDev& P, bool failed) {
  if (!P.commit) return;
  __syncwarp();
  StepStateView st{P.accept.state, P.accept.t_max, P.accept.g};
  if (st.done()) return;
  if (failed) { if ((threadIdx.x & 31) == 0) fail_state(st, kErrBarrier); return; }   // a wait of this launch ran out: nothing to commit
  if (!P.state && st.prefill_left() == 0u && (st.verify_len() != static_cast<uint32_t>(P.n_draft) || st.t_this_step() != static_cast<uint32_t>(P.n_draft) + 1u)) {
    if ((threadIdx.x & 31) == 0) fail_state(st, kErrRoundMismatch);        // the round came from the arguments and the state describes another
    return;
  }
  __threadfence();
  round_close(P.accept);
}

constexpr int kConsumeSlots = 4;                        // words one thread may hold: rows x grid (rounded up to 32) <= 4096

// Consumes words[r][g] for r < R, g < G (row stride kVerifyMaxGrid) and reduces each row over g (SUM false: maximum, true:
// sum) into out[r] (shared memory). Warps take 32 consecutive blocks of one row at a time. The values a thread consumed stay
// in vals[] (0 where it had none), vals[k] belonging to word k * kVerifyBlock + tid of the R x Gp index space. Every thread calls.
template <bool SUM>
__device__ __forceinline__ void consume_rows(const unsigned long long* words, int R, int G, unsigned long long* out, uint64_t (*red)[32],
                                             unsigned limit, bool* failed, uint64_t vals[kConsumeSlots]) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int Gp = (G + 31) & ~31, n = R * Gp;
  // Every word of this thread is in flight at once, on the first look and on every further one: a word that is not there yet
  // costs one more round trip for all of the thread's words together, not one each.
  const unsigned long long* addr[kConsumeSlots];
  unsigned long long got[kConsumeSlots];
#pragma unroll
  for (int k = 0; k < kConsumeSlots; k++) {
    const int idx = k * kVerifyBlock + tid, r = idx / Gp, g = idx - r * Gp;
    addr[k] = (idx < n && g < G) ? words + static_cast<size_t>(r) * kVerifyMaxGrid + g : nullptr;
    got[k] = addr[k] ? peek(addr[k]) : kTagged;
  }
  for (unsigned spins = 0;; spins++) {
    bool all = true;
#pragma unroll
    for (int k = 0; k < kConsumeSlots; k++) all = all && (got[k] & kTagged) != 0ull;
    if (all) break;
    if (spins >= limit) { *failed = true; break; }
    if (spins > 64u) __nanosleep(100);                                    // a long wait: leave the memory system to the blocks still working
#pragma unroll
    for (int k = 0; k < kConsumeSlots; k++) if (!(got[k] & kTagged)) got[k] = peek(addr[k]);
  }
#pragma unroll
  for (int k = 0; k < kConsumeSlots; k++) {
    const int idx = k * kVerifyBlock + tid, r = idx / Gp, g = idx - r * Gp;
    const uint64_t v = (got[k] & kTagged) ? (got[k] & ~kTagged) : 0ull;
    vals[k] = v;
    if (k * kVerifyBlock < n) {                                           // block-uniform
      const uint64_t w = SUM ? warp_sum_u64(v) : warp_max_u64(v);
      if (lane == 0 && idx < n) red[r][g >> 5] = w;
    }
  }
  __syncthreads();
  if (tid < R) {
    uint64_t acc = 0ull;
    for (int k = 0; k < Gp / 32; k++) { const uint64_t x = red[tid][k]; acc = SUM ? acc + x : (x > acc ? x : acc); }
    out[tid] = acc;
  }
  __syncthreads();
}

// kStats: the launch was given the rows' maxima and masses (compiled apart: the launch that has to find them runs code that is
// laid out as if the other did not exist, and the step is short enough for that to show).
template <bool kStats>
__global__ void __launch_bounds__(kVerifyBlock, 1) verify_kernel(VerifyDev P, int cached) {
  extern __shared__ __align__(16) float v_smem[];
  __shared__ uint64_t scratch[32];
  __shared__ uint64_t s_red[kVerifyMaxRows][32];
  __shared__ int s_j, s_token, s_j2;
  __shared__ unsigned long long s_pre2;
  __shared__ int s_drafts[kVerifyMaxRows];
  __shared__ unsigned long long s_best[kVerifyMaxRows], s_mass[kVerifyMaxRows], s_own[kVerifyMaxRows];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, G = gridDim.x, b = blockIdx.x;
  const int V = P.vocab;
  const bool stochastic = P.mode == LM_VERIFY_STOCHASTIC;
  const bool gumbel_draw = stochastic && P.draw == LM_DRAW_GUMBEL;
  // the bank of this launch (the load is in flight under phase 0; its value is first needed when the row maxima are published)
  unsigned long long launches;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(launches) : "l"(&P.ws->exits) : "memory");
  const unsigned bank_id = static_cast<unsigned>((launches / static_cast<unsigned long long>(G)) & 1ull);
  VerifyBank* ws = &P.ws->bank[bank_id];
  const unsigned limit = P.wait_limit ? P.wait_limit : kVerifyWaitLimit;
  bool failed = false;

  // ---- the round: from the arguments, or from the StepState ---------------------------------------------------------------
  int L = P.n_draft, row0 = 0;
  uint64_t seed = P.seed; uint32_t step = P.step;
  bool idle = false, mismatch = false;                                    // idle: the state is done, or this step is a prefill chunk
  bool prefill = false;
  if (P.state) {
    StepStateView st{P.state, P.t_max, P.g};
    if (st.done()) idle = true;
    else if (st.prefill_left() > 0u) { idle = true; prefill = true; }
    else {
      const uint32_t len = st.verify_len(), rows = st.t_this_step();
      if (len > static_cast<uint32_t>(P.n_draft) || rows < len + 1u || rows > static_cast<uint32_t>(P.n_draft) + 1u) mismatch = true;
      else { L = static_cast<int>(len); row0 = static_cast<int>(rows - 1u - len); }
    }
    seed = st.seed(); step = st.step();
  }
  const int R = L + 1;
  // this block's words of the other bank (the previous launch's) are cleared for the next launch; block 0 also clears the shared ones
  auto clean_other_bank = [&]() {
    VerifyBank* other = &P.ws->bank[bank_id ^ 1u];
    if (tid < kVerifyMaxRows) { other->best[tid][b] = 0ull; other->mass[tid][b] = 0ull; }
    if (tid < 2) other->resid[tid][b] = 0ull;
    if (b == 0 && tid < kVerifyMaxRows) other->draft_w[tid] = 0ull;
    if (b == 0 && tid == 0) other->error = 0u;
  };
  if (idle || mismatch) {
    clean_other_bank();                                                   // (the launch still counts: the banks keep alternating)
    // nothing is verified; block 0 still closes a prefill chunk (the scan's prefill branch) or reports the caller's error
    if (b == 0 && warp == 0) {
      if (mismatch) {
        if (lane == 0) { P.out_accept[0] = -1; P.out_final[0] = -1; StepStateView st{P.state, P.t_max, P.g}; fail_state(st, kErrRoundMismatch); }
      } else if (prefill) verify_commit(P, false);
    }
  } else {
  // this block's vocabulary slice, a multiple of 8 elements
  const int per = ((V + G - 1) / G + 7) & ~7;
  const int lo = min(V, b * per), hi = min(V, lo + per);
  const int len = hi - lo;
  const int chunks = (len + 7) / 8;                                        // 8-element load items of one row of the slice
  float* zs = cached ? v_smem : nullptr;
  float* qs = (cached && stochastic) ? v_smem + (P.n_draft + 1) * per : nullptr;
  const float c2 = stochastic ? exp2_scale(P.temperature) : 0.0f;
  VerifySlice S{&P, zs, qs, per, lo, row0, c2};

  const bool given_max = kStats || (stochastic && P.row_max != nullptr);              // the sampler already knows the rows' maxima: nothing to find or exchange
  const bool given_mass = kStats;                                         // ... and the masses of their kept sets: only the draw is left to do together

  // ---- phase 0: the only HBM pass. Slices of every target row and every draft row into shared memory.
  // The scalars the accept test needs later are fetched now, so their latency hides behind the slice loads.
  int my_draft = -1; float my_q = 0.0f, my_u = 0.0f;
  if (tid < L) {
    my_draft = P.state ? StepStateView{P.state, P.t_max, P.g}.pending(row0 + tid + 1) : P.drafts[tid];
    s_drafts[tid] = my_draft;
  }
  if (stochastic && tid < L) {
    my_u = P.u_accept ? P.u_accept[tid] : uniform01(seed, step, 3000u + static_cast<uint32_t>(tid), 0u);
    if (my_draft >= 0 && my_draft < V) my_q = verify_q(P, tid, my_draft, c2);
  }
  unsigned long long my_mass = 0ull; float my_zd = -INFINITY;              // given the masses: the row's mass and the draft's own logit, fetched now too
  if (given_mass) {
    if (tid < R) my_mass = P.row_mass[row0 + tid];
    if (tid < L && my_draft >= 0 && my_draft < V) my_zd = verify_load(P, row0 + tid, my_draft);
  }
  if (cached) {
    // 8 elements per load item (one 16-byte load of BF16 logits, two of FP32 logits or draft probabilities), every item of
    // a thread issued before the first is used: the whole slice arrives in one memory round trip
    const int n_q = stochastic ? L : 0;
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
        const int r = item / chunks, ci = item - r * chunks, c8 = ci * 8;
        if (item >= n_items) continue;
        const bool full = c8 + 8 <= len;
        if (r < R) {
          if (P.dtype == LM_DTYPE_BF16) {
            const uint16_t* src = reinterpret_cast<const uint16_t*>(P.target) + static_cast<int64_t>(row0 + r) * P.row_stride + lo + c8;
            if (full && z_vec) va[k] = __ldg(reinterpret_cast<const float4*>(src));      // eight BF16 codes, widened below
          } else {
            const float* src = reinterpret_cast<const float*>(P.target) + static_cast<int64_t>(row0 + r) * P.row_stride + lo + c8;
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
        const int r = item / chunks, ci = item - r * chunks, c8 = ci * 8;
        const bool full = c8 + 8 <= len;
        float* dst = (r < R ? zs + r * per : qs + (r - R) * per) + c8;
        const bool vec = full && (r < R ? z_vec : q_vec);
        if (!vec) {                                                       // a ragged last chunk or an unaligned tensor: element by element
          for (int e = 0; e < 8 && c8 + e < len; e++)
            dst[e] = r < R ? verify_load(P, row0 + r, lo + c8 + e) : verify_q(P, r - R, lo + c8 + e, c2);
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
  // ---- row maxima of the slice (lowest index on ties: the greedy pick), published one word per row -----------------------
  // A block of 1024 threads keeps every scheduler of the SM busy, so what counts is the total number of instructions: the rows
  // are walked four elements per shared-memory load, a warp staying inside one row (rows padded to 32 groups of four), and only
  // the warps that hold data reduce.
  const int n4 = (len + 3) / 4, n4p = (n4 + 31) & ~31;                      // groups of four elements per row of the slice
  const int split = max(1, kVerifyWarps / R);                              // without the shared-memory copy every row is shared by `split` warps
  const int n_red = cached ? n4p / 32 : split;                             // partial results per row in s_red
  if (given_max) {
    if (tid < R) s_best[tid] = pack52(canon_zero(P.row_max[row0 + tid]), 0u);
  } else if (cached) {
    // stochastic: the value alone (a 32-bit key); greedy: value and lowest index together (the 52-bit pack)
    for (int i0 = 0; i0 < R * n4p; i0 += kVerifyBlock) {
      const int r0 = (i0 + (tid & ~31)) / n4p;
      if (r0 >= R) break;                                                 // warp-uniform
      const int item = i0 + tid, c4 = item - r0 * n4p;
      const int left = len - 4 * c4;                                      // 4 except in a ragged last group
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c4 < n4) x = reinterpret_cast<const float4*>(zs + r0 * per)[c4];
      if (stochastic) {
        uint32_t key = 0u;
        if (c4 < n4) {
          key = fkey(x.x);
          if (left > 1) key = max(key, fkey(x.y));
          if (left > 2) key = max(key, fkey(x.z));
          if (left > 3) key = max(key, fkey(x.w));
        }
        key = warp_max_u32(key);
        if (lane == 0) s_red[r0][c4 >> 5] = static_cast<uint64_t>(key) << 20;
      } else {
        uint64_t best = 0ull;
        if (c4 < n4) {
          const uint32_t i4 = static_cast<uint32_t>(lo + 4 * c4);
          best = pack52(x.x, i4);
          if (left > 1) { const uint64_t p = pack52(x.y, i4 + 1u); best = p > best ? p : best; }
          if (left > 2) { const uint64_t p = pack52(x.z, i4 + 2u); best = p > best ? p : best; }
          if (left > 3) { const uint64_t p = pack52(x.w, i4 + 3u); best = p > best ? p : best; }
        }
        best = warp_max_u64(best);
        if (lane == 0) s_red[r0][c4 >> 5] = best;
      }
    }
    __syncthreads();
    if (tid < R && !(P.withhold && b == 0)) {
      uint64_t best = 0ull;
      for (int k = 0; k < n_red; k++) best = s_red[tid][k] > best ? s_red[tid][k] : best;
      publish(&ws->best[tid][b], best);
    }
  } else {
    for (int item = warp; item < R * split; item += kVerifyWarps) {
      const int r = item / split, part = item - r * split;
      uint64_t best = 0ull;
      for (int i = part * 32 + lane; i < len; i += 32 * split) {
        const uint64_t p = pack52(S.z(r, i), static_cast<uint32_t>(lo + i));
        best = p > best ? p : best;
      }
      best = warp_max_u64(best);
      if (lane == 0) s_red[r][part] = best;
    }
    __syncthreads();
    if (tid < R && !(P.withhold && b == 0)) {
      uint64_t best = 0ull;
      for (int k = 0; k < n_red; k++) best = s_red[tid][k] > best ? s_red[tid][k] : best;
      publish(&ws->best[tid][b], best);
    }
  }
  clean_other_bank();
  __syncthreads();                                                        // s_red is reused below

  uint64_t vals[kConsumeSlots] = {0ull, 0ull, 0ull, 0ull};
  const int Gp = (G + 31) & ~31;
  if (!stochastic) {
    // ---- greedy: block 0 gathers every row's pick and votes; the others are done --------------------------------------------
    if (b == 0) {
      consume_rows<false>(&ws->best[0][0], R, G, s_best, s_red, limit, &failed, vals);
      const bool bad = __syncthreads_or(failed) != 0;
      if (bad && tid == 0) atomicExch(&ws->error, 1u);
      if (tid < 32) {
        const int pick = tid < R ? static_cast<int>(pack52_index(s_best[tid])) : -1;
        const uint32_t miss = __ballot_sync(kFull, tid < L && pick != s_drafts[tid]);
        const int acc = miss ? (__ffs(miss) - 1) : L;
        const int fin = __shfl_sync(kFull, pick, acc);
        if (tid == 0) { P.out_accept[0] = bad ? -1 : acc; P.out_final[0] = bad ? -1 : fin; }
        if (P.out_tokens && tid < R) P.out_tokens[row0 + tid] = bad ? -1 : (tid < acc ? s_drafts[tid] : (tid == acc ? fin : -1));
        verify_commit(P, bad);
      }
    }
  } else {
    // ---- phase 1: every block learns the row maxima; fixed-point mass of every row's kept set; the drafts' own weights -------
    if (!given_max) consume_rows<false>(&ws->best[0][0], R, G, s_best, s_red, limit, &failed, vals);
    if (given_mass) {
      // nothing to sum: the sampler's masses, and every block evaluates the drafts' weights itself (one logit each)
    } else if (cached) {
      // the same walk as for the maxima: four elements per load, two packed weight evaluations, one warp sum per 128 elements
      for (int i0 = 0; i0 < R * n4p; i0 += kVerifyBlock) {
        const int r0 = (i0 + (tid & ~31)) / n4p;
        if (r0 >= R) break;                                               // warp-uniform
        const int item = i0 + tid, c4 = item - r0 * n4p;
        uint64_t w = 0ull;
        if (c4 < n4) {
          const float vmax = pack52_value(s_best[r0]);
          const float tau = P.tau ? P.tau[row0 + r0] : -INFINITY;
          const float4 x = reinterpret_cast<const float4*>(zs + r0 * per)[c4];
          const int left = len - 4 * c4;
          uint64_t w0, w1, w2, w3;
          weight_q40_x2(x.x, x.y, vmax, c2, w0, w1);
          weight_q40_x2(x.z, x.w, vmax, c2, w2, w3);
          if (x.x >= tau) w += w0;
          if (left > 1 && x.y >= tau) w += w1;
          if (left > 2 && x.z >= tau) w += w2;
          if (left > 3 && x.w >= tau) w += w3;
        }
        const uint32_t wl = warp_sum_u32(static_cast<uint32_t>(w) & 0x3FFFFFu), wh = warp_sum_u32(static_cast<uint32_t>(w >> 22));
        if (lane == 0) s_red[r0][c4 >> 5] = static_cast<uint64_t>(wl) + (static_cast<uint64_t>(wh) << 22);
      }
      if (tid < L) {                                                      // the drafts' own weights: the block whose slice holds the draft
        const int d = s_drafts[tid];
        if (d >= lo && d < hi) {
          const float z = S.z(tid, d - lo), tau = P.tau ? P.tau[row0 + tid] : -INFINITY;
          publish(&ws->draft_w[tid], (z >= tau) ? weight_q40(z, pack52_value(s_best[tid]), c2) : 0ull);
        } else if ((d < 0 || d >= V) && b == 0) publish(&ws->draft_w[tid], 0ull);     // an id outside the vocabulary: probability 0
      }
    } else {
    for (int item = warp; item < R * split; item += kVerifyWarps) {
      const int r = item / split, part = item - r * split;
      const float vmax = pack52_value(s_best[r]);
      const float tau = P.tau ? P.tau[row0 + r] : -INFINITY;
      uint64_t w = 0ull;
      for (int i = part * 32 + lane; i < len; i += 32 * split) {
        const float z = S.z(r, i);
        if (z >= tau) w += weight_q40(z, vmax, c2);
      }
      w = warp_sum_u64(w);
      if (lane == 0) {
        s_red[r][part] = w;
        if (part == 0 && r < L) {
          const int d = s_drafts[r];
          if (d >= lo && d < hi) {
            const float z = S.z(r, d - lo);
            publish(&ws->draft_w[r], (z >= tau) ? weight_q40(z, vmax, c2) : 0ull);
          } else if ((d < 0 || d >= V) && b == 0) publish(&ws->draft_w[r], 0ull);   // an id outside the vocabulary: probability 0
        }
      }
    }
    }
    __syncthreads();
    if (tid < R && !given_mass) {
      uint64_t w = 0ull;
      for (int k = 0; k < n_red; k++) w += s_red[tid][k];
      s_own[tid] = w;
      publish(&ws->mass[tid][b], w);
    }
    if (tid < R && given_mass) s_mass[tid] = my_mass;
    __syncthreads();
    // ---- phase 2: row masses; accept tests (every block, identically); this slice's share of the residual -------------------
    const unsigned long long dw_first = (tid < L && !given_mass) ? peek(&ws->draft_w[tid]) : 0ull;   // in flight while the masses are consumed
    if (!given_mass) consume_rows<true>(&ws->mass[0][0], R, G, s_mass, s_red, limit, &failed, vals);
    if (tid < 32) {
      bool reject = false;
      if (tid < L) {
        uint64_t dw;
        if (given_mass) {                                                  // the draft's own weight, straight from its logit
          const float tau = P.tau ? P.tau[row0 + tid] : -INFINITY;
          dw = (my_zd >= tau) ? weight_q40(my_zd, pack52_value(s_best[tid]), c2) : 0ull;
        } else dw = consume(&ws->draft_w[tid], limit, &failed, dw_first);
        const uint64_t mass = s_mass[tid];
        const float pd = (my_draft >= 0 && my_draft < V && mass > 0ull) ? prob_q40(dw, mass) : 0.0f;
        reject = __fmul_rn(my_u, my_q) >= pd;
        if (b == 0 && P.out_p_draft) P.out_p_draft[tid] = pd;
      }
      const uint32_t rejects = __ballot_sync(kFull, reject);
      if (tid == 0) s_j = rejects ? (__ffs(rejects) - 1) : L;
    }
    __syncthreads();
    const int j = s_j;
    const float vmax_j = pack52_value(s_best[j]);
    const float tau_j = P.tau ? P.tau[row0 + j] : -INFINITY;
    const uint64_t mass_j = s_mass[j];
    const bool has_q = j < L;
    // this block's exclusive prefix over the blocks' masses of row j (the draw over p itself needs it)
    uint64_t pre_w = 0ull;
    if (!given_mass) {
#pragma unroll
      for (int k = 0; k < kConsumeSlots; k++) {
        const int idx = k * kVerifyBlock + tid, r = idx / Gp, g = idx - r * Gp;
        if (r == j && g < b) pre_w += vals[k];
      }
      pre_w = block_sum_u64(pre_w, scratch);
    }
    uint64_t own_w = given_mass ? 0ull : s_own[j];                         // this block's share of row j's mass (the draw over p itself)
    // residual weight of element i of this slice (0 when not kept or not positive)
    auto residual_of = [&](const VerifySlice& V2, int i) -> uint64_t {
      const float z = V2.z(j, i);
      if (!(z >= tau_j)) return 0ull;
      const float p = prob_q40(weight_q40(z, vmax_j, c2), mass_j);
      const float res = has_q ? __fsub_rn(p, V2.q(j, i)) : p;
      return res > 0.0f ? residual_q40(res) : 0ull;
    };
    auto residual = [&](int i) -> uint64_t { return residual_of(S, i); };
    // the token inside a slice (lo2, len2, read through V2): the first element, in index order, at which the running weight -- the
    // residual's, or the row's own when the residual is empty -- passes the target; `base` = the weight of everything before the slice
    auto locate = [&](const VerifySlice& V2, int lo2, int len2, uint64_t base, bool use_res, uint64_t target) -> int {
      if (tid == 0) s_token = -2;
      __syncthreads();
      for (int i0 = 0; i0 < len2; i0 += kVerifyBlock) {                     // uniform trip count: block-wide scans inside
        const int i = i0 + tid;
        uint64_t w = 0ull;
        if (i < len2) {
          if (use_res) w = residual_of(V2, i);
          else { const float z = V2.z(j, i); if (z >= tau_j) w = weight_q40(z, vmax_j, c2); }
        }
        uint64_t sweep = 0ull;
        const uint64_t excl = block_exclusive_scan_u64(w, scratch, &sweep);
        if (w && base + excl <= target && target < base + excl + w) s_token = lo2 + i;
        base += sweep;
        __syncthreads();
        if (s_token != -2) break;
      }
      return s_token;
    };
    const uint32_t t_row = static_cast<uint32_t>(row0 + j);
    const float inv_t32 = __double2float_rn(1.0 / static_cast<double>(P.temperature));
    uint64_t total_r = 0ull, mine_r = 0ull;
    int token = -2;
    if (gumbel_draw) {
      // the reference's draws (kernels/common/sample.metal:322-346): argmax of ln(p - q) + noise of stream 4000 over the positive
      // residual; with nothing rejected, or an empty residual, the row's own Gumbel-max draw on its stream (the sampler's token)
      uint64_t best_res = 0ull, best_own = 0ull;
      if (mass_j > 0ull) for (int i = tid; i < len; i += kVerifyBlock) {
        const float z = S.z(j, i);
        if (!(z >= tau_j)) continue;
        const uint32_t idx = static_cast<uint32_t>(lo + i);
        const uint64_t own = pack52(__fadd_rn(__fmul_rn(z, inv_t32), gumbel(seed, step, t_row, idx)), idx);
        best_own = own > best_own ? own : best_own;
        if (has_q) {
          const float res = __fsub_rn(prob_q40(weight_q40(z, vmax_j, c2), mass_j), S.q(j, i));
          if (res > 0.0f) { const uint64_t k = pack52(__fadd_rn(logf(res), gumbel(seed, step, 4000u, idx)), idx); best_res = k > best_res ? k : best_res; }
        }
      }
      best_res = block_max_u64(best_res, scratch);
      best_own = block_max_u64(best_own, scratch);
      if (tid == 0) { publish(&ws->resid[0][b], best_res); publish(&ws->resid[1][b], best_own); }
      if (b == 0) {                                                       // block 0 gathers the blocks' best keys
        uint64_t kr = 0ull, ko = 0ull;
        for (int g = tid; g < G; g += kVerifyBlock) {
          const uint64_t a = consume(&ws->resid[0][g], limit, &failed), c = consume(&ws->resid[1][g], limit, &failed);
          kr = a > kr ? a : kr; ko = c > ko ? c : ko;
        }
        kr = block_max_u64(kr, scratch); ko = block_max_u64(ko, scratch);
        token = kr ? static_cast<int>(pack52_index(kr)) : (ko ? static_cast<int>(pack52_index(ko)) : -1);
      }
    } else if (given_mass) {
      // ---- the one exchange of a launch that was given the masses: this slice's share of row j's mass and of its residual --------
      uint64_t w = 0ull, wo = 0ull;
      if (mass_j > 0ull) for (int i = tid; i < len; i += kVerifyBlock) {
        const float z = S.z(j, i);
        if (z >= tau_j) wo += weight_q40(z, vmax_j, c2);
        if (has_q) w += residual(i);
      }
      mine_r = block_sum_u64(w, scratch); own_w = block_sum_u64(wo, scratch);
      if (tid == 0) { publish(&ws->resid[0][b], mine_r); publish(&ws->resid[1][b], own_w); }
      // Block 0 alone gathers the shares (148 blocks polling each other's words from the moment they have published cost more than
      // the draw itself); it then reads the one slice that holds the crossing straight from L2. Every other block is done.
      if (b == 0) {
        uint64_t* a_res = &s_red[0][0];                                    // G <= 256 shares each: s_red is free from here on
        uint64_t* a_own = &s_red[8][0];
        uint64_t tr = 0ull;
        for (int g = tid; g < G; g += kVerifyBlock) {
          const uint64_t v = consume(&ws->resid[0][g], limit, &failed), o = consume(&ws->resid[1][g], limit, &failed);
          a_res[g] = v; a_own[g] = o; tr += v;
        }
        total_r = block_sum_u64(tr, scratch);                              // (its barriers also publish a_res / a_own to the block)
      }
    } else if (has_q) {
      // ---- the residual's total: one more exchange (skipped when every draft was accepted: the bonus row draws from p). Block 0
      // gathers, as above; the blocks' shares of row j's mass are still in the workspace from the exchange before.
      uint64_t w = 0ull;
      if (mass_j > 0ull) for (int i = tid; i < len; i += kVerifyBlock) w += residual(i);
      mine_r = block_sum_u64(w, scratch);
      if (tid == 0) publish(&ws->resid[0][b], mine_r);
      if (b == 0) {
        uint64_t* a_res = &s_red[0][0];
        uint64_t* a_own = &s_red[8][0];
        uint64_t tr = 0ull;
        for (int g = tid; g < G; g += kVerifyBlock) {
          const uint64_t v = consume(&ws->resid[0][g], limit, &failed), o = consume(&ws->mass[j][g], limit, &failed);
          a_res[g] = v; a_own[g] = o; tr += v;
        }
        total_r = block_sum_u64(tr, scratch);
      }
    }
    const bool bad = __syncthreads_or(failed) != 0;
    if (bad && tid == 0) atomicExch(&ws->error, 1u);

    // ---- phase 3: locate the draw; the block whose slice holds it writes the outputs ---------------------------------------
    bool writer = false;
    if (gumbel_draw) {
      writer = b == 0;
    } else if (given_mass || has_q) {                                       // the shares were gathered by block 0: it draws
      if (b == 0) {
        writer = true;
        const bool use_res = total_r > 0ull;                             // an empty residual: draw from the row's own kept softmax
        const uint64_t total = use_res ? total_r : mass_j;
        token = -1;                                                      // (a row with no weight at all: empty or all -inf)
        if (total > 0ull && !bad) {
          const float u = P.u_final ? P.u_final[0] : uniform01(seed, step, 4000u, 0u);
          const uint64_t target = cdf_target(u, total);
          // the block whose share holds the crossing: an exclusive prefix over the shares, one per thread
          const uint64_t mine = tid < G ? (use_res ? (&s_red[0][0])[tid] : (&s_red[8][0])[tid]) : 0ull;
          const uint64_t before = block_exclusive_scan_u64(mine, scratch, nullptr);
          if (tid == 0) s_j2 = -1;
          __syncthreads();
          if (mine && before <= target && target < before + mine) { s_j2 = tid; s_pre2 = before; }
          __syncthreads();
          if (s_j2 >= 0) {
            const int lo2 = min(V, s_j2 * per), len2 = min(V, lo2 + per) - lo2;
            const VerifySlice V2{&P, (s_j2 == 0) ? zs : nullptr, (s_j2 == 0) ? qs : nullptr, per, lo2, row0, c2};   // block 0's own slice is in shared memory
            token = locate(V2, lo2, len2, s_pre2, use_res, target);
          }
        }
      }
    } else {
      // every draft accepted: the bonus row's own kept softmax; each block knows its share and its prefix from the masses' exchange
      if (mass_j > 0ull) {
        const float u = P.u_final ? P.u_final[0] : uniform01(seed, step, 4000u, 0u);
        const uint64_t target = cdf_target(u, mass_j);
        if (own_w > 0ull && pre_w <= target && target < pre_w + own_w) {   // the crossing lies in this block's slice
          writer = true;
          token = locate(S, lo, len, pre_w, false, target);
        }
      } else if (b == 0) { writer = true; token = -1; }                   // a row with no weight at all (empty or all -inf)
    }
    if (bad) writer = b == 0;                                             // a wait ran out: block 0 reports it
    if (writer && warp == 0) {
      if (lane == 0) {
        P.out_accept[0] = bad ? -1 : j; P.out_final[0] = bad ? -1 : token;
        if (P.out_tokens) for (int r = 0; r < R; r++) P.out_tokens[row0 + r] = bad ? -1 : (r < j ? s_drafts[r] : (r == j ? token : -1));
      }
      verify_commit(P, bad);
    }
  }
  }
  // ---- on the way out: one more block of this launch has left (nobody waits for the reply) -----------------------------------
  __syncthreads();
  if (tid == 0) asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(&P.ws->exits), "l"(1ull) : "memory");
}

}  // namespace lm
