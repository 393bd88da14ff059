// The step-closing kernels of GPU-resident generation control. They keep the decode loop on the device: the host never reads
// a token to decide what runs next. Each works on the reference's StepState record, a binary contract
// (monolith/core/step_state.py:38-62: 4-byte fields, fixed order, sized by t_max / gamma_max), and must leave exactly the
// bytes the reference's kernels leave:
//   round_close     what accept_scan does  (kernels/common/spec_ops.metal:148-195)  prefix match, ring commit, state advance
//   round_select    what verify_select does (kernels/common/spec_ops.metal:108-146) stage drafts, pick the verify length
//   step_advance    what advance does       (kernels/common/advance.metal:15-37)    close a plain decode step
//   confidence      the DSpark confidence head (kernels/common/spec_ops.metal:85-106) that feeds round_select
// Each runs as ONE WARP: the per-draft work (token compares, stop-token tests, ring slots, staging) is spread over the lanes
// and joined with votes; the state record is then updated by lane 0.
#pragma once
#include "common.cuh"

namespace lm {

// Field access on a StepState buffer laid out as StepStateLayout(t_max, gamma_max) lays it out.
struct StepStateView {
  uint32_t* w; int t_max; int g;                                           // g = max(gamma_max, 1)
  __device__ __forceinline__ uint32_t& step() { return w[0]; }
  __device__ __forceinline__ uint32_t& position() { return w[1]; }
  __device__ __forceinline__ uint32_t& kv_len() { return w[2]; }
  __device__ __forceinline__ uint32_t& t_this_step() { return w[3]; }
  __device__ __forceinline__ int32_t& pending(int i) { return reinterpret_cast<int32_t*>(w)[4 + i]; }
  __device__ __forceinline__ uint32_t& rng_lo() { return w[4 + t_max]; }
  __device__ __forceinline__ uint32_t& rng_hi() { return w[5 + t_max]; }
  __device__ __forceinline__ int32_t& anchor() { return reinterpret_cast<int32_t*>(w)[6 + t_max]; }
  __device__ __forceinline__ uint32_t& gamma() { return w[7 + t_max]; }
  __device__ __forceinline__ int32_t& draft(int i) { return reinterpret_cast<int32_t*>(w)[8 + t_max + i]; }
  __device__ __forceinline__ float& confidence(int i) { return reinterpret_cast<float*>(w)[8 + t_max + g + i]; }
  __device__ __forceinline__ uint32_t& tail(int i) { return w[8 + t_max + 2 * g + i]; }
  __device__ __forceinline__ uint32_t& verify_len() { return tail(0); }
  __device__ __forceinline__ uint32_t& accepted() { return tail(1); }
  __device__ __forceinline__ uint32_t& checkpoint_index() { return tail(2); }
  __device__ __forceinline__ uint32_t& drafter_ctx_len() { return tail(3); }
  __device__ __forceinline__ uint32_t& done() { return tail(4); }
  __device__ __forceinline__ uint32_t& error() { return tail(5); }
  __device__ __forceinline__ uint32_t& ring_head() { return tail(6); }
  __device__ __forceinline__ uint32_t& ring_tail() { return tail(7); }
  __device__ __forceinline__ uint32_t& prefill_left() { return tail(8); }
  __device__ __forceinline__ uint32_t& n_inject() { return tail(9); }
  __device__ __forceinline__ uint32_t& stop_at() { return tail(10); }
  __device__ __forceinline__ uint32_t& n_chain() { return tail(11); }
  __device__ __forceinline__ uint64_t seed() { return (static_cast<uint64_t>(rng_hi()) << 32) | rng_lo(); }
};

constexpr uint32_t kErrRingFull = 1u, kErrContextFull = 2u, kErrBarrier = 3u, kErrRoundMismatch = 4u;

struct EosSet { int32_t eos; const int32_t* list; int n; };                 // eos < 0 and n == 0: no stop token
__device__ __forceinline__ bool is_eos(const EosSet& e, int32_t tok) {
  bool hit = e.eos >= 0 && tok == e.eos;
  for (int i = 0; i < e.n; i++) hit = hit || tok == e.list[i];
  return hit;
}

// Ends a generation with an error code; lane 0 only.
__device__ __forceinline__ void fail_state(StepStateView& st, uint32_t code) { st.error() = code; st.done() = 1u; }
// One entry of the token ring: the sequence number of the token (1-based) above the token id.
__device__ __forceinline__ unsigned long long ring_entry(uint32_t seq, int32_t tok) {
  return (static_cast<unsigned long long>(seq) << 32) | static_cast<unsigned long long>(static_cast<uint32_t>(tok));
}

struct AcceptDev {
  const int32_t* token; uint32_t* state; int t_max, g; unsigned long long* ring; uint32_t ring_cap; EosSet eos;
  uint32_t* log; uint32_t log_cap; uint32_t ctx_cap; int lm;
};

// Closes a speculative round. All 32 lanes of one warp call it with the same arguments; `p.token` holds the target's pick
// for every row of the step (written before the call and visible to the warp).
//   lanes r < L     compare the pick of row base + r with draft r (pending[base + r + 1]); the first mismatch is the accept count
//   lanes k <= acc  hold the k-th token to commit (accepted draft, or the pick after the last accepted one), test it against the
//                   stop tokens, and, up to the first stop token, publish it in ring slot head + k
//   lane 0          writes the log entry and moves the state on
__device__ void round_close(const AcceptDev& p) {
  const int lane = threadIdx.x & 31;
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  const uint32_t rows = st.t_this_step();
  if (st.prefill_left() > 0u) {
    // prompt rows only: no draft was checked and nothing is published; the rows become injected context
    if (lane == 0) {
      if (p.log_cap) p.log[st.step() % p.log_cap] = (rows << 16) | 0xFFFFu;
      const uint32_t pos = st.position() + rows;
      st.position() = pos; st.step() += 1u;
      st.n_inject() = rows; st.checkpoint_index() = rows; st.n_chain() = 0u;
      if (p.ctx_cap && pos >= p.ctx_cap) fail_state(st, kErrContextFull);
    }
    return;
  }
  const uint32_t L = st.verify_len(), base = rows - 1u - L;
  // accept count: the number of leading drafts the target agrees with (32 drafts per vote)
  uint32_t acc = L;
  for (uint32_t r0 = 0; r0 < L; r0 += 32u) {
    const uint32_t r = r0 + lane;
    const bool differs = r < L && p.token[base + r] != st.pending(base + r + 1u);
    const uint32_t votes = __ballot_sync(kFull, differs);
    if (votes) { acc = r0 + static_cast<uint32_t>(__ffs(votes)) - 1u; break; }
  }
  const uint32_t head = st.ring_head();
  if (head + acc + 1u - st.ring_tail() > p.ring_cap) {                      // the consumer has not drained the ring: stop rather than overwrite
    if (lane == 0) fail_state(st, kErrRingFull);
    return;
  }
  // the tokens of this round in commit order, cut after the first stop token
  uint32_t n_commit = acc + 1u; bool stop = false; int32_t last = 0;
  for (uint32_t k0 = 0; k0 <= acc; k0 += 32u) {
    const uint32_t k = k0 + lane;
    const bool mine = k <= acc;
    const int32_t tok = mine ? (k < acc ? st.pending(base + k + 1u) : p.token[base + acc]) : 0;
    const uint32_t stops = __ballot_sync(kFull, mine && is_eos(p.eos, tok));
    const uint32_t upto = stops ? k0 + static_cast<uint32_t>(__ffs(stops)) : acc + 1u;   // tokens committed, counted from 0
    if (k < upto) p.ring[(head + k) % p.ring_cap] = ring_entry(head + k + 1u, tok);
    const uint32_t last_lane = (upto - 1u) - k0;
    if (last_lane < 32u) last = __shfl_sync(kFull, tok, static_cast<int>(last_lane));
    if (stops) { n_commit = upto; stop = true; break; }
  }
  if (lane == 0) {
    if (p.log_cap) p.log[st.step() % p.log_cap] = (n_commit << 16) | (L << 8) | acc;
    const uint32_t new_head = head + n_commit, fed = base + n_commit, pos = st.position() + fed;
    st.ring_head() = new_head;
    st.accepted() = acc; st.anchor() = last;
    st.position() = pos; st.step() += 1u;
    st.verify_len() = 0u; st.t_this_step() = 1u;
    st.checkpoint_index() = fed; st.n_chain() = 1u;
    st.n_inject() = p.lm ? (pos > st.drafter_ctx_len() ? pos - st.drafter_ctx_len() : 0u) : fed;
    if (stop || (st.stop_at() && new_head >= st.stop_at())) st.done() = 1u;
    if (p.ctx_cap && pos >= p.ctx_cap) fail_state(st, kErrContextFull);
  }
}

__global__ void accept_scan_kernel(AcceptDev p) {
  if (blockIdx.x == 0 && threadIdx.x < 32) round_close(p);
}

struct SelectDev {
  const int32_t* drafts; const float* conf; uint32_t* state; int t_max, g; uint32_t gamma; float threshold; uint32_t mode; float cost[16];
  float* conf_log; uint32_t log_cap; uint32_t ctx_cap; int lm; uint32_t t_limit;
};

// Prepares the next round: lanes k < gamma copy draft k and its confidence into the state (and the confidence log); the verify
// length L comes from the confidences (mode 0: the confident prefix, by vote; mode 1: the length with the best expected tokens
// per unit cost, a running product that lane 0 forms in the reference's order; mode 2: a fixed length); lanes k < L then stage
// draft k as pending token k + 1 behind the anchor. One warp.
__global__ void verify_select_kernel(SelectDev p) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const uint32_t lane = threadIdx.x;
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  const bool prefill = st.prefill_left() > 0u;
  const uint32_t pos = st.position(), step = st.step();
  __syncwarp();
  if (lane == 0) {
    // how much context the drafter has seen: an LM drafter is fed up to the position (plus its own drafts in a decode round),
    // a head drafter exactly what the last step injected
    st.drafter_ctx_len() = p.lm ? pos + (prefill ? 0u : p.gamma) : st.drafter_ctx_len() + st.n_inject();
    st.n_inject() = 0u;
  }
  if (prefill) return;                                                    // the next prompt chunk comes from the host; nothing to stage
  const float my_conf = lane < p.gamma ? p.conf[lane] : 0.0f;
  if (lane < p.gamma) {
    st.draft(lane) = p.drafts[lane];
    st.confidence(lane) = my_conf;
    if (p.log_cap) p.conf_log[(step % p.log_cap) * 16u + lane] = my_conf;
  }
  // the longest length the step program and the context leave room for
  uint32_t room = min(p.gamma, p.t_limit - 1u);
  if (p.ctx_cap) {
    if (pos >= p.ctx_cap) { if (lane == 0) fail_state(st, kErrContextFull); return; }
    room = min(room, p.ctx_cap - pos - 1u);
  }
  uint32_t L;
  if (p.mode == 2u) {
    L = min(static_cast<uint32_t>(fmaxf(p.threshold, 0.0f)), room);
  } else if (p.mode == 1u) {
    // expected tokens of verifying l drafts = 1 + conf_0 + conf_0 conf_1 + ...; its cost = cost[l]; ties keep the shorter length
    uint32_t best_l = 0u;
    if (lane == 0) {
      float reach = 1.0f, tokens = 1.0f, best = __fdiv_rn(1.0f, p.cost[0]);
      for (uint32_t l = 1; l <= room; l++) {
        reach = __fmul_rn(reach, p.conf[l - 1u]);
        tokens = __fadd_rn(tokens, reach);
        const float rate = __fdiv_rn(tokens, p.cost[l]);
        if (rate > best) { best = rate; best_l = l; }
      }
    }
    L = __shfl_sync(kFull, best_l, 0);
  } else if (p.threshold <= 0.0f) {
    L = room;
  } else {
    const uint32_t unsure = __ballot_sync(kFull, lane < room && !(my_conf >= p.threshold));
    L = unsure ? static_cast<uint32_t>(__ffs(unsure)) - 1u : room;
  }
  if (lane < L) st.pending(lane + 1u) = p.drafts[lane];
  if (lane == 0) {
    st.gamma() = p.gamma; st.verify_len() = L;
    st.pending(0) = st.anchor();
    st.t_this_step() = 1u + L;
  }
}

struct AdvanceDev { const int32_t* token; uint32_t* state; int t_max, g; unsigned long long* ring; uint32_t ring_cap; EosSet eos; uint32_t ctx_cap; };

// Closes a step that verified nothing: the last row's token is the step's token. The lanes share the stop-token test (one list
// entry each per vote); lane 0 publishes the token and moves the state on. One warp.
__global__ void advance_kernel(AdvanceDev p) {
  if (blockIdx.x != 0 || threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  const uint32_t rows = st.t_this_step();
  const bool prefill = st.prefill_left() > 0u;
  const int32_t tok = prefill ? 0 : p.token[rows - 1u];
  bool stop_tok = false;
  if (!prefill) {
    bool hit = lane == 0 && p.eos.eos >= 0 && tok == p.eos.eos;
    for (int i = lane; i < p.eos.n; i += 32) hit = hit || tok == p.eos.list[i];
    stop_tok = __any_sync(kFull, hit);
  }
  if (lane != 0) return;
  const uint32_t pos = st.position() + rows;
  if (!prefill) {
    const uint32_t head = st.ring_head();
    if (head - st.ring_tail() >= p.ring_cap) { fail_state(st, kErrRingFull); return; }
    p.ring[head % p.ring_cap] = ring_entry(head + 1u, tok);
    st.ring_head() = head + 1u;
    st.pending(0) = tok;
    st.t_this_step() = 1u;
    if (stop_tok || (st.stop_at() && head + 1u >= st.stop_at())) st.done() = 1u;
  }
  st.position() = pos; st.step() += 1u;
  if (p.ctx_cap && pos >= p.ctx_cap) fail_state(st, kErrContextFull);
}

// The confidence head: conf[k] = sigmoid(bf16(bf16(w . [hidden_k ; emb_k]) + b) / sts[k]) for the gamma draft positions, one
// warp per position. The sum is formed the way the reference's kernel forms it, because the two BF16 roundings make the order
// visible in the result: lane l takes elements l, l + 32, ... of the hidden row and then of the embedding row with one FP32
// FMA each, and the lanes meet in a butterfly. The sigmoid runs on the library's fixed exp2 (common.cuh), so a CPU restatement
// gives the same bits; the reference calls the Metal exp (its test bar: 2e-3).
struct ConfDev { const uint16_t* hidden; const uint16_t* emb; const float* w; const float* b; const float* sts; float* conf; uint32_t* state; int t_max, g; int gamma, n_hidden, rank; };

__device__ __forceinline__ float round_bf16(float x) {                     // round to nearest even on the bit pattern
  const uint32_t u = __float_as_uint(x);
  return __uint_as_float((u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u);
}
// acc += row[i] * w[i] over this lane's elements of a BF16 row
__device__ __forceinline__ float lane_dot_bf16(const uint16_t* row, const float* w, int n, int lane, float acc) {
  for (int i = lane; i < n; i += 32) acc = __fmaf_rn(__uint_as_float(static_cast<uint32_t>(__ldg(row + i)) << 16), __ldg(w + i), acc);
  return acc;
}

__global__ void confidence_kernel(ConfDev p) {
  const int lane = threadIdx.x & 31, k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (k >= p.gamma) return;
  if (p.state) { StepStateView st{p.state, p.t_max, p.g}; if (st.done()) return; }
  float dot = lane_dot_bf16(p.hidden + static_cast<int64_t>(k) * p.n_hidden, p.w, p.n_hidden, lane, 0.0f);
  dot = lane_dot_bf16(p.emb + static_cast<int64_t>(k) * p.rank, p.w + p.n_hidden, p.rank, lane, dot);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot = __fadd_rn(dot, __shfl_xor_sync(kFull, dot, o));
  if (lane != 0) return;
  const float logit = __fdiv_rn(round_bf16(__fadd_rn(round_bf16(dot), p.b[0])), p.sts ? p.sts[k] : 1.0f);
  const float e = spec_exp2(__fmul_rn(-fabsf(logit), 1.44269502f));        // exp(-|logit|) in (0, 1]: no overflow on either side
  p.conf[k] = __fdiv_rn(logit >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
}

}  // namespace lm
