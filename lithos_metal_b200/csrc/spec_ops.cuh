// The scalar step-closing kernels of GPU-resident generation control, on the reference's StepState layout:
//   accept_scan   (kernels/common/spec_ops.metal:148-195)  greedy prefix match, commit to the token ring, advance the state
//   verify_select (kernels/common/spec_ops.metal:108-146)  stage the next round's drafts and pick the verify length
//   advance       (kernels/common/advance.metal:15-37)     close a plain decode step
//   confidence    (kernels/common/spec_ops.metal:85-106)   the DSpark confidence head that feeds verify_select
// One thread each: they are a few dozen dependent scalar operations; what matters is that they run on the device,
// in stream order, so the host never has to read a token to keep the loop going. The state is the reference's
// binary contract (monolith/core/step_state.py:38-62): 4-byte fields, same order, for any t_max / gamma_max.
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
};

struct EosSet { int32_t eos; const int32_t* list; int n; };                 // eos < 0 and n == 0: no stop token
__device__ __forceinline__ bool is_eos(const EosSet& e, int32_t tok) {
  if (e.eos >= 0 && tok == e.eos) return true;
  for (int i = 0; i < e.n; i++) if (tok == e.list[i]) return true;
  return false;
}

struct AcceptDev {
  const int32_t* token; uint32_t* state; int t_max, g; unsigned long long* ring; uint32_t ring_cap; EosSet eos;
  uint32_t* log; uint32_t log_cap; uint32_t ctx_cap; int lm;
};

// The accept scan proper; one thread. Also the last act of the verify kernel when a round is committed there.
__device__ void accept_scan_body(const AcceptDev& p) {
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  const uint32_t t = st.t_this_step();
  if (st.prefill_left() > 0u) {                                           // a prefill chunk: nothing to verify, inject its positions
    if (p.log_cap) p.log[st.step() % p.log_cap] = (t << 16) | 0xFFFFu;
    st.position() += t;
    st.step() += 1u;
    st.n_inject() = t;
    st.checkpoint_index() = t;
    st.n_chain() = 0u;
    if (p.ctx_cap && st.position() >= p.ctx_cap) { st.error() = 2u; st.done() = 1u; }
    return;
  }
  const uint32_t L = st.verify_len();
  const uint32_t base = t - 1u - L;
  uint32_t acc = 0u;
  while (acc < L && p.token[base + acc] == st.pending(base + acc + 1u)) acc++;
  const int32_t bonus = p.token[base + acc];
  uint32_t head = st.ring_head();
  if (head + acc + 1u - st.ring_tail() > p.ring_cap) { st.error() = 1u; st.done() = 1u; return; }   // the host fell behind
  uint32_t committed = 0u;
  int32_t last = bonus;
  bool stop = false;
  for (uint32_t k = 0; k <= acc; k++) {
    const int32_t tok = (k < acc) ? st.pending(base + k + 1u) : bonus;
    p.ring[head % p.ring_cap] = (static_cast<unsigned long long>(head + 1u) << 32) | static_cast<unsigned long long>(static_cast<uint32_t>(tok));
    head++; committed++; last = tok;
    if (is_eos(p.eos, tok)) { stop = true; break; }                       // nothing after the first stop token is committed
  }
  if (p.log_cap) p.log[st.step() % p.log_cap] = (committed << 16) | (L << 8) | acc;
  st.ring_head() = head;
  if (st.stop_at() && head >= st.stop_at()) stop = true;
  st.accepted() = acc;
  st.anchor() = last;
  st.position() += base + committed;
  st.step() += 1u;
  st.verify_len() = 0u;
  st.t_this_step() = 1u;
  st.n_inject() = base + committed;
  st.checkpoint_index() = base + committed;
  st.n_chain() = 1u;
  if (p.lm) st.n_inject() = (st.position() > st.drafter_ctx_len()) ? st.position() - st.drafter_ctx_len() : 0u;
  if (stop) st.done() = 1u;
  if (p.ctx_cap && st.position() >= p.ctx_cap) { st.error() = 2u; st.done() = 1u; }
}

__global__ void accept_scan_kernel(AcceptDev p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  accept_scan_body(p);
}

struct SelectDev {
  const int32_t* drafts; const float* conf; uint32_t* state; int t_max, g; uint32_t gamma; float threshold; uint32_t mode; float cost[16];
  float* conf_log; uint32_t log_cap; uint32_t ctx_cap; int lm; uint32_t t_limit;
};

__global__ void verify_select_kernel(SelectDev p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  if (p.lm) st.drafter_ctx_len() = st.position() + ((st.prefill_left() > 0u) ? 0u : p.gamma);
  else st.drafter_ctx_len() = st.drafter_ctx_len() + st.n_inject();
  st.n_inject() = 0u;
  if (st.prefill_left() > 0u) return;                                     // the host feeds the next chunk
  for (uint32_t k = 0; k < p.gamma; k++) {
    st.draft(k) = p.drafts[k];
    st.confidence(k) = p.conf[k];
    if (p.log_cap) p.conf_log[(st.step() % p.log_cap) * 16u + k] = p.conf[k];
  }
  uint32_t L = 0u;
  uint32_t lmax = min(p.gamma, p.t_limit - 1u);
  if (p.ctx_cap) {                                                        // the verify rows must fit the target's caches
    if (st.position() >= p.ctx_cap) { st.error() = 2u; st.done() = 1u; return; }
    lmax = min(lmax, p.ctx_cap - st.position() - 1u);
  }
  if (p.mode == 2u) {
    L = min(static_cast<uint32_t>(fmaxf(p.threshold, 0.0f)), lmax);
  } else if (p.mode == 1u) {
    float a = 1.0f, expect = 1.0f, best = __fdiv_rn(1.0f, p.cost[0]);
    for (uint32_t l = 1; l <= lmax; l++) {
      a = __fmul_rn(a, p.conf[l - 1u]);
      expect = __fadd_rn(expect, a);
      const float score = __fdiv_rn(expect, p.cost[l]);
      if (score > best) { best = score; L = l; }
    }
  } else if (p.threshold <= 0.0f) {
    L = lmax;
  } else {
    while (L < lmax && p.conf[L] >= p.threshold) L++;
  }
  st.gamma() = p.gamma;
  st.verify_len() = L;
  st.pending(0) = st.anchor();
  for (uint32_t k = 0; k < L; k++) st.pending(k + 1u) = p.drafts[k];
  st.t_this_step() = 1u + L;
}

struct AdvanceDev { const int32_t* token; uint32_t* state; int t_max, g; unsigned long long* ring; uint32_t ring_cap; EosSet eos; uint32_t ctx_cap; };

__global__ void advance_kernel(AdvanceDev p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  StepStateView st{p.state, p.t_max, p.g};
  if (st.done()) return;
  const uint32_t t = st.t_this_step();
  if (st.prefill_left() > 0u) {
    st.position() += t;
    st.step() += 1u;
    if (p.ctx_cap && st.position() >= p.ctx_cap) { st.error() = 2u; st.done() = 1u; }
    return;
  }
  const int32_t tok = p.token[t - 1u];
  const uint32_t head = st.ring_head();
  if (head - st.ring_tail() >= p.ring_cap) { st.error() = 1u; st.done() = 1u; return; }
  p.ring[head % p.ring_cap] = (static_cast<unsigned long long>(head + 1u) << 32) | static_cast<unsigned long long>(static_cast<uint32_t>(tok));
  st.ring_head() = head + 1u;
  if (st.stop_at() && st.ring_head() >= st.stop_at()) st.done() = 1u;
  st.pending(0) = tok;
  st.position() += t;
  st.step() += 1u;
  st.t_this_step() = 1u;
  if (is_eos(p.eos, tok)) st.done() = 1u;
  if (p.ctx_cap && st.position() >= p.ctx_cap) { st.error() = 2u; st.done() = 1u; }
}

// The confidence head: conf[k] = sigmoid(bf16(bf16(w . [hidden_k ; emb_k]) + b) / sts[k]) for the gamma draft positions.
// One warp per position, the reference's arithmetic step by step: lane l accumulates elements l, l + 32, ... of the hidden
// row and then of the embedding row with one FMA each (FP32), the lanes meet in a butterfly sum, the dot product and the
// biased sum are each rounded to BF16 (round to nearest even on the bit pattern). The sigmoid is evaluated on the library's
// fixed exp2 (common.cuh) so that a CPU gives the same bits; the reference calls the Metal exp (test bar there: 2e-3).
struct ConfDev { const uint16_t* hidden; const uint16_t* emb; const float* w; const float* b; const float* sts; float* conf; uint32_t* state; int t_max, g; int gamma, n_hidden, rank; };

__device__ __forceinline__ float round_bf16(float x) {
  uint32_t u = __float_as_uint(x);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return __uint_as_float(u & 0xFFFF0000u);
}

__global__ void confidence_kernel(ConfDev p) {
  const int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (k >= p.gamma) return;
  if (p.state) { StepStateView st{p.state, p.t_max, p.g}; if (st.done()) return; }
  float acc = 0.0f;
  for (int i = lane; i < p.n_hidden; i += 32) acc = __fmaf_rn(__uint_as_float(static_cast<uint32_t>(__ldg(p.hidden + static_cast<int64_t>(k) * p.n_hidden + i)) << 16), __ldg(p.w + i), acc);
  for (int i = lane; i < p.rank; i += 32) acc = __fmaf_rn(__uint_as_float(static_cast<uint32_t>(__ldg(p.emb + static_cast<int64_t>(k) * p.rank + i)) << 16), __ldg(p.w + p.n_hidden + i), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(kFull, acc, o));
  if (lane == 0) {
    const float z = round_bf16(__fadd_rn(round_bf16(acc), p.b[0]));
    const float x = __fdiv_rn(z, p.sts ? p.sts[k] : 1.0f);
    const float e = spec_exp2(__fmul_rn(-fabsf(x), 1.44269502f));          // exp(-|x|), in (0, 1]
    p.conf[k] = x >= 0.0f ? __fdiv_rn(1.0f, __fadd_rn(1.0f, e)) : __fdiv_rn(e, __fadd_rn(1.0f, e));
  }
}

}  // namespace lm
