// The two draws over a row's kept set {z >= tau}, shared by the row samplers. One thread block per row.
//   inverse CDF  -- integer fixed-point weights, descending value order (equal values by ascending index), caller-supplied uniform (no reference
//                   counterpart; the arithmetic is fixed operation by operation so a CPU gives the same bits);
//   Gumbel-max   -- argmax of z * fl32(1/T) + g(seed, step, row, index), ties -> lowest index
//                   (monolith/nn/sampling_ref.py:55-62; kernels/common/sample.metal:164-198).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace lm {

constexpr int kMaxSweeps = LM_MAX_VOCAB / (kBlock * kChunk) + 1;

struct DrawSmem {
  uint64_t scratch[32];
  uint64_t sweep_total[kMaxSweeps];     // per sweep of the block over the row: how many logits equal the drawn value
  uint64_t wbin[256];                   // fixed-point weight per digit of the value key (the radix descent of the draw)
  uint64_t found_base;
  int found_sweep;
  int token;
};

// Smallest BF16 code whose value is >= t: for BF16-valued z, (z >= t) <=> (z >= that value).
__device__ __forceinline__ uint32_t ceil_bf16_code(float t) {
  const uint32_t u = __float_as_uint(t);
  uint32_t code = u >> 16;
  if ((u & 0xFFFFu) && !(u & 0x80000000u)) code += 1u;
  return code;
}

// Chunk c of the row: the bit mask of its kept elements (bit e <=> element 8c + e exists and z >= tau) and, for
// those, the widened (penalised) values. BF16 rows take a packed compare first and widen only on a hit.
__device__ __forceinline__ uint32_t kept_chunk(const RowView& rv, int c, float tau, uint32_t tau_code2, float z[kChunk]) {
  const int base = c * kChunk;
  if (base >= rv.vocab) return 0u;
  if (rv.dtype == LM_DTYPE_BF16 && rv.aligned && base + kChunk <= rv.vocab) {
    const uint32_t pen = rv.pen ? ((rv.pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu) : 0u;
    if (pen == 0u) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(rv.row) + base));
      const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&tau_code2);
      const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.x), t2);
      const uint32_t m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.y), t2);
      const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.z), t2);
      const uint32_t m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.w), t2);
      if ((m0 | m1 | m2 | m3) == 0u) return 0u;
      z[0] = bf16_lo(q.x); z[1] = bf16_hi(q.x); z[2] = bf16_lo(q.y); z[3] = bf16_hi(q.y);
      z[4] = bf16_lo(q.z); z[5] = bf16_hi(q.z); z[6] = bf16_lo(q.w); z[7] = bf16_hi(q.w);
      return (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) |
             ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
    }
  }
  const int n = load_chunk(rv, c, z);
  uint32_t mask = 0u;
#pragma unroll
  for (int e = 0; e < kChunk; e++) if (e < n && z[e] >= tau) mask |= 1u << e;
  return mask;
}

// The inverse-CDF draw: the kept set in descending value order, equal values by ascending index. Equal values have equal weights,
// so the draw is: the distinct value v at which the cumulative weight first exceeds the target (a 4 x 8-bit radix descent on the
// monotone value keys, every level one sweep of the row that sums the weights per digit), then the
// floor((target - weight above v) / w(v))-th smallest index among the logits equal to v (one sweep that counts them per sweep of
// the block, one look at the sweep that holds it). Every thread of the block calls; every thread gets the token (-1 if the kept
// set has no weight).
// The kept set's total fixed-point weight. Every thread of the block calls; every thread gets the total.
__device__ uint64_t kept_weight_total(const RowView& rv, float tau, float vmax, float temperature, DrawSmem& d) {
  const int tid = threadIdx.x;
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  const int n_sweeps = (n_chunks + kBlock - 1) / kBlock;
  const float c2 = exp2_scale(temperature);
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  uint64_t mine = 0ull;
  for (int it = 0; it < n_sweeps; it++) {
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, it * kBlock + tid, tau, tau2, z);
    if (mask) {
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) mine += weight_q40(z[e], vmax, c2);
    }
  }
  return block_sum_u64(mine, d.scratch);
}

__device__ int draw_inverse_cdf(const RowView& rv, float tau, float vmax, float temperature, float u, DrawSmem& d, uint64_t* out_total = nullptr) {
  const int tid = threadIdx.x;
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  const int n_sweeps = (n_chunks + kBlock - 1) / kBlock;
  const float c2 = exp2_scale(temperature);
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  if (tid == 0) d.token = -1;
  const uint64_t total = kept_weight_total(rv, tau, vmax, temperature, d);
  if (out_total) *out_total = total;
  if (total == 0ull) { __syncthreads(); return -1; }
  const uint64_t target = cdf_target(u, total);
  // ---- the value: digits of its key from the top
  uint32_t prefix = 0u;
  uint64_t before = 0ull;                                                  // weight of the kept logits above every value with this prefix
  for (int level = 0; level < 4; level++) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < 256; i += kBlock) d.wbin[i] = 0ull;
    __syncthreads();
    for (int it = 0; it < n_sweeps; it++) {
      float z[kChunk];
      const uint32_t mask = kept_chunk(rv, it * kBlock + tid, tau, tau2, z);
      if (!mask) continue;
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) {
        const uint32_t key = fkey(z[e]);
        if ((key & hi_mask) != prefix) continue;
        const uint64_t w = weight_q40(z[e], vmax, c2);
        if (w) atomicAdd(reinterpret_cast<unsigned long long*>(&d.wbin[(key >> shift) & 0xFFu]), static_cast<unsigned long long>(w));
      }
    }
    __syncthreads();
    if (tid == 0) {
      uint64_t run = before; int b = 255;
      for (; b > 0; b--) { if (run + d.wbin[b] > target) break; run += d.wbin[b]; }
      d.found_base = run; d.found_sweep = b;
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(d.found_sweep) << shift; before = d.found_base;
    __syncthreads();
  }
  const float v = fkey_inv(prefix);
  const uint64_t each = weight_q40(v, vmax, c2);
  const uint32_t want = each ? static_cast<uint32_t>((target - before) / each) : 0u;   // 0-based rank by index among the logits equal to v
  // ---- how many of them every sweep of the block holds
  for (int i = tid; i < n_sweeps; i += kBlock) d.sweep_total[i] = 0ull;
  __syncthreads();
  for (int it = 0; it < n_sweeps; it++) {
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, it * kBlock + tid, tau, tau2, z);
    uint32_t n = 0u;
    if (mask) {
#pragma unroll
      for (int e = 0; e < kChunk; e++) n += (((mask >> e) & 1u) && z[e] == v) ? 1u : 0u;
    }
    if (__any_sync(kFull, n != 0u)) {
      n = warp_sum_u32(n);
      if ((tid & 31) == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&d.sweep_total[it]), static_cast<unsigned long long>(n));
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint64_t run = 0ull;
    d.found_sweep = -1; d.found_base = 0ull;
    for (int it = 0; it < n_sweeps; it++) {
      if (run + d.sweep_total[it] > want) { d.found_sweep = it; d.found_base = want - run; break; }
      run += d.sweep_total[it];
    }
  }
  __syncthreads();
  const int it = d.found_sweep;
  if (it >= 0) {
    const uint32_t local = static_cast<uint32_t>(d.found_base);          // the (local)-th match, in index order, within this sweep
    const int c = it * kBlock + tid;
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, c, tau, tau2, z);
    uint32_t hit = 0u;
#pragma unroll
    for (int e = 0; e < kChunk; e++) if (((mask >> e) & 1u) && z[e] == v) hit |= 1u << e;
    const uint64_t excl = block_exclusive_scan_u64(static_cast<uint64_t>(__popc(hit)), d.scratch, nullptr);
    if (excl <= local && local < excl + __popc(hit)) {
      uint32_t run = static_cast<uint32_t>(excl);
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((hit >> e) & 1u) { if (run == local) { d.token = c * kChunk + e; break; } run++; }
    }
  }
  __syncthreads();
  return d.token;
}

// The Gumbel-max draw; *near_tie is set when another candidate lies within 4e-6 of the winning key.
__device__ int draw_gumbel(const RowView& rv, float tau, float temperature, uint64_t seed, uint32_t step, uint32_t t_id, DrawSmem& d, bool* near_tie) {
  const int tid = threadIdx.x;
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  const float inv_t32 = __double2float_rn(1.0 / static_cast<double>(temperature));
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  uint64_t b1 = 0ull;
  float second = -INFINITY;
  for (int c = tid; c < n_chunks; c += kBlock) {
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, c, tau, tau2, z);
    if (!mask) continue;
#pragma unroll
    for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) {
      const uint32_t i = static_cast<uint32_t>(c * kChunk + e);
      const float key = __fadd_rn(__fmul_rn(z[e], inv_t32), gumbel(seed, step, t_id, i));
      const uint64_t p = pack_best(key, i);
      if (p > b1) { if (b1) second = fmaxf(second, best_value(b1)); b1 = p; } else second = fmaxf(second, key);
    }
  }
  const uint64_t win = block_max_u64(b1, d.scratch);
  bool tie = false;
  int token = -1;
  if (win) {
    const float wkey = best_value(win);
    const float rival = (b1 == win) ? second : (b1 ? best_value(b1) : -INFINITY);   // this thread's best candidate other than the winner
    tie = __syncthreads_or(rival >= wkey - 4e-6f) != 0;
    token = static_cast<int>(best_index(win));
  }
  *near_tie = tie;
  return token;
}

}  // namespace lm
