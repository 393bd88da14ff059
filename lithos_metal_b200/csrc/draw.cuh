// The two draws over a row's kept set {z >= tau}, shared by the row samplers. One thread block per row.
//   inverse CDF  -- integer fixed-point weights, ascending index order, caller-supplied uniform (no reference
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
  uint64_t sweep_total[kMaxSweeps];     // fixed-point mass of each sweep of the block over the row
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

// Penalised logits kept aside by the streaming kernel: (index, penalised value) pairs in shared memory. When a draw
// is given such a list, its sweeps skip the penalised positions (no per-lane slow path in the hot loop) and the
// list's entries are added densely afterwards.
struct SideList { const int* idx; const float* val; uint32_t n; };

// BF16 rows, aligned, vocab a multiple of 8: kept mask of the loaded chunk c with the penalised positions removed.
__device__ __forceinline__ uint32_t kept_from_q(const RowView& rv, int c, const uint4 q, uint32_t tau_code2, float z[kChunk]) {
  const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&tau_code2);
  const uint32_t m0 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.x), t2);
  const uint32_t m1 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.y), t2);
  const uint32_t m2 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.z), t2);
  const uint32_t m3 = __hge2_mask(*reinterpret_cast<const __nv_bfloat162*>(&q.w), t2);
  if ((m0 | m1 | m2 | m3) == 0u) return 0u;
  uint32_t mask = (m0 & 1u) | ((m0 >> 15) & 2u) | ((m1 & 1u) << 2) | ((m1 >> 13) & 8u) | ((m2 & 1u) << 4) | ((m2 >> 11) & 32u) |
                  ((m3 & 1u) << 6) | ((m3 >> 9) & 128u);
  if (rv.pen) mask &= ~((rv.pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu);
  if (mask == 0u) return 0u;
  z[0] = bf16_lo(q.x); z[1] = bf16_hi(q.x); z[2] = bf16_lo(q.y); z[3] = bf16_hi(q.y);
  z[4] = bf16_lo(q.z); z[5] = bf16_hi(q.z); z[6] = bf16_lo(q.w); z[7] = bf16_hi(q.w);
  return mask;
}

constexpr int kDrawBatch = 4;            // sweeps whose loads are issued together (the row sits in L2: latency, not bandwidth)

// The inverse-CDF draw. Every thread of the block calls; every thread gets the token (-1 if the kept set has no weight).
template <bool SIDE>
__device__ int draw_inverse_cdf(const RowView& rv, float tau, float vmax, float temperature, float u, DrawSmem& d, SideList side = SideList{nullptr, nullptr, 0u},
                                uint64_t* sweep_part = nullptr, uint32_t* side_limb = nullptr) {
  const int tid = threadIdx.x;
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  const int n_sweeps = (n_chunks + kBlock - 1) / kBlock;
  const float c2 = exp2_scale(temperature);
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  for (int i = tid; i < n_sweeps; i += kBlock) d.sweep_total[i] = 0ull;
  if (SIDE) for (int i = tid; i < n_sweeps * 3; i += kBlock) side_limb[i] = 0u;
  if (tid == 0) d.token = -1;
  __syncthreads();
  if (SIDE) {
    const uint4* p4 = reinterpret_cast<const uint4*>(rv.row);
    const uint4 neg = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);   // -inf: never kept unless tau is -inf, masked below
    for (int it0 = 0; it0 < n_sweeps; it0 += kDrawBatch) {
      uint4 q[kDrawBatch];
#pragma unroll
      for (int j = 0; j < kDrawBatch; j++) { const int cc = (it0 + j) * kBlock + tid; q[j] = (cc < n_chunks) ? __ldg(p4 + cc) : neg; }
#pragma unroll
      for (int j = 0; j < kDrawBatch; j++) {
        const int it = it0 + j, cc = it * kBlock + tid;
        if (it >= n_sweeps) break;
        float z[kChunk];
        const uint32_t mask = (cc < n_chunks) ? kept_from_q(rv, cc, q[j], tau2, z) : 0u;
        uint64_t w = 0ull;
        if (mask) {
#pragma unroll
          for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) w += weight_q40(z[e], vmax, c2);
        }
        // per-warp partial of this sweep: plain stores, summed in warp order below (no 64-bit shared-memory atomics)
        if (__any_sync(kFull, w != 0ull)) w = warp_sum_u64(w);
        if ((tid & 31) == 0) sweep_part[it * 32 + (tid >> 5)] = w;
      }
    }
  } else {
    for (int it = 0; it < n_sweeps; it++) {
      float z[kChunk];
      const uint32_t mask = kept_chunk(rv, it * kBlock + tid, tau, tau2, z);
      uint64_t w = 0ull;
      if (mask) {
#pragma unroll
        for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) w += weight_q40(z[e], vmax, c2);
      }
      if (__any_sync(kFull, w != 0ull)) {
        w = warp_sum_u64(w);
        if ((tid & 31) == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&d.sweep_total[it]), static_cast<unsigned long long>(w));
      }
    }
  }
  if (SIDE) {
    // the kept penalised logits join the sweep their index falls in: three 16-bit limbs, native 32-bit atomics
    // (a limb sum stays below 2^16 * list length < 2^32; integer adds are exact in any order)
    for (uint32_t i = tid; i < side.n; i += kBlock) {
      const float v = side.val[i];
      if (v >= tau) {
        const uint64_t w = weight_q40(v, vmax, c2);
        if (w) {
          uint32_t* l = side_limb + 3 * ((side.idx[i] / kChunk) / kBlock);
          atomicAdd(l, static_cast<uint32_t>(w & 0xFFFFull)); atomicAdd(l + 1, static_cast<uint32_t>((w >> 16) & 0xFFFFull));
          atomicAdd(l + 2, static_cast<uint32_t>(w >> 32));
        }
      }
    }
    __syncthreads();
    if (tid < n_sweeps) {
      uint64_t t = 0ull;
      for (int w = 0; w < kWarps; w++) t += sweep_part[tid * 32 + w];
      t += static_cast<uint64_t>(side_limb[3 * tid]) + (static_cast<uint64_t>(side_limb[3 * tid + 1]) << 16) + (static_cast<uint64_t>(side_limb[3 * tid + 2]) << 32);
      d.sweep_total[tid] = t;
    }
  }
  __syncthreads();
  if (tid == 0) {
    uint64_t total = 0ull;
    for (int it = 0; it < n_sweeps; it++) total += d.sweep_total[it];
    d.found_sweep = -1; d.found_base = 0ull;
    if (total > 0ull) {
      const uint64_t target = cdf_target(u, total);
      uint64_t run = 0ull;
      for (int it = 0; it < n_sweeps; it++) {
        if (run + d.sweep_total[it] > target) { d.found_sweep = it; d.found_base = target - run; break; }
        run += d.sweep_total[it];
      }
    }
  }
  __syncthreads();
  const int it = d.found_sweep;
  if (it >= 0) {
    const uint64_t local_target = d.found_base;                         // the first cumulative weight > local_target, within this sweep
    const int c = it * kBlock + tid;
    float z[kChunk];
    const uint32_t mask = kept_chunk(rv, c, tau, tau2, z);
    uint64_t w[kChunk];
    uint64_t mine = 0ull;
#pragma unroll
    for (int e = 0; e < kChunk; e++) { w[e] = ((mask >> e) & 1u) ? weight_q40(z[e], vmax, c2) : 0ull; mine += w[e]; }
    const uint64_t excl = block_exclusive_scan_u64(mine, d.scratch, nullptr);
    if (excl <= local_target && local_target < excl + mine) {
      uint64_t run = excl;
#pragma unroll
      for (int e = 0; e < kChunk; e++) { run += w[e]; if (w[e] && run > local_target) { d.token = c * kChunk + e; break; } }
    }
  }
  __syncthreads();
  return d.token;
}

// The Gumbel-max draw; *near_tie is set when another candidate lies within 4e-6 of the winning key.
template <bool SIDE>
__device__ int draw_gumbel(const RowView& rv, float tau, float temperature, uint64_t seed, uint32_t step, uint32_t t_id, DrawSmem& d, bool* near_tie,
                           SideList side = SideList{nullptr, nullptr, 0u}) {
  const int tid = threadIdx.x;
  const int n_chunks = (rv.vocab + kChunk - 1) / kChunk;
  const float inv_t32 = __double2float_rn(1.0 / static_cast<double>(temperature));
  const uint32_t tc = ceil_bf16_code(tau);
  const uint32_t tau2 = tc | (tc << 16);
  uint64_t b1 = 0ull;
  float second = -INFINITY;
  for (int c0 = tid; c0 < n_chunks; c0 += kBlock * kDrawBatch) {
    uint4 q[kDrawBatch];
    if (SIDE) {
#pragma unroll
      for (int j = 0; j < kDrawBatch; j++) { const int c = c0 + j * kBlock; if (c < n_chunks) q[j] = __ldg(reinterpret_cast<const uint4*>(rv.row) + c); }
    }
#pragma unroll
    for (int j = 0; j < kDrawBatch; j++) {
      const int c = c0 + j * kBlock;
      if (c >= n_chunks) break;
      float z[kChunk];
      const uint32_t mask = SIDE ? kept_from_q(rv, c, q[j], tau2, z) : kept_chunk(rv, c, tau, tau2, z);
      if (!mask) continue;
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((mask >> e) & 1u) {
        const uint32_t i = static_cast<uint32_t>(c * kChunk + e);
        const float key = __fadd_rn(__fmul_rn(z[e], inv_t32), gumbel(seed, step, t_id, i));
        const uint64_t p = pack_best(key, i);
        if (p > b1) { if (b1) second = fmaxf(second, best_value(b1)); b1 = p; } else second = fmaxf(second, key);
      }
    }
  }
  if (SIDE) {
    for (uint32_t j = tid; j < side.n; j += kBlock) {
      const float v = side.val[j];
      if (!(v >= tau)) continue;
      const uint32_t i = static_cast<uint32_t>(side.idx[j]);
      const float key = __fadd_rn(__fmul_rn(v, inv_t32), gumbel(seed, step, t_id, i));
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
