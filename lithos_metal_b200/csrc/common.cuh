// Device helpers shared by the generation-control kernels (sm_100a).
//
// Everything that feeds an integer decision (token ids, kept sets, accept counts) is written with explicit
// round-to-nearest intrinsics so that the compiler cannot contract or reorder it: the same sequence of IEEE
// operations on a CPU gives the same bits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lithos_b200.h"

namespace lm {

#ifndef LM_BLOCK
#define LM_BLOCK 1024
#endif
constexpr int kBlock = LM_BLOCK;       // threads per block of the row kernels
constexpr int kWarps = kBlock / 32;
constexpr int kChunk = 8;              // consecutive logits one thread takes per step (one 128-bit load of BF16)
constexpr uint32_t kFull = 0xFFFFFFFFu;

// ---- element access ----------------------------------------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Monotone 32-bit key of a float: a > b  <=>  fkey(a) > fkey(b) (for non-NaN, with -0 canonicalised to +0 first).
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
__device__ __forceinline__ float canon_zero(float z) { return z == 0.0f ? 0.0f : z; }

// Repetition then presence penalty on one widened logit (both binary32, round to nearest).
__device__ __forceinline__ float penalise(float z, float rho, float pi) {
  z = (z > 0.0f) ? __fdiv_rn(z, rho) : __fmul_rn(z, rho);
  return __fsub_rn(z, pi);
}

// One row of logits as the kernels see it: widened to float, penalties applied on the fly from a bitmap of the
// row's distinct history ids (shared memory), -0 folded into +0.
struct RowView {
  const void* row;
  int dtype;
  int vocab;
  bool aligned;            // row start is 16-byte aligned: 128-bit loads are legal
  const uint32_t* pen;     // bitmap over [0, vocab) or nullptr
  float rho, pi;
};

// Elements [8c, 8c + 8) of the row; returns how many of them exist (0..8).
__device__ __forceinline__ int load_chunk(const RowView& rv, int c, float z[kChunk]) {
  const int base = c * kChunk;
  const int n = min(kChunk, rv.vocab - base);
  if (n <= 0) return 0;
  if (rv.dtype == LM_DTYPE_BF16) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(rv.row) + base;
    if (n == kChunk && rv.aligned) {
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(p));
      z[0] = bf16_lo(q.x); z[1] = bf16_hi(q.x); z[2] = bf16_lo(q.y); z[3] = bf16_hi(q.y);
      z[4] = bf16_lo(q.z); z[5] = bf16_hi(q.z); z[6] = bf16_lo(q.w); z[7] = bf16_hi(q.w);
    } else {
#pragma unroll
      for (int e = 0; e < kChunk; e++) z[e] = (e < n) ? __uint_as_float(static_cast<uint32_t>(__ldg(p + e)) << 16) : 0.0f;
    }
  } else {
    const float* p = reinterpret_cast<const float*>(rv.row) + base;
    if (n == kChunk && rv.aligned) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
      z[0] = a.x; z[1] = a.y; z[2] = a.z; z[3] = a.w; z[4] = b.x; z[5] = b.y; z[6] = b.z; z[7] = b.w;
    } else {
#pragma unroll
      for (int e = 0; e < kChunk; e++) z[e] = (e < n) ? __ldg(p + e) : 0.0f;
    }
  }
  if (rv.pen != nullptr) {
    const uint32_t bits = (rv.pen[c >> 2] >> ((c & 3) * 8)) & 0xFFu;
    if (bits) {
#pragma unroll
      for (int e = 0; e < kChunk; e++) if ((bits >> e) & 1u) z[e] = penalise(z[e], rv.rho, rv.pi);
    }
  }
#pragma unroll
  for (int e = 0; e < kChunk; e++) z[e] = canon_zero(z[e]);
  return n;
}

// ---- the counter-based noise of the reference's draw --------------------------------------------------------

__host__ __device__ __forceinline__ float uniform01(uint64_t seed, uint32_t step, uint32_t t, uint32_t i) {
  uint64_t x = seed + static_cast<uint64_t>(step) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(t) * 0xC2B2AE3D27D4EB4Full +
               static_cast<uint64_t>(i) * 0x165667B19E3779F9ull;
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 27; x *= 0x94D049BB133111EBull; x ^= x >> 31;
  return (static_cast<float>((x >> 41) & 0x7FFFFFull) + 0.5f) * (1.0f / 8388608.0f);
}
__device__ __forceinline__ float gumbel(uint64_t seed, uint32_t step, uint32_t t, uint32_t i) {
  return -logf(-logf(uniform01(seed, step, t, i)));
}

// ---- the integer-exact weights of the inverse-CDF draw ------------------------------------------------------

// 2^x for x <= 0: round-to-nearest split, degree-5 polynomial with fused multiply-adds, exact power-of-two scaling.
__device__ __forceinline__ float spec_exp2(float x) {
  if (!(x > -100.0f)) return 0.0f;
  x = fminf(x, 0.0f);
  const float n = rintf(x);
  const float f = __fsub_rn(x, n);
  float p = 0x1.5bba20p-10f;
  p = __fmaf_rn(p, f, 0x1.3cea88p-7f);
  p = __fmaf_rn(p, f, 0x1.c6b752p-5f);
  p = __fmaf_rn(p, f, 0x1.ebf9bcp-3f);
  p = __fmaf_rn(p, f, 0x1.62e42ap-1f);
  p = __fmaf_rn(p, f, 1.0f);
  return __fmul_rn(p, __int_as_float((static_cast<int>(n) + 127) << 23));
}
// log2(e) / T as a binary32: divided in binary64, rounded once.
__device__ __forceinline__ float exp2_scale(float temperature) {
  return __double2float_rn(__ddiv_rn(1.4426950408889634, static_cast<double>(temperature)));
}
// floor(2^40 * spec_exp2(fl32(fl32(z - vmax) * c)))
__device__ __forceinline__ uint64_t weight_q40(float z, float vmax, float c) {
  const float x = __fmul_rn(__fsub_rn(z, vmax), c);
  return __float2ull_rz(__fmul_rn(spec_exp2(x), 1099511627776.0f));
}
// Two weights at once on the packed binary32 instructions of sm_100 (fma.rn.f32x2 and friends): element for element the
// operations of weight_q40, so the same bits. (z - vmax is formed as z + (-vmax); the two exact power-of-two scalings, by 2^n
// and by 2^40, are one multiplication by 2^(n + 40).)
__device__ __forceinline__ void weight_q40_x2(float z0, float z1, float vmax, float c, uint64_t& w0, uint64_t& w1) {
  const float2 x = __fmul2_rn(__fadd2_rn(make_float2(z0, z1), make_float2(-vmax, -vmax)), make_float2(c, c));
  const float x0 = fminf(x.x, 0.0f), x1 = fminf(x.y, 0.0f);
  // round to nearest (ties to even) by adding and subtracting 1.5 * 2^23: for -100 < x <= 0 the sum has an ulp of 1, so this is
  // rintf(x) exactly, and the integer sits in the low bits of the sum (no conversion instructions, which run at a quarter of the rate)
  const float kMagic = 12582912.0f;
  const float2 t = __fadd2_rn(make_float2(x0, x1), make_float2(kMagic, kMagic));
  const float2 n = __fadd2_rn(t, make_float2(-kMagic, -kMagic));
  const int n0 = __float_as_int(t.x) - 0x4B400000, n1 = __float_as_int(t.y) - 0x4B400000;
  const float2 f = __fadd2_rn(make_float2(x0, x1), make_float2(-n.x, -n.y));
  float2 p = make_float2(0x1.5bba20p-10f, 0x1.5bba20p-10f);
  p = __ffma2_rn(p, f, make_float2(0x1.3cea88p-7f, 0x1.3cea88p-7f));
  p = __ffma2_rn(p, f, make_float2(0x1.c6b752p-5f, 0x1.c6b752p-5f));
  p = __ffma2_rn(p, f, make_float2(0x1.ebf9bcp-3f, 0x1.ebf9bcp-3f));
  p = __ffma2_rn(p, f, make_float2(0x1.62e42ap-1f, 0x1.62e42ap-1f));
  p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
  const float2 r = __fmul2_rn(p, make_float2(__int_as_float((n0 + 167) << 23), __int_as_float((n1 + 167) << 23)));
  w0 = (x.x > -100.0f) ? __float2ull_rz(r.x) : 0ull;                        // also NaN: weight 0
  w1 = (x.y > -100.0f) ? __float2ull_rz(r.y) : 0ull;
}
// floor(floor(u * 2^24) * total / 2^24), u clamped to [0, 1 - 2^-24]
__device__ __forceinline__ uint64_t cdf_target(float u, uint64_t total) {
  long long u24 = (u > 0.0f) ? __float2ll_rz(__fmul_rn(u, 16777216.0f)) : 0ll;
  if (u24 > 16777215ll) u24 = 16777215ll;
  const uint64_t a = static_cast<uint64_t>(u24);
  return (__umul64hi(total, a) << 40) | ((total * a) >> 24);
}
// binary32 probability of one token: fl32(double(w) / double(k))
__device__ __forceinline__ float prob_q40(uint64_t w, uint64_t k) {
  return __double2float_rn(__ddiv_rn(__ull2double_rn(w), __ull2double_rn(k)));
}
// fixed-point residual weight floor(2^40 * r) for a positive binary32 r <= 1
__device__ __forceinline__ uint64_t residual_q40(float r) { return __float2ull_rz(__fmul_rn(r, 1099511627776.0f)); }

// ---- block-wide reductions over kBlock threads (scratch: 32 entries of the type in shared memory) --------------

// 32-bit warp reductions by butterfly shuffles. (The single-instruction warp reduction, redux.sync, measured about 0.3 us per
// use on B200 when every warp of a block issues it: far slower than five shuffles.)
__device__ __forceinline__ uint32_t warp_sum_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}
__device__ __forceinline__ uint32_t warp_max_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(kFull, v, o));
  return v;
}
__device__ __forceinline__ uint32_t warp_min_u32(uint32_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(kFull, v, o));
  return v;
}
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { const uint64_t t = __shfl_xor_sync(kFull, v, o); v = t > v ? t : v; }
  return v;
}
__device__ __forceinline__ uint64_t warp_sum_u64(uint64_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

// All threads of the block must call; every thread gets the result. `scratch` holds blockDim.x/32 entries.
__device__ __forceinline__ uint64_t block_max_u64(uint64_t v, uint64_t* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max_u64(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  uint64_t r = (lane < nw) ? scratch[lane] : 0ull;
  return warp_max_u64(r);
}
__device__ __forceinline__ uint64_t block_sum_u64(uint64_t v, uint64_t* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum_u64(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  uint64_t r = (lane < nw) ? scratch[lane] : 0ull;
  return warp_sum_u64(r);
}
__device__ __forceinline__ double block_sum_f64(double v, uint64_t* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  double* s = reinterpret_cast<double*>(scratch);
  v = warp_sum_f64(v);
  __syncthreads();
  if (lane == 0) s[warp] = v;
  __syncthreads();
  double r = (lane < nw) ? s[lane] : 0.0;
  return warp_sum_f64(r);
}
// Exclusive prefix sum over the block's threads in thread order; *total gets the block sum.
__device__ __forceinline__ uint64_t block_exclusive_scan_u64(uint64_t v, uint64_t* scratch, uint64_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  uint64_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const uint64_t t = __shfl_up_sync(kFull, incl, o); if (lane >= o) incl += t; }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  uint64_t w = (lane < nw) ? scratch[lane] : 0ull;
  uint64_t winc = w;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) { const uint64_t t = __shfl_up_sync(kFull, winc, o); if (lane >= o) winc += t; }
  const uint64_t warp_base = __shfl_sync(kFull, winc - w, warp);
  if (total) *total = __shfl_sync(kFull, winc, nw - 1);
  return warp_base + incl - v;
}

// Packed (value, index) for argmax with ties -> lowest index: larger packed value wins.
__device__ __forceinline__ uint64_t pack_best(float v, uint32_t idx) { return (static_cast<uint64_t>(fkey(v)) << 32) | (0xFFFFFFFFu - idx); }
__device__ __forceinline__ uint32_t best_index(uint64_t p) { return 0xFFFFFFFFu - static_cast<uint32_t>(p); }
__device__ __forceinline__ float best_value(uint64_t p) { return fkey_inv(static_cast<uint32_t>(p >> 32)); }

}  // namespace lm
