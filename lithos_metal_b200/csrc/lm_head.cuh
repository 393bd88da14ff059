// The vocabulary projection of a decode step: logits[t, v] = bf16(sum_k x[t, k] * W[v, k]) for the T <= 8 rows of a step
// (one token, or the verification rows of a speculative round), with the final RMSNorm fused on the input
// (monolith/nn/lm_head.py:50-60: the `lm_head` op, norm = stat + weight, out = bf16; its semantics are
// monolith/nn/oracle.py:20-32: FP32 accumulation and one rounding to BF16; the norm's output rounded to BF16 first).
//
// With at most 8 rows this is a matrix-vector product: every weight is read once from HBM and used 8 times, so the kernel is
// bound by the weight stream (V x H BF16: 1.24 GB for 151,936 x 4096), not by arithmetic. The rows sit in shared memory as BF16;
// a warp takes 16 vocabulary rows at a time and walks the hidden dimension 64 elements per step: 32 bytes of W per thread and
// row (rows g and g + 8 of the tile, at element offset 16 * t: a whole 128-byte line per row and quad), 32 bytes of x from
// shared memory, four mma.sync m16n8k16 (BF16 in, FP32 accumulate) whose k slots are fed in the order the loads deliver --
// the same permutation of k on both operands, so the sums are over the same products. (The tensor-core instruction is here for
// the 8 FMAs per weight, which the FP32 pipes could not do at the rate HBM delivers weights; its throughput is nowhere near a
// limit.) Every vocabulary row's sum is formed in the same order wherever the row sits, so a shard of the weight gives the
// bits of the whole. The logits go to memory (2.4 MB for 8 x 151,936: they stay in L2 for the sampler that is launched behind).
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"

namespace lm {

constexpr int kHeadThreads = 256;
constexpr int kHeadWarps = kHeadThreads / 32;
constexpr int kHeadRows = 8;                 // rows of x (the n dimension of the mma)
constexpr int kHeadTile = 16;                // vocabulary rows per warp tile (the m dimension)
constexpr int kHeadStep = 64;                // hidden elements per step: 32 bytes per thread and row, a whole 128-byte line per row and quad
constexpr int kHeadPad = 8;                  // elements between the rows of x in shared memory beyond H: a 16-byte skew, so that the
                                             // 16-byte loads of a quarter warp (two rows, four offsets 32 bytes apart) fall on different banks
constexpr int kHeadUnroll = 8;               // steps whose loads are in flight together (32 x 16 bytes per thread): a batch
constexpr int kHeadMaxBatches = 25;          // batches of the longest row that fits (hidden 12,736)

struct HeadDev {
  const uint16_t* x; int64_t x_stride; int rows;
  const uint16_t* w; int64_t w_stride; int hidden; int vocab;
  const uint16_t* gamma; float eps; int one_plus;
  uint16_t* logits; int64_t logits_stride;
};

__host__ __device__ inline size_t head_smem_bytes(int hidden) { return static_cast<size_t>(kHeadRows) * (hidden + kHeadPad) * 2; }

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint16_t f32_to_bf16_rn(float f) {                // round to nearest even (NaN stays NaN)
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  return static_cast<uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

__global__ void __launch_bounds__(kHeadThreads) lm_head_kernel(HeadDev P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);                    // [kHeadRows][H + kHeadPad] BF16, rows beyond P.rows zero
  __shared__ float s_part[kHeadRows][kHeadWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = P.hidden, ld = H + kHeadPad;
  // ---- the rows of x into shared memory, normalised on the way if a norm is fused (every block for itself: 64 KB from L2)
  float inv_rms = 1.0f;
  for (int r = 0; r < kHeadRows; r++) {
    if (r < P.rows && P.gamma) {
      float ss = 0.0f;
      for (int k = tid; k < H; k += kHeadThreads) { const float v = bf16_hi(static_cast<uint32_t>(P.x[r * P.x_stride + k]) << 16); ss = __fmaf_rn(v, v, ss); }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(kFull, ss, o);
      if (lane == 0) s_part[r][warp] = ss;
    }
  }
  __syncthreads();
  for (int r = 0; r < kHeadRows; r++) {
    if (r < P.rows && P.gamma) {
      float ss = 0.0f;
#pragma unroll
      for (int q = 0; q < kHeadWarps; q++) ss += s_part[r][q];
      inv_rms = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(H)), P.eps));
    }
    for (int k = tid; k < ld; k += kHeadThreads) {
      uint16_t out = 0u;
      if (r < P.rows && k < H) {
        out = P.x[r * P.x_stride + k];
        if (P.gamma) {
          const float v = __fmul_rn(bf16_hi(static_cast<uint32_t>(out) << 16), inv_rms);
          const float g = bf16_hi(static_cast<uint32_t>(P.gamma[k]) << 16);
          out = f32_to_bf16_rn(__fmul_rn(v, P.one_plus ? __fadd_rn(1.0f, g) : g));
        }
      }
      xs[r * ld + k] = out;
    }
  }
  __syncthreads();
  // ---- the tiles: 16 vocabulary rows per warp and turn
  // A tile's sums are formed batch by batch (kHeadUnroll steps into a fresh accumulator, then added to the total), the batches in
  // order: the same additions whether one warp walks the whole row or, for the few tiles left over after the last full round, the
  // warps of a block take a batch each and one of them adds the partial sums up in that order.
  const int g = lane >> 2, t = lane & 3;
  const int n_tiles = (P.vocab + kHeadTile - 1) / kHeadTile;
  const int steps = H / kHeadStep, batches = (steps + kHeadUnroll - 1) / kHeadUnroll;
  const uint4* xrow = reinterpret_cast<const uint4*>(xs + g * ld) + 2 * t;  // this thread's 32 bytes of x per step: row g, elements 16 t ..
  auto batch_sum = [&](const uint4* wa, const uint4* wb, int batch, float (&c)[4]) {
    const int s0 = batch * kHeadUnroll;
    uint4 a[kHeadUnroll][2], b[kHeadUnroll][2];
#pragma unroll
    for (int u = 0; u < kHeadUnroll; u++) {
      const int s = s0 + u;
      if (s < steps) {                                                    // streamed: every weight is used once
        a[u][0] = __ldcs(wa + 8 * s); a[u][1] = __ldcs(wa + 8 * s + 1);
        b[u][0] = __ldcs(wb + 8 * s); b[u][1] = __ldcs(wb + 8 * s + 1);
      } else { a[u][0] = a[u][1] = b[u][0] = b[u][1] = make_uint4(0u, 0u, 0u, 0u); }
    }
    c[0] = c[1] = c[2] = c[3] = 0.0f;
#pragma unroll
    for (int u = 0; u < kHeadUnroll; u++) {
      const int s = s0 + u;
      if (s >= steps) break;
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const uint4 x = xrow[8 * s + h];
        mma_bf16_16816(c, a[u][h].x, b[u][h].x, a[u][h].y, b[u][h].y, x.x, x.y);
        mma_bf16_16816(c, a[u][h].z, b[u][h].z, a[u][h].w, b[u][h].w, x.z, x.w);
      }
    }
  };
  // c[0], c[1]: vocabulary row v0 + g, rows 2 t and 2 t + 1 of x; c[2], c[3]: vocabulary row v0 + g + 8
  auto store = [&](int v0, const float (&c)[4]) {
    const int r0 = 2 * t, r1 = 2 * t + 1;
    if (v0 + g < P.vocab) {
      if (r0 < P.rows) P.logits[r0 * P.logits_stride + v0 + g] = f32_to_bf16_rn(c[0]);
      if (r1 < P.rows) P.logits[r1 * P.logits_stride + v0 + g] = f32_to_bf16_rn(c[1]);
    }
    if (v0 + g + 8 < P.vocab) {
      if (r0 < P.rows) P.logits[r0 * P.logits_stride + v0 + g + 8] = f32_to_bf16_rn(c[2]);
      if (r1 < P.rows) P.logits[r1 * P.logits_stride + v0 + g + 8] = f32_to_bf16_rn(c[3]);
    }
  };
  auto rows_of = [&](int tile, const uint4*& wa, const uint4*& wb) {
    const int v0 = tile * kHeadTile;
    const int ra = min(v0 + g, P.vocab - 1), rb = min(v0 + g + 8, P.vocab - 1);    // (rows beyond the vocabulary: loaded again, never stored)
    wa = reinterpret_cast<const uint4*>(P.w + static_cast<int64_t>(ra) * P.w_stride) + 2 * t;
    wb = reinterpret_cast<const uint4*>(P.w + static_cast<int64_t>(rb) * P.w_stride) + 2 * t;
  };
  const int all_warps = gridDim.x * kHeadWarps;
  const int full = n_tiles / all_warps * all_warps;                        // tiles of the full rounds: one warp each
  for (int tile = blockIdx.x * kHeadWarps + warp; tile < full; tile += all_warps) {
    const uint4 *wa, *wb;
    rows_of(tile, wa, wb);
    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c[4];
    for (int batch = 0; batch < batches; batch++) {
      batch_sum(wa, wb, batch, c);
#pragma unroll
      for (int e = 0; e < 4; e++) total[e] = __fadd_rn(total[e], c[e]);
    }
    store(tile * kHeadTile, total);
  }
  // the tiles left over: one block each, a batch per warp and turn, the partial sums added up in batch order by warp 0
  __shared__ float part[kHeadMaxBatches][32][4];
  for (int tile = full + blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const uint4 *wa, *wb;
    rows_of(tile, wa, wb);
    for (int batch = warp; batch < batches; batch += kHeadWarps) {
      float c[4];
      batch_sum(wa, wb, batch, c);
#pragma unroll
      for (int e = 0; e < 4; e++) part[batch][lane][e] = c[e];
    }
    __syncthreads();
    if (warp == 0) {
      float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int batch = 0; batch < batches; batch++) {
#pragma unroll
        for (int e = 0; e < 4; e++) total[e] = __fadd_rn(total[e], part[batch][lane][e]);
      }
      store(tile * kHeadTile, total);
    }
    __syncthreads();
  }
}

}  // namespace lm
