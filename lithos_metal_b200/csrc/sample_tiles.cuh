// Sampling from logits that arrive TILE BY TILE: the boundary between the vocabulary projection (lm_head) and the sampler.
//
// The reference lowers lm_head to a GEMV / GEMM that writes logits [T, V] in BF16 to memory, and the sampler reads them back
// (monolith/nn/lm_head.py:50-60). On B200 the projection is a tensor-core GEMM whose epilogue holds a tile of logits
// [rows, 128..256 columns] in registers / shared memory; what the sampler needs from a tile is small: per row the running
// maximum, the running softmass, and the few logits that can still be among the row's top_k. This file is that consumer:
//
//   tile_consume_row   (device, block-cooperative)  one row of one tile -> the row's running state and candidate list
//   tile_consume_kernel                             the same as a launch, for tiles that lie in (L2-resident) memory
//   tile_finish_kernel                              the exact phases of the candidate path (sample_topk.cuh, topk_finish) on
//                                                   the collected candidates: thresholds, draw, token
//
// so that [rows, V] never has to exist. A GEMM epilogue calls tile_consume_row on the tile it holds (BF16 codes, rounded as
// lm_head would store them), the launch form serves producers that stage tiles in a small buffer, and the test feeds tiles cut
// from a materialised tensor and must get lm_sample's tokens.
//
// The row state is (m, s) = running maximum and sum_i 2^((z_i - m) c) in FP64 (each tile's share is summed in FP32 relative to
// the tile's own maximum and joined in FP64, so the error does not grow with the number of tiles), a cutoff value, and a list of
// every logit seen so far at or above the cutoff. The cutoff starts at -inf and only ever rises to the value of the k'-th
// largest logit seen so far (k' = top_k + top_k / 3 + 150, a compaction when the list fills), so the list always holds the
// row's top_k. Penalties are applied as the logits arrive (a bitmap of the row's distinct history ids in the state, built by
// tile_begin_kernel); greedy rows keep a running argmax. Rows without a top_k, or whose candidates do not fit the exact phases,
// are DECLINED (status bit): the caller materialises those rows and calls lm_sample.
#pragma once
#include "common.cuh"
#include "sample_topk.cuh"

namespace lm {

constexpr int kTileListCap = 8192;          // entries of a row's candidate list in the state buffer
constexpr int kTileMaxCols = 2048;          // columns of one tile
constexpr int kTileFill = kTileListCap - kTileMaxCols;   // a list longer than this is compacted before the next tile is added
constexpr int kTileBlock = 256;
constexpr uint32_t kTileDeclined = 1u;      // TileRow.flags

struct TileRow {                            // 48 bytes per row; all zero = nothing seen yet
  double m;                                 // running maximum (valid when something was seen)
  double s;                                 // sum_i 2^((z_i - m) c) over everything seen
  double s_pen;                             // the part of s that penalised logits contributed
  unsigned long long best;                  // packed (value, lowest index) of the running maximum: the greedy pick
  float cutoff;                             // every logit >= cutoff seen so far is in the list (valid when the cutoff bit is set)
  uint32_t n;                               // entries in the list
  uint32_t flags;                           // bit 0: declined; bit 1: cutoff set; bit 2: something seen
  uint32_t pad;
};

struct TileDev {
  const void* tile; int dtype; int rows; int vocab; int64_t tile_stride; int col0; int cols;
  const float* temperature; float temperature_s; const int32_t* top_k; int32_t top_k_s;
  TileRow* rows_state; unsigned long long* lists;      // lists[row * kTileListCap + i]
  uint32_t* pen_bits; int pen_words;                   // per row: bitmap of its distinct history ids (pen_words words), or nullptr
  const int32_t* history; int hist_len; int64_t hist_stride; float rho, pi;
};

__device__ __forceinline__ uint32_t f32_to_bf16_code(float f) {            // round to nearest even, as a BF16 store of the logit would
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x0040u;         // NaN stays NaN
  return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}

// The value key of the k-th largest entry (k >= 1, k <= n) of list[0 .. n): a 4 x 8-bit radix descent on the 32-bit monotone
// value keys, counting in shared memory. Every thread of the block calls; hist: 256 counters; pick: 2 words.
__device__ uint32_t tile_kth_key(const unsigned long long* list, int n, int k, uint32_t* hist, uint32_t* pick) {
  uint32_t prefix = 0u, above = 0u;                                       // `above`: entries whose key is larger than every key with this prefix
  for (int level = 0; level < 4; level++) {
    const int shift = 24 - 8 * level;
    const uint32_t hi_mask = level == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = static_cast<uint32_t>(list[i] >> 32);
      if ((key & hi_mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xFFu], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {                                               // 256 bins from the top: the bin where the count reaches k
      uint32_t run = above; int b = 255;
      for (; b > 0; b--) { if (run + hist[b] >= static_cast<uint32_t>(k)) break; run += hist[b]; }
      pick[0] = static_cast<uint32_t>(b); pick[1] = run;
    }
    __syncthreads();
    prefix |= pick[0] << shift; above = pick[1];
    __syncthreads();
  }
  return prefix;
}

// Keeps the entries of list[0 .. n) whose value key is >= min_key, in their order; returns how many. Every thread calls.
__device__ int tile_filter(unsigned long long* list, int n, uint32_t min_key, uint32_t* warp_cnt) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int out = 0;
  for (int i0 = 0; i0 < n; i0 += blockDim.x) {                            // a batch is read completely before any of it is written
    const int i = i0 + threadIdx.x;
    const unsigned long long e = i < n ? list[i] : 0ull;
    const bool keep = i < n && static_cast<uint32_t>(e >> 32) >= min_key;
    const uint32_t votes = __ballot_sync(kFull, keep);
    if (lane == 0) warp_cnt[warp] = __popc(votes);
    __syncthreads();
    int base = out, total = 0;
    for (int w = 0; w < nw; w++) { if (w < warp) base += warp_cnt[w]; total += warp_cnt[w]; }
    if (keep) list[base + __popc(votes & ((1u << lane) - 1u))] = e;      // base + rank <= i: never ahead of an unread entry of a later batch
    out += total;
    __syncthreads();
  }
  return out;
}

// One row of one tile. codes: the row's `cols` BF16 codes of columns col0 .. col0 + cols (shared or global memory). Every thread
// of the block calls with the same arguments. scratch: 256 + 2 + 32 words and 32 doubles of shared memory (TileScratch).
struct TileScratch { uint32_t hist[256]; uint32_t pick[2]; uint32_t warp_cnt[32]; double warp_d[32]; double warp_p[32]; uint64_t warp_m[32]; uint32_t n_now; };

__device__ void tile_consume_row(TileRow* st, unsigned long long* list, const uint16_t* codes, int cols, int col0, float temperature, int top_k,
                                 const uint32_t* pen_bits, float rho, float pi, TileScratch& t) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  if (st->flags & kTileDeclined) return;
  // the logit of column j of the tile, as the sampler sees it: widened, penalised if the row's history holds its id, -0 folded into +0
  auto logit = [&](int j, bool* penalised) -> float {
    float z = __uint_as_float(static_cast<uint32_t>(codes[j]) << 16);
    const int id = col0 + j;
    const bool p = pen_bits != nullptr && ((pen_bits[id >> 5] >> (id & 31)) & 1u);
    if (p) z = penalise(z, rho, pi);
    *penalised = p;
    return canon_zero(z);
  };
  if (temperature == 0.0f) {                                               // greedy: the running argmax is all there is
    uint64_t gb = 0ull; bool gnan = false;
    for (int j = tid; j < cols; j += blockDim.x) {
      bool p; const float z = logit(j, &p);
      gnan = gnan || (z != z);
      const uint64_t k = pack_best(z, static_cast<uint32_t>(col0 + j));
      gb = k > gb ? k : gb;
    }
    gb = warp_max_u64(gb);
    if (lane == 0) t.warp_m[warp] = gb;
    const bool any = __syncthreads_or(gnan) != 0;
    if (tid == 0) {
      uint64_t bb = st->best;
      for (int w = 0; w < nw; w++) bb = t.warp_m[w] > bb ? t.warp_m[w] : bb;
      st->best = bb; st->flags |= 4u | (any ? kTileDeclined : 0u);
    }
    __syncthreads();
    return;
  }
  if (top_k < 1 || top_k > kTopkMaxK || !(temperature > 0.0f)) { if (tid == 0) st->flags |= kTileDeclined; return; }
  const double c64 = 1.4426950408889634 / static_cast<double>(temperature);
  const float c2a = static_cast<float>(c64);
  // ---- the list makes room first: everything below the k'-th largest logit seen so far goes, and the cutoff rises to it
  int n = static_cast<int>(st->n);
  float cutoff = (st->flags & 2u) ? st->cutoff : -INFINITY;
  if (n > kTileFill) {
    const int keep_k = min(n, top_k + top_k / 3 + 150);
    const uint32_t kkey = tile_kth_key(list, n, keep_k, t.hist, t.pick);
    n = tile_filter(list, n, kkey, t.warp_cnt);
    cutoff = fkey_inv(kkey);
    if (n > kTileFill) { if (tid == 0) st->flags |= kTileDeclined; return; }   // ties by the thousand: not this path's row
  }
  // ---- the tile's maximum and its softmass relative to that maximum
  uint64_t best = 0ull; bool nan = false;
  for (int j = tid; j < cols; j += blockDim.x) {
    bool pz; const float z = logit(j, &pz);
    nan = nan || (z != z);
    const uint64_t p = pack_best(z, static_cast<uint32_t>(j));
    best = p > best ? p : best;
  }
  best = warp_max_u64(best);
  if (lane == 0) t.warp_m[warp] = best;
  const bool any_nan = __syncthreads_or(nan) != 0;
  uint64_t bb = 0ull;
  for (int w = 0; w < nw; w++) bb = t.warp_m[w] > bb ? t.warp_m[w] : bb;
  const float tmax = best_value(bb);
  if (any_nan || tmax == INFINITY) { if (tid == 0) st->flags |= kTileDeclined; return; }   // NaN / +inf: the exact path reports them
  float acc = 0.0f, acc_pen = 0.0f;
  for (int j = tid; j < cols; j += blockDim.x) {
    bool p; const float z = logit(j, &p);
    const float e = ex2_approx(__fmul_rn(__fsub_rn(z, tmax), c2a));       // z - tmax is exact for BF16 values within 16 binades
    if (p) acc_pen += e; else acc += e;                                   // (a penalised logit is not on the BF16 grid: its term is counted apart)
  }
  const double sd = warp_sum_f64(static_cast<double>(acc)), sp = warp_sum_f64(static_cast<double>(acc_pen));
  if (lane == 0) { t.warp_d[warp] = sd; t.warp_p[warp] = sp; }
  if (tid == 0) t.n_now = static_cast<uint32_t>(n);
  __syncthreads();
  // ---- the logits at or above the cutoff join the list
  for (int j0 = 0; j0 < cols; j0 += blockDim.x) {                         // uniform trip count: warp votes inside
    const int j = j0 + tid;
    bool p = false;
    const float z = j < cols ? logit(j, &p) : -INFINITY;
    const bool take = j < cols && z >= cutoff;
    const uint32_t votes = __ballot_sync(kFull, take);
    uint32_t base = 0u;
    if (lane == 0 && votes) base = atomicAdd(&t.n_now, __popc(votes));
    base = __shfl_sync(kFull, base, 0);
    if (take) {
      const uint32_t slot = base + __popc(votes & ((1u << lane) - 1u));
      if (slot < static_cast<uint32_t>(kTileListCap)) list[slot] = (static_cast<unsigned long long>(fkey(z)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(col0 + j));
    }
  }
  __syncthreads();
  if (tid == 0) {
    double ts = 0.0, tp = 0.0;
    for (int w = 0; w < nw; w++) { ts += t.warp_d[w]; tp += t.warp_p[w]; }
    const bool seen = (st->flags & 4u) != 0u;
    const double m_old = seen ? st->m : -INFINITY, tm = static_cast<double>(tmax);
    const double m_new = tm > m_old ? tm : m_old;
    const double f_tile = exp2((tm - m_new) * c64), f_old = seen ? exp2((m_old - m_new) * c64) : 0.0;
    st->s = (ts + tp) * f_tile + (seen ? st->s * f_old : 0.0);
    st->s_pen = tp * f_tile + (seen ? st->s_pen * f_old : 0.0);
    st->m = m_new;
    st->cutoff = cutoff; st->n = min(t.n_now, static_cast<uint32_t>(kTileListCap));
    st->flags |= 4u | (cutoff > -INFINITY ? 2u : 0u) | (t.n_now > static_cast<uint32_t>(kTileListCap) ? kTileDeclined : 0u);
  }
  __syncthreads();
}

// A tile that lies in memory: one block per row. FP32 tiles are rounded to BF16 first (what lm_head stores).
__global__ void __launch_bounds__(kTileBlock) tile_consume_kernel(TileDev P) {
  __shared__ TileScratch t;
  __shared__ uint16_t codes[kTileMaxCols];
  const int row = blockIdx.x;
  if (row >= P.rows) return;
  for (int j = threadIdx.x; j < P.cols; j += blockDim.x) {
    codes[j] = P.dtype == LM_DTYPE_BF16 ? __ldg(reinterpret_cast<const uint16_t*>(P.tile) + static_cast<int64_t>(row) * P.tile_stride + j)
                                        : static_cast<uint16_t>(f32_to_bf16_code(__ldg(reinterpret_cast<const float*>(P.tile) + static_cast<int64_t>(row) * P.tile_stride + j)));
  }
  __syncthreads();
  tile_consume_row(P.rows_state + row, P.lists + static_cast<size_t>(row) * kTileListCap, codes, P.cols, P.col0,
                   P.temperature ? P.temperature[row] : P.temperature_s, P.top_k ? P.top_k[row] : P.top_k_s,
                   P.pen_bits ? P.pen_bits + static_cast<size_t>(row) * P.pen_words : nullptr, P.rho, P.pi, t);
}

// Clears the rows' states and, with a history, builds each row's bitmap of distinct history ids. One block per row.
__global__ void __launch_bounds__(kTileBlock) tile_begin_kernel(TileDev P) {
  const int row = blockIdx.x;
  if (row >= P.rows) return;
  if (threadIdx.x < sizeof(TileRow) / 8) reinterpret_cast<unsigned long long*>(P.rows_state + row)[threadIdx.x] = 0ull;
  if (P.pen_bits == nullptr) return;
  uint32_t* bits = P.pen_bits + static_cast<size_t>(row) * P.pen_words;
  for (int i = threadIdx.x; i < P.pen_words; i += blockDim.x) bits[i] = 0u;
  __syncthreads();
  const int32_t* h = P.history + static_cast<int64_t>(row) * P.hist_stride;
  for (int i = threadIdx.x; i < P.hist_len; i += blockDim.x) {
    const int id = __ldg(h + i);
    if (id >= 0 && id < P.vocab) atomicOr(&bits[id >> 5], 1u << (id & 31));
  }
}

// The rows' tokens from their states and lists: a last compaction to what the exact phases hold, the candidates into shared
// memory with their code bins, then topk_finish. A row that cannot be finished here gets token -1 and LM_STATUS_TILE_DECLINED.
__global__ void __launch_bounds__(kTB, kTopkPerSM) tile_finish_kernel(SampleDev P, TileRow* states, unsigned long long* lists) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TopkSmem& c = *reinterpret_cast<TopkSmem*>(smem_raw);
  __shared__ TileScratch t;
  apply_step_state(P);
  const int tid = threadIdx.x;
  for (int row = blockIdx.x; row < P.rows; row += gridDim.x) {
    TileRow* st = states + row;
    unsigned long long* list = lists + static_cast<size_t>(row) * kTileListCap;
    const int top_k = P.top_k ? P.top_k[row] : P.top_k_s;
    const float T = P.temperature ? P.temperature[row] : P.temperature_s;
    if (T == 0.0f && !(st->flags & kTileDeclined) && (st->flags & 4u)) {     // greedy: the running argmax
      if (tid == 0) {
        P.out_tokens[row] = static_cast<int>(best_index(st->best));
        if (P.out_tau) P.out_tau[row] = -INFINITY;
        if (P.out_status) P.out_status[row] = 0u;
        if (P.out_vmax) P.out_vmax[row] = best_value(st->best);
        if (P.out_mass) P.out_mass[row] = 0ull;
      }
      __syncthreads();
      continue;
    }
    bool ok = !(st->flags & kTileDeclined) && (st->flags & 4u) && top_k >= 1 && top_k <= kTopkMaxK && T > 0.0f && static_cast<int>(st->n) >= top_k;
    int n = static_cast<int>(st->n);
    uint32_t cut_key = 0u;
    if (ok) {
      // the k'-th largest logit of the row is the cutoff of the exact phases (the list holds every logit at or above it)
      const int keep_k = min(n, top_k + top_k / 3 + 150);
      cut_key = tile_kth_key(list, n, keep_k, t.hist, t.pick);
      n = tile_filter(list, n, cut_key, t.warp_cnt);
      const float cut_val = fkey_inv(cut_key);
      ok = n <= kTopkCap && cut_val > 0.0f && (__float_as_uint(cut_val) >> 16) >= 0x0080u;    // a positive, normal BF16 cutoff
    }
    if (ok) {
      const uint32_t cut_code = __float_as_uint(fkey_inv(cut_key)) >> 16;
      for (int i = tid; i < kTopkBins; i += kTB) c.bins[i] = 0u;
      if (tid == 0) { c.n = static_cast<uint32_t>(n); c.wide = 0u; c.hit = kTopkCap; c.token = -1; c.cross_bin = 0u; c.n_hit = 0u; }
      __syncthreads();
      for (int i = tid; i < n; i += kTB) {
        const unsigned long long e = list[i];
        c.key[i] = e;
        const uint32_t rel = (__float_as_uint(fkey_inv(static_cast<uint32_t>(e >> 32))) >> 16) - cut_code;
        if (rel >= kTopkBins) c.wide = 1u; else atomicAdd(&c.bins[rel], 1u);
      }
      __syncthreads();
      RowMass zm;
      zm.need = true; zm.z_tilde = st->s; zm.z_raw = st->s - st->s_pen; zm.z_corr = st->s_pen;
      zm.shift = st->m * (1.4426950408889634 / static_cast<double>(T));
      zm.ref = static_cast<float>(st->m); zm.acc_terms = static_cast<double>(kTileMaxCols / kTileBlock) + 1.0;
      ok = topk_finish(P, row, c, cut_code, zm);
      __syncthreads();
    }
    if (!ok && tid == 0) {
      P.out_tokens[row] = -1;
      if (P.out_tau) P.out_tau[row] = -INFINITY;
      if (P.out_status) P.out_status[row] = LM_STATUS_TILE_DECLINED;
      if (P.out_vmax) P.out_vmax[row] = (st->flags & 4u) ? static_cast<float>(st->m) : -INFINITY;
      if (P.out_mass) P.out_mass[row] = 0ull;
    }
    __syncthreads();
  }
}

}  // namespace lm
