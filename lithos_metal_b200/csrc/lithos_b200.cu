// C ABI of the B200 generation-control library (declared in include/lithos_b200.h): argument checks, launch
// geometry, kernel launches. No allocation, no synchronisation, no CPU arithmetic on the data path.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "sample_generic.cuh"
#include "sample_hist.cuh"
#include "sample_topk.cuh"
#include "sample_tiles.cuh"
#include "sample_sliced.cuh"
#include "verify.cuh"
#include "draft_q.cuh"
#include "vocab_parallel.cuh"
#include "spec_ops.cuh"
#include "lm_head.cuh"

namespace lm {

static_assert(kBlock == 512 || kBlock == 1024, "the row kernels are written for 512 or 1024 threads per block");

// ---- greedy argmax: rows x splits blocks, packed (value, lowest index) maxima meet in the workspace --------------
constexpr int kArgmaxBlock = 512;

struct ArgmaxWs { unsigned long long best; unsigned arrivals; unsigned pad; };   // one per row, zero when idle

__global__ void __launch_bounds__(kArgmaxBlock) argmax_kernel(const void* logits, int dtype, int rows, int vocab, int64_t row_stride, int splits,
                                                             int32_t* out_tokens, ArgmaxWs* ws) {
  __shared__ uint64_t scratch[32];
  const int row = blockIdx.y, split = blockIdx.x, tid = threadIdx.x;
  RowView rv;
  rv.dtype = dtype; rv.vocab = vocab; rv.pen = nullptr; rv.rho = 1.0f; rv.pi = 0.0f;
  rv.row = static_cast<const char*>(logits) + static_cast<size_t>(row) * static_cast<size_t>(row_stride) * (dtype == LM_DTYPE_BF16 ? 2 : 4);
  rv.aligned = (reinterpret_cast<uintptr_t>(rv.row) & 15u) == 0;
  const int n_chunks = (vocab + kChunk - 1) / kChunk;
  uint64_t best = 0ull;
  for (int c = split * kArgmaxBlock + tid; c < n_chunks; c += splits * kArgmaxBlock) {
    float z[kChunk];
    const int n = load_chunk(rv, c, z);
#pragma unroll
    for (int e = 0; e < kChunk; e++) if (e < n) {
      const uint64_t p = pack_best(z[e], static_cast<uint32_t>(c * kChunk + e));
      best = p > best ? p : best;
    }
  }
  best = block_max_u64(best, scratch);
  if (tid != 0) return;
  if (splits == 1) { out_tokens[row] = best ? static_cast<int>(best_index(best)) : -1; return; }
  if (best) atomicMax(&ws[row].best, static_cast<unsigned long long>(best));
  __threadfence();
  if (atomicAdd(&ws[row].arrivals, 1u) == static_cast<unsigned>(splits) - 1u) {   // the last block of the row
    __threadfence();
    const unsigned long long b = atomicExch(&ws[row].best, 0ull);
    ws[row].arrivals = 0u;
    out_tokens[row] = b ? static_cast<int>(best_index(b)) : -1;
  }
}

// ---- the generic sampler: one block per row, grid-stride over rows, or over the rows an earlier kernel listed ---------------
__global__ void __launch_bounds__(kBlock, 1) sample_generic_kernel(SampleDev P, const int* list, const int* n_list) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  GenericSmem& s = *reinterpret_cast<GenericSmem*>(smem_raw);
  uint32_t* pen_bits = reinterpret_cast<uint32_t*>(smem_raw + sizeof(GenericSmem));
  apply_step_state(P);
  const int n = list ? min(*n_list, P.rows) : P.rows;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int row = list ? list[i] : i;
    if (row >= 0 && row < P.rows) sample_row_generic(P, row, s, pen_bits);
    __syncthreads();
  }
}

// Scratch of lm_argmax_static: a fixed array in the library image (zero at load). In host code this name is only a
// handle for cudaGetSymbolAddress; the kernels get the device address that call returns.
static __device__ __align__(256) ArgmaxWs g_argmax_static_ws[LM_ARGMAX_STATIC_MAX_ROWS];

thread_local char g_cuda_error[256] = "";

static int cuda_fail(cudaError_t e) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return LM_E_CUDA;
}

constexpr int kOverlapRowsPerSM = 5;    // up to this many rows per SM the two sampler kernels run side by side (lm_sample)
constexpr int kAloneRowsPerSM = 2;      // ... and up to this many the histogram kernel's blocks have their SM to themselves
constexpr size_t kAloneSmemBytes = 140 * 1024;   // more than an SM's shared memory less a block of the top-k kernel

static int sm_count(int* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  static thread_local int cached_dev = -1, cached = 0;
  if (cached_dev != dev) {
    e = cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    cached_dev = dev;
  }
  *out = cached;
  return LM_OK;
}

// Kernels that need more than 48 KB of dynamic shared memory must be told so once per device (the attribute belongs to the
// device's copy of the function); remembered per device and kernel, raised when a call needs more.
enum KernelSlot { kSlotFast, kSlotTopk, kSlotGeneric, kSlotVocabLocal, kSlotVerify, kSlotVerifyStats, kSlotDraftQ, kSlotTileFinish, kSlotSlice, kSlotSliceSmall, kSlotSliceTiny, kSlotSlicedMerge, kSlotHead, kSlotCount };

static int ensure_dynamic_smem(KernelSlot slot, const void* func, size_t bytes) {
  if (bytes <= 48 * 1024) return LM_OK;
  constexpr int kMaxDevices = 64;
  static std::mutex mutex;
  static size_t granted[kMaxDevices][kSlotCount] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  std::lock_guard<std::mutex> lock(mutex);
  const bool tracked = dev >= 0 && dev < kMaxDevices;
  if (tracked && bytes <= granted[dev][slot]) return LM_OK;
  e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e != cudaSuccess) return cuda_fail(e);
  if (tracked) granted[dev][slot] = bytes;
  return LM_OK;
}

static bool sample_has_penalties(const lm_sample_args* a) {
  return a->history != nullptr && a->hist_len > 0 && !(a->repetition_penalty == 1.0f && a->presence_penalty == 0.0f);
}

// The device-side view of a validated lm_sample_args.
static SampleDev sample_dev(const lm_sample_args* a) {
  SampleDev P;
  P.logits = a->logits; P.dtype = a->dtype; P.rows = static_cast<int>(a->rows); P.vocab = static_cast<int>(a->vocab); P.row_stride = a->row_stride;
  P.temperature = a->temperature; P.temperature_s = a->temperature_s; P.top_k = a->top_k; P.top_k_s = a->top_k_s;
  P.top_p = a->top_p; P.top_p_s = a->top_p_s; P.min_p = a->min_p; P.min_p_s = a->min_p_s;
  P.flags = a->flags; P.draw = a->draw;
  const bool pen = sample_has_penalties(a);
  P.history = pen ? a->history : nullptr; P.hist_len = static_cast<int>(a->hist_len); P.hist_stride = a->hist_stride;
  P.rho = a->repetition_penalty; P.pi = a->presence_penalty;
  P.uniforms = a->uniforms; P.seed = a->seed; P.step = a->step; P.row_offset = a->row_offset;
  P.out_tokens = a->out_tokens; P.out_tau = a->out_tau; P.out_stats = a->out_stats; P.out_probs = a->out_probs; P.probs_stride = a->probs_stride;
  P.out_status = a->out_status; P.out_vmax = a->out_vmax; P.out_mass = reinterpret_cast<unsigned long long*>(a->out_mass);
  P.state = static_cast<const uint32_t*>(a->step_state); P.t_max = a->t_max; P.g = a->gamma_max > 1 ? a->gamma_max : 1;
  return P;
}

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

}  // namespace lm

using namespace lm;

extern "C" {


int lm_abi_version(void) { return LM_ABI_VERSION; }

const char* lm_error_string(int code) {
  switch (code) {
    case LM_OK: return "ok";
    case LM_E_INVALID: return "invalid argument";
    case LM_E_WORKSPACE: return "workspace missing, misaligned or too small";
    case LM_E_CUDA: return "CUDA runtime error";
    case LM_E_UNSUPPORTED: return "size outside the supported range";
    default: return "unknown error";
  }
}

const char* lm_last_cuda_error(void) { return g_cuda_error; }

int lm_device_sm_count(void) {
  int n = 0;
  const int rc = sm_count(&n);
  return rc == LM_OK ? n : rc;
}

float lm_uniform01(uint64_t seed, uint32_t step, uint32_t t, uint32_t index) { return uniform01(seed, step, t, index); }

size_t lm_workspace_bytes(int64_t rows, int64_t vocab) {
  (void)vocab;
  if (rows < 0) rows = 0;
  // argmax partials | rows for the generic kernel | rows that are not the top-k kernel's | rows the top-k kernel left | counters
  //   | the slice records of a call of a few rows
  return align256(static_cast<size_t>(rows) * sizeof(ArgmaxWs)) + 3 * align256(static_cast<size_t>(rows) * sizeof(uint32_t)) + 256 + kSlicedWsBytes;
}

size_t lm_verify_workspace_bytes(int32_t n_draft, int64_t vocab) {
  (void)n_draft; (void)vocab;
  // lm_verify and lm_draft_q may share it: the verify kernel's words (which keep a launch count between calls) come first, the
  // draft kernel's (all zero between calls) behind them
  return align256(sizeof(VerifyWs)) + align256(sizeof(DraftQWs));
}

int lm_argmax(const void* logits, int32_t dtype, int64_t rows, int64_t vocab, int64_t row_stride, int32_t* out_tokens, void* workspace,
              size_t workspace_bytes, void* stream) {
  if (rows < 0 || vocab < 0 || (dtype != LM_DTYPE_BF16 && dtype != LM_DTYPE_F32)) return LM_E_INVALID;
  if (rows == 0) return LM_OK;
  if (!logits || !out_tokens || row_stride < vocab) return LM_E_INVALID;
  if (vocab > LM_MAX_VOCAB || rows > 65535 * 32) return LM_E_UNSUPPORTED;
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  const int n_chunks = static_cast<int>((vocab + kChunk - 1) / kChunk);
  // enough blocks to cover the machine twice; a block needs at least one sweep of work
  int splits = static_cast<int>((2 * sms + rows - 1) / rows);
  const int max_splits = (n_chunks + kArgmaxBlock - 1) / kArgmaxBlock;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < lm_workspace_bytes(rows, vocab)))
    return LM_E_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (splits > 1) {
    // one entry per row, zero when the kernel starts. A workspace that also served lm_sample with another row count holds that
    // call's row lists where these entries lie, so they are cleared here rather than trusted.
    const cudaError_t e = cudaMemsetAsync(workspace, 0, static_cast<size_t>(rows) * sizeof(ArgmaxWs), st);
    if (e != cudaSuccess) return cuda_fail(e);
  }
  for (int64_t r0 = 0; r0 < rows; r0 += 65535) {                          // gridDim.y limit
    const int nr = static_cast<int>(rows - r0 < 65535 ? rows - r0 : 65535);
    const size_t esz = dtype == LM_DTYPE_BF16 ? 2 : 4;
    argmax_kernel<<<dim3(splits, nr), kArgmaxBlock, 0, st>>>(static_cast<const char*>(logits) + static_cast<size_t>(r0) * row_stride * esz, dtype, nr,
                                                            static_cast<int>(vocab), row_stride, splits, out_tokens + r0,
                                                            static_cast<ArgmaxWs*>(workspace) + r0);
  }
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

// The allocation-free variant of lm_argmax: the same kernel, its workspace in g_argmax_static_ws.
int lm_argmax_static(const void* logits, int32_t dtype, int64_t rows, int64_t vocab, int64_t row_stride, int32_t* out_tokens, void* stream) {
  if (rows < 0 || vocab < 0 || (dtype != LM_DTYPE_BF16 && dtype != LM_DTYPE_F32)) return LM_E_INVALID;
  if (rows == 0) return LM_OK;
  if (!logits || !out_tokens || row_stride < vocab) return LM_E_INVALID;
  if (rows > LM_ARGMAX_STATIC_MAX_ROWS || vocab > LM_MAX_VOCAB) return LM_E_UNSUPPORTED;   // beyond the fixed scratch
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  // set-up, once per device, with that device current: the device address of the scratch array
  constexpr int kMaxDevices = 64;
  static void* ws_addr[kMaxDevices] = {nullptr};
  static std::mutex ws_mutex;
  if (dev < 0 || dev >= kMaxDevices) return LM_E_UNSUPPORTED;
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(ws_mutex);
    if (ws_addr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_argmax_static_ws);
      if (e != cudaSuccess) return cuda_fail(e);
      ws_addr[dev] = p;
    }
    ws = ws_addr[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // lm_argmax touches one ArgmaxWs entry per row and nothing else of a workspace (it clears the entries it uses on the stream
  // before its kernel: the array keeps whatever the last call left); the size given here only has to pass its general check
  return lm_argmax(logits, dtype, rows, vocab, row_stride, out_tokens, ws, lm_workspace_bytes(rows, vocab), st);
}

// The merge's thread geometry and the FP64 reciprocal of a scalar temperature, once per call on the host.
static void merge_geometry(VpMergeDev& M) {
  M.per = kVpMaxCandidates / M.shards;
  M.per_log2 = -1;
  for (int b = 0; b <= 10; b++) if ((1 << b) == M.per) M.per_log2 = b;
  M.inv_t_s = M.temperature == nullptr ? 1.0 / static_cast<double>(M.temperature_s) : 0.0;
}

int lm_sample(const lm_sample_args* a) {
  if (!a || a->struct_size != sizeof(lm_sample_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->vocab < 0 || (a->dtype != LM_DTYPE_BF16 && a->dtype != LM_DTYPE_F32)) return LM_E_INVALID;
  if (a->draw != LM_DRAW_GUMBEL && a->draw != LM_DRAW_INVERSE_CDF) return LM_E_INVALID;
  if (a->rows == 0) return LM_OK;
  if (!a->logits || !a->out_tokens || a->row_stride < a->vocab) return LM_E_INVALID;
  if (a->vocab > LM_MAX_VOCAB || a->rows > 0x7FFFFFFF || a->hist_len > 0x7FFFFFFF) return LM_E_UNSUPPORTED;
  if (a->temperature == nullptr && !(a->temperature_s >= 0.0f)) return LM_E_INVALID;
  if (a->history != nullptr && (a->hist_len < 0 || a->hist_stride < a->hist_len)) return LM_E_INVALID;
  if (a->history != nullptr && !(a->repetition_penalty > 0.0f)) return LM_E_INVALID;
  if (a->out_probs != nullptr && a->probs_stride < a->vocab) return LM_E_INVALID;
  if (a->step_state != nullptr && lm_step_state_bytes(a->t_max, a->gamma_max) == 0) return LM_E_INVALID;
  // an all-greedy call needs no uniforms; a stochastic inverse-CDF call does
  if (a->draw == LM_DRAW_INVERSE_CDF && a->uniforms == nullptr && (a->temperature != nullptr || a->temperature_s > 0.0f)) return LM_E_INVALID;

  const bool pen = sample_has_penalties(a);
  SampleDev P = sample_dev(a);

  int sms = 0;
  int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(a->stream);
  const int* redo_list = nullptr; const int* redo_n = nullptr;
  // BF16 rows that only need tokens (and tau) stream through the one-pass kernel; it marks the rows it cannot take
  // and the generic kernel behind it handles exactly those.
  // A call of a few rows with one top_k for all of them: the rows are cut into slices over the whole GPU (sample_sliced.cuh).
  const size_t ws_base = lm_workspace_bytes(a->rows, a->vocab) - kSlicedWsBytes;
  const bool sliced = a->rows <= kSlicedMaxRows && a->vocab >= kSlicedMinVocab && a->temperature == nullptr && a->temperature_s > 0.0f &&
                      a->top_k == nullptr && a->top_k_s >= 1 && a->top_k_s <= 64 && a->out_stats == nullptr && a->out_probs == nullptr &&
                      !(a->flags & LM_FLAG_EXACT_ONLY) && (!pen || a->hist_len <= 65536) &&
                      a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0 && a->workspace_bytes >= ws_base + kSlicedWsBytes;
  if (sliced) {
    SliceDev S;
    // a record holds twice the top_k (16 at least): only a slice with that many logits at or above its own bound overflows it
    S.slices = kSlices;
    S.cap = a->top_k_s <= 8 ? 16 : 2 * a->top_k_s;
    S.slice_len = static_cast<int>(((a->vocab + S.slices - 1) / S.slices + 7) / 8 * 8);
    if (S.slice_len <= kSliceMaxLen) {
      char* ws = static_cast<char*>(a->workspace) + ws_base;
      S.logits = a->logits; S.dtype = a->dtype; S.rows = P.rows; S.vocab = P.vocab; S.row_stride = a->row_stride;
      S.temperature = a->temperature_s; S.top_k = a->top_k_s;
      S.temperature_rows = nullptr; S.top_k_rows = nullptr; S.exact_mass = 0; S.index_base = 0;
      S.history = P.history; S.hist_len = P.hist_len; S.hist_stride = P.hist_stride; S.rho = P.rho; S.pi = P.pi;
      S.records = reinterpret_cast<unsigned char*>(ws); S.record_bytes = static_cast<int64_t>(lm_vocab_record_bytes(S.cap));
      S.state = P.state; S.t_max = P.t_max; S.g = P.g;
      const size_t gsmem = sizeof(GenericSmem) + (pen ? static_cast<size_t>((a->vocab + 31) / 32) * 4 : 0) + 16;   // a row handed on to the generic algorithm
      S.need_mass = (a->top_p != nullptr || (a->top_p_s > 0.0f && a->top_p_s < 1.0f)) && !(a->flags & LM_FLAG_TOPP_IN_TOPK);
      const size_t slice_smem = slice_smem_bytes(S.slice_len);
      // threads per slice: 1024 when every slice has an SM to itself (the latency of one or two rows), else 128 (or 256 for a large
      // top_k, whose bound needs more threads' maxima to stay close): with several slices per SM the launch is bound by instruction
      // issue, and the per-warp work of the selection is most of a slice's instructions
      const int threads = static_cast<long long>(S.slices) * P.rows <= sms ? kSliceBlockBig : (a->top_k_s <= kSliceTinyMaxK ? kSliceBlockTiny : kSliceBlockSmall);
      const void* slice_fn = threads == kSliceBlockBig ? reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockBig>)
                           : threads == kSliceBlockSmall ? reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockSmall>)
                                                         : reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockTiny>);
      rc = ensure_dynamic_smem(threads == kSliceBlockBig ? kSlotSlice : (threads == kSliceBlockSmall ? kSlotSliceSmall : kSlotSliceTiny), slice_fn, slice_smem);
      if (rc == LM_OK) rc = ensure_dynamic_smem(kSlotSlicedMerge, reinterpret_cast<const void*>(sliced_merge_kernel), gsmem);
      if (rc != LM_OK) return rc;
      if (threads == kSliceBlockBig) slice_local_kernel<kSliceBlockBig><<<dim3(S.slices, P.rows), kSliceBlockBig, slice_smem, st>>>(S);
      else if (threads == kSliceBlockSmall) slice_local_kernel<kSliceBlockSmall><<<dim3(S.slices, P.rows), kSliceBlockSmall, slice_smem, st>>>(S);
      else slice_local_kernel<kSliceBlockTiny><<<dim3(S.slices, P.rows), kSliceBlockTiny, slice_smem, st>>>(S);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e);
      VpMergeDev M;
      M.bases = nullptr; M.pieces = 1;
      M.records = S.records; M.shards = S.slices; M.rows = P.rows; M.cap = S.cap; M.record_bytes = S.record_bytes;
      M.temperature = nullptr; M.temperature_s = a->temperature_s; M.top_k = nullptr; M.top_k_s = a->top_k_s;
      M.top_p = a->top_p; M.top_p_s = a->top_p_s; M.min_p = a->min_p; M.min_p_s = a->min_p_s;
      M.flags = a->flags; M.draw = a->draw; M.uniforms = a->uniforms; M.seed = a->seed; M.step = a->step; M.row_offset = a->row_offset;
      M.out_tokens = a->out_tokens; M.out_tau = a->out_tau; M.out_status = a->out_status; M.out_vmax = a->out_vmax; M.out_mass = reinterpret_cast<unsigned long long*>(a->out_mass);
      M.hand_on = 1; M.path_status = LM_STATUS_SLICED_PATH;
      merge_geometry(M);
      M.mass_band = S.need_mass ? slice_mass_band(S.slice_len, threads) : 0.0;
      // the merge is launched with programmatic stream serialization: its blocks are resident and waiting when the slices complete
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(P.rows); cfg.blockDim = dim3(kVpMaxCandidates); cfg.dynamicSmemBytes = gsmem; cfg.stream = st; cfg.attrs = attr; cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, sliced_merge_kernel, M, P);
      return e == cudaSuccess ? LM_OK : cuda_fail(e);
    }
  }
  const bool fast = a->dtype == LM_DTYPE_BF16 && a->out_stats == nullptr && a->out_probs == nullptr && a->vocab <= kHistMaxVocab &&
                    (a->vocab % kChunk) == 0 && (!pen || a->hist_len <= 65536);
  if (fast) {
    if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255u) || a->workspace_bytes < lm_workspace_bytes(a->rows, a->vocab))
      return LM_E_WORKSPACE;
    const size_t rows_bytes = align256(static_cast<size_t>(a->rows) * sizeof(uint32_t));
    char* ws = static_cast<char*>(a->workspace) + align256(static_cast<size_t>(a->rows) * sizeof(ArgmaxWs));
    int* redo = reinterpret_cast<int*>(ws);                                // rows for the generic kernel
    int* list_other = reinterpret_cast<int*>(ws + rows_bytes);             // rows that are not the top-k kernel's
    int* list_left = reinterpret_cast<int*>(ws + 2 * rows_bytes);          // rows the top-k kernel left
    int* counters = reinterpret_cast<int*>(ws + 3 * rows_bytes);
    // counters: 0 next row of the top-k kernel, 1 length of list_left, 2 next item of the histogram kernel, 3 length of redo,
    //           4 length of list_other, 5 next item of the histogram kernel's second launch
    const size_t hist_smem = hist_smem_bytes(static_cast<int>(a->vocab));
    rc = ensure_dynamic_smem(kSlotFast, reinterpret_cast<const void*>(sample_hist_kernel), hist_smem);
    if (rc == LM_OK) rc = ensure_dynamic_smem(kSlotTopk, reinterpret_cast<const void*>(sample_topk_kernel), sizeof(TopkSmem));
    if (rc != LM_OK) return rc;
    const int limit = static_cast<int>((a->flags >> 8) & 0xFFu);
    const bool topk = !(a->flags & LM_FLAG_EXACT_ONLY) && a->vocab >= kTopkMinVocab && (a->top_k != nullptr || (a->top_k_s >= 1 && a->top_k_s <= kTopkMaxK)) &&
                      (a->temperature != nullptr || a->temperature_s > 0.0f) && (!pen || a->hist_len <= kTopkHist);
    {
      const cudaError_t e = cudaMemsetAsync(counters, 0, 8 * sizeof(int), st);
      if (e != cudaSuccess) return cuda_fail(e);
    }
    const long long hist_per_sm = 2 * (hist_smem + 1024) <= 233472 ? 2 : 1;   // blocks of the histogram kernel that fit one SM's shared memory
    int grid = static_cast<int>(a->rows < hist_per_sm * sms ? a->rows : hist_per_sm * sms);
    if (limit > 0 && grid > limit) grid = limit;
    int grid1 = static_cast<int>(a->rows < static_cast<long long>(kTopkPerSM) * sms ? a->rows : static_cast<long long>(kTopkPerSM) * sms);
    if (limit > 0 && grid1 > limit) grid1 = limit;
    if (!topk) {
      sample_hist_kernel<<<grid, kHB, hist_smem, st>>>(P, nullptr, nullptr, counters + 2, redo, counters + 3);
    } else if (a->rows > static_cast<int64_t>(kOverlapRowsPerSM) * sms) {
      // Many rows per SM: the top-k kernel first (it lists the rows it does not take or cannot finish), then the histogram
      // kernel on that list. The few rows the top-k kernel hands on are absorbed among the histogram kernel's other rows.
      sample_topk_kernel<<<grid1, kTB, sizeof(TopkSmem), st>>>(P, list_left, counters, 1);
      sample_hist_kernel<<<grid, kHB, hist_smem, st>>>(P, list_left, counters + 1, counters + 2, redo, counters + 3);
    } else {
      // Few rows per SM: the length of a launch is the length of its longest rows, so the two kernels, which work on different
      // rows, share the GPU. The histogram kernel (long rows, one block per SM) goes first on the rows a one-thread-per-row
      // kernel lists for it; the top-k kernel is launched behind it with programmatic stream serialization and takes the SMs
      // as the histogram kernel's blocks leave them (at once, for the SMs it has no rows for); a second launch of the histogram
      // kernel takes what the top-k kernel handed on (usually nothing: it leaves at once).
      sample_classify_kernel<<<static_cast<int>((a->rows + 255) / 256), 256, 0, st>>>(P, list_other, counters + 4);
      // With at most kAloneRowsPerSM rows per SM the histogram kernel's blocks ask for so much shared memory that nothing else fits
      // beside them: a long row then has its SM to itself, and the blocks that find no row leave their SM to the top-k kernel at
      // once (256 rows of the benchmark mix: 112 -> 106 us per call; from 3 rows per SM on it costs time).
      size_t hist_smem_first = hist_smem; int grid_first = grid;
      if (a->rows <= static_cast<int64_t>(kAloneRowsPerSM) * sms && hist_smem < kAloneSmemBytes) {
        hist_smem_first = kAloneSmemBytes; grid_first = static_cast<int>(a->rows < sms ? a->rows : sms);
        rc = ensure_dynamic_smem(kSlotFast, reinterpret_cast<const void*>(sample_hist_kernel), hist_smem_first);
        if (rc != LM_OK) return rc;
      }
      sample_hist_kernel<<<grid_first, kHB, hist_smem_first, st>>>(P, list_other, counters + 4, counters + 2, redo, counters + 3);
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(grid1); cfg.blockDim = dim3(kTB); cfg.dynamicSmemBytes = sizeof(TopkSmem); cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      e = cudaLaunchKernelEx(&cfg, sample_topk_kernel, P, list_left, counters, 0);
      if (e != cudaSuccess) return cuda_fail(e);
      sample_hist_kernel<<<grid, kHB, hist_smem, st>>>(P, list_left, counters + 1, counters + 5, redo, counters + 3);
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e);
    redo_list = redo; redo_n = counters + 3;
  }
  const size_t smem = sizeof(GenericSmem) + (pen ? static_cast<size_t>((a->vocab + 31) / 32) * 4 : 0) + 16;
  rc = ensure_dynamic_smem(kSlotGeneric, reinterpret_cast<const void*>(sample_generic_kernel), smem);
  if (rc != LM_OK) return rc;
  const long long cap = fast ? sms : 8LL * sms;
  const int grid = static_cast<int>(a->rows < cap ? a->rows : cap);
  sample_generic_kernel<<<grid, kBlock, smem, st>>>(P, redo_list, redo_n);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

static size_t tile_lists_offset(int64_t rows) { return align256(static_cast<size_t>(rows) * sizeof(TileRow)); }
static size_t tile_bits_offset(int64_t rows) { return tile_lists_offset(rows) + static_cast<size_t>(rows) * kTileListCap * sizeof(unsigned long long); }
static int tile_pen_words(int64_t vocab) { return static_cast<int>((vocab + 127) / 128 * 4); }

size_t lm_tile_state_bytes(int64_t rows, int64_t vocab, int32_t with_history) {
  if (rows <= 0 || vocab < 0) return 0;
  return tile_bits_offset(rows) + (with_history ? static_cast<size_t>(rows) * tile_pen_words(vocab) * sizeof(uint32_t) : 0);
}

// The checks lm_tile_begin and lm_tile_consume share, and the device-side view of the arguments.
static int tile_dev(const lm_tile_args* a, bool consume, TileDev* out) {
  if (!a || a->struct_size != sizeof(lm_tile_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->vocab < 0) return LM_E_INVALID;
  if (a->rows == 0) return LM_OK;
  if (a->vocab > LM_MAX_VOCAB || a->rows > 0x7FFFFFFF || a->hist_len > 0x7FFFFFFF) return LM_E_UNSUPPORTED;
  if (a->history != nullptr && (a->hist_len < 0 || a->hist_stride < a->hist_len || !(a->repetition_penalty > 0.0f))) return LM_E_INVALID;
  if (consume) {
    if (a->dtype != LM_DTYPE_BF16 && a->dtype != LM_DTYPE_F32) return LM_E_INVALID;
    if (!a->tile || a->cols < 1 || a->col0 < 0 || a->col0 + a->cols > a->vocab || a->tile_stride < a->cols) return LM_E_INVALID;
    if (a->cols > LM_TILE_MAX_COLS) return LM_E_UNSUPPORTED;
  }
  const bool pen = a->history != nullptr && a->hist_len > 0 && !(a->repetition_penalty == 1.0f && a->presence_penalty == 0.0f);
  if (!a->state || (reinterpret_cast<uintptr_t>(a->state) & 255u) || a->state_bytes < lm_tile_state_bytes(a->rows, a->vocab, pen ? 1 : 0)) return LM_E_WORKSPACE;
  TileDev& T = *out;
  T.tile = a->tile; T.dtype = a->dtype; T.rows = static_cast<int>(a->rows); T.vocab = static_cast<int>(a->vocab); T.tile_stride = a->tile_stride;
  T.col0 = static_cast<int>(a->col0); T.cols = static_cast<int>(a->cols);
  T.temperature = a->temperature; T.temperature_s = a->temperature_s; T.top_k = a->top_k; T.top_k_s = a->top_k_s;
  char* base = static_cast<char*>(a->state);
  T.rows_state = reinterpret_cast<TileRow*>(base);
  T.lists = reinterpret_cast<unsigned long long*>(base + tile_lists_offset(a->rows));
  T.pen_bits = pen ? reinterpret_cast<uint32_t*>(base + tile_bits_offset(a->rows)) : nullptr;
  T.pen_words = tile_pen_words(a->vocab);
  T.history = pen ? a->history : nullptr; T.hist_len = static_cast<int>(a->hist_len); T.hist_stride = a->hist_stride;
  T.rho = a->repetition_penalty; T.pi = a->presence_penalty;
  return LM_OK;
}

int lm_tile_begin(const lm_tile_args* a) {
  TileDev T;
  const int rc = tile_dev(a, false, &T);
  if (rc != LM_OK || a->rows == 0) return rc;
  tile_begin_kernel<<<T.rows, kTileBlock, 0, static_cast<cudaStream_t>(a->stream)>>>(T);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_tile_consume(const lm_tile_args* a) {
  TileDev T;
  const int rc = tile_dev(a, true, &T);
  if (rc != LM_OK || a->rows == 0) return rc;
  tile_consume_kernel<<<T.rows, kTileBlock, 0, static_cast<cudaStream_t>(a->stream)>>>(T);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_tile_finish(const lm_sample_args* a, void* state, size_t state_bytes) {
  if (!a || a->struct_size != sizeof(lm_sample_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->vocab < 0) return LM_E_INVALID;
  if (a->draw != LM_DRAW_GUMBEL && a->draw != LM_DRAW_INVERSE_CDF) return LM_E_INVALID;
  if (a->rows == 0) return LM_OK;
  if (!a->out_tokens || a->out_stats != nullptr || a->out_probs != nullptr) return LM_E_INVALID;
  if (a->vocab > kTopkMaxVocab || a->rows > 0x7FFFFFFF) return LM_E_UNSUPPORTED;
  if (a->step_state != nullptr && lm_step_state_bytes(a->t_max, a->gamma_max) == 0) return LM_E_INVALID;
  if (a->draw == LM_DRAW_INVERSE_CDF && a->uniforms == nullptr && (a->temperature != nullptr || a->temperature_s > 0.0f)) return LM_E_INVALID;
  if (!state || (reinterpret_cast<uintptr_t>(state) & 255u) || state_bytes < lm_tile_state_bytes(a->rows, a->vocab, 0)) return LM_E_WORKSPACE;
  SampleDev P = sample_dev(a);
  P.logits = nullptr; P.history = nullptr;
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  rc = ensure_dynamic_smem(kSlotTileFinish, reinterpret_cast<const void*>(tile_finish_kernel), sizeof(TopkSmem));
  if (rc != LM_OK) return rc;
  const long long cap = static_cast<long long>(kTopkPerSM) * sms;
  const int grid = static_cast<int>(a->rows < cap ? a->rows : cap);
  tile_finish_kernel<<<grid, kTB, sizeof(TopkSmem), static_cast<cudaStream_t>(a->stream)>>>(
      P, static_cast<TileRow*>(state), reinterpret_cast<unsigned long long*>(static_cast<char*>(state) + tile_lists_offset(a->rows)));
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

size_t lm_vocab_record_bytes(int32_t cap) { return cap > 0 ? static_cast<size_t>(kVpHeader) + 8u * static_cast<size_t>(cap) : 0; }

int32_t lm_vocab_candidate_cap(int32_t top_k) { return top_k > 0 ? (top_k + 64 + 7) / 8 * 8 : 0; }

// Pieces a shard is cut into by the local step (each with a record of its own). As many as the merge still takes with the other
// shards' (shards * pieces <= 64 records per row, cap <= 8 * (1024 / (shards * pieces))), pieces of at least 2048 logits, and only
// for records of at most 128 candidates (a top_k up to 64): beyond that a piece's bound, taken from its threads' maxima, is no
// longer close to its k-th largest logit. More pieces also mean more bytes in the all-gather behind the step, which soon costs more
// than the local step gains: beyond the pieces a shard needs for its length (at most 32768 logits each), no more than keep the
// gathered records of all GPUs and rows under 1 MB.
int32_t lm_vocab_pieces(int32_t shards, int32_t cap, int64_t vocab_local, int64_t rows) {
  if (shards < 1 || cap < 1 || cap > 128 || vocab_local < 1) return 1;
  if (rows < 1) rows = 1;
  int32_t need = 1;                                                        // the fewest pieces that fit the slice kernel
  while (vocab_local / need > kSliceMaxLen) need *= 2;
  const int64_t record = static_cast<int64_t>(lm_vocab_record_bytes(cap));
  int32_t p = 1;
  while (2 * p * shards <= kVpMaxShards && cap <= kVpPerThread * (kVpMaxCandidates / (2 * p * shards)) && vocab_local / (2 * p) >= 2048 &&
         (2 * p <= need || static_cast<int64_t>(2 * p) * shards * rows * record <= (1 << 20))) p *= 2;
  return p >= need ? p : 1;
}

int lm_vocab_local(const lm_vocab_args* a) {
  if (!a || a->struct_size != sizeof(lm_vocab_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->vocab_local < 1 || (a->dtype != LM_DTYPE_BF16 && a->dtype != LM_DTYPE_F32)) return LM_E_INVALID;
  if (a->rows == 0) return LM_OK;
  if (!a->logits || !a->records || a->row_stride < a->vocab_local || a->cap < 1 || a->shard_start < 0) return LM_E_INVALID;
  if (a->temperature == nullptr && !(a->temperature_s > 0.0f)) return LM_E_INVALID;
  if (a->top_k == nullptr && a->top_k_s < 1) return LM_E_INVALID;
  if (a->vocab_local > LM_MAX_VOCAB || a->rows > 0x7FFFFFFF || a->shard_start + a->vocab_local > 0x7FFFFFFF) return LM_E_UNSUPPORTED;
  VpLocalDev P;
  P.logits = a->logits; P.dtype = a->dtype; P.rows = static_cast<int>(a->rows); P.vocab_local = static_cast<int>(a->vocab_local);
  P.row_stride = a->row_stride; P.shard_start = static_cast<int>(a->shard_start);
  P.temperature = a->temperature; P.temperature_s = a->temperature_s; P.top_k = a->top_k; P.top_k_s = a->top_k_s;
  P.cap = a->cap; P.records = static_cast<unsigned char*>(a->records); P.record_bytes = static_cast<int64_t>(lm_vocab_record_bytes(a->cap));
  int sms = 0;
  const int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  if (a->pieces > 1) {
    // the shard in pieces, one block each (the few-row path's slice kernel, with FP64 masses: no exact path stands behind this merge)
    if (a->pieces > kVpMaxShards || a->cap > 128) return LM_E_UNSUPPORTED;
    SliceDev S;
    S.logits = a->logits; S.dtype = a->dtype; S.rows = P.rows; S.vocab = P.vocab_local; S.row_stride = a->row_stride;
    S.slices = a->pieces;
    S.slice_len = static_cast<int>(((a->vocab_local + S.slices - 1) / S.slices + 7) / 8 * 8);
    if (S.slice_len > kSliceMaxLen) return LM_E_UNSUPPORTED;
    S.temperature = a->temperature_s; S.top_k = a->top_k_s; S.cap = a->cap; S.need_mass = 1;
    S.temperature_rows = a->temperature; S.top_k_rows = a->top_k; S.exact_mass = 1; S.index_base = P.shard_start;
    S.history = nullptr; S.hist_len = 0; S.hist_stride = 0; S.rho = 1.0f; S.pi = 0.0f;
    S.records = P.records; S.record_bytes = P.record_bytes;
    S.state = nullptr; S.t_max = 0; S.g = 0;
    const size_t slice_smem = slice_smem_bytes(S.slice_len);
    cudaStream_t st = static_cast<cudaStream_t>(a->stream);
    // threads per piece as on the few-row path; a record of cap candidates serves a top_k up to cap - 64
    const int threads = (static_cast<long long>(S.slices) * P.rows <= sms || S.slice_len >= 8192) ? kSliceBlockBig
                        : (a->cap - 64 <= kSliceTinyMaxK ? kSliceBlockTiny : kSliceBlockSmall);      // (long pieces: many logits per thread otherwise)
    int rs;
    if (threads == kSliceBlockBig) {
      rs = ensure_dynamic_smem(kSlotSlice, reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockBig>), slice_smem);
      if (rs == LM_OK) slice_local_kernel<kSliceBlockBig><<<dim3(S.slices, P.rows), kSliceBlockBig, slice_smem, st>>>(S);
    } else if (threads == kSliceBlockSmall) {
      rs = ensure_dynamic_smem(kSlotSliceSmall, reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockSmall>), slice_smem);
      if (rs == LM_OK) slice_local_kernel<kSliceBlockSmall><<<dim3(S.slices, P.rows), kSliceBlockSmall, slice_smem, st>>>(S);
    } else {
      rs = ensure_dynamic_smem(kSlotSliceTiny, reinterpret_cast<const void*>(slice_local_kernel<kSliceBlockTiny>), slice_smem);
      if (rs == LM_OK) slice_local_kernel<kSliceBlockTiny><<<dim3(S.slices, P.rows), kSliceBlockTiny, slice_smem, st>>>(S);
    }
    if (rs != LM_OK) return rs;
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? LM_OK : cuda_fail(e);
  }
  const size_t smem = sizeof(GenericSmem) + 16;
  const int rs = ensure_dynamic_smem(kSlotVocabLocal, reinterpret_cast<const void*>(vocab_local_kernel), smem);
  if (rs != LM_OK) return rs;
  const int grid = static_cast<int>(a->rows < 2LL * sms ? a->rows : 2LL * sms);
  vocab_local_kernel<<<grid, kBlock, smem, static_cast<cudaStream_t>(a->stream)>>>(P);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_vocab_merge(const lm_vocab_args* a) {
  if (!a || a->struct_size != sizeof(lm_vocab_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->shards < 1 || a->cap < 1) return LM_E_INVALID;
  if (a->draw != LM_DRAW_GUMBEL && a->draw != LM_DRAW_INVERSE_CDF) return LM_E_INVALID;
  if (a->rows == 0) return LM_OK;
  if ((!a->records && !a->record_ptrs) || !a->out_tokens) return LM_E_INVALID;
  if (a->temperature == nullptr && !(a->temperature_s > 0.0f)) return LM_E_INVALID;
  if (a->top_k == nullptr && a->top_k_s < 1) return LM_E_INVALID;
  if (a->draw == LM_DRAW_INVERSE_CDF && a->uniforms == nullptr) return LM_E_INVALID;
  if (a->shards > kVpMaxShards || a->cap > kVpPerThread * (kVpMaxCandidates / a->shards) || a->rows > 0x7FFFFFFF) return LM_E_UNSUPPORTED;
  VpMergeDev P;
  P.records = static_cast<const unsigned char*>(a->records); P.shards = a->shards; P.rows = static_cast<int>(a->rows); P.cap = a->cap;
  P.bases = static_cast<const unsigned long long*>(a->record_ptrs); P.pieces = a->pieces > 0 ? a->pieces : 1;
  if (P.bases && (a->shards % P.pieces) != 0) return LM_E_INVALID;
  P.record_bytes = static_cast<int64_t>(lm_vocab_record_bytes(a->cap));
  P.temperature = a->temperature; P.temperature_s = a->temperature_s; P.top_k = a->top_k; P.top_k_s = a->top_k_s;
  P.top_p = a->top_p; P.top_p_s = a->top_p_s; P.min_p = a->min_p; P.min_p_s = a->min_p_s;
  P.flags = a->flags; P.draw = a->draw; P.uniforms = a->uniforms; P.seed = a->seed; P.step = a->step; P.row_offset = a->row_offset;
  P.out_tokens = a->out_tokens; P.out_tau = a->out_tau; P.out_status = a->out_status; P.out_vmax = nullptr; P.out_mass = nullptr;
  P.hand_on = 0; P.path_status = 0u; P.mass_band = 0.0;
  merge_geometry(P);
  int sms = 0;
  const int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  const int grid = static_cast<int>(a->rows < 4LL * sms ? a->rows : 4LL * sms);
  vocab_merge_kernel<<<grid, kVpMaxCandidates, 0, static_cast<cudaStream_t>(a->stream)>>>(P);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_head(const lm_head_args* a) {
  if (!a || a->struct_size != sizeof(lm_head_args)) return LM_E_INVALID;
  if (a->rows < 0 || a->vocab < 0 || a->hidden_dim < 1) return LM_E_INVALID;
  if (a->rows == 0 || a->vocab == 0) return LM_OK;
  if (!a->hidden || !a->weight || !a->logits || a->hidden_stride < a->hidden_dim || a->weight_stride < a->hidden_dim || a->logits_stride < a->vocab) return LM_E_INVALID;
  if (a->rows > LM_HEAD_MAX_ROWS || a->vocab > LM_MAX_VOCAB || (a->hidden_dim % kHeadStep) != 0 || head_smem_bytes(static_cast<int>(a->hidden_dim < 65536 ? a->hidden_dim : 65536)) > 200 * 1024) return LM_E_UNSUPPORTED;   // the rows of x must fit shared memory (hidden up to 12,736)
  if ((reinterpret_cast<uintptr_t>(a->weight) & 15u) || (a->weight_stride % 8) != 0) return LM_E_UNSUPPORTED;      // 16-byte loads of the weights
  HeadDev P;
  P.x = static_cast<const uint16_t*>(a->hidden); P.x_stride = a->hidden_stride; P.rows = a->rows;
  P.w = static_cast<const uint16_t*>(a->weight); P.w_stride = a->weight_stride; P.hidden = static_cast<int>(a->hidden_dim); P.vocab = static_cast<int>(a->vocab);
  P.gamma = static_cast<const uint16_t*>(a->norm_weight); P.eps = a->eps; P.one_plus = a->one_plus;
  P.logits = static_cast<uint16_t*>(a->logits); P.logits_stride = a->logits_stride;
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  const size_t smem = head_smem_bytes(P.hidden);
  rc = ensure_dynamic_smem(kSlotHead, reinterpret_cast<const void*>(lm_head_kernel), smem);
  if (rc != LM_OK) return rc;
  int per_sm = 1;                                                          // blocks of the kernel that one SM holds (registers and shared memory)
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lm_head_kernel, kHeadThreads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  const long long tiles = (a->vocab + kHeadTile - 1) / kHeadTile, want = (tiles + kHeadWarps - 1) / kHeadWarps;
  const int grid = static_cast<int>(want < static_cast<long long>(per_sm) * sms ? want : static_cast<long long>(per_sm) * sms);
  lm_head_kernel<<<grid, kHeadThreads, smem, static_cast<cudaStream_t>(a->stream)>>>(P);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

size_t lm_step_state_bytes(int32_t t_max, int32_t gamma_max) {
  if (t_max < 1 || gamma_max < 0 || t_max < gamma_max + 1) return 0;
  const size_t g = gamma_max > 1 ? gamma_max : 1;
  const size_t words = 4 + static_cast<size_t>(t_max) + 4 + 2 * g + 12;
  return (words * 4 + 15) / 16 * 16;
}

static int step_args_ok(const lm_step_args* a) {
  if (!a || a->struct_size != sizeof(lm_step_args)) return LM_E_INVALID;
  if (lm_step_state_bytes(a->t_max, a->gamma_max) == 0 || !a->step_state) return LM_E_INVALID;
  if (a->n_eos < 0 || (a->n_eos > 0 && !a->eos_list)) return LM_E_INVALID;
  return LM_OK;
}

int lm_accept_scan(const lm_step_args* a) {
  int rc = step_args_ok(a);
  if (rc != LM_OK) return rc;
  if (!a->tokens || !a->ring || a->ring_cap == 0 || (a->log_cap && !a->log)) return LM_E_INVALID;
  AcceptDev p{a->tokens, static_cast<uint32_t*>(a->step_state), a->t_max, a->gamma_max > 1 ? a->gamma_max : 1,
              reinterpret_cast<unsigned long long*>(a->ring), a->ring_cap, EosSet{a->eos, a->eos_list, a->n_eos}, a->log, a->log_cap, a->ctx_cap, a->lm};
  accept_scan_kernel<<<1, 32, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_verify_select(const lm_step_args* a) {
  int rc = step_args_ok(a);
  if (rc != LM_OK) return rc;
  if (!a->drafts || !a->conf || a->gamma > 16u || static_cast<int>(a->gamma) > (a->gamma_max > 1 ? a->gamma_max : 1) || a->mode > 2u) return LM_E_INVALID;
  if (a->conf_log_cap && !a->conf_log) return LM_E_INVALID;
  if (a->mode == 1u) {                                                     // the cost rule: positive costs relative to cost[0] = 1 (kernels.py:820-822)
    if (std::fabs(a->cost[0] - 1.0f) > 1e-6f) return LM_E_INVALID;
    for (int i = 0; i < 16; i++) if (!(a->cost[i] > 0.0f)) return LM_E_INVALID;
  }
  SelectDev p;
  if (a->t_limit > static_cast<uint32_t>(a->t_max)) return LM_E_INVALID;
  p.drafts = a->drafts; p.conf = a->conf; p.state = static_cast<uint32_t*>(a->step_state); p.t_max = a->t_max; p.t_limit = a->t_limit ? a->t_limit : static_cast<uint32_t>(a->t_max); p.g = a->gamma_max > 1 ? a->gamma_max : 1;
  p.gamma = a->gamma; p.threshold = a->threshold; p.mode = a->mode;
  for (int i = 0; i < 16; i++) p.cost[i] = a->cost[i];
  p.conf_log = a->conf_log; p.log_cap = a->conf_log_cap; p.ctx_cap = a->ctx_cap; p.lm = a->lm;
  verify_select_kernel<<<1, 32, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_advance(const lm_step_args* a) {
  int rc = step_args_ok(a);
  if (rc != LM_OK) return rc;
  if (!a->tokens || !a->ring || a->ring_cap == 0) return LM_E_INVALID;
  AdvanceDev p{a->tokens, static_cast<uint32_t*>(a->step_state), a->t_max, a->gamma_max > 1 ? a->gamma_max : 1,
               reinterpret_cast<unsigned long long*>(a->ring), a->ring_cap, EosSet{a->eos, a->eos_list, a->n_eos}, a->ctx_cap};
  advance_kernel<<<1, 32, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_verify(const lm_verify_args* a) {
  if (!a || a->struct_size != sizeof(lm_verify_args)) return LM_E_INVALID;
  if (a->mode != LM_VERIFY_GREEDY && a->mode != LM_VERIFY_STOCHASTIC) return LM_E_INVALID;
  if (a->dtype != LM_DTYPE_BF16 && a->dtype != LM_DTYPE_F32) return LM_E_INVALID;
  if (a->n_draft < 1 || a->n_draft > LM_MAX_DRAFT) return LM_E_INVALID;
  if (!a->target_logits || !a->out_accept || !a->out_final || a->vocab < 1 || a->row_stride < a->vocab) return LM_E_INVALID;
  if (!a->draft_ids && !a->step_state) return LM_E_INVALID;                 // the drafts come from the arguments or from the state
  if (a->vocab > LM_MAX_VOCAB) return LM_E_UNSUPPORTED;
  if (a->step_state && (lm_step_state_bytes(a->t_max, a->gamma_max) == 0 || a->t_max < a->n_draft + 1)) return LM_E_INVALID;
  if (a->mode == LM_VERIFY_STOCHASTIC) {
    if (!(a->temperature > 0.0f)) return LM_E_INVALID;
    if (a->residual_draw != LM_RESIDUAL_INVERSE_CDF && a->residual_draw != LM_RESIDUAL_GUMBEL) return LM_E_INVALID;
    if (a->draft_probs) { if (a->probs_stride < a->vocab) return LM_E_INVALID; }
    else if (!a->draft_logits || a->draft_logits_stride < a->vocab || !a->draft_vmax || !a->draft_mass) return LM_E_INVALID;
  }
  if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255u) || a->workspace_bytes < lm_verify_workspace_bytes(a->n_draft, a->vocab))
    return LM_E_WORKSPACE;
  int sms = 0;
  int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  VerifyDev P;
  P.mode = a->mode; P.dtype = a->dtype; P.n_draft = a->n_draft; P.vocab = static_cast<int>(a->vocab); P.row_stride = a->row_stride;
  P.draw = a->residual_draw == LM_RESIDUAL_GUMBEL ? LM_DRAW_GUMBEL : LM_DRAW_INVERSE_CDF;
  P.target = a->target_logits; P.drafts = a->draft_ids; P.q = a->draft_probs; P.q_stride = a->probs_stride; P.temperature = a->temperature;
  P.q_logits = static_cast<const uint16_t*>(a->draft_logits); P.q_logits_stride = a->draft_logits_stride;
  P.q_vmax = a->draft_vmax; P.q_mass = reinterpret_cast<const unsigned long long*>(a->draft_mass);
  P.tau = a->tau; P.u_accept = a->u_accept; P.u_final = a->u_final; P.seed = a->seed; P.step = a->step;
  P.row_max = a->mode == LM_VERIFY_STOCHASTIC ? a->target_vmax : nullptr;
  P.row_mass = P.row_max ? reinterpret_cast<const unsigned long long*>(a->target_mass) : nullptr;
  P.out_accept = a->out_accept; P.out_final = a->out_final; P.out_tokens = a->out_tokens; P.out_p_draft = a->out_p_draft;
  P.ws = static_cast<VerifyWs*>(a->workspace);
  P.state = static_cast<uint32_t*>(const_cast<void*>(a->step_state)); P.t_max = a->t_max; P.g = a->gamma_max > 1 ? a->gamma_max : 1;
  P.wait_limit = a->wait_limit; P.withhold = (a->selftest & LM_VERIFY_SELFTEST_WITHHOLD) ? 1u : 0u;
  P.commit = 0;
  if (a->commit) {
    const lm_step_args* c = a->commit;
    rc = step_args_ok(c);
    if (rc != LM_OK) return rc;
    if (!a->out_tokens || !c->ring || c->ring_cap == 0 || (c->log_cap && !c->log)) return LM_E_INVALID;
    if (a->step_state && (a->step_state != c->step_state || a->t_max != c->t_max || a->gamma_max != c->gamma_max)) return LM_E_INVALID;
    P.commit = 1;
    P.accept = AcceptDev{a->out_tokens, static_cast<uint32_t*>(c->step_state), c->t_max, c->gamma_max > 1 ? c->gamma_max : 1,
                         reinterpret_cast<unsigned long long*>(c->ring), c->ring_cap, EosSet{c->eos, c->eos_list, c->n_eos}, c->log, c->log_cap,
                         c->ctx_cap, c->lm};
  }
  // one block per SM, all resident at once (the blocks wait for one another's partial results): a cooperative launch guarantees it
  // (the same grid for every call on a device, whatever the vocabulary: the workspace's launch count is in units of it; blocks
  // beyond a small vocabulary hold empty slices)
  const int grid = sms < 256 ? sms : 256;                                  // consume_rows holds rows x grid words in kConsumeSlots per thread
  // the block's slices of all rows in shared memory when they fit (they do for every vocabulary up to ~700k at 148 SMs)
  const int per = (static_cast<int>((a->vocab + grid - 1) / grid) + 7) & ~7;
  const size_t rows_cached = static_cast<size_t>(a->n_draft + 1) + (a->mode == LM_VERIFY_STOCHASTIC ? a->n_draft : 0);
  size_t smem = rows_cached * static_cast<size_t>(per) * sizeof(float);
  int cached = smem <= 200 * 1024 ? 1 : 0;
  if (!cached) smem = 0;
  const bool stats = P.row_max != nullptr && P.row_mass != nullptr;
  const void* kernel = stats ? reinterpret_cast<const void*>(verify_kernel<true>) : reinterpret_cast<const void*>(verify_kernel<false>);
  rc = ensure_dynamic_smem(stats ? kSlotVerifyStats : kSlotVerify, kernel, smem);
  if (rc != LM_OK) return rc;
  void* params[] = {&P, &cached};
  const cudaError_t e = cudaLaunchCooperativeKernel(const_cast<void*>(kernel), dim3(grid), dim3(kVerifyBlock), params, smem, static_cast<cudaStream_t>(a->stream));
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_draft_q(const lm_draft_q_args* a) {
  if (!a || a->struct_size != sizeof(lm_draft_q_args)) return LM_E_INVALID;
  if (a->rows < 1 || a->rows > LM_MAX_DRAFT + 1 || a->first_position < 0 || (a->dtype != LM_DTYPE_BF16 && a->dtype != LM_DTYPE_F32)) return LM_E_INVALID;
  if (!a->logits || !a->out_tokens || a->vocab < 1 || a->row_stride < a->vocab || !(a->temperature > 0.0f)) return LM_E_INVALID;
  if (a->out_q_logits && a->q_logits_stride < a->vocab) return LM_E_INVALID;
  if (a->vocab > LM_MAX_VOCAB) return LM_E_UNSUPPORTED;
  if (a->step_state && lm_step_state_bytes(a->t_max, a->gamma_max) == 0) return LM_E_INVALID;
  if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255u) || a->workspace_bytes < lm_verify_workspace_bytes(a->rows, a->vocab))
    return LM_E_WORKSPACE;
  int sms = 0;
  const int rc = sm_count(&sms);
  if (rc != LM_OK) return rc;
  DraftQDev P;
  P.dtype = a->dtype; P.rows = a->rows; P.first_position = a->first_position; P.vocab = static_cast<int>(a->vocab); P.row_stride = a->row_stride;
  P.logits = a->logits; P.temperature = a->temperature; P.seed = a->seed; P.step = a->step;
  P.out_tokens = a->out_tokens; P.out_lse = a->out_lse; P.out_vmax = a->out_vmax; P.out_mass = reinterpret_cast<unsigned long long*>(a->out_mass);
  P.out_status = a->out_status; P.out_q_logits = a->out_q_logits; P.q_logits_stride = a->q_logits_stride;
  P.ws = reinterpret_cast<DraftQWs*>(static_cast<char*>(a->workspace) + align256(sizeof(VerifyWs)));
  P.state = static_cast<const uint32_t*>(a->step_state); P.t_max = a->t_max; P.g = a->gamma_max > 1 ? a->gamma_max : 1;
  // one block per SM, all resident at once (one grid barrier), each holding its slice of every row in shared memory;
  // more blocks than that never, fewer when the slices would not fit
  int grid = sms < 1024 ? sms : 1024;
  constexpr int kPerThread = 4;
  {
    // a single row is ~150 logits per SM: fewer blocks with a few logits per thread meet sooner at the barrier
    const long long want = (static_cast<long long>(a->rows) * a->vocab + kDraftQBlock * kPerThread - 1) / (kDraftQBlock * kPerThread);
    if (want < grid) grid = static_cast<int>(want < 1 ? 1 : want);
  }
  const int per = (static_cast<int>((a->vocab + grid - 1) / grid) + 7) & ~7;
  const size_t smem = static_cast<size_t>(a->rows) * static_cast<size_t>(per) * sizeof(float);
  if (smem > 200 * 1024) return LM_E_UNSUPPORTED;                          // rows x vocabulary beyond what the SMs can hold between the phases
  const int rs = ensure_dynamic_smem(kSlotDraftQ, reinterpret_cast<const void*>(draft_q_kernel), smem);
  if (rs != LM_OK) return rs;
  void* params[] = {&P};
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(draft_q_kernel), dim3(grid), dim3(kDraftQBlock), params, smem,
                                                    static_cast<cudaStream_t>(a->stream));
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

int lm_confidence(const lm_confidence_args* a) {
  if (!a || a->struct_size != sizeof(lm_confidence_args)) return LM_E_INVALID;
  if (a->gamma < 0 || a->gamma > 16 || a->hidden < 0 || a->rank < 0 || a->hidden + a->rank < 1) return LM_E_INVALID;
  if (a->gamma == 0) return LM_OK;
  if (!a->w || !a->b || !a->out_conf || (a->hidden > 0 && !a->hidden_rows) || (a->rank > 0 && !a->emb_rows)) return LM_E_INVALID;
  if (a->step_state && (a->t_max < 1 || a->gamma_max < 0 || a->t_max < a->gamma_max + 1)) return LM_E_INVALID;
  ConfDev P;
  P.hidden = static_cast<const uint16_t*>(a->hidden_rows); P.emb = static_cast<const uint16_t*>(a->emb_rows); P.w = a->w; P.b = a->b; P.sts = a->sts;
  P.conf = a->out_conf; P.state = static_cast<uint32_t*>(a->step_state); P.t_max = a->t_max; P.g = a->gamma_max > 1 ? a->gamma_max : 1;
  P.gamma = a->gamma; P.n_hidden = a->hidden; P.rank = a->rank;
  confidence_kernel<<<(a->gamma + 3) / 4, 128, 0, static_cast<cudaStream_t>(a->stream)>>>(P);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? LM_OK : cuda_fail(e);
}

}  // extern "C"
