// One pre-norm block of grouped-query attention and a gated (SwiGLU) feed-forward as one call: the ten or so launches of a layer issued from here, without a
// return to the interpreter between them.  Nothing new is computed: the same kernels, in the order and with
// the choices (which attention kernel, which product) that the Python parts make one by one
// (parts/block.py, parts/attention.py, parts/mlp.py, kernels/attention.py, kernels/gemm.py); the parts use
// this call when every part of the block is one of the built-in kinds, and their own sequence otherwise.
//
//   n  = rmsnorm(residual += pending)                      add_rmsnorm
//   qkv = n . Wqkv^T; q, k -> rotary; k, v -> pages        product, rope_append
//   a  = attention(q, pages)                               prefill (tcgen05 / mma.sync) and decode (TMA / cp.async)
//   o  = a . Wo^T                                          product
//   n  = rmsnorm(residual += o)                            add_rmsnorm
//   out = (silu(n . Wg^T) * (n . Wu^T)) . Wd^T             products, swiglu (or the activation in the product's epilogue)
// A product is the hand-written swap-AB tcgen05 kernel up to the number of rows its weight asks for, else the library's.
// `out` is left pending: the next block's (or the final) norm adds it
// (src/torchinferno/models/llama3/pipeline.py:190-198; the pending add: tensor_parallel.py:7430-7435).
#include "common.cuh"
#include <mutex>
#include <vector>

extern "C" {
int tib_add_rmsnorm(const void*, float*, const int*, const float*, void*, int, int, float, int, cudaStream_t);
int tib_swiglu(const void*, void*, int, int, int, int, cudaStream_t);
int tib_rope_append(const void*, void*, void*, const int*, const int*, const int*, int, const float*, int, int, int, int, int,
                    int, int, int64_t, int, int, int*, int, cudaStream_t);
int tib_prefill_attention_tcgen05_supports(int, int, int);
int tib_prefill_attention_tcgen05(const void*, const void*, void*, const int*, const int*, const int*, const int*, int, int, int,
                                  int, int, int, int, int, int64_t, int, int, float, int, int*, cudaStream_t);
int tib_prefill_attention(const void*, const void*, void*, const int*, const int*, const int*, const int*, int, int, int, int,
                          int, int, int, int64_t, int, int, float, int, cudaStream_t);
int tib_attention_mma_supports(int, int);
int tib_decode_attention_tma_supports(int, int, int);
int tib_decode_attention_tma(const void*, const void*, void*, float*, float*, const int*, const int*, const int*, const int*,
                             int, int, int, int, int, int, int64_t, int, int, float, int, int, int*, int*, cudaStream_t);
int tib_decode_attention_tma_rope(const void*, void*, void*, float*, float*, const int*, const int*, const int*, const int*,
                                  int, int, int, int, int, int, int64_t, int, int, float, int, int, int*, int*, const float*, int, int,
                                  cudaStream_t);
int tib_decode_attention(const void*, const void*, void*, float*, float*, const int*, const int*, const int*, const int*, int,
                         int, int, int, int, int, int64_t, int, int, float, int, int, cudaStream_t);
int tib_gemm_tcgen05_swapab_supports(int, int, int);
int tib_gemm_tcgen05_swapab(const void*, const void*, void*, int, int, int, int64_t, int64_t, int64_t, int, int, int, int*, cudaStream_t);
int tib_blas_gemm(const void*, const void*, void*, int, int, int, int64_t, int64_t, int64_t, int, int, cudaStream_t);
int tib_gemm_decode_supports(int, int, int, int, int, int);
int tib_gemm_decode(const void*, const void*, void*, int, int, int, int64_t, int64_t, int64_t, int, int, int, int, int, int*, cudaStream_t);
}

// What a block is made of: sizes, constants and weights.  Filled once when the weights are bound.
struct TibPrenormBlockWeights {
  int hidden, heads, kv_heads, head_dim, intermediate;
  int rot_dim, interleaved;              // rotary: rotated width (0: none), pairing
  int qkv_kn, o_kn, gate_up_kn, down_kn; // 1: the matrix is stored [in, out]
  int qkv_few_rows, o_few_rows, gate_up_few_rows, down_few_rows;   // rows up to which a projection goes to a few-rows kernel (0: never)
  int qkv_features, o_features, gate_up_features, down_features;   // the few-rows kernel's tile width (128 or 256) ...
  int qkv_splits, o_splits, gate_up_splits, down_splits;           // ... K split (0: the older swap-AB kernel) ...
  int qkv_stages, o_stages, gate_up_stages, down_stages;           // ... and ring depth (0: the kernel's default)
  float eps_mixer, eps_feed_forward, scale;
  const float* norm_mixer;               // [hidden]
  const float* norm_feed_forward;        // [hidden]
  const float* inv_freq;                 // [rot_dim / 2]
  const void* qkv;                       // (heads + 2 kv_heads) * head_dim x hidden
  const void* o;                         // hidden x heads * head_dim
  const void* gate_up;                   // 2 intermediate x hidden
  const void* down;                      // hidden x intermediate
};

// What a step brings: the batch arrays and the buffers the block works in (all of them for n_tokens rows).
struct TibPrenormBlockStep {
  int n_tokens, n_entries, max_q_len, n_single, n_multi;
  int decode_splits;
  int decode_rotates;                    // 1: a step of single tokens may go to the decode kernel unrotated
  int own_launches;                      // (out) kernels of this library the call launched (library products not counted)
  const int* positions;
  const int* token_slot;
  const int* q_start;
  const int* kv_start;
  const int* slots;
  float* residual;                       // [n_tokens, hidden] fp32
  void* normed;                          // [n_tokens, hidden]
  void* qkv;                             // [n_tokens, (heads + 2 kv_heads) * head_dim]
  void* q;                               // [n_tokens, heads * head_dim]
  void* attn;                            // [n_tokens, heads * head_dim]
  void* o_out;                           // [n_tokens, hidden]
  void* gate_up;                         // [n_tokens, 2 intermediate]
  void* act;                             // [n_tokens, intermediate]
  void* out;                             // [n_tokens, hidden]: the block's result, left pending
  float* split_scratch;                  // decode_splits > 1: n_entries * heads * decode_splits * (head_dim + 2) floats
  int* split_counters;                   // zeros, n_entries * kv_heads (or null: merge by a second kernel)
  int* error_word;
};

#define TIB_TRY(call)        \
  do {                       \
    const int rc__ = (call); \
    if (rc__ != TIB_OK) return rc__; \
  } while (0)

// --- optional timers per kernel class -------------------------------------------------------------------------
// Off by default and free when off.  When on (tib_kernel_timers(1)), every launch of the block is bracketed by two
// CUDA events on the launching stream; tib_kernel_timers_read() waits for the events recorded so far and adds
// their elapsed times up by class (the reference keeps such per-class timers around its layer's launches:
// src/torchinferno/models/llama3/tensor_parallel.py:4058-4069, 4462-4480).  Nothing is recorded while the
// stream is being captured into a graph: a captured step has no per-kernel times, run it uncaptured to time it.
namespace {
enum KernelClass { KC_NORM, KC_QKV, KC_ROPE_APPEND, KC_ATTENTION_PREFILL, KC_ATTENTION_DECODE, KC_O, KC_GATE_UP, KC_SWIGLU, KC_DOWN, KC_COUNT };
struct PendingTime { int kind; cudaEvent_t begin, end; };
struct KernelTimers {
  bool on = false;
  std::mutex guard;
  std::vector<PendingTime> pending;
  std::vector<cudaEvent_t> spare;
  double ms[KC_COUNT] = {0};
  long long count[KC_COUNT] = {0};
  cudaEvent_t event() {
    if (!spare.empty()) { cudaEvent_t e = spare.back(); spare.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};
KernelTimers& timers() { static KernelTimers t; return t; }

struct TimedScope {
  int kind; cudaStream_t stream; cudaEvent_t begin = nullptr;
  TimedScope(int k, cudaStream_t s) : kind(k), stream(s) {
    KernelTimers& t = timers();
    if (!t.on) return;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) return;
    std::lock_guard<std::mutex> lock(t.guard);
    begin = t.event();
    if (begin) cudaEventRecord(begin, s);
  }
  ~TimedScope() {
    if (!begin) return;
    KernelTimers& t = timers();
    std::lock_guard<std::mutex> lock(t.guard);
    cudaEvent_t end = t.event();
    if (end) cudaEventRecord(end, stream);
    t.pending.push_back({kind, begin, end});
  }
};
}  // namespace

#define TIB_TIMED(kind, call)            \
  do {                                   \
    TimedScope scope__(kind, stream);    \
    TIB_TRY(call);                       \
  } while (0)

// A launch of one of this library's own kernels (counted for the caller; the library products are not).
#define TIB_OWN(kind, call)   \
  do {                        \
    TIB_TIMED(kind, call);    \
    ++s->own_launches;        \
  } while (0)

// Switch the per-class timers on (1) or off (0); returns the setting before.
TIB_API int tib_kernel_timers(int on) {
  KernelTimers& t = timers();
  std::lock_guard<std::mutex> lock(t.guard);
  const int before = t.on ? 1 : 0;
  t.on = on != 0;
  return before;
}

// Waits for every pair of events recorded so far, adds the times up and copies the totals: ms[n], count[n] for the
// classes in the order of KernelClass (norm, qkv, rope_append, attention_prefill, attention_decode, o, gate_up,
// swiglu, down).  reset != 0 clears the totals afterwards.  Returns the number of classes.
TIB_API int tib_kernel_timers_read(double* ms, long long* count, int n, int reset) {
  KernelTimers& t = timers();
  std::lock_guard<std::mutex> lock(t.guard);
  for (const PendingTime& p : t.pending) {
    float elapsed = 0.f;
    if (p.end && cudaEventSynchronize(p.end) == cudaSuccess && cudaEventElapsedTime(&elapsed, p.begin, p.end) == cudaSuccess) {
      t.ms[p.kind] += elapsed;
      t.count[p.kind] += 1;
    }
    t.spare.push_back(p.begin);
    if (p.end) t.spare.push_back(p.end);
  }
  t.pending.clear();
  for (int i = 0; i < KC_COUNT && i < n; ++i) {
    if (ms) ms[i] = t.ms[i];
    if (count) count[i] = t.count[i];
  }
  if (reset) for (int i = 0; i < KC_COUNT; ++i) { t.ms[i] = 0; t.count[i] = 0; }
  return KC_COUNT;
}

// --- which kernel takes what ------------------------------------------------------------------------------------
// Asked by this file and by the Python parts alike (kernels/attention.py, kernels/gemm.py), so that the two ways of
// running a block cannot come to choose differently.

// Attention of a step in bfloat16.  group: query heads per kv head; packed: the layer's pages lie back to back as
// [2][kv_heads][page_size][head_dim]; allow: TIB_ALLOW_* bits (what the caller lets the plan use; rotary_table in
// TIB_ALLOW_DECODE_ROTATES means the position encoding is a rotary table the decode kernel can apply itself).
// *prefill, *decode: a TIB_ATTENTION_* kernel each, TIB_ATTENTION_NONE where the step has no such entries; where the
// tensor-core kernels do not take the shape both are TIB_ATTENTION_SIMT (one kernel for the whole step).
enum { TIB_ATTENTION_NONE = 0, TIB_ATTENTION_PREFILL_TCGEN05 = 1, TIB_ATTENTION_PREFILL_MMA = 2, TIB_ATTENTION_DECODE_TMA_ROTATES = 3,
       TIB_ATTENTION_DECODE_TMA = 4, TIB_ATTENTION_DECODE_CP_ASYNC = 5, TIB_ATTENTION_SIMT = 6 };
enum { TIB_ALLOW_PREFILL_TCGEN05 = 1, TIB_ALLOW_DECODE_ROTATES = 2, TIB_ALLOW_DECODE_TMA = 4 };
// Single tokens go to the decode kernel unrotated in steps of up to this many requests.  With few requests the step
// is a chain of short kernels and one link less is a gain (8 requests at 2,100 tokens, 8B sizes: 3.54 -> 3.51 ms a
// step); with many the attention kernel streams long enough that the head start it has under the rotary kernel (older
// keys are fetched while that runs) is worth more than the link (32 requests: 4.47 -> 4.52 ms, 64: 5.92 -> 6.01; 4 and
// 16: no difference).
constexpr int kDecodeRotatesMaxEntries = 8;

TIB_API int tib_plan_attention(int head_dim, int group, int page_size, int packed, int n_entries, int n_single, int n_multi,
                               int allow, int* prefill, int* decode) {
  if (!prefill || !decode || group < 1 || n_entries < 0 || n_single < 0 || n_multi < 0) return TIB_E_ARG;
  *prefill = *decode = TIB_ATTENTION_NONE;
  if (!tib_attention_mma_supports(head_dim, group)) {
    *prefill = *decode = TIB_ATTENTION_SIMT;
    return TIB_OK;
  }
  if (n_multi)
    *prefill = (allow & TIB_ALLOW_PREFILL_TCGEN05) && packed && tib_prefill_attention_tcgen05_supports(head_dim, group, page_size)
                   ? TIB_ATTENTION_PREFILL_TCGEN05 : TIB_ATTENTION_PREFILL_MMA;
  if (n_single) {
    const bool tma = (allow & TIB_ALLOW_DECODE_TMA) && packed && tib_decode_attention_tma_supports(head_dim, group, page_size);
    if (tma && (allow & TIB_ALLOW_DECODE_ROTATES) && !n_multi && n_single == n_entries && n_entries <= kDecodeRotatesMaxEntries)
      *decode = TIB_ATTENTION_DECODE_TMA_ROTATES;
    else
      *decode = tma ? TIB_ATTENTION_DECODE_TMA : TIB_ATTENTION_DECODE_CP_ASYNC;
  }
  return TIB_OK;
}

// A bf16 product of `rows` rows with a weight [N, K] or (kn) [K, N] that goes to a few-rows kernel up to few_rows rows
// (0: never) with tiles of `features` and K over `splits` blocks (splits 0: the older swap-AB kernel); epilogue 1: the
// weight holds gate and up columns interleaved and the activation is wanted; aligned: 16-byte pointers, row strides
// that are multiples of 8.  Returns the kernel: TIB_PRODUCT_DECODE (gemm_decode.cu, with the activation in its
// epilogue when asked), TIB_PRODUCT_SWAPAB (gemm_tcgen05.cu) or TIB_PRODUCT_LIBRARY (followed by the SwiGLU kernel when
// the activation is wanted, as after TIB_PRODUCT_SWAPAB).
enum { TIB_PRODUCT_LIBRARY = 0, TIB_PRODUCT_DECODE = 1, TIB_PRODUCT_SWAPAB = 2 };

TIB_API int tib_plan_product(int rows, int N, int K, int kn, int few_rows, int features, int splits, int epilogue, int aligned) {
  if (!(few_rows > 0 && rows > 0 && rows <= few_rows && aligned)) return TIB_PRODUCT_LIBRARY;
  if (epilogue) {
    if (kn && splits == 1 && tib_gemm_decode_supports(rows, N, K, features, 1, 1)) return TIB_PRODUCT_DECODE;
  } else if (kn && splits > 0 && tib_gemm_decode_supports(rows, N, K, features, splits, 0)) {
    return TIB_PRODUCT_DECODE;
  }
  return tib_gemm_tcgen05_swapab_supports(rows, N, K) ? TIB_PRODUCT_SWAPAB : TIB_PRODUCT_LIBRARY;
}

// out[n, N] = x[n, K] . w^T, w stored [N, K] or (kn) [K, N], by the kernel tib_plan_product names.
static int project(const void* x, const void* w, void* out, int n, int N, int K, int kn, int few_rows, int features, int splits,
                   int stages, int* error_word, int* own_launches, cudaStream_t stream) {
  const int kernel = tib_plan_product(n, N, K, kn, few_rows, features, splits, 0, 1);
  *own_launches += kernel != TIB_PRODUCT_LIBRARY;
  switch (kernel) {
    case TIB_PRODUCT_DECODE:
      return tib_gemm_decode(x, w, out, n, N, K, K, N, N, TIB_BF16, features, splits, 0, stages, error_word, stream);
    case TIB_PRODUCT_SWAPAB:
      return tib_gemm_tcgen05_swapab(x, w, out, n, N, K, K, kn ? N : K, N, kn, TIB_BF16, 0, error_word, stream);
    default:
      return tib_blas_gemm(x, w, out, n, N, K, K, kn ? N : K, N, kn, TIB_BF16, stream);
  }
}

// pending: the result of the block before (bf16 [n_tokens, hidden]) or null for the first.  pool: this layer's
// pages [pages, 2, kv_heads, page_size, head_dim] (page_stride elements apart); window 0: every key.
TIB_API int tib_prenorm_gqa_glu_block(const TibPrenormBlockWeights* w, TibPrenormBlockStep* s, const void* pending, void* pool,
                            const int* block_table, int table_stride, int page_size, int64_t page_stride, int num_pages,
                            int window, cudaStream_t stream) {
  if (!w || !s || !pool || !block_table) return TIB_E_ARG;
  const int n = s->n_tokens;
  s->own_launches = 0;
  if (n == 0) return TIB_OK;
  const int h = w->heads, k = w->kv_heads, d = w->head_dim, group = h / k;
  const int qkv_width = (h + 2 * k) * d, q_width = h * d;
  const bool packed = page_stride == (int64_t)2 * k * page_size * d;

  TIB_OWN(KC_NORM, tib_add_rmsnorm(pending, s->residual, nullptr, w->norm_mixer, s->normed, n, w->hidden, w->eps_mixer, TIB_BF16, stream));
  TIB_TIMED(KC_QKV, project(s->normed, w->qkv, s->qkv, n, qkv_width, w->hidden, w->qkv_kn, w->qkv_few_rows, w->qkv_features, w->qkv_splits, w->qkv_stages, s->error_word, &s->own_launches, stream));
  int prefill_kernel = 0, decode_kernel = 0;
  TIB_TRY(tib_plan_attention(d, group, page_size, packed, s->n_entries, s->n_single, s->n_multi,
                             TIB_ALLOW_PREFILL_TCGEN05 | TIB_ALLOW_DECODE_TMA | (s->decode_rotates ? TIB_ALLOW_DECODE_ROTATES : 0),
                             &prefill_kernel, &decode_kernel));
  if (prefill_kernel == TIB_ATTENTION_SIMT) return TIB_E_SIZE;      // (the caller keeps such shapes to the part-by-part sequence)
  // a step of single tokens only: the decode kernel rotates and stores the newest token itself (no rotary kernel)
  const bool fused_rope = decode_kernel == TIB_ATTENTION_DECODE_TMA_ROTATES;
  if (!fused_rope)
    TIB_OWN(KC_ROPE_APPEND, tib_rope_append(s->qkv, s->q, pool, s->positions, s->token_slot, block_table, table_stride, w->inv_freq, n, h, k, d,
                            w->rot_dim, w->interleaved, page_size, page_stride, num_pages, 1, s->error_word, TIB_BF16, stream));
  if (prefill_kernel == TIB_ATTENTION_PREFILL_TCGEN05)
    TIB_OWN(KC_ATTENTION_PREFILL, tib_prefill_attention_tcgen05(s->q, pool, s->attn, s->q_start, s->kv_start, s->slots, block_table, table_stride,
                                          s->n_entries, s->max_q_len, n, h, k, d, page_size, page_stride, num_pages, window,
                                          w->scale, s->n_single > 0, s->error_word, stream));
  else if (prefill_kernel == TIB_ATTENTION_PREFILL_MMA)
    TIB_OWN(KC_ATTENTION_PREFILL, tib_prefill_attention(s->q, pool, s->attn, s->q_start, s->kv_start, s->slots, block_table, table_stride,
                                  s->n_entries, s->max_q_len, h, k, d, page_size, page_stride, num_pages, window, w->scale,
                                  s->n_single > 0, stream));
  if (decode_kernel != TIB_ATTENTION_NONE) {
    const int splits = s->decode_splits < 1 ? 1 : s->decode_splits;
    float* scratch_o = splits > 1 ? s->split_scratch : nullptr;
    float* scratch_ml = splits > 1 ? s->split_scratch + (size_t)s->n_entries * h * splits * d : nullptr;
    if (splits > 1 && !scratch_o) return TIB_E_ARG;
    if (decode_kernel == TIB_ATTENTION_DECODE_TMA_ROTATES)
      TIB_OWN(KC_ATTENTION_DECODE, tib_decode_attention_tma_rope(s->qkv, pool, s->attn, scratch_o, scratch_ml, s->q_start, s->kv_start, s->slots,
                                              block_table, table_stride, s->n_entries, h, k, d, page_size, page_stride, num_pages,
                                              window, w->scale, splits, 0, splits > 1 ? s->split_counters : nullptr, s->error_word,
                                              w->inv_freq, w->rot_dim, w->interleaved, stream));
    else if (decode_kernel == TIB_ATTENTION_DECODE_TMA)
      TIB_OWN(KC_ATTENTION_DECODE, tib_decode_attention_tma(s->q, pool, s->attn, scratch_o, scratch_ml, s->q_start, s->kv_start, s->slots, block_table,
                                       table_stride, s->n_entries, h, k, d, page_size, page_stride, num_pages, window, w->scale,
                                       splits, 0, splits > 1 ? s->split_counters : nullptr, s->error_word, stream));
    else
      TIB_OWN(KC_ATTENTION_DECODE, tib_decode_attention(s->q, pool, s->attn, scratch_o, scratch_ml, s->q_start, s->kv_start, s->slots, block_table,
                                   table_stride, s->n_entries, h, k, d, page_size, page_stride, num_pages, window, w->scale,
                                   splits, 0, stream));
  }
  TIB_TIMED(KC_O, project(s->attn, w->o, s->o_out, n, w->hidden, q_width, w->o_kn, w->o_few_rows, w->o_features, w->o_splits, w->o_stages, s->error_word, &s->own_launches, stream));
  TIB_OWN(KC_NORM, tib_add_rmsnorm(s->o_out, s->residual, nullptr, w->norm_feed_forward, s->normed, n, w->hidden, w->eps_feed_forward,
                          TIB_BF16, stream));
  const int inter = w->intermediate;
  // gate and up rows are interleaved in the weight; at few rows the few-rows kernel writes silu(gate) * up itself
  if (tib_plan_product(n, 2 * inter, w->hidden, w->gate_up_kn, w->gate_up_few_rows, w->gate_up_features, w->gate_up_splits, 1, 1) ==
      TIB_PRODUCT_DECODE) {
    TIB_OWN(KC_GATE_UP, tib_gemm_decode(s->normed, w->gate_up, s->act, n, 2 * inter, w->hidden, w->hidden, 2 * inter, inter, TIB_BF16,
                                          w->gate_up_features, 1, 1, w->gate_up_stages, s->error_word, stream));
  } else {
    TIB_TIMED(KC_GATE_UP, project(s->normed, w->gate_up, s->gate_up, n, 2 * inter, w->hidden, w->gate_up_kn, w->gate_up_few_rows,
                                  w->gate_up_features, w->gate_up_splits, w->gate_up_stages, s->error_word, &s->own_launches, stream));
    TIB_OWN(KC_SWIGLU, tib_swiglu(s->gate_up, s->act, n, inter, TIB_BF16, 1, stream));
  }
  TIB_TIMED(KC_DOWN, project(s->act, w->down, s->out, n, w->hidden, inter, w->down_kn, w->down_few_rows, w->down_features, w->down_splits, w->down_stages, s->error_word, &s->own_launches, stream));
  return TIB_OK;
}
