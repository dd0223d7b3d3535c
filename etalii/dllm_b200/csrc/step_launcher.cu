// The host side of a prefill-sized step, in C++: one call issues every launch of every pre-norm layer
// (RMSNorm, q/k/v product with rotation and cache write, attention, output product + residual, RMSNorm, gate/up
// product with SwiGLU, down product + residual), where the same step driven from Python pays an interpreter round
// trip of 7 to 10 microseconds per launch. Where the norms' weights were folded into the weights of the products
// that follow them, the norms are folded around those products too and a layer is five launches, not seven.
// No kernels live here: the entry points of the kernel libraries are given once as a table of function pointers,
// and the rules that choose between kernels are the ones the Python parts apply
// (etalii/dllm_b200/parts/attention.py, kernels/ops.py::gemm), restated for the case this file takes: bfloat16, more
// than 64 tokens, every product on the tcgen05 tile kernel. Layers with other parts keep the Python path.
#include "common.cuh"

extern "C" {
// Entry points of the other libraries (signatures as exported there).
struct DllmKernelTable {
  int (*rmsnorm)(void* out, const float* x, const float* weight, const int* rows, int n_rows, int hidden, float eps,
                 int out_dtype, cudaStream_t stream);
  int (*gemm_tcgen05)(void* c, const void* a, const void* w, int M, int N, int K, int epilogue, int tile_n,
                      int* status, cudaStream_t stream);
  int (*gemm_tcgen05_qkv_rope)(const void* a, const void* w, int M, int K, void* q_out, void* cache_base,
                               const int* page_table, int max_pages, int page_size, int heads, int kv_heads,
                               int head_dim, const float* table, int rotary_dim, int table_positions,
                               const int* tok_seq, const int* tok_pos, const int* slots, int write_cache, int* status,
                               cudaStream_t stream);
  int (*attention_prefill)(void* out, const void* q, void* cache_base, const int* page_table, int max_pages,
                           int page_size, int heads, int kv_heads, int head_dim, const int* tile_seq,
                           const int* tile_first, const int* cu_seqlens, const int* start, const int* slots,
                           int tiles, float scale, int window, cudaStream_t stream);
  int (*attention_prefill_tcgen05)(void* out, const void* q, int tokens, void* cache_base, long long cache_pages,
                                   const int* page_table, int max_pages, int page_size, int heads, int kv_heads,
                                   int head_dim, const int* tile_seq, const int* tile_first, const int* cu_seqlens,
                                   const int* start, const int* slots, int tiles, float scale, int window,
                                   int* status, cudaStream_t stream);
  // the products with an RMSNorm folded around them (gemm_tcgen05.cu) and what prepares a step's first rows for them
  int (*cast_ssq)(void* copy, float* ssq, const float* x, int n_rows, int hidden, cudaStream_t stream);
  int (*gemm_tcgen05_normed)(void* c, const void* a, const void* w, int M, int N, int K, int epilogue,
                             const float* ssq_in, int parts_in, float eps, int* status, cudaStream_t stream);
  int (*gemm_tcgen05_qkv_rope_normed)(const void* a, const void* w, int M, int K, void* q_out, void* cache_base,
                                      const int* page_table, int max_pages, int page_size, int heads, int kv_heads,
                                      int head_dim, const float* table, int rotary_dim, int table_positions,
                                      const int* tok_seq, const int* tok_pos, const int* slots, int write_cache,
                                      const float* ssq_in, int parts_in, float eps, int* status, cudaStream_t stream);
  int (*gemm_tcgen05_residual_norm)(void* x, void* copy_out, float* ssq_out, int* parts_out, const void* a,
                                    const void* w, int M, int N, int K, int* status, cudaStream_t stream);
};

// One pre-norm layer: norm -> attention (rotary or no position encoding) -> norm -> SwiGLU, as its parts were bound.
struct DllmPreNormLayer {
  const float* mixer_norm_weight;
  const float* feed_forward_norm_weight;
  const void* w_qkv;       // [(heads + 2 kv_heads) * head_dim, hidden]
  const void* w_o;         // [hidden, heads * head_dim]
  const void* w_gate_up;   // [2 * intermediate, hidden], gate and up rows interleaved
  const void* w_down;      // [hidden, intermediate]
  const float* rotary_table;  // [rotary_dim / 2, rotary_positions, (cos, sin)] (pair by pair) or null
  void* cache_base;
  const int* page_table;
  long long cache_pages;
  float mixer_norm_eps, feed_forward_norm_eps, scale;
  int hidden, heads, kv_heads, head_dim, intermediate, rotary_dim, window;
  int max_pages, page_size;
  int tcgen05_attention_from;  // contexts above this take the tcgen05 attention kernel; negative: never
  int rotary_positions;        // positions the rotary table covers
};

// The step: the residual stream, work buffers (sized for the widest layer) and the step's metadata on the device.
struct DllmPrefillStep {
  float* x;          // [tokens, hidden] float32, in and out
  void* normed;      // [tokens, hidden] bfloat16
  void* q;           // [tokens, heads * head_dim] bfloat16
  void* attended;    // [tokens, heads * head_dim] bfloat16
  void* activations; // [tokens, intermediate] bfloat16
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
  const int* cu_seqlens;
  const int* start;
  const int* tile_seq;
  const int* tile_first;
  int* status;       // the kernels' shared status word
  float* row_ssq;    // [up to ceil(hidden / 16)][tokens] sums of squares (folded norms), or null
  int tokens, tiles, max_context;
  int norms_folded;  // the norms' weights live in the columns of w_qkv and w_gate_up: five launches a layer
};
}

namespace {
constexpr int EPI_RESIDUAL = 2, EPI_SWIGLU = 3;
}

// Issues the launches of layers[0 .. n_layers) for the step. Returns 0, or the first refusal of a kernel entry
// point (negative), with *failed_at = 16 * layer + stage (stages 0..6 in launch order). *launched counts launches.
DLLM_EXPORT int dllm_prefill_pre_norm_layers(const DllmKernelTable* k, const DllmPreNormLayer* layers, int n_layers,
                                             const DllmPrefillStep* s, int* launched, int* failed_at,
                                             cudaStream_t stream) {
  if (k == nullptr || layers == nullptr || s == nullptr || launched == nullptr || failed_at == nullptr)
    return DLLM_BAD_ARGUMENT;
  *launched = 0;
  *failed_at = -1;
#define DLLM_STAGE(stage, call)                   \
  do {                                            \
    int status_ = (call);                         \
    if (status_ != DLLM_OK) {                     \
      *failed_at = 16 * i + (stage);              \
      return status_;                             \
    }                                             \
    ++*launched;                                  \
  } while (0)
  if (s->norms_folded) {
    // No norm kernels: the products that write the residual also write its bfloat16 copy (into `normed`) and the
    // rows' sums of squares; the products that read it scale their rows. Only the step's first rows need a pass.
    int parts = 1;
    {
      int i = 0;
      DLLM_STAGE(0, k->cast_ssq(s->normed, s->row_ssq, s->x, s->tokens, layers[0].hidden, stream));
    }
    for (int i = 0; i < n_layers; ++i) {
      const DllmPreNormLayer& l = layers[i];
      int q_size = l.heads * l.head_dim;
      DLLM_STAGE(1, k->gemm_tcgen05_qkv_rope_normed(s->normed, l.w_qkv, s->tokens, l.hidden, s->q, l.cache_base,
                                                    l.page_table, l.max_pages, l.page_size, l.heads, l.kv_heads,
                                                    l.head_dim, l.rotary_table, l.rotary_table ? l.rotary_dim : 0,
                                                    l.rotary_positions, s->tok_seq, s->tok_pos, s->slots, 1,
                                                    s->row_ssq, parts,
                                                    l.mixer_norm_eps, s->status, stream));
      if (l.tcgen05_attention_from >= 0 && s->max_context > l.tcgen05_attention_from)
        DLLM_STAGE(2, k->attention_prefill_tcgen05(s->attended, s->q, s->tokens, l.cache_base, l.cache_pages,
                                                   l.page_table, l.max_pages, l.page_size, l.heads, l.kv_heads,
                                                   l.head_dim, s->tile_seq, s->tile_first, s->cu_seqlens, s->start,
                                                   s->slots, s->tiles, l.scale, l.window, s->status, stream));
      else
        DLLM_STAGE(2, k->attention_prefill(s->attended, s->q, l.cache_base, l.page_table, l.max_pages, l.page_size,
                                           l.heads, l.kv_heads, l.head_dim, s->tile_seq, s->tile_first,
                                           s->cu_seqlens, s->start, s->slots, s->tiles, l.scale, l.window, stream));
      DLLM_STAGE(3, k->gemm_tcgen05_residual_norm(s->x, s->normed, s->row_ssq, &parts, s->attended, l.w_o, s->tokens,
                                                  l.hidden, q_size, s->status, stream));
      DLLM_STAGE(5, k->gemm_tcgen05_normed(s->activations, s->normed, l.w_gate_up, s->tokens, 2 * l.intermediate,
                                           l.hidden, EPI_SWIGLU, s->row_ssq, parts, l.feed_forward_norm_eps,
                                           s->status, stream));
      DLLM_STAGE(6, k->gemm_tcgen05_residual_norm(s->x, s->normed, s->row_ssq, &parts, s->activations, l.w_down,
                                                  s->tokens, l.hidden, l.intermediate, s->status, stream));
    }
    return DLLM_OK;
  }
  for (int i = 0; i < n_layers; ++i) {
    const DllmPreNormLayer& l = layers[i];
    int q_size = l.heads * l.head_dim;
    DLLM_STAGE(0, k->rmsnorm(s->normed, s->x, l.mixer_norm_weight, nullptr, s->tokens, l.hidden, l.mixer_norm_eps,
                             DLLM_BF16, stream));
    DLLM_STAGE(1, k->gemm_tcgen05_qkv_rope(s->normed, l.w_qkv, s->tokens, l.hidden, s->q, l.cache_base, l.page_table,
                                           l.max_pages, l.page_size, l.heads, l.kv_heads, l.head_dim, l.rotary_table,
                                           l.rotary_table ? l.rotary_dim : 0, l.rotary_positions, s->tok_seq,
                                           s->tok_pos, s->slots, 1, s->status, stream));
    if (l.tcgen05_attention_from >= 0 && s->max_context > l.tcgen05_attention_from)
      DLLM_STAGE(2, k->attention_prefill_tcgen05(s->attended, s->q, s->tokens, l.cache_base, l.cache_pages,
                                                 l.page_table, l.max_pages, l.page_size, l.heads, l.kv_heads,
                                                 l.head_dim, s->tile_seq, s->tile_first, s->cu_seqlens, s->start,
                                                 s->slots, s->tiles, l.scale, l.window, s->status, stream));
    else
      DLLM_STAGE(2, k->attention_prefill(s->attended, s->q, l.cache_base, l.page_table, l.max_pages, l.page_size,
                                         l.heads, l.kv_heads, l.head_dim, s->tile_seq, s->tile_first, s->cu_seqlens,
                                         s->start, s->slots, s->tiles, l.scale, l.window, stream));
    DLLM_STAGE(3, k->gemm_tcgen05(s->x, s->attended, l.w_o, s->tokens, l.hidden, q_size, EPI_RESIDUAL, 0, s->status,
                                  stream));
    DLLM_STAGE(4, k->rmsnorm(s->normed, s->x, l.feed_forward_norm_weight, nullptr, s->tokens, l.hidden,
                             l.feed_forward_norm_eps, DLLM_BF16, stream));
    DLLM_STAGE(5, k->gemm_tcgen05(s->activations, s->normed, l.w_gate_up, s->tokens, 2 * l.intermediate, l.hidden,
                                  EPI_SWIGLU, 0, s->status, stream));
    DLLM_STAGE(6, k->gemm_tcgen05(s->x, s->activations, l.w_down, s->tokens, l.hidden, l.intermediate, EPI_RESIDUAL,
                                  0, s->status, stream));
  }
#undef DLLM_STAGE
  return DLLM_OK;
}
