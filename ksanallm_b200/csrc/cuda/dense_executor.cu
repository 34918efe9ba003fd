// Native per-step executor for dense decoder layers: one host call launches every kernel of the layer range.
// The Python model layer costs 15-25 microseconds of interpreter, allocator and ctypes time per kernel; with ~8
// kernels per layer that is more than the GPU time of a decode step once the model is sharded over 4-8 GPUs. Here
// a launch costs the driver call plus a tensor-map encode. The reference's equivalent is its C++ layer stack
// (src/ksana_llm/models/common/simple_decoder_layer.cpp:22-100 driven by common_model.cpp:424-513).
#include "dense_executor.h"

#include "host_common.h"

extern "C" {
int ksana_gemm_bf16(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw,
                    int ldc, int out_fp32, int bn, int force_splits, float* ws, long long ws_floats,
                    unsigned int* counters, int num_counters, cudaStream_t stream);
int ksana_rms_norm(const void* x, int ldx, void* residual, int ldr, const void* w, void* out, int ldo, int T, int H,
                   float eps, cudaStream_t stream);
int ksana_silu_mul(const void* x, int ldx, void* out, int ldo, int T, int I, cudaStream_t stream);
int ksana_rope_cache(void* q, int ldq, void* k, int ldk, const void* v, int ldv, const int* positions,
                     const float* cos_sin, const int* slots, void* cache, const void* qw, const void* kw, float eps,
                     int T, int h, int hk, int d, int rd, int interleaved, int block_size, int cache_kind,
                     float k_scale, float v_scale, cudaStream_t stream);
int ksana_paged_prefill(const void* q, int ldq, int total_tokens, const void* cache, int num_blocks,
                        const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int seq_base,
                        int num_seqs, int max_q_len, int h, int hk, int d, int block_size, float scale,
                        const float* alibi, void* out, int ldo, cudaStream_t stream);
int ksana_paged_decode(const void* q, int ldq, const void* cache, int cache_kind, const int* block_tables,
                       int max_blocks, const int* cu_q, const int* kv_lens, int seq_base, int num_seqs, int max_q_len,
                       int max_kv_len, int h, int hk, int d, int block_size, float scale, const float* alibi,
                       float k_scale, float v_scale, void* out, int ldo, float* workspace, long long workspace_floats,
                       cudaStream_t stream);
int ksana_rs_norm_ag(int rank, int ws, void* const* partial, void* const* hbuf, void* const* sig, void* partial_mc,
                     void* hbuf_mc, int T, int H, void* residual, const void* norm_w, float eps, unsigned int epoch,
                     int mode, int max_ctas, cudaStream_t stream);
int ksana_gemm_rs_norm_ag(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank, int ws,
                          void* const* recv, void* const* hbuf, void* const* sig, void* hbuf_mc, int rows_cap,
                          void* residual, const void* norm_w, float eps, unsigned int epoch, int mode, int comm_ctas,
                          int force_splits, cudaStream_t stream);
int ksana_gemm_ll_reduce_norm(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank, int ws,
                              void* const* recv, void* const* hbuf, void* const* flags, void* hbuf_mc, int rows_cap,
                              void* residual, const void* norm_w, float eps, unsigned int epoch, int mode,
                              int force_splits, cudaStream_t stream);
}

#define KSANA_STEP(n, call)                      \
  do {                                           \
    const int code__ = (call);                   \
    ++(*launches);                               \
    if (code__ != 0) {                           \
      *fail_code = code__;                       \
      return (L + 1) * 100 + (n);                \
    }                                            \
  } while (0)

KSANA_API int ksana_dense_forward(const KsanaDenseModel* m, const KsanaDenseStep* s, const void* h_in, void* residual,
                                  int first, int last, unsigned int* epoch_io, void** out_h, int* fail_code,
                                  int* launches, cudaStream_t stream) {
  const int T = s->total_tokens, H = m->hidden, h = m->heads, hk = m->kv_heads, d = m->head_dim, I = m->inter;
  const int nq = h * d, nk = hk * d, nqkv = nq + 2 * nk;
  const char* hcur = static_cast<const char*>(h_in);
  int pp = 0;
  *fail_code = 0;
  *launches = 0;
  if (T <= 0) {
    *out_h = const_cast<void*>(h_in);
    return 0;
  }
  // Small steps on many ranks are latency-bound: there the plain GEMM followed by the reduce/norm/gather kernel beats
  // the single fused kernel (8 ranks, 64 tokens: 48 us against 81 us), large steps are the other way round.
  const bool two_kernel = m->ws > 1 && T <= m->two_kernel_max_tokens && m->partial != nullptr;
  // decode-sized steps: one kernel whose chain of NVLink round trips is as short as it gets
  const bool ll_path = m->ws > 1 && T <= m->ll_max_tokens && m->ll_recv != nullptr;
  unsigned int epoch = epoch_io != nullptr ? *epoch_io : 0;
  auto next_epoch = [&]() -> unsigned int {
    if (++epoch == 0) ++epoch;
    return epoch;
  };
  auto row_parallel = [&](const void* a, const void* wt, int K, const void* norm_w, unsigned int ep) -> int {
    if (ll_path)
      return ksana_gemm_ll_reduce_norm(a, wt, T, H, K, K, K, m->rank, m->ws, m->ll_recv, m->hbuf, m->ll_flags,
                                       m->hbuf_mc, m->ll_rows_cap, residual, norm_w, m->eps, ep, 3, 0, stream);
    if (two_kernel) {
      const int c = ksana_gemm_bf16(a, wt, m->partial[m->rank], nullptr, T, H, K, K, K, H, 0, 0, 0, m->gemm_ws,
                                    m->gemm_ws_floats, m->gemm_counters, m->n_counters, stream);
      if (c != 0) return c;
      ++(*launches);
      return ksana_rs_norm_ag(m->rank, m->ws, m->partial, m->hbuf, m->sig, m->partial_mc, m->hbuf_mc, T, H, residual,
                              norm_w, m->eps, ep, 3, 0, stream);
    }
    return ksana_gemm_rs_norm_ag(a, wt, T, H, K, K, K, m->rank, m->ws, m->recv, m->hbuf, m->sig, m->hbuf_mc, m->rows_cap,
                                 residual, norm_w, m->eps, ep, 3, m->comm_ctas, 0, stream);
  };
  for (int L = first; L < last; ++L) {
    const KsanaDenseLayer& w = m->layers[L];
    char* qkv = static_cast<char*>(m->qkv_buf);
    KSANA_STEP(1, ksana_gemm_bf16(hcur, w.wqkv, qkv, w.bqkv, T, nqkv, H, H, H, nqkv, 0, 0, 0, m->gemm_ws,
                                  m->gemm_ws_floats, m->gemm_counters, m->n_counters, stream));
    char* q = qkv;
    char* k = qkv + static_cast<size_t>(nq) * 2;
    char* v = qkv + static_cast<size_t>(nq + nk) * 2;
    KSANA_STEP(2, ksana_rope_cache(q, nqkv, k, nqkv, v, nqkv, s->positions, m->rope_cache, s->slot_mapping, w.kv_cache,
                                   w.q_norm, w.k_norm, m->eps, T, h, hk, d, m->rope_cache ? m->rotary_dim : 0,
                                   m->rope_interleaved, m->block_size, m->kv_kind, m->k_scale, m->v_scale, stream));
    if (s->num_prefill > 0)
      KSANA_STEP(3, ksana_paged_prefill(q, nqkv, T, w.kv_cache, m->num_blocks, s->block_tables, s->max_blocks, s->cu_q,
                                        s->kv_lens, 0, s->num_prefill, s->max_q_prefill, h, hk, d, m->block_size,
                                        m->attn_scale, nullptr, m->attn_buf, nq, stream));
    if (s->num_decode > 0)
      KSANA_STEP(4, ksana_paged_decode(q, nqkv, w.kv_cache, m->kv_kind, s->block_tables, s->max_blocks, s->cu_q,
                                       s->kv_lens, s->num_prefill, s->num_decode, s->max_q_decode, s->max_kv_decode, h,
                                       hk, d, m->block_size, m->attn_scale, nullptr, m->k_scale, m->v_scale,
                                       m->attn_buf, nq, m->attn_ws, m->attn_ws_floats, stream));
    const char* h2;
    if (m->ws > 1) {
      KSANA_STEP(5, row_parallel(m->attn_buf, w.wo, nq, w.ln2, next_epoch()));
      h2 = static_cast<const char*>(m->hbuf[m->rank]);
    } else {
      KSANA_STEP(5, ksana_gemm_bf16(m->attn_buf, w.wo, m->proj_buf, nullptr, T, H, nq, nq, nq, H, 0, 0, 0, m->gemm_ws,
                                    m->gemm_ws_floats, m->gemm_counters, m->n_counters, stream));
      KSANA_STEP(6, ksana_rms_norm(m->proj_buf, H, residual, H, w.ln2, m->h_buf[pp], H, T, H, m->eps, stream));
      h2 = static_cast<const char*>(m->h_buf[pp]);
      pp ^= 1;
    }
    KSANA_STEP(7, ksana_gemm_bf16(h2, w.wgu, m->gu_buf, nullptr, T, 2 * I, H, H, H, 2 * I, 0, 0, 0, m->gemm_ws,
                                  m->gemm_ws_floats, m->gemm_counters, m->n_counters, stream));
    KSANA_STEP(8, ksana_silu_mul(m->gu_buf, 2 * I, m->act_buf, I, T, I, stream));
    if (m->ws > 1) {
      KSANA_STEP(9, row_parallel(m->act_buf, w.wdown, I, w.next_ln, next_epoch()));
      hcur = static_cast<const char*>(m->hbuf[m->rank]);
    } else {
      KSANA_STEP(9, ksana_gemm_bf16(m->act_buf, w.wdown, m->proj_buf, nullptr, T, H, I, I, I, H, 0, 0, 0, m->gemm_ws,
                                    m->gemm_ws_floats, m->gemm_counters, m->n_counters, stream));
      KSANA_STEP(10, ksana_rms_norm(m->proj_buf, H, residual, H, w.next_ln, m->h_buf[pp], H, T, H, m->eps, stream));
      hcur = static_cast<const char*>(m->h_buf[pp]);
      pp ^= 1;
    }
  }
  *out_h = const_cast<char*>(hcur);
  if (epoch_io != nullptr) *epoch_io = epoch;
  return 0;
}
