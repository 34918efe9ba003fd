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
int ksana_paged_decode_gqa(const void* q, int ldq, int total_tokens, const void* cache, int num_blocks,
                           const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int seq_base,
                           int num_seqs, int max_q_len, int max_kv_len, int h, int hk, int d, int block_size, float scale,
                           void* out, int ldo, float* workspace, long long workspace_floats, cudaStream_t stream);
int ksana_rs_norm_ag(int rank, int ws, void* const* partial, void* const* hbuf, void* const* sig, void* partial_mc,
                     void* hbuf_mc, int T, int H, void* residual, const void* norm_w, float eps, unsigned int epoch,
                     int mode, int max_ctas, cudaStream_t stream);
int ksana_gemm_rs_norm_ag(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank, int ws,
                          void* const* recv, void* const* hbuf, void* const* sig, void* hbuf_mc, int rows_cap,
                          void* residual, const void* norm_w, float eps, unsigned int epoch, int mode, int comm_ctas,
                          int force_splits, cudaStream_t stream);
int ksana_gemm_ll_reduce_norm(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank, int ws,
                              void* const* recv, long long recv_off, void* const* recv2, void* recv2_mc, void* hbuf,
                              int rows_cap, int one_shot, void* residual, const void* norm_w, float eps,
                              unsigned int epoch, int mode, int force_splits, cudaStream_t stream);
int ksana_ll_reduce_norm(const void* partial, int ldp, int M, int H, int rank, int ws, void* const* recv,
                         long long recv_off, void* const* recv2, void* recv2_mc, void* hbuf, int rows_cap, int one_shot,
                         void* residual, const void* norm_w, float eps, unsigned int epoch, int mode,
                         cudaStream_t stream);
int ksana_gemm_fp8_block(const void* A8, const float* sa, const void* W8, const float* sw, void* C, const void* bias,
                         int M, int N, int K, int lda, int ldw, int ldc, int out_fp32, int force_splits, float* ws,
                         long long ws_floats, unsigned int* counters, int num_counters, cudaStream_t stream);
int ksana_quant_fp8_group(const void* x, int ldx, void* q, int ldq, float* scales, int T, int K, cudaStream_t stream);
int ksana_silu_mul_quant_fp8(const void* x, int ldx, void* q, int ldq, float* scales, int T, int I,
                             cudaStream_t stream);
int ksana_quant_fp8_ue8m0(const void* x, int ldx, void* q, int ldq, float* scales, void* sfa, int T, int K,
                          cudaStream_t stream);
int ksana_silu_mul_quant_ue8m0(const void* x, int ldx, void* q, int ldq, float* scales, void* sfa, int T, int I,
                               cudaStream_t stream);
int ksana_gemm_mxf8(const void* A8, const void* sfa, const void* W8, const void* sfb, void* C, const void* bias, int M,
                    int N, int K, int lda, int ldw, int ldc, int variant, cudaStream_t stream);
int ksana_gemm_bf16_swiglu(const void* A, const void* W_interleaved, void* C, int M, int N, int K, int lda, int ldw,
                           int ldc, cudaStream_t stream);
void ksana_gemm_set_lane(int lane);
}

namespace {

// One half-batch (or the whole step): rows [r0, r0 + rows) of every [T, ...] buffer, prefill sequences
// [pre_base, pre_base + n_pre) and decode sequences [dec_base, dec_base + n_dec) of the step's sequence list.
struct Range {
  int r0, rows;
  int pre_base, n_pre, dec_base, n_dec;
  int max_q_prefill, max_q_decode, max_kv_decode;
  int lane;  // 0 / 1: which flag region, scratch half and stream this range uses
  cudaStream_t stream;
  const char* hcur;  // normalised input rows of the next layer (pointer to row r0)
  int pp;            // ws == 1: which of the two h buffers receives the next norm output
  const char* h2 = nullptr;  // normalised rows after the attention half, the MLP's input
};

struct Exec {
  const KsanaDenseModel* m;
  const KsanaDenseStep* s;
  char* residual;
  unsigned int epoch, ll_seq;
  int* launches;
  int fail_step, fail_code;
  void* sig_lane[2][8];
  // Two-batch overlap: the kernels that wait on peers form one chain across both streams (each starts after the
  // previous one of the chain has finished), in the same order on every rank. Without the chain, rank A can sit in
  // the first half's reduction while rank B sits in the second half's: each waits for a peer kernel that is queued
  // behind a GEMM which finds no room beside the waiting CTAs, and both run into the wait limit.
  cudaEvent_t chain_ev[2] = {nullptr, nullptr};
  cudaEvent_t chain_prev = nullptr;

  unsigned int next_epoch() {
    if (++epoch == 0) ++epoch;
    return epoch;
  }
  bool step(int n, int code) {
    ++(*launches);
    if (code != 0 && fail_step == 0) {
      fail_step = n;
      fail_code = code;
    }
    return code == 0;
  }

  // fp8 staging rows of one range (the two half-batches use disjoint row ranges of the same buffers)
  uint8_t* a8(const Range& g) const { return static_cast<uint8_t*>(m->a8_buf) + static_cast<size_t>(g.r0) * m->a8_cols; }
  // the second half-batch's scales start at a 128-row boundary: the packed layout covers whole 128-row groups
  float* sa(const Range& g) const {
    return m->sa_buf + static_cast<size_t>((g.r0 + 127) / 128 * 128) * (m->a8_cols / 128);
  }
  // the scaled tensor-core GEMM serves this product (its activations are then staged with packed scale bytes)
  bool use_mx(const Range& g, const void* sfb) const {
    return m->fp8_pow2 != 0 && sfb != nullptr && g.rows >= m->mx_min_rows;
  }

  // activations -> e4m3 staging rows, with the kind of scales the GEMM of this product wants
  int quant_f8(const Range& g, const void* a, int K, const void* sfb) {
    if (m->fp8_pow2 == 0) return ksana_quant_fp8_group(a, K, a8(g), K, sa(g), g.rows, K, g.stream);
    const bool mx = use_mx(g, sfb);
    return ksana_quant_fp8_ue8m0(a, K, a8(g), K, mx ? nullptr : sa(g), mx ? sa(g) : nullptr, g.rows, K, g.stream);
  }

  // block-scaled fp8 GEMM over activations that are already in the staging rows; half-batches never split K
  // (the split-K workspace is shared between the streams)
  int gemm_f8(const Range& g, const void* wt, const float* sw, const void* sfb, void* out, const void* bias, int N,
              int K, int ldc, bool whole_step) {
    if (use_mx(g, sfb)) return ksana_gemm_mxf8(a8(g), sa(g), wt, sfb, out, bias, g.rows, N, K, K, K, ldc, 0, g.stream);
    return ksana_gemm_fp8_block(a8(g), sa(g), wt, sw, out, bias, g.rows, N, K, K, K, ldc, 0, whole_step ? 0 : 1,
                                m->gemm_ws, m->gemm_ws_floats, m->gemm_counters, m->n_counters, g.stream);
  }

  // out[rows, N] = a[rows, K] * wt^T (+ bias), bf16 weights or (sw != null) block-scaled e4m3 weights
  int linear(const Range& g, const void* a, const void* wt, const float* sw, const void* sfb, void* out,
             const void* bias, int N, int K, int ldc, bool whole_step) {
    if (sw == nullptr)
      return ksana_gemm_bf16(a, wt, out, bias, g.rows, N, K, K, K, ldc, 0, 0, 0, m->gemm_ws, m->gemm_ws_floats,
                             m->gemm_counters, m->n_counters, g.stream);
    const int c = quant_f8(g, a, K, sfb);
    if (c != 0) return c;
    ++(*launches);
    return gemm_f8(g, wt, sw, sfb, out, bias, N, K, ldc, whole_step);
  }

  // row-parallel GEMM + reduce + residual add + RMSNorm + gather of one range; the output rows land in hbuf.
  // sw != null: e4m3 weights, `a` is ignored and the activations are taken from the fp8 staging rows.
  int row_parallel(const Range& g, const void* a, const void* wt, const float* sw, const void* sfb, int K,
                   const void* norm_w, bool whole_step) {
    const int H = m->hidden, T = g.rows;
    char* res = residual + static_cast<size_t>(g.r0) * H * 2;
    const unsigned int ep = next_epoch();
    if (sw != nullptr) {
      // fp8: the GEMM writes this rank's partial sum, a second kernel reduces it over the ranks
      const size_t off = static_cast<size_t>(g.r0) * H * 2;
      void* partial[8];
      void* hbuf[8];
      for (int i = 0; i < m->ws; ++i) {
        partial[i] = static_cast<char*>(m->partial[i]) + off;
        hbuf[i] = static_cast<char*>(m->hbuf[i]) + off;
      }
      const int c = gemm_f8(g, wt, sw, sfb, partial[m->rank], nullptr, H, K, H, whole_step);
      if (c != 0) return c;
      ++(*launches);
      if (whole_step && T <= m->ll_max_tokens && m->ll_recv != nullptr) {
        ++ll_seq;
        const long long loff = m->ll_one_shot ? static_cast<long long>(ll_seq & 1u) * m->ll_half_words : 0;
        return ksana_ll_reduce_norm(partial[m->rank], H, T, H, m->rank, m->ws, m->ll_recv, loff, m->ll_recv2,
                                    m->ll_recv2_mc, m->hbuf[m->rank], m->ll_rows_cap, m->ll_one_shot, res, norm_w,
                                    m->eps, ep, 3, g.stream);
      }
      return reduce_kernel(g, partial, hbuf, off, res, norm_w, ep, whole_step);
    }
    // decode-sized steps: one kernel whose chain of NVLink round trips is as short as it gets
    if (whole_step && T <= m->ll_max_tokens && m->ll_recv != nullptr) {
      ++ll_seq;
      const long long off = m->ll_one_shot ? static_cast<long long>(ll_seq & 1u) * m->ll_half_words : 0;
      return ksana_gemm_ll_reduce_norm(a, wt, T, H, K, K, K, m->rank, m->ws, m->ll_recv, off, m->ll_recv2,
                                       m->ll_recv2_mc, m->hbuf[m->rank], m->ll_rows_cap, m->ll_one_shot, res, norm_w,
                                       m->eps, ep, 3, 0, g.stream);
    }
    // Half-batches always take the GEMM + reduce kernel pair: the reduce kernel is small enough to stay resident next
    // to the other half's GEMM. Whole steps: the pair when latency-bound, else the single fused kernel.
    const bool two_kernel = !whole_step || (T <= m->two_kernel_max_tokens && m->partial != nullptr);
    if (two_kernel) {
      void* partial[8];
      void* hbuf[8];
      const size_t off = static_cast<size_t>(g.r0) * H * 2;
      for (int i = 0; i < m->ws; ++i) {
        partial[i] = static_cast<char*>(m->partial[i]) + off;
        hbuf[i] = static_cast<char*>(m->hbuf[i]) + off;
      }
      const int c = ksana_gemm_bf16(a, wt, partial[m->rank], nullptr, T, H, K, K, K, H, 0, 0, 0, m->gemm_ws,
                                    m->gemm_ws_floats, m->gemm_counters, m->n_counters, g.stream);
      if (c != 0) return c;
      ++(*launches);
      return reduce_kernel(g, partial, hbuf, off, res, norm_w, ep, whole_step);
    }
    return ksana_gemm_rs_norm_ag(a, wt, T, H, K, K, K, m->rank, m->ws, m->recv, m->hbuf, m->sig, m->hbuf_mc, m->rows_cap,
                                 res, norm_w, m->eps, ep, 3, m->comm_ctas, 0, g.stream);
  }

  // reduce over the ranks + residual add + RMSNorm + gather of a partial sum in the symmetric buffers
  int reduce_kernel(const Range& g, void* const* partial, void* const* hbuf, size_t off, char* res, const void* norm_w,
                    unsigned int ep, bool whole_step) {
    const bool chained = !whole_step && chain_ev[g.lane] != nullptr;
    if (chained && chain_prev != nullptr) cudaStreamWaitEvent(g.stream, chain_prev, 0);
    const int rc = ksana_rs_norm_ag(m->rank, m->ws, partial, hbuf, sig_lane[g.lane],
                                    m->partial_mc ? static_cast<char*>(m->partial_mc) + off : nullptr,
                                    m->hbuf_mc ? static_cast<char*>(m->hbuf_mc) + off : nullptr, g.rows, m->hidden, res,
                                    norm_w, m->eps, ep, 3, 0, g.stream);
    if (chained) {
      cudaEventRecord(chain_ev[g.lane], g.stream);
      chain_prev = chain_ev[g.lane];
    }
    return rc;
  }

  // one decoder layer over one range; part 1 = up to the attention output's reduction, part 2 = the MLP, 0 = both
  bool layer(int L, Range& g, bool whole_step, int part = 0) {
    const KsanaDenseLayer& w = m->layers[L];
    const int T = g.rows, H = m->hidden, h = m->heads, hk = m->kv_heads, d = m->head_dim, I = m->inter;
    const int nq = h * d, nk = hk * d, nqkv = nq + 2 * nk;
    cudaStream_t st = g.stream;
    ksana_gemm_set_lane(g.lane);
    char* qkv_all = static_cast<char*>(m->qkv_buf);
    char* qkv = qkv_all + static_cast<size_t>(g.r0) * nqkv * 2;
    char* attn_all = static_cast<char*>(m->attn_buf);
    char* attn = attn_all + static_cast<size_t>(g.r0) * nq * 2;
    char* gu = static_cast<char*>(m->gu_buf) + static_cast<size_t>(g.r0) * 2 * I * 2;
    char* act = static_cast<char*>(m->act_buf) + static_cast<size_t>(g.r0) * I * 2;
    char* res = residual + static_cast<size_t>(g.r0) * H * 2;
    if (part == 2) return mlp(w, g, whole_step, gu, act, res);
    if (!step(1, linear(g, g.hcur, w.wqkv, w.sqkv, w.fqkv, qkv, w.bqkv, nqkv, H, nqkv, whole_step))) return false;
    char* q = qkv;
    char* k = qkv + static_cast<size_t>(nq) * 2;
    char* v = qkv + static_cast<size_t>(nq + nk) * 2;
    if (!step(2, ksana_rope_cache(q, nqkv, k, nqkv, v, nqkv, s->positions + g.r0, m->rope_cache, s->slot_mapping + g.r0,
                                  w.kv_cache, w.q_norm, w.k_norm, m->eps, T, h, hk, d,
                                  m->rope_cache ? m->rotary_dim : 0, m->rope_interleaved, m->block_size, m->kv_kind,
                                  m->k_scale, m->v_scale, st)))
      return false;
    // the attention kernels index rows through the step's cu_q, so they get the base pointers of all rows
    if (g.n_pre > 0 &&
        !step(3, ksana_paged_prefill(qkv_all, nqkv, s->total_tokens, w.kv_cache, m->num_blocks, s->block_tables,
                                     s->max_blocks, s->cu_q, s->kv_lens, g.pre_base, g.n_pre, g.max_q_prefill, h, hk, d,
                                     m->block_size, m->attn_scale, nullptr, attn_all, nq, st)))
      return false;
    if (g.n_dec > 0) {
      const long long half = m->attn_ws_floats / 2;
      float* aws = m->attn_ws + (whole_step ? 0 : g.lane * half);
      const long long aws_floats = whole_step ? m->attn_ws_floats : half;
      int gqa = -1;
      if (m->kv_kind == 0 && h / hk >= 4 && (h / hk) * g.max_q_decode <= 128) {
        // grouped-query decode on the tensor cores; shapes it declines (-1) and workspace shortfalls (-6) fall through
        gqa = ksana_paged_decode_gqa(qkv_all, nqkv, s->total_tokens, w.kv_cache, m->num_blocks, s->block_tables,
                                     s->max_blocks, s->cu_q, s->kv_lens, g.dec_base, g.n_dec, g.max_q_decode,
                                     g.max_kv_decode, h, hk, d, m->block_size, m->attn_scale, attn_all, nq, aws,
                                     aws_floats, st);
        if (gqa != 0 && gqa != -1 && gqa != -6) return step(4, gqa);
        if (gqa == 0) ++(*launches);
      }
      if (gqa != 0 && !step(4, ksana_paged_decode(qkv_all, nqkv, w.kv_cache, m->kv_kind, s->block_tables, s->max_blocks, s->cu_q,
                                      s->kv_lens, g.dec_base, g.n_dec, g.max_q_decode, g.max_kv_decode, h, hk, d,
                                      m->block_size, m->attn_scale, nullptr, m->k_scale, m->v_scale, attn_all, nq,
                                      aws, aws_floats, st)))
        return false;
    }
    if (w.so != nullptr && !step(5, quant_f8(g, attn, nq, w.fo))) return false;
    if (m->ws > 1) {
      if (!step(5, row_parallel(g, attn, w.wo, w.so, w.fo, nq, w.ln2, whole_step))) return false;
      g.h2 = static_cast<const char*>(m->hbuf[m->rank]) + static_cast<size_t>(g.r0) * H * 2;
    } else {
      char* proj = static_cast<char*>(m->proj_buf) + static_cast<size_t>(g.r0) * H * 2;
      char* hb = static_cast<char*>(m->h_buf[g.pp]) + static_cast<size_t>(g.r0) * H * 2;
      const int c = w.so != nullptr ? gemm_f8(g, w.wo, w.so, w.fo, proj, nullptr, H, nq, H, whole_step)
                                    : ksana_gemm_bf16(attn, w.wo, proj, nullptr, T, H, nq, nq, nq, H, 0, 0, 0, m->gemm_ws,
                                                      m->gemm_ws_floats, m->gemm_counters, m->n_counters, st);
      if (!step(5, c)) return false;
      if (!step(6, ksana_rms_norm(proj, H, res, H, w.ln2, hb, H, T, H, m->eps, st))) return false;
      g.h2 = hb;
      g.pp ^= 1;
    }
    return part == 1 ? true : mlp(w, g, whole_step, gu, act, res);
  }

  bool mlp(const KsanaDenseLayer& w, Range& g, bool whole_step, char* gu, char* act, char* res) {
    const int T = g.rows, H = m->hidden, I = m->inter;
    cudaStream_t st = g.stream;
    // bf16, prefill-sized (the CTA-pair GEMM's range) and an interleaved weight copy at hand: the activation is the
    // GEMM's epilogue
    const bool fused_act = w.wgu_il != nullptr && w.sgu == nullptr && w.sdown == nullptr && T >= 384;
    if (fused_act) {
      if (!step(7, ksana_gemm_bf16_swiglu(g.h2, w.wgu_il, act, T, 2 * I, H, H, H, I, st))) return false;
    } else if (!step(7, linear(g, g.h2, w.wgu, w.sgu, w.fgu, gu, nullptr, 2 * I, H, 2 * I, whole_step))) {
      return false;
    }
    // fp8 down projection: SiLU * up is written once, already quantised
    int c8;
    if (fused_act) {
      c8 = 0;
      --(*launches);
    } else if (w.sdown == nullptr) {
      c8 = ksana_silu_mul(gu, 2 * I, act, I, T, I, st);
    } else if (m->fp8_pow2 == 0) {
      c8 = ksana_silu_mul_quant_fp8(gu, 2 * I, a8(g), I, sa(g), T, I, st);
    } else {
      const bool mx = use_mx(g, w.fdown);
      c8 = ksana_silu_mul_quant_ue8m0(gu, 2 * I, a8(g), I, mx ? nullptr : sa(g), mx ? sa(g) : nullptr, T, I, st);
    }
    if (!step(8, c8)) return false;
    if (m->ws > 1) {
      if (!step(9, row_parallel(g, act, w.wdown, w.sdown, w.fdown, I, w.next_ln, whole_step))) return false;
      g.hcur = static_cast<const char*>(m->hbuf[m->rank]) + static_cast<size_t>(g.r0) * H * 2;
    } else {
      char* proj = static_cast<char*>(m->proj_buf) + static_cast<size_t>(g.r0) * H * 2;
      char* hb = static_cast<char*>(m->h_buf[g.pp]) + static_cast<size_t>(g.r0) * H * 2;
      const int c = w.sdown != nullptr ? gemm_f8(g, w.wdown, w.sdown, w.fdown, proj, nullptr, H, I, H, whole_step)
                                       : ksana_gemm_bf16(act, w.wdown, proj, nullptr, T, H, I, I, I, H, 0, 0, 0,
                                                         m->gemm_ws, m->gemm_ws_floats, m->gemm_counters, m->n_counters,
                                                         st);
      if (!step(9, c)) return false;
      if (!step(10, ksana_rms_norm(proj, H, res, H, w.next_ln, hb, H, T, H, m->eps, st))) return false;
      g.hcur = hb;
      g.pp ^= 1;
    }
    return true;
  }
};

// second stream + events of the two-batch overlap, one set per device, created on first use
struct OverlapStreams {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr, chain[2] = {nullptr, nullptr};
};
OverlapStreams g_overlap[64];

OverlapStreams* overlap_streams() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  OverlapStreams* o = &g_overlap[dev];
  if (o->side == nullptr) {
    if (cudaStreamCreateWithFlags(&o->side, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&o->fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&o->join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < 2; ++i)
      if (cudaEventCreateWithFlags(&o->chain[i], cudaEventDisableTiming) != cudaSuccess) return nullptr;
  }
  return o;
}

}  // namespace

KSANA_API int ksana_dense_forward(const KsanaDenseModel* m, const KsanaDenseStep* s, const void* h_in, void* residual,
                                  int first, int last, unsigned int* epoch_io, void** out_h, int* fail_code,
                                  int* launches, cudaStream_t stream) {
  const int T = s->total_tokens, H = m->hidden;
  *fail_code = 0;
  *launches = 0;
  if (T <= 0) {
    *out_h = const_cast<void*>(h_in);
    return 0;
  }
  Exec ex;
  ex.m = m;
  ex.s = s;
  ex.residual = static_cast<char*>(residual);
  ex.epoch = epoch_io != nullptr ? epoch_io[0] : 0;
  ex.ll_seq = epoch_io != nullptr ? epoch_io[1] : 0;
  ex.launches = launches;
  ex.fail_step = ex.fail_code = 0;
  for (int i = 0; i < 8; ++i) {
    ex.sig_lane[0][i] = (m->ws > 1 && i < m->ws) ? m->sig[i] : nullptr;
    ex.sig_lane[1][i] = (m->ws > 1 && i < m->ws) ? static_cast<char*>(m->sig[i]) + static_cast<size_t>(m->sig_words) * 4
                                                 : nullptr;
  }
  const bool overlap = m->ws > 1 && s->split_seq > 0 && s->split_row > 0 && s->split_row < T && m->sig_words > 0 &&
                       m->partial != nullptr;
  OverlapStreams* os = overlap ? overlap_streams() : nullptr;
  int failed_layer = -1;
  if (overlap && os != nullptr) {
    // ---- two half-batches on two streams; kernels are issued layer by layer, alternating between the halves ----
    const int n_seq_a = s->split_seq;
    Range a{0, s->split_row, 0, s->num_prefill, s->num_prefill, s->num_decode, s->max_q_prefill, s->max_q_decode,
            s->max_kv_decode, 0, stream, static_cast<const char*>(h_in), 0};
    // the sequence list is "prefill sequences, then decode sequences"; the second half starts at sequence split_seq
    Range b{s->split_row, T - s->split_row, n_seq_a, s->num_prefill_b, n_seq_a + s->num_prefill_b, s->num_decode_b,
            s->max_q_prefill_b, s->max_q_decode_b, s->max_kv_decode_b, 1, os->side,
            static_cast<const char*>(h_in) + static_cast<size_t>(s->split_row) * H * 2, 0};
    cudaEventRecord(os->fork, stream);
    cudaStreamWaitEvent(os->side, os->fork, 0);
    ex.chain_ev[0] = os->chain[0];
    ex.chain_ev[1] = os->chain[1];
    for (int L = first; L < last && failed_layer < 0; ++L) {
      if (!ex.layer(L, a, false, 1) || !ex.layer(L, b, false, 1) || !ex.layer(L, a, false, 2) ||
          !ex.layer(L, b, false, 2))
        failed_layer = L;
    }
    ksana_gemm_set_lane(0);
    cudaEventRecord(os->join, os->side);
    cudaStreamWaitEvent(stream, os->join, 0);
    *out_h = m->hbuf[m->rank];
  } else {
    Range g{0, T, 0, s->num_prefill, s->num_prefill, s->num_decode, s->max_q_prefill, s->max_q_decode,
            s->max_kv_decode, 0, stream, static_cast<const char*>(h_in), 0};
    for (int L = first; L < last && failed_layer < 0; ++L) {
      if (!ex.layer(L, g, true)) failed_layer = L;
    }
    *out_h = const_cast<char*>(g.hcur);
  }
  if (epoch_io != nullptr) {
    epoch_io[0] = ex.epoch;
    epoch_io[1] = ex.ll_seq;
  }
  if (failed_layer >= 0) {
    *fail_code = ex.fail_code;
    return (failed_layer + 1) * 100 + ex.fail_step;
  }
  return 0;
}
