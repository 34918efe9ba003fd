// Native forward pass of the dense decoder stack (Llama / Qwen family blocks: RMSNorm, fused-QKV attention with RoPE
// over the paged cache, gated FFN), driven from ONE call per step. Declared here so that the Python side can mirror
// the structs with ctypes.
#pragma once
#include <cuda_runtime.h>

extern "C" {

struct KsanaDenseLayer {
  const void* wqkv;     // [(h + 2 hk) d, H] bf16
  const void* bqkv;     // optional bias [(h + 2 hk) d]
  const void* wo;       // [H, h d]
  const void* ln2;      // post-attention RMSNorm weight [H]
  const void* wgu;      // [2 I, H] gate rows then up rows
  const void* wdown;    // [H, I]
  const void* next_ln;  // the norm applied after this layer's FFN: next layer's input norm, or the final norm
  const void* q_norm;   // optional per-head RMSNorm weights [d]
  const void* k_norm;
  void* kv_cache;       // [num_blocks, 2, hk, block_size, d]
  // 128 x 128 block scales (fp32, [ceil(N / 128), K / 128]) of the four weights when they are e4m3; all null: bf16
  const float* sqkv;
  const float* so;
  const float* sgu;
  const float* sdown;
  // the same scales as packed power-of-two bytes for the scaled tensor-core GEMM (gemm_mxf8.cu); null: not available
  const void* fqkv;
  const void* fo;
  const void* fgu;
  const void* fdown;
  // optional copy of wgu with gate / up rows interleaved in groups of 16: prefill-sized steps then run the gated FFN's
  // first GEMM with the SiLU-mul epilogue (ksana_gemm_bf16_swiglu) instead of GEMM + activation kernel
  const void* wgu_il;
};

struct KsanaDenseModel {
  int hidden, heads, kv_heads, head_dim, inter;  // per-rank heads and FFN width
  int n_layers;
  float eps;
  int rotary_dim, rope_interleaved;
  int block_size, num_blocks, kv_kind;  // kv_kind 0 bf16, 1 fp8 e4m3
  float attn_scale, k_scale, v_scale;
  const float* rope_cache;  // [max_pos, rotary_dim] cos | sin, or null
  // tensor parallel (ws == 1: everything below up to comm_ctas is ignored)
  int rank, ws, rows_cap, comm_ctas;
  void* const* recv;
  void* const* hbuf;
  void* const* sig;
  void* hbuf_mc;
  void* const* partial;  // two-kernel path: GEMM into this rank's symmetric `partial`, then the reduce/norm/gather kernel
  void* partial_mc;
  int two_kernel_max_tokens;  // steps with at most this many tokens take the two-kernel path (0: never)
  // decode-sized steps: word-flagged single-kernel path (gemm_ll_fused.cu); ll_max_tokens 0 switches it off
  void* const* ll_recv;
  void* const* ll_recv2;
  void* ll_recv2_mc;
  long long ll_half_words;  // 8-byte words of one hop-1 buffer half (one-hop mode alternates between two halves)
  int ll_rows_cap, ll_max_tokens, ll_one_shot;
  // scratch, all sized for max_tokens rows
  void* qkv_buf;   // [T, (h + 2 hk) d]
  void* attn_buf;  // [T, h d]
  void* gu_buf;    // [T, 2 I]
  void* act_buf;   // [T, I]
  void* proj_buf;  // [T, H]   (ws == 1)
  void* h_buf[2];  // [T, H]   (ws == 1) normalised activations, ping-pong
  float* gemm_ws;
  long long gemm_ws_floats;
  unsigned int* gemm_counters;
  int n_counters;
  float* attn_ws;
  long long attn_ws_floats;
  int sig_words;  // uint32 words of one flag region in `sig`; the second half-batch uses the region after the first
  // fp8 weights: the activations of each GEMM are quantised (e4m3, one scale per token per 128 channels) into these
  void* a8_buf;   // [T, a8_cols] bytes
  float* sa_buf;  // [T + 256, a8_cols / 128]: fp32 scales, or the packed scale bytes of the scaled tensor-core GEMM
  int a8_cols;    // max(H, h d, I)
  int fp8_pow2;     // the weights' block scales are powers of two: activations get power-of-two group scales
  int mx_min_rows;  // products with at least this many rows (and packed weight scales) take the scaled GEMM
  const KsanaDenseLayer* layers;
};

struct KsanaDenseStep {
  const int* positions;
  const int* slot_mapping;
  const int* block_tables;
  const int* cu_q;
  const int* kv_lens;
  int total_tokens, num_prefill, num_decode, max_blocks;
  int max_q_prefill, max_q_decode, max_kv_decode;
  // Two-batch overlap (tensor parallel, prefill-sized steps): when split_seq > 0 the step's sequences [0, split_seq)
  // (rows [0, split_row)) and [split_seq, n) (rows [split_row, total_tokens)) run as two independent half-batches on
  // two streams, so the NVLink collectives of one half overlap the GEMMs and attention of the other. The halves
  // hold different sequences, so they never read each other's rows or cache blocks. The maxima of the second half
  // follow; the fields above then describe the first half.
  int split_seq, split_row;
  int num_prefill_b, num_decode_b, max_q_prefill_b, max_q_decode_b, max_kv_decode_b;
};

// h: normalised input of layer `first` ([T, H] bf16; for ws > 1 it may be any buffer), residual: [T, H] running
// residual stream (updated in place; row-sharded across ranks when ws > 1). Runs layers [first, last). *epoch_io: the
// last collective epoch used on the shared buffers (ws > 1); two more are consumed per layer (0 is skipped) and the
// last one used is written back; epoch_io[1] counts the small-step calls (selects the buffer half) the same way.
// *out_h receives the pointer of the normalised output
// (one of the scratch buffers or this rank's hbuf). Returns 0, or (layer + 1) * 100 + step on failure with
// *fail_code holding the failing call's code. Has no counterpart in the reference (its per-layer C++ forward is
// CommonModel::LayerForward, src/ksana_llm/models/common/common_model.cpp).
int ksana_dense_forward(const KsanaDenseModel* m, const KsanaDenseStep* s, const void* h, void* residual, int first,
                        int last, unsigned int* epoch_io, void** out_h, int* fail_code, int* launches,
                        cudaStream_t stream);
}
