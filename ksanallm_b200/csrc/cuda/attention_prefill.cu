// Paged flash-attention prefill for sm_100a (tcgen05 + TMEM + TMA), causal, with prefix offset and GQA.
//
// Replaces the external flash-attn library the reference dlopen()s for multi-token requests
// (src/ksana_llm/utils/attention_backend/flash_attention_backend.cpp:197-203, 339-401; AttenVarlen,
// src/ksana_llm/kernels/nvidia/attention_kernel_wrapper.cpp:141-400) including its "gather the cached prefix back
// into contiguous K/V" step: this kernel attends directly over the pages (K/V of the new tokens were appended
// to the cache by the fused RoPE kernel), so chunked prefill and prefix-cache hits need no extra copies.
//
// One CTA = 128 query rows of one (sequence, head). Per 128-token KV tile:
//   TMA: eight 16-token pages of K and of V (block table gather), 128-byte swizzle, double buffered;
//   S = Q K^T   tcgen05.mma (128 x 128 x 16, both operands K-major from shared memory) -> TMEM (fp32);
//   softmax     thread r owns TMEM lane r: tcgen05.ld, scale/mask, running max with lazy rescale of O
//               (only when a row's max grew by more than 2^8), exp2, bf16 P written to shared memory in the
//               same swizzled K-major layout TMA would produce;
//   O += P V    tcgen05.mma (128 x D x 16; A = P K-major, B = V as MN-major operand straight from the page
//               layout [token][d]) -> TMEM.
// Epilogue: O / l, bf16, direct global stores of the valid rows.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int PF_BQ = 128;   // query rows per CTA
constexpr int PF_BKV = 128;  // kv tokens per tile
constexpr int PF_PAGE = 16;

__host__ __device__ constexpr uint32_t idesc_pv(int n) {
  // bf16 x bf16 -> f32, A K-major, B MN-major (bit 16)
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(128 >> 4) << 24);
}

// MN-major 128-byte-swizzled operand: 64 elements contiguous along MN (one 128-byte row), 8 K-rows per 1024 bytes,
// next 8 K-rows at +1024 (SBO), next 64 MN elements at +lbo_bytes (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

template <int D>
struct PrefillSmem {
  static constexpr int HALVES = D / 64;
  static constexpr int Q_BYTES = PF_BQ * D * 2;
  static constexpr int KV_BYTES = PF_BKV * D * 2;  // one K or V tile
  static constexpr int P_BYTES = PF_BQ * PF_BKV * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(128, 1)
paged_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                     const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                     const int* __restrict__ kv_lens, int seq_base, int h, int hk, float scale_log2,
                     const float* __restrict__ alibi, __nv_bfloat16* __restrict__ out, int ldo, unsigned int* err) {
  using L_ = PrefillSmem<D>;
  const int b = blockIdx.y + seq_base;
  const int head = blockIdx.z;
  const int qt = blockIdx.x;
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  if (qt * PF_BQ >= q_len) return;
  const int L = kv_lens[b];
  const int q_start = L - q_len;
  const int kh = head / (h / hk);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L_::OFF_Q;
  uint8_t* sK = smem + L_::OFF_K;
  uint8_t* sV = smem + L_::OFF_V;
  uint8_t* sP = smem + L_::OFF_P;
  uint64_t* q_bar = reinterpret_cast<uint64_t*>(smem + L_::OFF_BAR);
  uint64_t* k_full = q_bar + 1;   // [2]
  uint64_t* v_full = k_full + 2;  // [2]
  uint64_t* s_done = v_full + 2;
  uint64_t* o_done = s_done + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  constexpr uint32_t TMEM_COLS = (PF_BKV + D) <= 256 ? 256 : 512;
  if (tid == 0) {
    mbar_init(q_bar, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
    }
    mbar_init(s_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + PF_BKV;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

  const int row0 = q0 + qt * PF_BQ;
  const int q_idx = qt * PF_BQ + tid;
  const bool valid = q_idx < q_len;
  const int q_pos = valid ? q_start + q_idx : L - 1;
  const int kv_end = min(L, q_start + (qt + 1) * PF_BQ);
  const int n_tiles = (kv_end + PF_BKV - 1) / PF_BKV;
  const int n_pages = (L + PF_PAGE - 1) / PF_PAGE;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const float slope = alibi ? alibi[head] * 1.4426950408889634f : 0.f;

  auto load_kv_tile = [&](int kt, int stage) {
    // thread 0 only: 8 pages x HALVES boxes for K and for V
    mbar_expect_tx(&k_full[stage], L_::KV_BYTES);
    mbar_expect_tx(&v_full[stage], L_::KV_BYTES);
    for (int p = 0; p < PF_BKV / PF_PAGE; ++p) {
      int pg = kt * (PF_BKV / PF_PAGE) + p;
      if (pg >= n_pages) pg = n_pages - 1;  // finite filler; those columns are masked to p = 0
      const int blk = bt[pg];
      const int krow = ((blk * 2 + 0) * hk + kh) * PF_PAGE;
      const int vrow = ((blk * 2 + 1) * hk + kh) * PF_PAGE;
#pragma unroll
      for (int hf = 0; hf < L_::HALVES; ++hf) {
        tma_load_2d(sK + stage * L_::KV_BYTES + hf * (PF_BKV * 128) + p * (PF_PAGE * 128), &tmKV, &k_full[stage],
                    hf * 64, krow);
        tma_load_2d(sV + stage * L_::KV_BYTES + hf * (PF_BKV * 128) + p * (PF_PAGE * 128), &tmKV, &v_full[stage],
                    hf * 64, vrow);
      }
    }
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
    mbar_expect_tx(q_bar, L_::Q_BYTES);
#pragma unroll
    for (int hf = 0; hf < L_::HALVES; ++hf)
      tma_load_2d(sQ + hf * (PF_BQ * 128), &tmQ, q_bar, head * D + hf * 64, row0);
    load_kv_tile(0, 0);
  }

  float m_ref = -INFINITY;  // max used as exponent reference (log2 domain, already scaled)
  float l_sum = 0.f;
  int bad = 0;

  if (!mbar_wait_bounded(q_bar, 0, abort_flag, err)) bad = 1;

  for (int kt = 0; kt < n_tiles; ++kt) {
    const int stage = kt & 1;
    const uint32_t ph = (kt >> 1) & 1;
    if (tid == 0 && !bad) {
      if (kt + 1 < n_tiles) load_kv_tile(kt + 1, stage ^ 1);
      if (mbar_wait_bounded(&k_full[stage], ph, abort_flag, err)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, PF_BKV, 1, 1);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * (PF_BQ * 128) + (k & 3) * 32;
          umma_f16(tmem_S, umma_desc_k128(smem_u32(sQ) + off),
                   umma_desc_k128(smem_u32(sK + stage * L_::KV_BYTES) + off), idesc, k > 0 ? 1u : 0u);
        }
        umma_commit(s_done);
      } else {
        bad = 1;
      }
    }
    if (!bad && !mbar_wait_bounded(s_done, kt & 1, abort_flag, err)) bad = 1;
    if (__syncthreads_or(bad)) {
      bad = 1;
      break;
    }
    tc_fence_after();

    // ---- pass 1: row max of the masked, scaled scores ----
    const int kv0 = kt * PF_BKV;
    float m_tile = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < PF_BKV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_S + lane_off + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = kv0 + c * 32 + j;
        float s = __uint_as_float(r[j]) * scale_log2 + slope * static_cast<float>(kpos - q_pos);
        if (kpos > q_pos) s = -INFINITY;
        m_tile = fmaxf(m_tile, s);
      }
    }
    const float m_new = fmaxf(m_ref, m_tile);
    // lazy rescale: exponents stay relative to m_ref until some row's max has grown by more than 8 (x256)
    const int want = (kt > 0) && (m_new - m_ref > 8.f);
    if (kt == 0) m_ref = m_new;
    if (__syncthreads_or(want)) {
      const float f = (m_new > m_ref) ? exp2f(m_ref - m_new) : 1.f;
      if (m_new > m_ref) {
        m_ref = m_new;
        l_sum *= f;
      }
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_O + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
        tmem_st32(tmem_O + lane_off + c * 32, r);
      }
      tmem_wait_st();
    }
    // ---- pass 2: P = exp2(S - m_ref) -> bf16 -> shared memory (swizzled K-major), row sums ----
#pragma unroll 1
    for (int c = 0; c < PF_BKV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_S + lane_off + c * 32, r);
      tmem_wait_ld();
      float p[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = kv0 + c * 32 + j;
        float s = __uint_as_float(r[j]) * scale_log2 + slope * static_cast<float>(kpos - q_pos);
        p[j] = (kpos > q_pos) ? 0.f : exp2f(s - m_ref);
        l_sum += p[j];
      }
      // 32 columns = 4 chunks of 8 bf16 (16 bytes); column c*32 + j lives in half (c >> 1), chunk ((c & 1) * 4 + j / 8)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 o;
        o.x = pack_bf16(p[ch * 8 + 0], p[ch * 8 + 1]);
        o.y = pack_bf16(p[ch * 8 + 2], p[ch * 8 + 3]);
        o.z = pack_bf16(p[ch * 8 + 4], p[ch * 8 + 5]);
        o.w = pack_bf16(p[ch * 8 + 6], p[ch * 8 + 7]);
        const int chunk = (c & 1) * 4 + ch;
        uint8_t* dst = sP + (c >> 1) * (PF_BQ * 128) + tid * 128 + ((chunk ^ (tid & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = o;
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      if (mbar_wait_bounded(&v_full[stage], ph, abort_flag, err)) {
        tc_fence_after();
        constexpr uint32_t idesc = idesc_pv(D);
#pragma unroll
        for (int k = 0; k < PF_BKV / 16; ++k) {
          const uint64_t da = umma_desc_k128(smem_u32(sP) + (k >> 2) * (PF_BQ * 128) + (k & 3) * 32);
          const uint64_t db = umma_desc_mn128(smem_u32(sV + stage * L_::KV_BYTES) + k * (16 * 128), PF_BKV * 128);
          umma_f16(tmem_O, da, db, idesc, (kt > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(o_done);
      } else {
        bad = 1;
      }
    }
    if (!bad && !mbar_wait_bounded(o_done, kt & 1, abort_flag, err)) bad = 1;
    if (__syncthreads_or(bad)) {
      bad = 1;
      break;
    }
    tc_fence_after();
  }

  if (!bad) {
    // tcgen05.ld is warp-collective: all lanes load, only rows inside the sequence store
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
    __nv_bfloat16* orow = out + static_cast<size_t>(q0 + (valid ? q_idx : 0)) * ldo + head * D;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_O + lane_off + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o;
        o.x = pack_bf16(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
        o.y = pack_bf16(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
        o.z = pack_bf16(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
        o.w = pack_bf16(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
        if (valid) *reinterpret_cast<uint4*>(orow + c * 32 + j) = o;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace ksana

using namespace ksana;

// Prefill attention for sequences [seq_base, seq_base + num_seqs) (each with q_len <= max_q_len new tokens whose
// K/V are already in the cache). q: [T, h, d] bf16 (token pitch ldq elements, multiple of 8); cache: one layer
// [num_blocks][2][hk][16][d] bf16; out: [T, h, d] bf16 (token pitch ldo, multiple of 8). total_tokens = T.
KSANA_API int ksana_paged_prefill(const void* q, int ldq, int total_tokens, const void* cache, int num_blocks,
                                  const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens,
                                  int seq_base, int num_seqs, int max_q_len, int h, int hk, int d, int block_size,
                                  float scale, const float* alibi, void* out, int ldo, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if ((d != 128 && d != 64) || block_size != PF_PAGE || h % hk != 0 || (ldq & 7) || (ldo & 7)) return -1;
  CUtensorMap tmQ, tmKV;
  if (make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_tokens, static_cast<uint64_t>(h) * d, ldq, PF_BQ,
                   64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmKV, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   static_cast<uint64_t>(num_blocks) * 2 * hk * PF_PAGE, d, d, PF_PAGE, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  dim3 grid((max_q_len + PF_BQ - 1) / PF_BQ, num_seqs, h);
  const float scale_log2 = scale * 1.4426950408889634f;
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  if (d == 128) {
    auto kern = paged_prefill_kernel<128>;
    if (KSANA_SMEM_ONCE(kern, PrefillSmem<128>::TOTAL) != 0) return -4;
    kern<<<grid, 128, PrefillSmem<128>::TOTAL, stream>>>(tmQ, tmKV, block_tables, max_blocks, cu_q, kv_lens, seq_base, h,
                                                         hk, scale_log2, alibi, O, ldo, error_word());
  } else {
    auto kern = paged_prefill_kernel<64>;
    if (KSANA_SMEM_ONCE(kern, PrefillSmem<64>::TOTAL) != 0) return -4;
    kern<<<grid, 128, PrefillSmem<64>::TOTAL, stream>>>(tmQ, tmKV, block_tables, max_blocks, cu_q, kv_lens, seq_base, h,
                                                        hk, scale_log2, alibi, O, ldo, error_word());
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
