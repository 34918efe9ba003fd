// Absorbed multi-head latent attention (MLA) over the compressed latent KV cache, sm_100a (tcgen05 + TMEM + TMA).
//
// Cache row per token: [kv_lora_rank = 512 latent | 64 rope] bf16 (576 values, shared by all heads). With the
// up-projections absorbed into the query / output, every head attends with the SAME keys and values:
//   S[h, t] = q_cat[h, :576] . c[t, :576]        O[h, :512] = softmax(S)[h, :] . c[:, :512]
// so the 128 heads of a token are exactly the M = 128 rows of a tcgen05 tile. This replaces FlashMLA (sm90a only in
// the reference: 3rdparty/LLM_kernels/csrc/kernels/nvidia/flash_mla/kernels/splitkv_mla.cu, driver flash_mla.cu:113-225,
// layer src/ksana_llm/layers/nvidia/paged_mla_attention_layer.cpp:23-77; empty stubs for any other arch).
//
// One CTA = (sequence, query token, KV split, half of the 512 output dims). Per 32-token half page:
//   TMA   9 boxes of 32 tokens x 64 dims (128-byte swizzle), double buffered;
//   S     36 x tcgen05.mma 128 x 32 x 16 (K = 576), both operands K-major        -> TMEM (32 columns)
//   softmax in registers (thread r = head r), lazy rescale of O, bf16 P -> shared memory
//   O +=  2 x tcgen05.mma 128 x 256 x 16, B = the SAME shared-memory page read as an MN-major operand (columns
//         [half * 256, +256) of the latent)                                          -> TMEM (256 columns)
// The two "halves" recompute S (cheap next to keeping 512 + 32 accumulator columns, which TMEM cannot hold).
// Shared memory: Q 144 KB + 2 x 36 KB pages + 8 KB P. Splits are merged by mla_combine_kernel.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int MLA_DQK = 576, MLA_DV = 512, MLA_DVH = 256, MLA_TOK = 32, MLA_PAGE = 64;
constexpr int MLA_CHUNKS = MLA_DQK / 64;               // 9
constexpr int MLA_Q_BYTES = 128 * MLA_DQK * 2;         // 147456
constexpr int MLA_KV_BYTES = MLA_TOK * MLA_DQK * 2;    // 36864
constexpr int MLA_P_BYTES = 128 * MLA_TOK * 2;         // 8192
constexpr int MLA_OFF_KV = MLA_Q_BYTES;
constexpr int MLA_OFF_P = MLA_OFF_KV + 2 * MLA_KV_BYTES;
constexpr int MLA_OFF_BAR = MLA_OFF_P + MLA_P_BYTES;
constexpr int MLA_SMEM = MLA_OFF_BAR + 128 + 1024;

__device__ __forceinline__ uint64_t mla_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(128, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_lens, int seq_base, int h, float scale_log2, int splits, int max_q_len,
                  float* __restrict__ part_o, float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                  unsigned int* err) {
  const int half = blockIdx.z & 1;
  const int split = blockIdx.z >> 1;
  const int b = blockIdx.x + seq_base;
  const int j = blockIdx.y;  // query token within the sequence
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  if (j >= q_len) return;
  const int L = kv_lens[b];
  const int q_pos = L - q_len + j;
  const int n_ctx = q_pos + 1;                             // tokens visible to this query
  const int n_tiles_total = (n_ctx + MLA_TOK - 1) / MLA_TOK;
  const int tiles_per_split = (n_tiles_total + splits - 1) / splits;
  const int tile_begin = split * tiles_per_split;
  const int tile_end = min(tile_begin + tiles_per_split, n_tiles_total);
  const int tid = threadIdx.x, warp = tid >> 5;
  const size_t prow = ((static_cast<size_t>(blockIdx.x) * max_q_len + j) * splits + split) * h;

  if (tile_begin >= tile_end) {
    // empty split: contribute "nothing" (m = -inf) so the merge ignores it
    if (half == 0 && splits > 1 && tid < h) {
      part_ml[(prow + tid) * 2 + 0] = -INFINITY;
      part_ml[(prow + tid) * 2 + 1] = 0.f;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + MLA_OFF_KV;
  uint8_t* sP = smem + MLA_OFF_P;
  uint64_t* q_bar = reinterpret_cast<uint64_t*>(smem + MLA_OFF_BAR);
  uint64_t* kv_full = q_bar + 1;  // [2]
  uint64_t* s_done = kv_full + 2;
  uint64_t* o_done = s_done + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  if (tid == 0) {
    mbar_init(q_bar, 1);
    mbar_init(&kv_full[0], 1);
    mbar_init(&kv_full[1], 1);
    mbar_init(s_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base;            // 32 columns
  const uint32_t tmem_O = tmem_base + 64;       // 256 columns
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;

  auto load_tile = [&](int t, int stage) {
    // 32 tokens starting at token t * 32: half of one 64-token page
    const int tok0 = t * MLA_TOK;
    const int blk = bt[tok0 / MLA_PAGE];
    const int row = blk * MLA_PAGE + (tok0 % MLA_PAGE);
    mbar_expect_tx(&kv_full[stage], MLA_KV_BYTES);
#pragma unroll
    for (int c = 0; c < MLA_CHUNKS; ++c)
      tma_load_2d(sKV + stage * MLA_KV_BYTES + c * (MLA_TOK * 128), &tmKV, &kv_full[stage], c * 64, row);
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
    mbar_expect_tx(q_bar, MLA_Q_BYTES);
#pragma unroll
    for (int c = 0; c < MLA_CHUNKS; ++c)
      tma_load_2d(sQ + c * (128 * 128), &tmQ, q_bar, c * 64, (q0 + j) * h);
    load_tile(tile_begin, 0);
  }

  float m_ref = -INFINITY, l_sum = 0.f;
  int bad = 0;
  if (!mbar_wait_bounded(q_bar, 0, abort_flag, err)) bad = 1;

  for (int t = tile_begin; t < tile_end; ++t) {
    const int it = t - tile_begin;
    const int stage = it & 1;
    const uint32_t ph = (it >> 1) & 1;
    if (tid == 0 && !bad) {
      if (t + 1 < tile_end) load_tile(t + 1, stage ^ 1);
      if (mbar_wait_bounded(&kv_full[stage], ph, abort_flag, err)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, MLA_TOK, 1, 1);
#pragma unroll
        for (int k = 0; k < MLA_DQK / 16; ++k) {
          const uint32_t qa = smem_u32(sQ) + (k >> 2) * (128 * 128) + (k & 3) * 32;
          const uint32_t ka = smem_u32(sKV + stage * MLA_KV_BYTES) + (k >> 2) * (MLA_TOK * 128) + (k & 3) * 32;
          umma_f16(tmem_S, umma_desc_k128(qa), umma_desc_k128(ka), idesc, k > 0 ? 1u : 0u);
        }
        umma_commit(s_done);
      } else {
        bad = 1;
      }
    }
    if (!bad && !mbar_wait_bounded(s_done, it & 1, abort_flag, err)) bad = 1;
    if (__syncthreads_or(bad)) {
      bad = 1;
      break;
    }
    tc_fence_after();
    // ---- softmax over this tile's 32 tokens (row = head) ----
    uint32_t r[32];
    tmem_ld32(tmem_S + lane_off, r);
    tmem_wait_ld();
    float s[32];
    float m_tile = -INFINITY;
    const int tok0 = t * MLA_TOK;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      s[c] = (tok0 + c <= q_pos) ? __uint_as_float(r[c]) * scale_log2 : -INFINITY;
      m_tile = fmaxf(m_tile, s[c]);
    }
    const float m_new = fmaxf(m_ref, m_tile);
    const int want = (it > 0) && (m_new - m_ref > 8.f);
    if (it == 0) m_ref = m_new;
    if (__syncthreads_or(want)) {
      const float f = (m_new > m_ref) ? exp2f(m_ref - m_new) : 1.f;
      if (m_new > m_ref) {
        m_ref = m_new;
        l_sum *= f;
      }
#pragma unroll 1
      for (int c = 0; c < MLA_DVH / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_O + lane_off + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 32; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * f);
        tmem_st32(tmem_O + lane_off + c * 32, o);
      }
      tmem_wait_st();
    }
    float p[32];
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      p[c] = (s[c] == -INFINITY) ? 0.f : exp2f(s[c] - m_ref);
      l_sum += p[c];
    }
    // P [128 x 32] bf16 in the un-swizzled K-major operand layout: 8 x 16-byte "core matrices" stored contiguously
    // (row r, k-chunk c of 8 values -> (r / 8) * 512 + c * 128 + (r % 8) * 16)
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      uint4 o;
      o.x = pack_bf16(p[ch * 8 + 0], p[ch * 8 + 1]);
      o.y = pack_bf16(p[ch * 8 + 2], p[ch * 8 + 3]);
      o.z = pack_bf16(p[ch * 8 + 4], p[ch * 8 + 5]);
      o.w = pack_bf16(p[ch * 8 + 6], p[ch * 8 + 7]);
      *reinterpret_cast<uint4*>(sP + (tid >> 3) * 512 + ch * 128 + (tid & 7) * 16) = o;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      // A = P (un-swizzled K-major: LBO = 128 bytes between the two k-chunks of one MMA, SBO = 512 bytes between
      // 8-row groups); B = latent columns [half * 256, +256) of the page read as an MN-major operand.
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                 (static_cast<uint32_t>(MLA_DVH >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
#pragma unroll
      for (int k = 0; k < MLA_TOK / 16; ++k) {
        uint64_t da = 0;
        da |= static_cast<uint64_t>(((smem_u32(sP) + k * 256) >> 4) & 0x3FFF);
        da |= static_cast<uint64_t>(128 >> 4) << 16;
        da |= static_cast<uint64_t>(512 >> 4) << 32;
        da |= static_cast<uint64_t>(1) << 46;
        const uint32_t vb = smem_u32(sKV + stage * MLA_KV_BYTES) + (half * 4) * (MLA_TOK * 128) + k * (16 * 128);
        const uint64_t db = mla_desc_mn(vb, MLA_TOK * 128, 1024);
        umma_f16(tmem_O, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(o_done);
    }
    if (!mbar_wait_bounded(o_done, it & 1, abort_flag, err)) bad = 1;
    if (__syncthreads_or(bad)) {
      bad = 1;
      break;
    }
    tc_fence_after();
  }

  if (!bad) {
    const bool row_ok = tid < h;
    if (splits == 1) {
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = out + (static_cast<size_t>(q0 + j) * h + (row_ok ? tid : 0)) * MLA_DV + half * MLA_DVH;
#pragma unroll 1
      for (int c = 0; c < MLA_DVH / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_O + lane_off + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 32; q += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[q]) * inv, __uint_as_float(o[q + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(o[q + 2]) * inv, __uint_as_float(o[q + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(o[q + 4]) * inv, __uint_as_float(o[q + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(o[q + 6]) * inv, __uint_as_float(o[q + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + q) = v;
          }
        }
      }
    } else {
      float* prow_o = part_o + (prow + (row_ok ? tid : 0)) * MLA_DV + half * MLA_DVH;
#pragma unroll 1
      for (int c = 0; c < MLA_DVH / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_O + lane_off + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int q = 0; q < 32; q += 4)
            *reinterpret_cast<float4*>(prow_o + c * 32 + q) =
                make_float4(__uint_as_float(o[q]), __uint_as_float(o[q + 1]), __uint_as_float(o[q + 2]),
                            __uint_as_float(o[q + 3]));
        }
      }
      if (half == 0 && row_ok) {
        part_ml[(prow + tid) * 2 + 0] = m_ref;
        part_ml[(prow + tid) * 2 + 1] = l_sum;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// out[token, head, :] = sum_s w_s O_s / sum_s w_s l_s with w_s = 2^(m_s - max m). One warp per (token, head).
__global__ void mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                   const int* __restrict__ cu_q, int seq_base, int h, int splits, int max_q_len,
                                   __nv_bfloat16* __restrict__ out) {
  const int bi = blockIdx.x, j = blockIdx.y;
  const int b = bi + seq_base;
  const int q0 = cu_q[b];
  if (j >= cu_q[b + 1] - q0) return;
  const int lane = threadIdx.x & 31;
  for (int head = threadIdx.x >> 5; head < h; head += blockDim.x >> 5) {
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s)
      mm = fmaxf(mm, part_ml[((static_cast<size_t>(bi) * max_q_len + j) * splits + s) * h * 2 + head * 2]);
    float den = 0.f;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int s = 0; s < splits; ++s) {
      const size_t row = ((static_cast<size_t>(bi) * max_q_len + j) * splits + s) * h + head;
      const float ms = part_ml[row * 2];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - mm);
      den += w * part_ml[row * 2 + 1];
      const float* o = part_o + row * MLA_DV;
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] += w * o[i * 32 + lane];
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    __nv_bfloat16* dst = out + (static_cast<size_t>(q0 + j) * h + head) * MLA_DV;
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  }
}

}  // namespace ksana

using namespace ksana;

// q_cat: [T, h, 576] bf16 contiguous ([absorbed latent query | rope query]); cache: one layer
// [num_blocks, 64, 576] bf16; out: [T, h, 512] bf16 contiguous. Sequences [seq_base, seq_base + num_seqs), each
// with at most max_q_len query tokens. workspace: fp32, num_seqs * max_q_len * splits * h * (512 + 2) floats when
// the KV range is split. h <= 128.
KSANA_API int ksana_mla_decode(const void* q_cat, int total_tokens, const void* cache, int num_blocks,
                               const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens,
                               int seq_base, int num_seqs, int max_q_len, int max_kv_len, int h, float scale, void* out,
                               float* workspace, long long workspace_floats, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (h < 1 || h > 128) return -1;
  CUtensorMap tmQ, tmKV;
  if (make_tmap_2d(&tmQ, q_cat, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(total_tokens) * h, MLA_DQK,
                   MLA_DQK, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmKV, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(num_blocks) * MLA_PAGE,
                   MLA_DQK, MLA_DQK, MLA_TOK, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  static bool once = false;
  if (!once) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM) != cudaSuccess)
      return -4;
    once = true;
  }
  const int sms = sm_count();
  const int n_tiles = (max_kv_len + MLA_TOK - 1) / MLA_TOK;
  int splits = 1;
  const int base = num_seqs * max_q_len * 2;
  if (base < sms) {
    splits = (sms + base - 1) / base;
    const int max_splits = (n_tiles + 3) / 4;  // at least 4 tiles (128 tokens) per split
    if (splits > max_splits) splits = max_splits;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (splits > 1) {
    const long long rows = static_cast<long long>(num_seqs) * max_q_len * splits * h;
    if (workspace == nullptr || rows * (MLA_DV + 2) > workspace_floats) return -6;
    part_o = workspace;
    part_ml = workspace + rows * MLA_DV;
  }
  dim3 grid(num_seqs, max_q_len, splits * 2);
  mla_decode_kernel<<<grid, 128, MLA_SMEM, stream>>>(tmQ, tmKV, block_tables, max_blocks, cu_q, kv_lens, seq_base, h,
                                                     scale * 1.4426950408889634f, splits, max_q_len, part_o, part_ml,
                                                     reinterpret_cast<__nv_bfloat16*>(out), error_word());
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (splits > 1) {
    dim3 cgrid(num_seqs, max_q_len);
    mla_combine_kernel<<<cgrid, 256, 0, stream>>>(part_o, part_ml, cu_q, seq_base, h, splits, max_q_len,
                                                  reinterpret_cast<__nv_bfloat16*>(out));
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}

// cache[slot] = [latent | k_rope] (bf16). One warp per token.
__global__ void mla_cache_append_kernel(const __nv_bfloat16* __restrict__ latent, int ld_l,
                                        const __nv_bfloat16* __restrict__ k_rope, int ld_r,
                                        const int* __restrict__ slots, __nv_bfloat16* __restrict__ cache, int T, int r,
                                        int dr) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  __nv_bfloat16* dst = cache + static_cast<size_t>(slots[t]) * (r + dr);
  for (int i = lane * 2; i < r; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = *reinterpret_cast<const __nv_bfloat162*>(latent + static_cast<size_t>(t) * ld_l + i);
  for (int i = lane * 2; i < dr; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(dst + r + i) = *reinterpret_cast<const __nv_bfloat162*>(k_rope + static_cast<size_t>(t) * ld_r + i);
}

KSANA_API int ksana_mla_cache_append(const void* latent, int ld_l, const void* k_rope, int ld_r, const int* slots,
                                     void* cache, int T, int r, int dr, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((r & 1) || (dr & 1) || (ld_l & 1) || (ld_r & 1)) return -1;
  mla_cache_append_kernel<<<(T + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(latent), ld_l,
                                                           reinterpret_cast<const __nv_bfloat16*>(k_rope), ld_r, slots,
                                                           reinterpret_cast<__nv_bfloat16*>(cache), T, r, dr);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
