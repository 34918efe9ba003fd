// Absorbed multi-head latent attention (MLA) over the compressed latent KV cache, sm_100a (tcgen05 + TMEM + TMA).
//
// Cache row per token: [kv_lora_rank = 512 latent | 64 rope] bf16 (576 values, shared by all heads). With the
// up-projections absorbed into the query / output, every head attends with the SAME keys and values:
//   S[h, t] = q_cat[h, :576] . c[t, :576]        O[h, :512] = softmax(S)[h, :] . c[:, :512]
// so the 128 heads of a token are exactly the M = 128 rows of a tcgen05 tile. This replaces FlashMLA (sm90a only in
// the reference: 3rdparty/LLM_kernels/csrc/kernels/nvidia/flash_mla/kernels/splitkv_mla.cu, driver flash_mla.cu:113-225,
// layer src/ksana_llm/layers/nvidia/paged_mla_attention_layer.cpp:23-77; empty stubs for any other arch).
//
// One CTA = (sequence, query token, KV split, half of the 512 output dims), 320 threads:
//   warps 0-7  softmax: thread (g, r) owns head r and the tokens [g * 64, +64) of the tile (g = warp / 4)
//   warp 8     TMA producer, warp 9 MMA issuer (one lane each)
// Per tile of 128 tokens = 2 pages:
//   TMA   18 boxes of 64 tokens x 64 dims (128-byte swizzle) into 9 chunk slots of 16 KB. The slots are single
//         buffered but refilled as they die: the 5 chunks only S needs (the other half's latent + rope) right after
//         S(t), the 4 chunks that are this half's V after PV(t); S(t+1) consumes chunks in that same order.
//   S     36 x tcgen05.mma 128 x 128 x 16 (K = 576): query chunks 0-3 are the A operand FROM TMEM (written once per
//         CTA), chunks 4-8 come from shared memory                                      -> TMEM (128 columns)
//   softmax in registers, lazy rescale of O, bf16 P written back over S in TMEM (64 columns)
//   O +=  8 x tcgen05.mma 128 x 256 x 16, A = P from TMEM, B = the SAME shared-memory chunks read as an MN-major
//         operand (columns [half * 256, +256) of the latent)                            -> TMEM (256 columns)
// An MMA of M = 128, K = 16 costs ~62 cycles for any N <= 128 (45 with A in TMEM), so the token tile is 128 wide and Q
// lives in TMEM as far as its 512 columns allow: O 256 | S/P 128 | Q 128. The two "halves" recompute S (TMEM cannot
// hold 512 + 128 accumulator columns). Shared memory: Q 80 KB + 144 KB of KV. Splits are merged by mla_combine_kernel.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int MLA_DQK = 576, MLA_DV = 512, MLA_DVH = 256, MLA_TOK = 128, MLA_PAGE = 64;
constexpr int MLA_CHUNKS = MLA_DQK / 64;               // 9
constexpr int MLA_QT = 4;                              // query chunks held in TMEM
constexpr int MLA_QS = MLA_CHUNKS - MLA_QT;            // query chunks in shared memory
constexpr int MLA_Q_BYTES = 128 * 128 * MLA_QS;        // 81920
constexpr int MLA_SLOT = MLA_TOK * 128;                // one chunk of a tile: 128 tokens x 64 dims, 16 KB
constexpr int MLA_KV_BYTES = MLA_CHUNKS * MLA_SLOT;    // 147456
constexpr int MLA_OFF_KV = MLA_Q_BYTES;
constexpr int MLA_OFF_BAR = MLA_OFF_KV + MLA_KV_BYTES;
constexpr int MLA_OFF_X = MLA_OFF_BAR + 128;           // 2 x 256 floats of row max / sum exchange, then 4 vote words
constexpr int MLA_USED = MLA_OFF_X + 2048 + 64;        // 231616
constexpr int MLA_SMEM = 232448;                       // the whole 227 KB: at most 832 bytes of alignment padding
constexpr int MLA_TM_O = 0, MLA_TM_S = 256, MLA_TM_Q = 384;  // TMEM columns
constexpr int MLA_THREADS = 320;

__device__ __forceinline__ uint64_t mla_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ void mla_bar_softmax() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// chunk processed at position i of a tile: first the 5 chunks only S reads, then this half's 4 V chunks
__device__ __forceinline__ int mla_chunk_at(int i, int half) {
  if (i < 4) return (1 - half) * 4 + i;
  if (i == 4) return 8;
  return half * 4 + (i - 5);
}

__global__ void __launch_bounds__(MLA_THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                  const __nv_bfloat16* __restrict__ q_cat, int total_rows, const int* __restrict__ block_tables,
                  int max_blocks, const int* __restrict__ cu_q, const int* __restrict__ kv_lens, int seq_base, int h,
                  float scale_log2, int splits, int max_q_len, float* __restrict__ part_o,
                  float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, unsigned int* err,
                  long long* __restrict__ trace) {
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
  const int n_pages = (n_ctx + MLA_PAGE - 1) / MLA_PAGE;
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
  if ((smem - smem_raw) + MLA_USED > MLA_SMEM) {  // uniform over the CTA: nothing has been set up yet
    if (tid == 0) atomicOr(err, KERR_BAD_SHAPE);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + MLA_OFF_KV;
  uint64_t* q_bar = reinterpret_cast<uint64_t*>(smem + MLA_OFF_BAR);
  uint64_t* kv_full = q_bar + 1;            // [9], one per chunk slot
  uint64_t* s_done = kv_full + MLA_CHUNKS;
  uint64_t* o_done = s_done + 1;
  uint64_t* p_ready = o_done + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(p_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* xch = reinterpret_cast<float*>(smem + MLA_OFF_X);              // [2][256] row max / row sum exchange
  volatile int* bad_vote = reinterpret_cast<volatile int*>(xch + 512);  // [3] rotating per tile + [1] final

  if (tid == 0) {
    mbar_init(q_bar, 1);
    for (int c = 0; c < MLA_CHUNKS; ++c) mbar_init(&kv_full[c], 1);
    mbar_init(s_done, 1);
    mbar_init(o_done, 1);
    mbar_init(p_ready, 8);
    *abort_flag = 0;
    bad_vote[0] = bad_vote[1] = bad_vote[2] = bad_vote[3] = 0;
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
  const uint32_t tmem_O = tmem_base + MLA_TM_O;
  const uint32_t tmem_S = tmem_base + MLA_TM_S;
  const uint32_t tmem_Q = tmem_base + MLA_TM_Q;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int n_it = tile_end - tile_begin;
#define MLA_TRACE(slot, who)                                                                                   \
  if (trace != nullptr && tid == (who) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && it < 16)   \
    trace[it * 8 + (slot)] = clock64();

  // ================= softmax warps =================
  const int g = (tid >> 7) & 1;                     // token half of the tile (warps 0-3: 0, warps 4-7: 1)
  const int r = tid & 127;                          // head
  const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
  float m_ref = -INFINITY, l_sum = 0.f;
  int bad = 0;
  if (warp < 8) {
    // query chunks 0-3 -> TMEM as packed bf16 pairs: thread (g, r) writes chunks 2g and 2g + 1 of head r
    const int grow = (q0 + j) * h + r;
    const bool ok = r < h && grow < total_rows;
    const uint4* src = reinterpret_cast<const uint4*>(q_cat + static_cast<size_t>(ok ? grow : 0) * MLA_DQK);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int c = 2 * g + cc;
      uint32_t v[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint4 u = make_uint4(0u, 0u, 0u, 0u);
        if (ok) u = src[c * 8 + i];
        v[4 * i] = u.x;
        v[4 * i + 1] = u.y;
        v[4 * i + 2] = u.z;
        v[4 * i + 3] = u.w;
      }
      tmem_st32(tmem_Q + lane_off + c * 32, v);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();  // Q is in TMEM: the MMA issuer's first tcgen05.mma comes after this barrier
  tc_fence_after();

  if (warp == 8) {
    // ================= TMA producer =================
    if ((tid & 31) == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmKV);
      mbar_expect_tx(q_bar, MLA_Q_BYTES);
#pragma unroll
      for (int c = 0; c < MLA_QS; ++c)
        tma_load_2d(sQ + c * (128 * 128), &tmQ, q_bar, (MLA_QT + c) * 64, (q0 + j) * h);
      auto load_chunk = [&](int t, int c) {
        // rows 0-63 of the slot: page 2t, rows 64-127: page 2t + 1 (past the context: any valid page, masked later)
        const int p0 = 2 * t, p1 = (2 * t + 1 < n_pages) ? 2 * t + 1 : 2 * t;
        mbar_expect_tx(&kv_full[c], MLA_SLOT);
        tma_load_2d(sKV + c * MLA_SLOT, &tmKV, &kv_full[c], c * 64, bt[p0] * MLA_PAGE);
        tma_load_2d(sKV + c * MLA_SLOT + MLA_PAGE * 128, &tmKV, &kv_full[c], c * 64, bt[p1] * MLA_PAGE);
      };
      for (int i = 0; i < MLA_CHUNKS; ++i) load_chunk(tile_begin, mla_chunk_at(i, half));
      for (int it = 0; it + 1 < n_it; ++it) {
        const int t = tile_begin + it;
        if (!mbar_wait_bounded(s_done, it & 1, abort_flag, err)) break;
        for (int i = 0; i < 5; ++i) load_chunk(t + 1, mla_chunk_at(i, half));
        if (!mbar_wait_bounded(o_done, it & 1, abort_flag, err)) break;
        for (int i = 5; i < MLA_CHUNKS; ++i) load_chunk(t + 1, mla_chunk_at(i, half));
      }
    }
  } else if (warp == 9) {
    // ================= MMA issuer =================
    if ((tid & 31) == 0) {
      bool ok = mbar_wait_bounded(q_bar, 0, abort_flag, err);
      // Q chunks 0-3 were written to TMEM by the softmax warps before the CTA-wide barrier above
      for (int it = 0; ok && it < n_it; ++it) {
        constexpr uint32_t idesc_s = umma_idesc(128, MLA_TOK, 1, 1);
        MLA_TRACE(0, 288)
        for (int i = 0; ok && i < MLA_CHUNKS; ++i) {
          const int c = mla_chunk_at(i, half);
          if (!mbar_wait_bounded(&kv_full[c], it & 1, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t kvb = smem_u32(sKV + c * MLA_SLOT);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t kb = umma_desc_k128(kvb + k * 32);
            const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
            if (c < MLA_QT) {
              umma_f16_ts(tmem_S, tmem_Q + c * 32 + k * 8, kb, idesc_s, acc);
            } else {
              umma_f16(tmem_S, umma_desc_k128(smem_u32(sQ) + (c - MLA_QT) * (128 * 128) + k * 32), kb, idesc_s, acc);
            }
          }
        }
        if (!ok) break;
        umma_commit(s_done);
        MLA_TRACE(1, 288)
        if (!mbar_wait_bounded(p_ready, it & 1, abort_flag, err)) break;
        MLA_TRACE(2, 288)
        tc_fence_after();
        // A = P from TMEM (8 columns per 16 tokens); B = latent columns [half * 256, +256) of the tile, MN-major.
        constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                     (static_cast<uint32_t>(MLA_DVH >> 3) << 17) |
                                     (static_cast<uint32_t>(128 >> 4) << 24);
#pragma unroll
        for (int k = 0; k < MLA_TOK / 16; ++k) {
          const uint32_t vb = smem_u32(sKV) + (half * 4) * MLA_SLOT + k * (16 * 128);
          umma_f16_ts(tmem_O, tmem_S + k * 8, mla_desc_mn(vb, MLA_SLOT, 1024), idesc_o, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(o_done);
        MLA_TRACE(3, 288)
      }
    }
  }


  if (warp < 8) {
    for (int it = 0; it < n_it; ++it) {
      const int t = tile_begin + it;
      if (!mbar_wait_bounded(s_done, it & 1, abort_flag, err)) bad = 1;
      tc_fence_after();
      MLA_TRACE(4, 0)
      const int tok0 = t * MLA_TOK + g * 64;
      float s[64];
      float m_tile = -INFINITY;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t raw[32];
        tmem_ld32(tmem_S + lane_off + g * 64 + q * 32, raw);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float v = (tok0 + q * 32 + c <= q_pos) ? __uint_as_float(raw[c]) * scale_log2 : -INFINITY;
          s[q * 32 + c] = v;
          m_tile = fmaxf(m_tile, v);
        }
      }
      // both token halves of a row agree on the tile maximum; every S read of the tile happens before this barrier
      xch[(it & 1) * 256 + g * 128 + r] = m_tile;
      if (bad) bad_vote[it % 3] = 1;
      mla_bar_softmax();
      m_tile = fmaxf(m_tile, xch[(it & 1) * 256 + (1 - g) * 128 + r]);
      // the vote slot of tile it + 2 is cleared here: its writers are past the NEXT barrier, its last readers
      // (tile it - 1) arrived at THIS barrier after reading it
      if (tid == 0) bad_vote[(it + 2) % 3] = 0;
      if (bad_vote[it % 3]) {
        bad = 1;
        break;
      }
      const float m_new = fmaxf(m_ref, m_tile);
      const bool want = (it > 0) && (m_new - m_ref > 8.f);
      if (it == 0) m_ref = m_new;
      if (__any_sync(0xffffffffu, want)) {
        // s_done(t) also covers PV(t - 1): O is stable. This thread rescales its 128 of the 256 columns.
        const float f = (m_new > m_ref) ? exp2f(m_ref - m_new) : 1.f;
        if (m_new > m_ref) {
          m_ref = m_new;
          l_sum *= f;
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_O + lane_off + g * 128 + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 32; ++q) o[q] = __float_as_uint(__uint_as_float(o[q]) * f);
          tmem_st32(tmem_O + lane_off + g * 128 + c * 32, o);
        }
      }
      MLA_TRACE(5, 0)
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float p0 = (s[2 * c] == -INFINITY) ? 0.f : exp2f(s[2 * c] - m_ref);
          const float p1 = (s[2 * c + 1] == -INFINITY) ? 0.f : exp2f(s[2 * c + 1] - m_ref);
          l_sum += p0 + p1;
          pk[c] = pack_bf16(p0, p1);
        }
        tmem_st32(tmem_S + lane_off + g * 32, pk);
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(p_ready);  // one arrival per warp
      MLA_TRACE(6, 0)
    }
    // every softmax thread leaves the loop at the same iteration (uniform votes), so the named barrier stays balanced
    if (!bad && !mbar_wait_bounded(o_done, (n_it - 1) & 1, abort_flag, err)) bad = 1;
    tc_fence_after();
    xch[(n_it & 1) * 256 + g * 128 + r] = l_sum;
    if (bad) bad_vote[3] = 1;
    mla_bar_softmax();
    l_sum += xch[(n_it & 1) * 256 + (1 - g) * 128 + r];
    if (bad_vote[3]) bad = 1;

    if (!bad) {
      const bool row_ok = r < h;
      if (splits == 1) {
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        __nv_bfloat16* orow = out + (static_cast<size_t>(q0 + j) * h + (row_ok ? r : 0)) * MLA_DV + half * MLA_DVH +
                              g * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_O + lane_off + g * 128 + c * 32, o);
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
        float* prow_o = part_o + (prow + (row_ok ? r : 0)) * MLA_DV + half * MLA_DVH + g * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_O + lane_off + g * 128 + c * 32, o);
          tmem_wait_ld();
          if (row_ok) {
#pragma unroll
            for (int q = 0; q < 32; q += 4)
              *reinterpret_cast<float4*>(prow_o + c * 32 + q) =
                  make_float4(__uint_as_float(o[q]), __uint_as_float(o[q + 1]), __uint_as_float(o[q + 2]),
                              __uint_as_float(o[q + 3]));
          }
        }
        if (half == 0 && g == 0 && row_ok) {
          part_ml[(prow + r) * 2 + 0] = m_ref;
          part_ml[(prow + r) * 2 + 1] = l_sum;
        }
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
  const int head = blockIdx.z * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= h) return;
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

}  // namespace ksana

using namespace ksana;

static long long* g_mla_trace = nullptr;
// Debug hook: 128 int64 slots receiving CTA 0's phase timeline (nullptr switches it off).
KSANA_API void ksana_mla_set_trace(void* buf) { g_mla_trace = reinterpret_cast<long long*>(buf); }

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
                   MLA_DQK, MLA_DQK, MLA_PAGE, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (reinterpret_cast<uintptr_t>(q_cat) & 15) return -1;
  if (KSANA_SMEM_ONCE(mla_decode_kernel, MLA_SMEM) != 0) return -4;
  const int sms = sm_count();
  const int n_tiles = (max_kv_len + MLA_TOK - 1) / MLA_TOK;
  // KV splits by a wave-count model: time ~ waves * (tiles per split + fixed per-CTA cost) (+ the merge when split)
  int splits = 1;
  {
    const int base = num_seqs * max_q_len * 2;
    float best = 1e30f;
    for (int sp = 1; sp <= 32 && sp <= n_tiles; ++sp) {
      if (sp > 1 && (base >= sms || workspace == nullptr ||
                     static_cast<long long>(num_seqs) * max_q_len * sp * h * (MLA_DV + 2) > workspace_floats))
        break;
      const int waves = (base * sp + sms - 1) / sms;
      const float cost = waves * ((n_tiles + sp - 1) / sp + 1.5f) + (sp > 1 ? 1.0f : 0.f);
      if (cost < best - 1e-3f) {
        best = cost;
        splits = sp;
      }
    }
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
  mla_decode_kernel<<<grid, MLA_THREADS, MLA_SMEM, stream>>>(
      tmQ, tmKV, reinterpret_cast<const __nv_bfloat16*>(q_cat), total_tokens * h, block_tables, max_blocks, cu_q, kv_lens,
      seq_base, h, scale * 1.4426950408889634f, splits, max_q_len, part_o, part_ml,
      reinterpret_cast<__nv_bfloat16*>(out), error_word(), g_mla_trace);
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (splits > 1) {
    dim3 cgrid(num_seqs, max_q_len, (h + 7) / 8);
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

// ---- fused MLA RoPE + cache append ---------------------------------------------------------------------------------
// One launch replaces the PyTorch rotary ops of the MLA layer and the separate cache append (reference:
// src/ksana_llm/modules/attention/multihead_latent_attention.cpp:276-284 rotary + FlashMLA cache copy):
//   warps 0 .. T*h-1 : rotate the rope part of query (token, head) and write it behind the absorbed latent query in
//                      q_cat[token][head][r .. r + dr) (the attention kernel reads [latent | rope] rows);
//   warps T*h ..     : rotate the token's shared rope key and write cache[slot] = [latent | rotated key] (the cache row
//                      may be wider: extra columns, e.g. an indexer key, are left alone).
// cos_sin: [max_pos, dr] = [cos(dr/2) | sin(dr/2)] fp32 rows. Pairs are (i, i + dr/2), or (2i, 2i + 1) when interleaved.
namespace ksana {

__global__ void __launch_bounds__(256)
mla_rope_append_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, int q_head_stride, int dn,
                       __nv_bfloat16* __restrict__ q_cat, const __nv_bfloat16* __restrict__ k_rope, int ld_k,
                       const __nv_bfloat16* __restrict__ latent, int ld_l, const int* __restrict__ positions,
                       const float* __restrict__ cos_sin, const int* __restrict__ slots,
                       __nv_bfloat16* __restrict__ cache, int cache_width, int T, int h, int r, int dr,
                       int interleaved) {
  const long long gw = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int half = dr >> 1;
  if (gw < static_cast<long long>(T) * h) {
    const int t = static_cast<int>(gw / h), hd = static_cast<int>(gw - static_cast<long long>(t) * h);
    const __nv_bfloat16* src = q + static_cast<size_t>(t) * q_row_stride + static_cast<size_t>(hd) * q_head_stride + dn;
    __nv_bfloat16* dst = q_cat + (static_cast<size_t>(t) * h + hd) * (r + dr) + r;
    const float* cs = cos_sin + static_cast<size_t>(positions[t]) * dr;
    for (int i = lane; i < half; i += 32) {
      const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
      const float a = __bfloat162float(src[i0]), b = __bfloat162float(src[i1]);
      const float c = cs[i], s = cs[half + i];
      dst[i0] = __float2bfloat16(a * c - b * s);
      dst[i1] = __float2bfloat16(b * c + a * s);
    }
    return;
  }
  const long long kt = gw - static_cast<long long>(T) * h;
  if (kt >= T) return;
  const int t = static_cast<int>(kt);
  __nv_bfloat16* row = cache + static_cast<size_t>(slots[t]) * cache_width;
  for (int i = lane * 2; i < r; i += 64)
    *reinterpret_cast<__nv_bfloat162*>(row + i) =
        *reinterpret_cast<const __nv_bfloat162*>(latent + static_cast<size_t>(t) * ld_l + i);
  const __nv_bfloat16* ksrc = k_rope + static_cast<size_t>(t) * ld_k;
  const float* cs = cos_sin + static_cast<size_t>(positions[t]) * dr;
  for (int i = lane; i < half; i += 32) {
    const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(ksrc[i0]), b = __bfloat162float(ksrc[i1]);
    const float c = cs[i], s = cs[half + i];
    row[r + i0] = __float2bfloat16(a * c - b * s);
    row[r + i1] = __float2bfloat16(b * c + a * s);
  }
}

}  // namespace ksana

// q: projected queries, element (t, head, j) at q + t * q_row_stride + head * q_head_stride + j with the rope part at
// j in [dn, dn + dr); q_cat: [T, h, r + dr] contiguous (its [.., :r] part is written by the absorb GEMM); k_rope:
// [T, dr] (pitch ld_k); latent: [T, r] (pitch ld_l); cache: rows of cache_width >= r + dr elements; r, ld_l even.
KSANA_API int ksana_mla_rope_append(const void* q, long long q_row_stride, int q_head_stride, int dn, void* q_cat,
                                    const void* k_rope, int ld_k, const void* latent, int ld_l, const int* positions,
                                    const float* cos_sin, const int* slots, void* cache, int cache_width, int T, int h,
                                    int r, int dr, int interleaved, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((r & 1) || (dr & 1) || (ld_l & 1) || cache_width < r + dr || (cache_width & 1)) return -1;
  const long long warps = static_cast<long long>(T) * h + T;
  ksana::mla_rope_append_kernel<<<static_cast<unsigned int>((warps + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(q), q_row_stride, q_head_stride, dn, reinterpret_cast<__nv_bfloat16*>(q_cat),
      reinterpret_cast<const __nv_bfloat16*>(k_rope), ld_k, reinterpret_cast<const __nv_bfloat16*>(latent), ld_l,
      positions, cos_sin, slots, reinterpret_cast<__nv_bfloat16*>(cache), cache_width, T, h, r, dr, interleaved);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
