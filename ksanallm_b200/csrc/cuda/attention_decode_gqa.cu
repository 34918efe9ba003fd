// Tensor-core decode attention for grouped-query models on sm_100a (tcgen05 + TMEM + TMA over the paged cache).
//
// The SIMT decode kernel (attention_decode.cu, the counterpart of the reference's
// 3rdparty/LLM_kernels/csrc/kernels/nvidia/paged_attention/paged_attention.cu:393-436) reads every K / V element
// once per query head of the group, from registers, and is instruction-bound when 8 query heads share one KV head
// (Llama-3-70B, Qwen3-32B). Here the whole group is ONE matrix operand: the q_len x G query rows of a
// (sequence, KV head) form the M side of S = Q K^T and O = P V, so a KV tile is read once from HBM and multiplied on
// the tensor cores for all heads of the group.
//
// One CTA = one (sequence, KV head, KV split), 128 threads. Per 128-token KV tile, as in the prefill kernel:
//   TMA   eight 16-token pages of K and of V through the block table, 128-byte swizzle, double buffered;
//         Q (q_len x G rows of 128) once, through a 3-d tensor map (dim, head, token);
//   S = Q K^T -> TMEM; softmax with thread r owning row r (token r / G, head kv * G + r % G), causal over the
//   sequence's own new tokens; P -> shared memory (bf16, swizzled K-major); O += P V -> TMEM.
// KV splits write normalised partial rows + log-sum-exp to the workspace in the layout of the SIMT kernel and are
// merged by the same combine kernel.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

int launch_decode_combine(const float* part_o, const float* part_lse, const int* cu_q, int seq_base, int h, int splits,
                          int max_rows, int num_seqs, void* out, int ldo, cudaStream_t stream);

constexpr int DG_BQ = 128, DG_BKV = 128, DG_PAGE = 16, DG_D = 128;
constexpr int DG_Q_BYTES = DG_BQ * DG_D * 2;
constexpr int DG_KV_BYTES = DG_BKV * DG_D * 2;
constexpr int DG_P_BYTES = DG_BQ * DG_BKV * 2;
constexpr int DG_OFF_Q = 0;
constexpr int DG_OFF_K = DG_OFF_Q + DG_Q_BYTES;
constexpr int DG_OFF_V = DG_OFF_K + 2 * DG_KV_BYTES;
constexpr int DG_OFF_P = DG_OFF_V + 2 * DG_KV_BYTES;
constexpr int DG_OFF_BAR = DG_OFF_P + DG_P_BYTES;
constexpr int DG_SMEM = DG_OFF_BAR + 256 + 1024;

__host__ __device__ constexpr uint32_t dg_idesc_pv() {
  // bf16 x bf16 -> f32, A K-major, B MN-major (bit 16), M = 128, N = 128
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(DG_D >> 3) << 17) |
         (static_cast<uint32_t>(128 >> 4) << 24);
}
__device__ __forceinline__ uint64_t dg_desc_mn128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(128, 1)
paged_decode_gqa_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                        const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                        const int* __restrict__ kv_lens, int seq_base, int h, int hk, int q_box, float scale_log2,
                        __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ part_o,
                        float* __restrict__ part_lse, int splits, int tiles_per_split, int max_rows,
                        unsigned int* err) {
  const int bi = blockIdx.x;
  const int b = bi + seq_base;
  const int kh = blockIdx.y;
  const int split = blockIdx.z;
  const int G = h / hk;
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  const int L = kv_lens[b];
  const int q_start = L - q_len;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int rows = q_len * G;
  const bool valid = tid < rows;
  const int qi = valid ? tid / G : 0;
  const int head = kh * G + (valid ? tid - qi * G : 0);
  const int q_pos = valid ? q_start + qi : L - 1;
  const int n_tiles_all = (L + DG_BKV - 1) / DG_BKV;
  const int t0 = split * tiles_per_split;
  const int t1 = min(n_tiles_all, t0 + tiles_per_split);
  const size_t prow = (static_cast<size_t>(bi) * max_rows + (static_cast<size_t>(qi) * h + head)) * splits + split;
  if (t0 >= t1) {
    // this split holds no tokens of this (shorter) sequence: its rows must not count in the merge
    if (valid && splits > 1) part_lse[prow] = -INFINITY;
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + DG_OFF_Q;
  uint8_t* sK = smem + DG_OFF_K;
  uint8_t* sV = smem + DG_OFF_V;
  uint8_t* sP = smem + DG_OFF_P;
  uint64_t* q_bar = reinterpret_cast<uint64_t*>(smem + DG_OFF_BAR);
  uint64_t* k_full = q_bar + 1;   // [2]
  uint64_t* v_full = k_full + 2;  // [2]
  uint64_t* s_done = v_full + 2;
  uint64_t* o_done = s_done + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  constexpr uint32_t TMEM_COLS = 256;
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
  const uint32_t tmem_O = tmem_base + DG_BKV;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

  const int n_pages = (L + DG_PAGE - 1) / DG_PAGE;
  const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;

  auto load_kv_tile = [&](int kt, int stage) {
    mbar_expect_tx(&k_full[stage], DG_KV_BYTES);
    mbar_expect_tx(&v_full[stage], DG_KV_BYTES);
    for (int p = 0; p < DG_BKV / DG_PAGE; ++p) {
      int pg = kt * (DG_BKV / DG_PAGE) + p;
      if (pg >= n_pages) pg = n_pages - 1;  // finite filler; those columns are masked to p = 0
      const int blk = bt[pg];
      const int krow = ((blk * 2 + 0) * hk + kh) * DG_PAGE;
      const int vrow = ((blk * 2 + 1) * hk + kh) * DG_PAGE;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        tma_load_2d(sK + stage * DG_KV_BYTES + hf * (DG_BKV * 128) + p * (DG_PAGE * 128), &tmKV, &k_full[stage], hf * 64,
                    krow);
        tma_load_2d(sV + stage * DG_KV_BYTES + hf * (DG_BKV * 128) + p * (DG_PAGE * 128), &tmKV, &v_full[stage], hf * 64,
                    vrow);
      }
    }
  };

  if (tid == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
    // rows of the tile = (token, head of the group): q_box tokens x G heads x 64 dims per box, two boxes (dim halves)
    mbar_expect_tx(q_bar, static_cast<uint32_t>(q_box) * G * DG_D * 2);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) tma_load_3d(sQ + hf * (DG_BQ * 128), &tmQ, q_bar, hf * 64, kh * G, q0);
    load_kv_tile(t0, 0);
  }

  float m_ref = -INFINITY;
  float l_sum = 0.f;
  int bad = 0;
  if (!mbar_wait_bounded(q_bar, 0, abort_flag, err)) bad = 1;

  for (int kt = t0; kt < t1; ++kt) {
    const int it = kt - t0;
    const int stage = it & 1;
    const uint32_t ph = (it >> 1) & 1;
    if (tid == 0 && !bad) {
      if (kt + 1 < t1) load_kv_tile(kt + 1, stage ^ 1);
      if (mbar_wait_bounded(&k_full[stage], ph, abort_flag, err)) {
        tc_fence_after();
        constexpr uint32_t idesc = umma_idesc(128, DG_BKV, 1, 1);
#pragma unroll
        for (int k = 0; k < DG_D / 16; ++k) {
          const uint32_t off = (k >> 2) * (DG_BQ * 128) + (k & 3) * 32;
          umma_f16(tmem_S, umma_desc_k128(smem_u32(sQ) + off), umma_desc_k128(smem_u32(sK + stage * DG_KV_BYTES) + off),
                   idesc, k > 0 ? 1u : 0u);
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

    const int kv0 = kt * DG_BKV;
    float m_tile = -INFINITY;
#pragma unroll 1
    for (int c = 0; c < DG_BKV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_S + lane_off + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = kv0 + c * 32 + j;
        const float s = (kpos > q_pos) ? -INFINITY : __uint_as_float(r[j]) * scale_log2;
        m_tile = fmaxf(m_tile, s);
      }
    }
    if (!valid) m_tile = 0.f;  // rows past the group hold whatever was in shared memory: keep their exponents finite
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
      for (int c = 0; c < DG_D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_O + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
        tmem_st32(tmem_O + lane_off + c * 32, r);
      }
      tmem_wait_st();
    }
#pragma unroll 1
    for (int c = 0; c < DG_BKV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_S + lane_off + c * 32, r);
      tmem_wait_ld();
      float p[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int kpos = kv0 + c * 32 + j;
        p[j] = (kpos > q_pos || !valid) ? 0.f : exp2f(__uint_as_float(r[j]) * scale_log2 - m_ref);
        l_sum += p[j];
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 o;
        o.x = pack_bf16(p[ch * 8 + 0], p[ch * 8 + 1]);
        o.y = pack_bf16(p[ch * 8 + 2], p[ch * 8 + 3]);
        o.z = pack_bf16(p[ch * 8 + 4], p[ch * 8 + 5]);
        o.w = pack_bf16(p[ch * 8 + 6], p[ch * 8 + 7]);
        const int chunk = (c & 1) * 4 + ch;
        uint8_t* dst = sP + (c >> 1) * (DG_BQ * 128) + tid * 128 + ((chunk ^ (tid & 7)) << 4);
        *reinterpret_cast<uint4*>(dst) = o;
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      if (mbar_wait_bounded(&v_full[stage], ph, abort_flag, err)) {
        tc_fence_after();
        constexpr uint32_t idesc = dg_idesc_pv();
#pragma unroll
        for (int k = 0; k < DG_BKV / 16; ++k) {
          const uint64_t da = umma_desc_k128(smem_u32(sP) + (k >> 2) * (DG_BQ * 128) + (k & 3) * 32);
          const uint64_t db = dg_desc_mn128(smem_u32(sV + stage * DG_KV_BYTES) + k * (16 * 128), DG_BKV * 128);
          umma_f16(tmem_O, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(o_done);
      } else {
        bad = 1;
      }
    }
    if (!bad && !mbar_wait_bounded(o_done, it & 1, abort_flag, err)) bad = 1;
    if (__syncthreads_or(bad)) {
      bad = 1;
      break;
    }
    tc_fence_after();
  }

  if (!bad) {
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
    __nv_bfloat16* orow = out + static_cast<size_t>(q0 + qi) * ldo + head * DG_D;
    float* prow_o = part_o != nullptr ? part_o + prow * DG_D : nullptr;
#pragma unroll 1
    for (int c = 0; c < DG_D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_O + lane_off + c * 32, r);  // warp-collective: every lane loads, only valid rows store
      tmem_wait_ld();
      if (valid) {
        if (splits == 1) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv);
            o.y = pack_bf16(__uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
            o.z = pack_bf16(__uint_as_float(r[j + 4]) * inv, __uint_as_float(r[j + 5]) * inv);
            o.w = pack_bf16(__uint_as_float(r[j + 6]) * inv, __uint_as_float(r[j + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + j) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(prow_o + c * 32 + j) =
                make_float4(__uint_as_float(r[j]) * inv, __uint_as_float(r[j + 1]) * inv,
                            __uint_as_float(r[j + 2]) * inv, __uint_as_float(r[j + 3]) * inv);
        }
      }
    }
    if (valid && splits > 1) part_lse[prow] = l_sum > 0.f ? m_ref + log2f(l_sum) : -INFINITY;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- the transposed form for small groups: at most 16 query rows (group x new tokens) ---------------------------------
// With 8 query heads and one new token only 8 of the 128 rows above are real, yet every thread scans 128 score columns
// twice: the softmax, not the memory system, sets the pace. Here the roles are swapped: S^T = K Q^T puts the 128 KV
// tokens of a tile on the MMA rows (one per thread) and the <= 16 query rows on the columns, so a thread handles 16
// scores per tile; the column maxima / sums go across threads (redux + shared memory), O^T = V^T P^T accumulates
// 128 head dims x 16 query rows in 16 TMEM columns, and rescaling the accumulator touches 16 values per thread. One
// CTA needs 73 KB of shared memory (one K tile, one V tile, Q, P) and 32 TMEM columns, so three CTAs share an SM and
// overlap each other's loads, MMAs and softmax; inside a CTA the next K tile is requested as soon as S is out and the
// next V tile as soon as O has been updated.
//   warps 0-3  thread t = KV token t of the tile (S^T row) and head dim t (O^T row)
//   warp 4     lane 0: TMA producer
constexpr int DT_N = 16;
constexpr int DT_Q_BYTES = DT_N * DG_D * 2;     // 4 KB: two 64-dim halves of [16 rows x 128 B]
constexpr int DT_P_BYTES = DT_N * DG_BKV * 2;   // 4 KB: two 64-token halves of [16 rows x 128 B]
constexpr int DT_OFF_K = 0;
constexpr int DT_OFF_V = DT_OFF_K + DG_KV_BYTES;
constexpr int DT_OFF_Q = DT_OFF_V + DG_KV_BYTES;
constexpr int DT_OFF_P = DT_OFF_Q + DT_Q_BYTES;
constexpr int DT_OFF_RED = DT_OFF_P + DT_P_BYTES;          // [4 warps][16] floats, twice (max, sum)
constexpr int DT_OFF_BAR = DT_OFF_RED + 2 * 4 * DT_N * 4;
constexpr int DT_SMEM = DT_OFF_BAR + 128 + 1024;

// order-preserving float <-> int so that redux.sync.max can reduce floats
__device__ __forceinline__ int dt_key(float f) {
  const int b = __float_as_int(f);
  return b ^ ((b >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float dt_unkey(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }

__global__ void __launch_bounds__(160, 3)
paged_decode_gqa_t_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                          const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                          const int* __restrict__ kv_lens, int seq_base, int h, int hk, int q_box, float scale_log2,
                          __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ part_o,
                          float* __restrict__ part_lse, int splits, int tiles_per_split, int max_rows,
                          unsigned int* err) {
  const int bi = blockIdx.x;
  const int b = bi + seq_base;
  const int kh = blockIdx.y;
  const int split = blockIdx.z;
  const int G = h / hk;
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  const int L = kv_lens[b];
  const int q_start = L - q_len;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int rows = q_len * G;  // real query rows, <= 16
  const int n_tiles_all = (L + DG_BKV - 1) / DG_BKV;
  const int t0 = split * tiles_per_split;
  const int t1 = min(n_tiles_all, t0 + tiles_per_split);
  if (t0 >= t1) {
    // this split holds no tokens of this (shorter) sequence: its rows must not count in the merge
    if (tid < rows && splits > 1) {
      const int qi = tid / G, head = kh * G + tid - qi * G;
      part_lse[(static_cast<size_t>(bi) * max_rows + (static_cast<size_t>(qi) * h + head)) * splits + split] = -INFINITY;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + DT_OFF_K;
  uint8_t* sV = smem + DT_OFF_V;
  uint8_t* sQ = smem + DT_OFF_Q;
  uint8_t* sP = smem + DT_OFF_P;
  float* red_max = reinterpret_cast<float*>(smem + DT_OFF_RED);  // [4][16]
  float* red_sum = red_max + 4 * DT_N;
  uint64_t* q_bar = reinterpret_cast<uint64_t*>(smem + DT_OFF_BAR);
  uint64_t* k_full = q_bar + 1;
  uint64_t* v_full = k_full + 1;
  uint64_t* k_free = v_full + 1;  // S^T is out: the K tile may be overwritten
  uint64_t* v_free = k_free + 1;  // O^T is updated: the V tile (and P) may be overwritten
  uint64_t* s_done = v_free + 1;
  uint64_t* o_done = s_done + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  if (tid == 0) {
    mbar_init(q_bar, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_free, 1);
    mbar_init(v_free, 1);
    mbar_init(s_done, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + DT_N;

  if (warp == 4) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmKV);
      const int n_pages = (L + DG_PAGE - 1) / DG_PAGE;
      const int* bt = block_tables + static_cast<size_t>(b) * max_blocks;
      mbar_expect_tx(q_bar, static_cast<uint32_t>(q_box) * G * DG_D * 2);
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) tma_load_3d(sQ + hf * (DT_N * 128), &tmQ, q_bar, hf * 64, kh * G, q0);
      bool ok = true;
      for (int kt = t0; kt < t1 && ok; ++kt) {
        const int it = kt - t0;
        for (int which = 0; which < 2 && ok; ++which) {  // 0: K, 1: V
          uint64_t* freeb = which ? v_free : k_free;
          uint64_t* fullb = which ? v_full : k_full;
          uint8_t* dst = which ? sV : sK;
          if (it > 0 && !mbar_wait_bounded(freeb, (it - 1) & 1, abort_flag, err)) {
            ok = false;
            break;
          }
          mbar_expect_tx(fullb, DG_KV_BYTES);
          for (int p = 0; p < DG_BKV / DG_PAGE; ++p) {
            int pg = kt * (DG_BKV / DG_PAGE) + p;
            if (pg >= n_pages) pg = n_pages - 1;  // finite filler; those tokens are masked
            const int row = ((bt[pg] * 2 + which) * hk + kh) * DG_PAGE;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
              tma_load_2d(dst + hf * (DG_BKV * 128) + p * (DG_PAGE * 128), &tmKV, fullb, hf * 64, row);
          }
        }
      }
    }
  } else {
    // ---------------- MMA issue (thread 0) + softmax (128 threads) ----------------
    float m_ref[DT_N], l_part[DT_N];
#pragma unroll
    for (int n = 0; n < DT_N; ++n) {
      m_ref[n] = -INFINITY;
      l_part[n] = 0.f;
    }
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    int bad = 0;
    if (!mbar_wait_bounded(q_bar, 0, abort_flag, err)) bad = 1;
    for (int kt = t0; kt < t1; ++kt) {
      const int it = kt - t0;
      const uint32_t ph = it & 1;
      if (tid == 0 && !bad) {
        if (mbar_wait_bounded(k_full, ph, abort_flag, err)) {
          tc_fence_after();
          constexpr uint32_t idesc = umma_idesc(128, DT_N, 1, 1);
#pragma unroll
          for (int k = 0; k < DG_D / 16; ++k)
            umma_f16(tmem_S, umma_desc_k128(smem_u32(sK) + (k >> 2) * (DG_BKV * 128) + (k & 3) * 32),
                     umma_desc_k128(smem_u32(sQ) + (k >> 2) * (DT_N * 128) + (k & 3) * 32), idesc, k > 0 ? 1u : 0u);
          umma_commit(k_free);
          umma_commit(s_done);
        } else {
          bad = 1;
        }
      }
      if (!bad && !mbar_wait_bounded(s_done, ph, abort_flag, err)) bad = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) {
        bad = 1;
        break;
      }
      tc_fence_after();

      // scores of KV token kv0 + tid against the 16 query rows
      uint32_t r[DT_N];
      tmem_ld16(tmem_S + lane_off, r);
      tmem_wait_ld();
      const int kpos = kt * DG_BKV + tid;
      float s[DT_N];
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        const int q_pos = q_start + n / G;
        s[n] = (n >= rows || kpos >= L || kpos > q_pos) ? -INFINITY : __uint_as_float(r[n]) * scale_log2;
      }
      // column maxima over the 128 tokens: redux inside the warp, shared memory across the four warps
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        const int k = __reduce_max_sync(0xffffffffu, dt_key(s[n]));
        if (lane == 0) red_max[warp * DT_N + n] = dt_unkey(k);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[DT_N];
      bool any_scale = false;
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        const float mt = fmaxf(fmaxf(red_max[n], red_max[DT_N + n]), fmaxf(red_max[2 * DT_N + n], red_max[3 * DT_N + n]));
        const float m_new = fmaxf(m_ref[n], mt);
        alpha[n] = (m_new > m_ref[n] && m_ref[n] != -INFINITY) ? exp2f(m_ref[n] - m_new) : 1.f;
        any_scale |= alpha[n] != 1.f;
        m_ref[n] = m_new;
        l_part[n] *= alpha[n];
      }
      // probabilities first (this overlaps the previous tile's PV product) ...
      float pr[DT_N];
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        pr[n] = (s[n] == -INFINITY) ? 0.f : exp2f(s[n] - m_ref[n]);
        l_part[n] += pr[n];
      }
      // ... then the previous PV product must be in: it reads P, and O^T is rescaled below
      if (it > 0) {
        if (!bad && !mbar_wait_bounded(o_done, (it - 1) & 1, abort_flag, err)) bad = 1;
        tc_fence_after();
        if (any_scale && !bad) {  // the maxima are the same in every thread: a uniform branch
          uint32_t o[DT_N];
          tmem_ld16(tmem_O + lane_off, o);
          tmem_wait_ld();
#pragma unroll
          for (int n = 0; n < DT_N; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * alpha[n]);
          tmem_st16(tmem_O + lane_off, o);
          tmem_wait_st();
        }
      }
      // P^T: thread = token (column of P), 16 query rows; bf16 into the K-major, 128-byte-swizzled B operand
      {
        uint8_t* base = sP + (tid >> 6) * (DT_N * 128) + (tid & 7) * 2;
        const int chunk = (tid & 63) >> 3;
#pragma unroll
        for (int n = 0; n < DT_N; ++n)
          *reinterpret_cast<__nv_bfloat16*>(base + n * 128 + ((chunk ^ (n & 7)) << 4)) = __float2bfloat16(pr[n]);
      }
      fence_async_smem();
      tc_fence_before();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) {
        bad = 1;
        break;
      }
      if (tid == 0) {
        if (mbar_wait_bounded(v_full, ph, abort_flag, err)) {
          tc_fence_after();
          // O^T[dim, row] += V^T[dim, token] P^T[token, row]: A = V tile read MN-major (dims contiguous), B = P
          constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) |
                                     (static_cast<uint32_t>(DT_N >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
#pragma unroll
          for (int k = 0; k < DG_BKV / 16; ++k)
            umma_f16(tmem_O, dg_desc_mn128(smem_u32(sV) + k * (16 * 128), DG_BKV * 128),
                     umma_desc_k128(smem_u32(sP) + (k >> 2) * (DT_N * 128) + (k & 3) * 32), idesc,
                     (it > 0 || k > 0) ? 1u : 0u);
          umma_commit(v_free);
          umma_commit(o_done);
        } else {
          bad = 1;
        }
      }
    }
    const int n_it = t1 - t0;
    if (!bad && !mbar_wait_bounded(o_done, (n_it - 1) & 1, abort_flag, err)) bad = 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*abort_flag) bad = 1;
    tc_fence_after();
    if (!bad) {
      // row sums over the 128 token-threads
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        float v = l_part[n];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) red_sum[warp * DT_N + n] = v;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      uint32_t o[DT_N];
      tmem_ld16(tmem_O + lane_off, o);  // thread = head dim tid, 16 query rows
      tmem_wait_ld();
#pragma unroll
      for (int n = 0; n < DT_N; ++n) {
        if (n < rows) {
          const float l = red_sum[n] + red_sum[DT_N + n] + red_sum[2 * DT_N + n] + red_sum[3 * DT_N + n];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          const int qi = n / G, head = kh * G + n - qi * G;
          const float v = __uint_as_float(o[n]) * inv;
          if (splits == 1) {
            out[static_cast<size_t>(q0 + qi) * ldo + head * DG_D + tid] = __float2bfloat16(v);
          } else {
            const size_t prow = (static_cast<size_t>(bi) * max_rows + (static_cast<size_t>(qi) * h + head)) * splits + split;
            part_o[prow * DG_D + tid] = v;
            if (tid == 0) part_lse[prow] = l > 0.f ? m_ref[n] + log2f(l) : -INFINITY;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}

}  // namespace ksana

using namespace ksana;

// 0: the transposed kernel for at most 16 query rows, the row kernel otherwise; 1: always the row kernel (tests, timing)
static int g_gqa_variant = 0;
KSANA_API void ksana_paged_decode_gqa_set_variant(int v) { g_gqa_variant = v; }

// Decode attention for grouped-query models: sequences [seq_base, seq_base + num_seqs) of the step, each with at most
// max_q_len new tokens; (h / hk) * max_q_len <= 128, d == 128, 16-token pages, bf16 cache
// [num_blocks][2][hk][16][128]. q / out: [total_tokens, h, 128] bf16 with token pitches ldq / ldo (multiples of 8).
// workspace (fp32): num_seqs * max_q_len * h * splits * 129 floats when the KV range is split (the launcher splits when
// there are fewer (sequence, KV head) pairs than SMs). Returns 0, -1 (shape not taken: use ksana_paged_decode),
// -6 (workspace too small) or another negative code.
KSANA_API int ksana_paged_decode_gqa(const void* q, int ldq, int total_tokens, const void* cache, int num_blocks,
                                     const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens,
                                     int seq_base, int num_seqs, int max_q_len, int max_kv_len, int h, int hk, int d,
                                     int block_size, float scale, void* out, int ldo, float* workspace,
                                     long long workspace_floats, cudaStream_t stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (d != DG_D || block_size != DG_PAGE || hk <= 0 || h % hk != 0 || (ldq & 7) || (ldo & 7)) return -1;
  const int G = h / hk;
  if (G * max_q_len > DG_BQ || G * max_q_len > 256) return -1;
  CUtensorMap tmQ, tmKV;
  {
    // (dim, head, token): heads are 128 elements apart, tokens ldq elements; one box = 64 dims x G heads x tokens
    const uint64_t dims[3] = {static_cast<uint64_t>(d), static_cast<uint64_t>(h), static_cast<uint64_t>(total_tokens)};
    const uint64_t strides[2] = {static_cast<uint64_t>(d) * 2, static_cast<uint64_t>(ldq) * 2};
    const uint32_t box[3] = {64, static_cast<uint32_t>(G), static_cast<uint32_t>(max_q_len)};
    if (make_tmap_nd(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return -2;
  }
  if (make_tmap_2d(&tmKV, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   static_cast<uint64_t>(num_blocks) * 2 * hk * DG_PAGE, d, d, DG_PAGE, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  const int sms = sm_count();
  const int n_tiles = (max_kv_len + DG_BKV - 1) / DG_BKV;
  const int base = num_seqs * hk;
  // at most 16 query rows: the transposed kernel, three CTAs per SM
  const bool transposed = G * max_q_len <= DT_N && g_gqa_variant != 1;
  // The transposed kernel keeps three CTAs per SM: with only a few more CTAs than the 3 x SMs slots the last wave
  // runs mostly empty (512 CTAs on 444 slots cost 40 %), so the KV range is cut until there are about four waves of
  // CTAs of at least two tiles each; the hardware then balances them as slots free up.
  const int want_ctas = transposed ? 12 * sms : sms;
  int splits = base >= want_ctas ? 1 : (want_ctas + base - 1) / base;
  if (transposed && splits > (n_tiles + 1) / 2) splits = (n_tiles + 1) / 2;
  if (splits > n_tiles) splits = n_tiles;
  if (splits < 1) splits = 1;
  int tiles_per_split = (n_tiles + splits - 1) / splits;
  if (tiles_per_split < 1) tiles_per_split = 1;
  splits = (n_tiles + tiles_per_split - 1) / tiles_per_split;
  if (splits < 1) splits = 1;
  const int max_rows = max_q_len * h;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    const long long rows = static_cast<long long>(num_seqs) * max_rows * splits;
    if (workspace == nullptr || rows * (d + 1) > workspace_floats) return -6;
    part_o = workspace;
    part_lse = workspace + rows * d;
  }
  dim3 grid(num_seqs, hk, splits);
  if (transposed) {
    if (KSANA_SMEM_ONCE(paged_decode_gqa_t_kernel, DT_SMEM) != 0) return -4;
    paged_decode_gqa_t_kernel<<<grid, 160, DT_SMEM, stream>>>(
        tmQ, tmKV, block_tables, max_blocks, cu_q, kv_lens, seq_base, h, hk, max_q_len, scale * 1.4426950408889634f,
        reinterpret_cast<__nv_bfloat16*>(out), ldo, part_o, part_lse, splits, tiles_per_split, max_rows, error_word());
    if (cudaGetLastError() != cudaSuccess) return -5;
    if (splits > 1)
      return launch_decode_combine(part_o, part_lse, cu_q, seq_base, h, splits, max_rows, num_seqs, out, ldo, stream);
    return 0;
  }
  if (KSANA_SMEM_ONCE(paged_decode_gqa_kernel, DG_SMEM) != 0) return -4;
  paged_decode_gqa_kernel<<<grid, 128, DG_SMEM, stream>>>(
      tmQ, tmKV, block_tables, max_blocks, cu_q, kv_lens, seq_base, h, hk, max_q_len, scale * 1.4426950408889634f,
      reinterpret_cast<__nv_bfloat16*>(out), ldo, part_o, part_lse, splits, tiles_per_split, max_rows, error_word());
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (splits > 1)
    return launch_decode_combine(part_o, part_lse, cu_q, seq_base, h, splits, max_rows, num_seqs, out, ldo, stream);
  return 0;
}
