// Weight-only int4 (group-quantised, asymmetric) x bf16 GEMM for sm_100a: C[M, N] = A[M, K] * dequant(Wq)[N, K]^T.
//
// Wq: int32 words holding 8 weights each (element j in bits [4j, 4j+4)), pre-tiled at load time as
// [K/64][ceil(N/128)][128 rows][8 words]: the 128 x 64 weights one pipeline stage needs are ONE contiguous 4 KB block,
// and the blocks that concurrently running CTAs fetch (neighbouring row tiles, same k-step) are adjacent in memory.
// Two layouts that were measured and dropped: row-major [N, K/8] (every stage = 128 separate 32-byte sectors) and
// tiles with the row tile as the OUTER dimension (every CTA's stream starts a power-of-two stride apart: the whole GPU
// delivered 0.87 TB/s, channel camping).
// (scale, zero) pairs: [N, K/group, 2] fp32 with w = (q - zero) * scale; the kernel rounds the scale to bf16 and the
// product once more (two packed bf16 instructions per pair of weights instead of a trip through fp32).
// The packed weights are the only thing streamed from HBM (K/2 bytes per output column): the dequantisation happens
// inside the pipeline, between the load stage and the tensor core, so no bf16 copy of the weights exists in memory.
// It stands in for the reference's int4 back-ends: CUTLASS fpA_intB (3rdparty/LLM_kernels/csrc/kernels/nvidia/
// asymmetric_gemm/fpA_intB_gemm), Marlin (gptq_marlin/marlin_template.h: mma.sync + cp.async) and Machete
// (machete/machete_mainloop.cuh: sm90 wgmma), chosen by src/ksana_llm/layers/matmul_layer_factory.cpp:87-212.
//
// CTA = 14 warps: warp 0 TMA producer (A tile 128 x 64 bf16 with 128-byte swizzle + raw packed W tile 128 x 32 bytes),
// warp 1 MMA issuer (tcgen05, accumulators double-buffered in TMEM), warps 2-9 dequantisers (two threads per W row:
// nibbles -> exact bf16 integers by bit tricks, minus zero, times scale in fp32, stored in the swizzled K-major layout
// the MMA descriptor expects), warps 10-13 epilogue. Split-K through the fp32 workspace (last arriver reduces in
// split order) keeps all SMs busy for decode-sized M.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int Q_BM = 128, Q_BK = 64;
constexpr int Q_A_BYTES = Q_BM * Q_BK * 2;
constexpr int Q_TILE_RAW = 128 * 32;  // one pre-tiled block: 128 weight rows x 64 weights
constexpr int Q_THREADS = 14 * 32;
template <int BN>
struct QCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 5;
  static constexpr int B_BYTES = BN * Q_BK * 2, RAW_BYTES = BN * 32;
  static constexpr int STAGE = Q_A_BYTES + B_BYTES + RAW_BYTES;
  static constexpr int BAR = STAGES * STAGE;
  static constexpr int SMEM = BAR + 256 + 1024;
};

// BN = 128: five stages, two dequantiser threads per weight row (decode-sized M: more tiles, shorter chains);
// BN = 256: four stages, one thread per row (large M: half the activation traffic per FLOP, 512-cycle MMA stages).
template <int BN>
__global__ void __launch_bounds__(Q_THREADS, 1)
gemm_int4_kernel(const __grid_constant__ CUtensorMap tmA, const uint8_t* __restrict__ wq_tiled,
                 const float2* __restrict__ sz, int groups_per_row, int group,
                 __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc,
                 int splits, float* __restrict__ ws, unsigned int* __restrict__ counters, unsigned int* err,
                 long long* __restrict__ trace, int dbg) {
#define Q_TRACE(slot, kbi)                                                        \
  if (trace != nullptr && blockIdx.x == 0 && (kbi) < 32) trace[(kbi) * 8 + (slot)] = clock64();
  constexpr int Q_BN = BN, Q_STAGES = QCfg<BN>::STAGES, Q_B_BYTES = QCfg<BN>::B_BYTES, Q_RAW_BYTES = QCfg<BN>::RAW_BYTES;
  constexpr int Q_STAGE = QCfg<BN>::STAGE, Q_BAR = QCfg<BN>::BAR;
  constexpr int WORDS = BN == 256 ? 8 : 4;  // packed words per dequantiser thread and k-block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* in_full = reinterpret_cast<uint64_t*>(smem + Q_BAR);  // A + raw W landed (TMA)
  uint64_t* b_full = in_full + Q_STAGES;                          // dequantised W written (one arrival per warp)
  uint64_t* empty_bar = b_full + Q_STAGES;                        // MMAs of the stage retired
  uint64_t* acc_full = empty_bar + Q_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + Q_BM - 1) / Q_BM, tiles_n = (N + Q_BN - 1) / Q_BN;
  const int num_kb = (K + Q_BK - 1) / Q_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_units = tiles_m * tiles_n * splits;
  const int n_tiles128 = (N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&in_full[s], 1);
      mbar_init(&b_full[s], 8);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 128);
    }
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * Q_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
        const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          Q_TRACE(0, kb - kb0)
          uint8_t* sa = smem + stage * Q_STAGE;
          mbar_expect_tx(&in_full[stage], Q_A_BYTES + ((dbg & 1) ? 0 : Q_RAW_BYTES));
          tma_load_2d(sa, &tmA, &in_full[stage], kb * Q_BK, m_idx * Q_BM);
          if (!(dbg & 1)) {
#pragma unroll
            for (int blk = 0; blk < BN / 128; ++blk) {
              // rows past the last weight tile only exist as padding of the output tile: re-read the last block
              const int nt = min(n_idx * (BN / 128) + blk, n_tiles128 - 1);
              bulk_load(sa + Q_A_BYTES + Q_B_BYTES + blk * Q_TILE_RAW,
                        wq_tiled + (static_cast<size_t>(kb) * n_tiles128 + nt) * Q_TILE_RAW, Q_TILE_RAW, &in_full[stage]);
            }
          }
          if (++stage == Q_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(Q_BM, Q_BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (kb1 <= kb0) continue;  // empty split: no barrier is touched on either side
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * Q_BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&in_full[stage], phase, abort_flag, err) ||
              !mbar_wait_bounded(&b_full[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          Q_TRACE(4, kb - kb0)
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Q_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + Q_A_BYTES);
#pragma unroll
          for (int k = 0; k < Q_BK / 16; ++k) umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          Q_TRACE(5, kb - kb0)
          if (++stage == Q_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
      }
    }
  } else if (warp < 10) {
    // ---------------- dequantisers: thread -> (W row of the tile, half of the 64-wide k-block) ----------------
    const int dt = threadIdx.x - 64;
    const int row = BN == 256 ? dt : dt >> 1, hf = BN == 256 ? 0 : dt & 1;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int n_idx = tile / tiles_m;
      const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
      const int n = n_idx * Q_BN + row;
      const int nn = n < N ? n : N - 1;
      // (scale, zero) pairs of this row, one 8-byte load per group. They are fetched TWO groups ahead into a small
      // register queue: a load consumed one k-block after its issue still stalled the whole TMA -> dequantise -> MMA
      // chain for ~600 cycles per k-block (measured with the phase timeline below).
      const float2* szrow = sz + static_cast<size_t>(nn) * groups_per_row;
      const int g_last = groups_per_row - 1;
      int g_cur = (kb0 * Q_BK) / group;
      float2 q0 = __ldg(szrow + min(g_cur, g_last));
      float2 q1 = __ldg(szrow + min(g_cur + 1, g_last));
      float2 q2 = __ldg(szrow + min(g_cur + 2, g_last));
      for (int kb = kb0; kb < kb1; ++kb) {
        const int g = (kb * Q_BK) / group;
        if (g != g_cur) {
          g_cur = g;
          q0 = q1;
          q1 = q2;
          q2 = __ldg(szrow + min(g + 2, g_last));
        }
        const float sc = q0.x;
        const int z = static_cast<int>(q0.y);
        if (!mbar_wait_bounded(&in_full[stage], phase, abort_flag, err)) {
          ok = false;
          break;
        }
        if (dt == 0) { Q_TRACE(1, kb - kb0) }
        uint8_t* sb = smem + stage * Q_STAGE + Q_A_BYTES;
        uint32_t words[WORDS];
#pragma unroll
        for (int q = 0; q < WORDS / 4; ++q) {
          const uint4 raw = *reinterpret_cast<const uint4*>(sb + Q_B_BYTES + row * 32 + hf * 16 + q * 16);
          words[4 * q] = raw.x;
          words[4 * q + 1] = raw.y;
          words[4 * q + 2] = raw.z;
          words[4 * q + 3] = raw.w;
        }
        if (!(dbg & 2)) {
        // bf16 bits 0x4300 | q are exactly 128 + q; subtracting 128 + z in bf16 is exact, and the product with the
        // (bf16) scale is rounded once: w = bf16((q - z) * bf16(scale))
        const uint32_t zb = 0x43004300u | static_cast<uint32_t>(z) | (static_cast<uint32_t>(z) << 16);
        const uint32_t sc2 = pack_bf16(sc, sc);
        uint8_t* drow = sb + row * 128;
#pragma unroll
        for (int wv = 0; wv < WORDS; ++wv) {
          const uint32_t v = words[wv];
          const uint32_t t = v & 0x0F0F0F0Fu;          // nibbles 0, 2, 4, 6 (one per byte)
          const uint32_t u = (v >> 4) & 0x0F0F0F0Fu;   // nibbles 1, 3, 5, 7
          uint32_t o[4];
#pragma unroll
          for (int p = 0; p < 4; ++p) {
            // pair (nibble 2p, nibble 2p + 1) -> bytes 0 and 2 of one word
            uint32_t x;
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(x) : "r"(t), "r"(u), "r"(0x4440u | (4u + p) << 8 | static_cast<uint32_t>(p)));
            x = (x & 0x00FF00FFu) | 0x43004300u;
            uint32_t d;
            asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(x), "r"(zb));
            asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[p]) : "r"(d), "r"(sc2));
          }
          const int chunk = hf * 4 + wv;  // 16-byte chunk (8 k values) of the row's 128 bytes
          *reinterpret_cast<uint4*>(drow + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        }
        if (dt == 0) { Q_TRACE(2, kb - kb0) }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[stage]);
        if (dt == 0) { Q_TRACE(3, kb - kb0) }  // one arrival per warp: 256 arrivals on one barrier serialise
        if (++stage == Q_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 10..13) ----------------
    const int quarter = warp & 3;  // warps 10..13 -> TMEM lane quarters 2, 3, 0, 1
    int it = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++it) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
      const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      const bool has_k = kb1 > kb0;  // a trailing split can be empty: it contributes zeros
      if (has_k) {
        uint32_t ok_in = mbar_wait_bounded(&acc_full[as], aphase, abort_flag, err) ? 1u : 0u, ok_all;
        asm volatile(
            "{\n\t.reg .pred pin, pout;\n\t"
            "setp.ne.u32 pin, %1, 0;\n\t"
            "bar.red.and.pred pout, 1, 128, pin;\n\t"
            "selp.u32 %0, 1, 0, pout;\n\t}"
            : "=r"(ok_all)
            : "r"(ok_in)
            : "memory");
        if (!ok_all) break;
      }
      tc_fence_after();
      const int row = m_idx * Q_BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * Q_BN;
      bool reduce_here = true;
      if (splits > 1) {
        float* wrow = ws + (static_cast<size_t>(split) * M + (row_ok ? row : 0)) * N + n_idx * Q_BN;
#pragma unroll 1
        for (int c = 0; c < Q_BN / 32; ++c) {
          uint32_t r[32];
          if (has_k) {
            tmem_ld32(t_row + c * 32, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              if (n_idx * Q_BN + c * 32 + j < N)
                *reinterpret_cast<float4*>(wrow + c * 32 + j) =
                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                __uint_as_float(r[j + 3]));
          }
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 320) {
          const unsigned int prev = atomicAdd(&counters[tile], 1u);
          const int last = (prev == static_cast<unsigned int>(splits - 1));
          if (last) counters[tile] = 0;
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        reduce_here = (*last_flag != 0);
        __threadfence();
      }
      if (reduce_here) {
        __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc;
#pragma unroll 1
        for (int c = 0; c < Q_BN / 32; ++c) {
          float v[32];
          if (splits > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            for (int s = 0; s < splits; ++s) {
              const float* wrow = ws + (static_cast<size_t>(s) * M + (row_ok ? row : 0)) * N + n_idx * Q_BN + c * 32;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                if (row_ok && n_idx * Q_BN + c * 32 + j < N) {
                  const float4 p = __ldcg(reinterpret_cast<const float4*>(wrow + j));
                  v[j] += p.x;
                  v[j + 1] += p.y;
                  v[j + 2] += p.z;
                  v[j + 3] += p.w;
                }
              }
            }
          } else {
            uint32_t r[32];
            tmem_ld32(t_row + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          }
          const int col0 = n_idx * Q_BN + c * 32;
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) v[j] += __bfloat162float(bias[col0 + j]);
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (row_ok && col0 + j < N) {
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]);
              o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]);
              o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(crow + col0 + j) = o;
            }
          }
        }
      }
      if (has_k) {
        tc_fence_before();
        mbar_arrive(&acc_empty[as]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * Q_BN);
  }
}

}  // namespace ksana

using namespace ksana;

static long long* g_int4_trace = nullptr;
static int g_int4_dbg = 0;
KSANA_API void ksana_gemm_int4_set_debug(int mode) { g_int4_dbg = mode; }
// Debug hook: 256 int64 slots receiving CTA 0's per-k-block timeline of its first work unit (nullptr: off).
KSANA_API void ksana_gemm_int4_set_trace(void* buf) { g_int4_trace = reinterpret_cast<long long*>(buf); }

// A: [M, K] bf16 (row stride lda); Wq: tiled int32 words (see the top of the file; rows past N are zero padding);
// sz: [N, K/group, 2] fp32 (scale, zero) pairs; C: [M, N] bf16.
// group must be a multiple of 64, K a multiple of 64, N a multiple of 8. ws / counters: split-K scratch as for the
// bf16 GEMM (splits * M * N floats, one counter per output tile, zero on entry and left zero).
KSANA_API int ksana_gemm_int4(const void* A, const void* Wq, const float* sz, const void* bias,
                              void* C, int M, int N, int K, int lda, int ldc, int group, float* ws,
                              long long ws_floats, unsigned int* counters, int force_splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % Q_BK) || (group % Q_BK) || (K % group) || (N & 7) || (lda & 7) || (ldc & 7)) return -1;
  CUtensorMap tmA;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, Q_BM, Q_BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -2;
  if (reinterpret_cast<uintptr_t>(Wq) & 15) return -3;
  const int sms = sm_count();
  const int num_kb = K / Q_BK;
  const int tiles_m = (M + Q_BM - 1) / Q_BM;
  const bool wide = tiles_m * ((N + 255) / 256) >= sms;  // enough 128 x 256 tiles to fill the machine
  const int bn = wide ? 256 : 128;
  const int tiles = tiles_m * ((N + bn - 1) / bn);
  int splits = 1;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (tiles < sms) {
    splits = sms / tiles;
    if (splits > num_kb / 4) splits = num_kb / 4;  // at least 4 k-blocks per split
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
  }
  if (splits > 1) {
    // no empty splits: shrink until every split owns at least one k-block
    while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
    if (ws == nullptr || counters == nullptr || static_cast<long long>(splits) * M * N > ws_floats) splits = 1;
  }
  int grid = tiles * splits;
  if (grid > sms) grid = sms;
  if (KSANA_SMEM_ONCE(gemm_int4_kernel<128>, QCfg<128>::SMEM) != 0 ||
      KSANA_SMEM_ONCE(gemm_int4_kernel<256>, QCfg<256>::SMEM) != 0)
    return -4;
  auto Cb = reinterpret_cast<__nv_bfloat16*>(C);
  auto Bb = reinterpret_cast<const __nv_bfloat16*>(bias);
  auto Wb = reinterpret_cast<const uint8_t*>(Wq);
  auto S2 = reinterpret_cast<const float2*>(sz);
  if (wide)
    gemm_int4_kernel<256><<<grid, Q_THREADS, QCfg<256>::SMEM, stream>>>(tmA, Wb, S2, K / group, group, Cb, Bb, M, N, K,
                                                                        ldc, splits, ws, counters, error_word(),
                                                                        g_int4_trace, g_int4_dbg);
  else
    gemm_int4_kernel<128><<<grid, Q_THREADS, QCfg<128>::SMEM, stream>>>(tmA, Wb, S2, K / group, group, Cb, Bb, M, N, K,
                                                                        ldc, splits, ws, counters, error_word(),
                                                                        g_int4_trace, g_int4_dbg);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ---- decode-sized M (<= 64 tokens): weights on the M side of the MMA, dequantised straight into TMEM -----------------
// C^T[n, m] = sum_k W[n, k] * A[m, k]: the 128 weight rows of a tile are the 128 TMEM lanes. Dequantiser thread r owns
// weight row r: it reads its 32 raw bytes per k-block directly from the pre-tiled layout (one coalesced 4 KB read per
// CTA, prefetched two k-blocks ahead in registers), converts, and writes the 64 bf16 values as 32 packed columns of
// the MMA's A operand in TMEM (tcgen05.st) - no shared-memory staging, no swizzle, no proxy fence. The activations
// (<= 64 rows) are the B operand, streamed by TMA in 64-wide k-blocks. One CTA = one (weight tile, K split); CTAs are
// small (160 threads, 128 TMEM columns, ~40 KB shared memory) so four of them share an SM and hide each other's
// latencies. Split-K partials meet in the fp32 workspace; the last CTA of a tile reduces them in split order.
namespace ksana {

constexpr int QS_STAGES = 4;
constexpr int QS_THREADS = 160;

template <int MP>  // padded token count: 16, 32 or 64
__global__ void __launch_bounds__(QS_THREADS, 4)
gemm_int4_small_kernel(const __grid_constant__ CUtensorMap tmA, const uint8_t* __restrict__ wq_tiled,
                       const float2* __restrict__ sz, int groups_per_row, int group, __nv_bfloat16* __restrict__ C,
                       const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc, int splits,
                       float* __restrict__ ws, unsigned int* __restrict__ counters, unsigned int* err) {
  constexpr int ACT_BYTES = MP * Q_BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* act_full = reinterpret_cast<uint64_t*>(smem + QS_STAGES * ACT_BYTES);
  uint64_t* act_empty = act_full + QS_STAGES;
  uint64_t* a_ready = act_empty + QS_STAGES;  // [2] dequantised k-block written to TMEM (one arrival per warp)
  uint64_t* a_free = a_ready + 2;             // [2] the MMAs that read it retired
  uint64_t* acc_done = a_free + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = K / Q_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int tile = blockIdx.x / splits, split = blockIdx.x - tile * splits;
  const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
  const int n_kb = kb1 - kb0;  // >= 1 (the host never creates empty splits)

  if (threadIdx.x == 0) {
    for (int s = 0; s < QS_STAGES; ++s) {
      mbar_init(&act_full[s], 1);
      mbar_init(&act_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&a_ready[s], 4);
      mbar_init(&a_free[s], 1);
    }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_holder, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_D = tmem_base;        // MP columns (<= 64)
  const uint32_t tmem_A = tmem_base + 64;   // 2 x 32 columns

  if (warp == 4) {
    if (lane == 0) {
      // activations: TMA producer and MMA issuer in one thread (the loads run QS_STAGES k-blocks ahead)
      tma_prefetch_desc(&tmA);
      constexpr uint32_t idesc = umma_idesc(128, MP, 1, 1);
      bool ok = true;
      const int pre = n_kb < QS_STAGES ? n_kb : QS_STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&act_full[i], ACT_BYTES);
        tma_load_2d(smem + i * ACT_BYTES, &tmA, &act_full[i], (kb0 + i) * Q_BK, 0);
      }
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % QS_STAGES, b = i & 1;
        if (!mbar_wait_bounded(&act_full[s], (i / QS_STAGES) & 1, abort_flag, err) ||
            !mbar_wait_bounded(&a_ready[b], (i >> 1) & 1, abort_flag, err)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t db = umma_desc_k128(smem_u32(smem + s * ACT_BYTES));
#pragma unroll
        for (int k = 0; k < Q_BK / 16; ++k)
          umma_f16_ts(tmem_D, tmem_A + b * 32 + k * 8, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(&a_free[b]);
        umma_commit(&act_empty[s]);
        if (i + QS_STAGES < n_kb) {
          // refill this activation stage once its MMAs retired
          if (!mbar_wait_bounded(&act_empty[s], (i / QS_STAGES) & 1, abort_flag, err)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&act_full[s], ACT_BYTES);
          tma_load_2d(smem + s * ACT_BYTES, &tmA, &act_full[s], (kb0 + i + QS_STAGES) * Q_BK, 0);
        }
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    // ---------------- dequantisers: thread = weight row of the tile = TMEM lane ----------------
    const int row = threadIdx.x;
    const int n = tile * 128 + row;
    const int nn = n < N ? n : N - 1;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
    const int n_tiles128 = (N + 127) / 128;
    const size_t kstep = static_cast<size_t>(n_tiles128) * 256;  // uint4 between consecutive k-blocks of one row tile
    const uint4* wsrc = reinterpret_cast<const uint4*>(wq_tiled + (static_cast<size_t>(kb0) * n_tiles128 + tile) * Q_TILE_RAW) +
                        row * 2;
    const float2* szrow = sz + static_cast<size_t>(nn) * groups_per_row;
    const int g_last = groups_per_row - 1;
    int g_cur = (kb0 * Q_BK) / group;
    float2 q0 = __ldg(szrow + min(g_cur, g_last));
    float2 q1 = __ldg(szrow + min(g_cur + 1, g_last));
    uint4 r0a = __ldg(wsrc), r0b = __ldg(wsrc + 1);  // k-block i
    uint4 r1a = r0a, r1b = r0b;                      // k-block i + 1
    if (n_kb > 1) {
      r1a = __ldg(wsrc + kstep);
      r1b = __ldg(wsrc + kstep + 1);
    }
    bool ok = true;
    for (int i = 0; i < n_kb; ++i) {
      const int b = i & 1;
      uint4 r2a = r1a, r2b = r1b;
      if (i + 2 < n_kb) {  // prefetch k-block i + 2
        r2a = __ldg(wsrc + (i + 2) * kstep);
        r2b = __ldg(wsrc + (i + 2) * kstep + 1);
      }
      const int g = ((kb0 + i) * Q_BK) / group;
      if (g != g_cur) {
        g_cur = g;
        q0 = q1;
        q1 = __ldg(szrow + min(g + 1, g_last));
      }
      const int z = static_cast<int>(q0.y);
      const uint32_t zb = 0x43004300u | static_cast<uint32_t>(z) | (static_cast<uint32_t>(z) << 16);
      const uint32_t sc2 = pack_bf16(q0.x, q0.x);
      const uint32_t words[8] = {r0a.x, r0a.y, r0a.z, r0a.w, r0b.x, r0b.y, r0b.z, r0b.w};
      uint32_t o[32];
#pragma unroll
      for (int wv = 0; wv < 8; ++wv) {
        const uint32_t v = words[wv];
        const uint32_t t = v & 0x0F0F0F0Fu;
        const uint32_t u = (v >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          uint32_t x;
          asm("prmt.b32 %0, %1, %2, %3;" : "=r"(x) : "r"(t), "r"(u), "r"(0x4440u | (4u + p) << 8 | static_cast<uint32_t>(p)));
          x = (x & 0x00FF00FFu) | 0x43004300u;
          uint32_t d;
          asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(x), "r"(zb));
          asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[wv * 4 + p]) : "r"(d), "r"(sc2));
        }
      }
      // the A buffer is free once the MMAs of k-block i - 2 retired
      if (i >= 2 && !mbar_wait_bounded(&a_free[b], ((i - 2) >> 1) & 1, abort_flag, err)) {
        ok = false;
        break;
      }
      tc_fence_after();
      tmem_st32(tmem_A + lane_off + b * 32, o);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[b]);
      r0a = r1a;
      r0b = r1b;
      r1a = r2a;
      r1b = r2b;
    }
    // ---------------- epilogue: lane = output column n, TMEM columns = tokens ----------------
    if (ok && !mbar_wait_bounded(acc_done, 0, abort_flag, err)) ok = false;
    tc_fence_after();
    uint32_t acc[MP];
    if (MP == 64) {
      tmem_ld32(tmem_D + lane_off, acc);
      tmem_ld32(tmem_D + lane_off + 32, acc + 32);
    } else if (MP == 32) {
      tmem_ld32(tmem_D + lane_off, acc);
    } else {
      tmem_ld16(tmem_D + lane_off, acc);
    }
    tmem_wait_ld();
    const bool n_ok = n < N;
    bool reduce_here = ok;
    if (splits > 1) {
      // ws[split][m][n]: lanes write consecutive n
      if (ok && n_ok) {
#pragma unroll
        for (int m = 0; m < MP; ++m)
          if (m < M) ws[(static_cast<size_t>(split) * M + m) * N + n] = __uint_as_float(acc[m]);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&counters[tile], 1u);
        const int last = (prev == static_cast<unsigned int>(splits - 1));
        if (last) counters[tile] = 0;
        *last_flag = last;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      reduce_here = ok && (*last_flag != 0);
      __threadfence();
    }
    if (reduce_here && n_ok) {
      const float bv = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int m = 0; m < MP; ++m) {
        if (m < M) {
          float v;
          if (splits > 1) {
            // partials are added in split order (deterministic); eight independent loads in flight at a time
            v = 0.f;
            for (int s0 = 0; s0 < splits; s0 += 8) {
              float t[8];
#pragma unroll
              for (int q = 0; q < 8; ++q)
                t[q] = (s0 + q < splits) ? __ldcg(ws + (static_cast<size_t>(s0 + q) * M + m) * N + n) : 0.f;
#pragma unroll
              for (int q = 0; q < 8; ++q) v += t[q];
            }
          } else {
            v = __uint_as_float(acc[m]);
          }
          C[static_cast<size_t>(m) * ldc + n] = __float2bfloat16(v + bv);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

template <int MP>
static int launch_int4_small(const void* A, const void* Wq, const float* sz, const void* bias, void* C, int M, int N,
                             int K, int lda, int ldc, int group, int splits, float* ws, unsigned int* counters,
                             cudaStream_t stream) {
  constexpr int SMEM = QS_STAGES * MP * Q_BK * 2 + 256 + 1024;
  CUtensorMap tmA;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, MP, Q_BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -2;
  auto kern = gemm_int4_small_kernel<MP>;
  if (KSANA_SMEM_ONCE(kern, SMEM) != 0) return -4;
  const int tiles = (N + 127) / 128;
  kern<<<tiles * splits, QS_THREADS, SMEM, stream>>>(tmA, reinterpret_cast<const uint8_t*>(Wq),
                                                    reinterpret_cast<const float2*>(sz), K / group, group,
                                                    reinterpret_cast<__nv_bfloat16*>(C),
                                                    reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, splits, ws,
                                                    counters, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ksana

// Same contract as ksana_gemm_int4 for M <= 64.
KSANA_API int ksana_gemm_int4_small(const void* A, const void* Wq, const float* sz, const void* bias, void* C, int M,
                                    int N, int K, int lda, int ldc, int group, float* ws, long long ws_floats,
                                    unsigned int* counters, int n_counters, int force_splits, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || (K % Q_BK) || (group % Q_BK) || (K % group) || (lda & 7)) return -1;
  if (reinterpret_cast<uintptr_t>(Wq) & 15) return -3;
  const int tiles = (N + 127) / 128, num_kb = K / Q_BK;
  int splits = force_splits > 0 ? force_splits : 1;
  if (force_splits <= 0) {
    // aim at ~4 CTAs per SM, at least 8 k-blocks per split
    const int want = (4 * sm_count()) / tiles;  // rounded down: one wave of four CTAs per SM
    splits = want < 1 ? 1 : want;
    if (splits > num_kb / 8) splits = num_kb / 8;
    if (splits > 32) splits = 32;
    if (splits < 1) splits = 1;
  }
  while (splits > 1 && (splits - 1) * ((num_kb + splits - 1) / splits) >= num_kb) --splits;
  if (splits > 1 && (ws == nullptr || counters == nullptr || tiles > n_counters ||
                     static_cast<long long>(splits) * M * N > ws_floats))
    splits = 1;
  if (M <= 16) return ksana::launch_int4_small<16>(A, Wq, sz, bias, C, M, N, K, lda, ldc, group, splits, ws, counters, stream);
  if (M <= 32) return ksana::launch_int4_small<32>(A, Wq, sz, bias, C, M, N, K, lda, ldc, group, splits, ws, counters, stream);
  return ksana::launch_int4_small<64>(A, Wq, sz, bias, C, M, N, K, lda, ldc, group, splits, ws, counters, stream);
}
