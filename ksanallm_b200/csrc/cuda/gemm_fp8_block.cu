// Block-scaled fp8 GEMM for sm_100a: C[M, N] = sum_kb (sa[m, kb] * sw[n / 128, kb]) * (A8[m, kb] . W8[n, kb]) (+ bias)
// with e4m3 activations quantised per token per 128 channels (sa: [M, K/128] fp32) and e4m3 weights scaled per
// 128 x 128 block (sw: [ceil(N/128), K/128] fp32 = the checkpoint's weight_scale_inv).
//
// Replaces the three back-ends the reference profiles at load time (DeepGEMM JIT, CUTLASS sm90 block-scaled,
// TRT-LLM fp8_blockscale_gemm: src/ksana_llm/layers/nvidia/blockwise_matmul_layer.cpp:71-301), none of which has
// an sm_100 build. Here the K loop is cut at the 128-wide scale blocks: each K-block is a fresh tcgen05
// accumulation (4 x kind::f8f6f4 MMAs of K = 32) into one of two TMEM buffers, and eight "promotion" warps fold
// the finished block into fp32 register accumulators with its scale product while the tensor core already works
// on the next block (2-level accumulation with exact fp32 scales, no UE8M0 rounding of the scales).
//   warp 0: TMA (128 x 128-byte A tile + 128 x 128-byte W tile per stage, 128-byte swizzle)
//   warp 1: TMEM alloc + MMA issue
//   warps 2-5 / 6-9: promotion + epilogue for columns [0, 64) / [64, 128) of the tile
// Split-K over an fp32 workspace as in the bf16 kernel.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int F8_BM = 128;
constexpr int F8_BN = 128;
constexpr int F8_BK = 128;  // bytes = elements
constexpr int F8_STAGES = 6;
constexpr int F8_STAGE_BYTES = (F8_BM + F8_BN) * F8_BK;
constexpr int F8_BAR_OFFSET = F8_STAGES * F8_STAGE_BYTES;
constexpr int F8_SMEM = F8_BAR_OFFSET + 256 + 1024;
constexpr int F8_THREADS = 320;

template <typename OutT>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const float* __restrict__ sa, const float* __restrict__ sw, OutT* __restrict__ C,
                      const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc, int splits,
                      float* __restrict__ ws, unsigned int* __restrict__ counters, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + F8_BAR_OFFSET);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* acc_full = empty_bar + F8_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + F8_BM - 1) / F8_BM;
  const int tiles_n = (N + F8_BN - 1) / F8_BN;
  const int num_kb = K / F8_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_units = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 256);
    }
    *abort_flag = 0;
    *last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * F8_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
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
          uint8_t* sA = smem + stage * F8_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], F8_STAGE_BYTES);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * F8_BK, m_idx * F8_BM);
          tma_load_2d(sA + F8_BM * F8_BK, &tmB, &full_bar[stage], kb * F8_BK, n_idx * F8_BN);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(F8_BM, F8_BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t blk = 0;  // running K-block counter -> TMEM buffer / phase
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
        for (int kb = kb0; kb < kb1; ++kb, ++blk) {
          const int buf = blk & 1;
          if (!mbar_wait_bounded(&acc_empty[buf], ((blk >> 1) & 1) ^ 1, abort_flag, err) ||
              !mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * F8_STAGE_BYTES);
          const uint64_t da = umma_desc_k128(sA);
          const uint64_t db = umma_desc_k128(sA + F8_BM * F8_BK);
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            umma_f8(tmem_base + buf * F8_BN, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&acc_full[buf]);
          if (++stage == F8_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // ---------------- promotion + epilogue: 8 warps, 64 columns per thread ----------------
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;  // 0: columns [0, 64), 1: [64, 128)
    const int kscales = K / F8_BK;
    uint32_t blk = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
      const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
      const int row = m_idx * F8_BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const float* sa_row = sa + static_cast<size_t>(row_ok ? row : 0) * kscales;
      const float* sw_row = sw + static_cast<size_t>(n_idx) * kscales;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      bool alive = true;
      for (int kb = kb0; kb < kb1; ++kb, ++blk) {
        const int buf = blk & 1;
        uint32_t ok_in = mbar_wait_bounded(&acc_full[buf], (blk >> 1) & 1, abort_flag, err) ? 1u : 0u, ok_all;
        asm volatile(
            "{\n\t.reg .pred pin, pout;\n\t"
            "setp.ne.u32 pin, %1, 0;\n\t"
            "bar.red.and.pred pout, 1, 256, pin;\n\t"
            "selp.u32 %0, 1, 0, pout;\n\t}"
            : "=r"(ok_all)
            : "r"(ok_in)
            : "memory");
        if (!ok_all) {
          alive = false;
          break;
        }
        tc_fence_after();
        const float scale = (row_ok ? __ldg(sa_row + kb) : 0.f) * __ldg(sw_row + kb);
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * F8_BN + col_half * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c * 32 + j] = fmaf(scale, __uint_as_float(r[j]), acc[c * 32 + j]);
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
      }
      if (!alive) break;
      const int col_base = n_idx * F8_BN + col_half * 64;
      bool reduce_here = true;
      if (splits > 1) {
        if (row_ok) {
          float* wrow = ws + (static_cast<size_t>(split) * M + row) * N + col_base;
#pragma unroll
          for (int j = 0; j < 64; j += 4)
            if (col_base + j < N)
              *reinterpret_cast<float4*>(wrow + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        }
        __threadfence();
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (threadIdx.x == 64) {
          const unsigned int prev = atomicAdd(&counters[tile], 1u);
          const int last = (prev == static_cast<unsigned int>(splits - 1));
          if (last) counters[tile] = 0;
          *last_flag = last;
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");
        reduce_here = (*last_flag != 0);
        __threadfence();
        if (reduce_here && row_ok) {
#pragma unroll
          for (int j = 0; j < 64; ++j) acc[j] = 0.f;
          for (int s = 0; s < splits; ++s) {
            const float* wrow = ws + (static_cast<size_t>(s) * M + row) * N + col_base;
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
              if (col_base + j < N) {
                const float4 p = __ldcg(reinterpret_cast<const float4*>(wrow + j));
                acc[j] += p.x;
                acc[j + 1] += p.y;
                acc[j + 2] += p.z;
                acc[j + 3] += p.w;
              }
            }
          }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");  // last_flag may be rewritten by the next unit
      }
      if (reduce_here && row_ok) {
        OutT* crow = C + static_cast<size_t>(row) * ldc;
        if (bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (col_base + j < N) acc[j] += __bfloat162float(bias[col_base + j]);
        }
        if constexpr (sizeof(OutT) == 2) {
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            if (col_base + j < N) {
              uint4 o;
              o.x = pack_bf16(acc[j], acc[j + 1]);
              o.y = pack_bf16(acc[j + 2], acc[j + 3]);
              o.z = pack_bf16(acc[j + 4], acc[j + 5]);
              o.w = pack_bf16(acc[j + 6], acc[j + 7]);
              *reinterpret_cast<uint4*>(crow + col_base + j) = o;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; j += 4)
            if (col_base + j < N)
              *reinterpret_cast<float4*>(crow + col_base + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * F8_BN);
  }
}

}  // namespace ksana

using namespace ksana;

// A8: [M, K] e4m3 (row pitch lda bytes), sa: [M, K/128] fp32; W8: [N, K] e4m3 (row pitch ldw), sw: [ceil(N/128), K/128].
// C: [M, N] bf16 (out_fp32 = 0) or fp32, row pitch ldc elements. K % 128 == 0, N % 8 == 0, lda/ldw % 16 == 0.
KSANA_API int ksana_gemm_fp8_block(const void* A8, const float* sa, const void* W8, const float* sw, void* C,
                                   const void* bias, int M, int N, int K, int lda, int ldw, int ldc, int out_fp32,
                                   int force_splits, float* ws, long long ws_floats, unsigned int* counters,
                                   int num_counters, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 127) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 3)) return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, F8_BM, F8_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldw, F8_BN, F8_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  const int sms = sm_count();
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int num_kb = K / F8_BK;
  int splits = 1;
  if (force_splits > 0) splits = force_splits;
  else if (tiles * 2 <= sms && num_kb >= 8) {
    splits = sms / tiles;
    if (splits > 8) splits = 8;
    if (splits > num_kb / 4) splits = num_kb / 4;
    if (splits < 1) splits = 1;
  }
  while (splits > 1 && ((num_kb + splits - 1) / splits) * (splits - 1) >= num_kb) --splits;
  if (splits > 1 && (ws == nullptr || counters == nullptr || static_cast<long long>(splits) * M * N > ws_floats ||
                     tiles > num_counters))
    splits = 1;
  int grid = tiles * splits;
  if (grid > sms) grid = sms;
  if (out_fp32) {
    auto kern = gemm_fp8_block_kernel<float>;
    if (KSANA_SMEM_ONCE(kern, F8_SMEM) != 0) return -4;
    kern<<<grid, F8_THREADS, F8_SMEM, stream>>>(tmA, tmB, sa, sw, reinterpret_cast<float*>(C),
                                                reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, splits, ws,
                                                counters, error_word());
  } else {
    auto kern = gemm_fp8_block_kernel<__nv_bfloat16>;
    if (KSANA_SMEM_ONCE(kern, F8_SMEM) != 0) return -4;
    kern<<<grid, F8_THREADS, F8_SMEM, stream>>>(tmA, tmB, sa, sw, reinterpret_cast<__nv_bfloat16*>(C),
                                                reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, splits, ws,
                                                counters, error_word());
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
