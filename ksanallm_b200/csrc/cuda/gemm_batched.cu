// Head-batched bf16 GEMM for sm_100a: C[t, b, :] = A[t, b, :] * W[b]^T for every batch entry b (attention head),
// with A and C addressed through (row, batch) strides, so token-major activations [T, heads, dim] are read and
// written in place.
//
// This is the "absorb" step of multi-head latent attention: the query's no-position part times W_UK^T per head
// before the attention over the latent cache, and the attention output times W_UV per head after it. The reference
// runs them as strided-batched cuBLAS calls (src/ksana_llm/modules/attention/multihead_latent_attention.cpp:276-284,
// 368-373; InvokeStridedBatchedMatMul in src/ksana_llm/kernels/nvidia/basic_kernel_wrapper.cpp).
//
// Same pipeline as the grouped expert GEMM (moe.cu): warp 0 TMA producer, warp 1 tcgen05 issuer, warps 2-5 epilogue,
// accumulator double-buffered in TMEM, persistent loop over (batch, m-tile, n-tile). A is loaded through a 3-d tensor
// map (k, token, batch): one 128 x 64 box per k-block, whatever the strides between tokens and heads.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int BG_BM = 128, BG_BN = 128, BG_BK = 64, BG_STAGES = 6;
constexpr int BG_A_BYTES = BG_BM * BG_BK * 2, BG_B_BYTES = BG_BN * BG_BK * 2, BG_STAGE = BG_A_BYTES + BG_B_BYTES;
constexpr int BG_BAR = BG_STAGES * BG_STAGE;
constexpr int BG_SMEM = BG_BAR + 256 + 1024;

__global__ void __launch_bounds__(192, 1)
gemm_bf16_batched_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         __nv_bfloat16* __restrict__ C, long long c_row_stride, long long c_batch_stride, int T, int B,
                         int N, int K, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + BG_BAR);
  uint64_t* empty_bar = full_bar + BG_STAGES;
  uint64_t* acc_full = empty_bar + BG_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (T + BG_BM - 1) / BG_BM;
  const int tiles_n = N / BG_BN;
  const int num_kb = (K + BG_BK - 1) / BG_BK;
  const int per_batch = tiles_m * tiles_n;
  const int total = per_batch * B;

  if (threadIdx.x == 0) {
    for (int s = 0; s < BG_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * BG_BN);
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
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int b = tile / per_batch, r = tile - b * per_batch;
        const int mt = r / tiles_n, nt = r - mt * tiles_n;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * BG_STAGE;
          mbar_expect_tx(&full_bar[stage], BG_STAGE);
          tma_load_3d(sa, &tmA, &full_bar[stage], kb * BG_BK, mt * BG_BM, b);
          tma_load_2d(sa + BG_A_BYTES, &tmB, &full_bar[stage], kb * BG_BK, b * N + nt * BG_BN);
          if (++stage == BG_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BG_BM, BG_BN, 1, 1);
      int stage = 0, n_it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++n_it) {
        const int as = n_it & 1;
        if (!mbar_wait_bounded(&acc_empty[as], ((n_it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * BG_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + BG_A_BYTES);
#pragma unroll
          for (int k = 0; k < BG_BK / 16; ++k)
            umma_f16(tmem_base + as * BG_BN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == BG_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int n_it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++n_it) {
      const int b = tile / per_batch, r = tile - b * per_batch;
      const int mt = r / tiles_n, nt = r - mt * tiles_n;
      const int as = n_it & 1;
      uint32_t ok_in = mbar_wait_bounded(&acc_full[as], (n_it >> 1) & 1, abort_flag, err) ? 1u : 0u, ok_all;
      asm volatile(
          "{\n\t.reg .pred pin, pout;\n\t"
          "setp.ne.u32 pin, %1, 0;\n\t"
          "bar.red.and.pred pout, 1, 128, pin;\n\t"
          "selp.u32 %0, 1, 0, pout;\n\t}"
          : "=r"(ok_all)
          : "r"(ok_in)
          : "memory");
      if (!ok_all) break;
      tc_fence_after();
      const int row = mt * BG_BM + quarter * 32 + lane;
      const bool row_ok = row < T;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BG_BN;
      __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * c_row_stride +
                            static_cast<size_t>(b) * c_batch_stride + nt * BG_BN;
#pragma unroll 1
      for (int c = 0; c < BG_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(t_row + c * 32, rr);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(rr[j]), __uint_as_float(rr[j + 1]));
            o.y = pack_bf16(__uint_as_float(rr[j + 2]), __uint_as_float(rr[j + 3]));
            o.z = pack_bf16(__uint_as_float(rr[j + 4]), __uint_as_float(rr[j + 5]));
            o.w = pack_bf16(__uint_as_float(rr[j + 6]), __uint_as_float(rr[j + 7]));
            *reinterpret_cast<uint4*>(crow + c * 32 + j) = o;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BG_BN);
  }
}

}  // namespace ksana

using namespace ksana;

// C[t, b, 0:N] = A[t, b, 0:K] * W[b]^T for t < T, b < B. A element (t, b, k) at A + t * a_row_stride +
// b * a_batch_stride + k; C element (t, b, n) at C + t * c_row_stride + b * c_batch_stride + n; W: [B, N, K] contiguous.
// All bf16; strides in elements and multiples of 8, base pointers 16-byte aligned, N % 128 == 0, K % 8 == 0.
KSANA_API int ksana_gemm_bf16_batched(const void* A, long long a_row_stride, long long a_batch_stride, const void* W,
                                      void* C, long long c_row_stride, long long c_batch_stride, int T, int B, int N,
                                      int K, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if ((N % BG_BN) || (K & 7) || (a_row_stride & 7) || (a_batch_stride & 7) || (c_row_stride & 7) || (c_batch_stride & 7) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return -1;
  CUtensorMap tmA, tmB;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(K), static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
    const uint64_t strides[2] = {static_cast<uint64_t>(a_row_stride) * 2, static_cast<uint64_t>(a_batch_stride) * 2};
    const uint32_t box[3] = {BG_BK, BG_BM, 1};
    if (make_tmap_nd(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return -2;
  }
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(B) * N, K, K, BG_BN, BG_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (KSANA_SMEM_ONCE(gemm_bf16_batched_kernel, BG_SMEM) != 0) return -4;
  const int total = ((T + BG_BM - 1) / BG_BM) * (N / BG_BN) * B;
  int grid = sm_count();
  if (grid > total) grid = total;
  gemm_bf16_batched_kernel<<<grid, 192, BG_SMEM, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), c_row_stride,
                                                          c_batch_stride, T, B, N, K, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
