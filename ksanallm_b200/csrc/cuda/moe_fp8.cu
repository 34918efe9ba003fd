// Block-scaled fp8 grouped expert GEMM and the fused SiLU * mul + 1 x 128 activation quantiser for sm_100a.
//
// The reference serves DeepSeek-style fp8 MoE layers through a Triton fused-MoE kernel with 128 x 128 weight
// blocks and per-token-group activation scales (src/ksana_llm/kernels/nvidia/moe_kernel_wrapper.cpp:463-655,
// 3rdparty/LLM_kernels/csrc/kernels/nvidia/moe/fused_moe/fused_moe.py, backend choice in
// src/ksana_llm/layers/moe_layer_factory.cpp:26-70) and quantises the SiLU output with a fused kernel
// (.../others/sglang/main/quantization/fp8/per_token_group_quant.cu:265-269). Here:
//
//  * moe_grouped_gemm_fp8_kernel: C[rows of expert e, N] = sum_kb sa[row, kb] * sw[e][n / 128][kb] *
//    (A8[row, kb] . W8[e][n, kb]) over the expert-sorted rows. Tile walk over (expert, m-tile, n-tile) from
//    device-side offsets as in the bf16 grouped kernel (moe.cu), K loop and two-level accumulation as in
//    gemm_fp8_block.cu: every 128-wide K block is a fresh tcgen05 kind::f8f6f4 accumulation into one of two TMEM
//    buffers; eight promotion warps fold it into fp32 registers with the exact fp32 scale product while the tensor
//    core works on the next block. No host synchronisation anywhere: ragged and empty experts cost nothing.
//  * silu_mul_quant_kernel: h[row, :I] = SiLU(gate) * up in fp32 -> e4m3 with one scale per 128 outputs, so the
//    activation between the two expert GEMMs is written once, as fp8.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int GF_BM = 128, GF_BN = 128, GF_BK = 128, GF_STAGES = 6;
constexpr int GF_STAGE = (GF_BM + GF_BN) * GF_BK;
constexpr int GF_BAR = GF_STAGES * GF_STAGE;
constexpr int GF_SMEM = GF_BAR + 256 + 1024;
constexpr int GF_THREADS = 320;

struct GroupedTileIterF8 {
  const int* offsets;
  int E, tiles_n, stride, next, e, base;
  __device__ GroupedTileIterF8(const int* off, int E_, int tiles_n_, int first, int stride_)
      : offsets(off), E(E_), tiles_n(tiles_n_), stride(stride_), next(first), e(0), base(0) {}
  __device__ bool get(int* expert, int* mt, int* nt) {
    while (e < E) {
      const int rows = offsets[e + 1] - offsets[e];
      const int tiles = ((rows + GF_BM - 1) / GF_BM) * tiles_n;
      if (next < base + tiles) {
        const int local = next - base;
        *expert = e;
        *mt = local / tiles_n;
        *nt = local - (*mt) * tiles_n;
        next += stride;
        return true;
      }
      base += tiles;
      ++e;
    }
    return false;
  }
};

__global__ void __launch_bounds__(GF_THREADS, 1)
moe_grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const float* __restrict__ sa, const float* __restrict__ sw,
                            __nv_bfloat16* __restrict__ C, const int* __restrict__ offsets, int E, int N, int K,
                            int ldc, int sa_stride, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + GF_BAR);
  uint64_t* empty_bar = full_bar + GF_STAGES;
  uint64_t* acc_full = empty_bar + GF_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + GF_BN - 1) / GF_BN;
  const int num_kb = K / GF_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GF_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 256);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * GF_BN);
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
      GroupedTileIterF8 it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
      int stage = 0, e, mt, nt;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && it.get(&e, &mt, &nt)) {
        const int row0 = offsets[e] + mt * GF_BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * GF_STAGE;
          mbar_expect_tx(&full_bar[stage], GF_STAGE);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * GF_BK, row0);
          tma_load_2d(sA + GF_BM * GF_BK, &tmB, &full_bar[stage], kb * GF_BK, e * N + nt * GF_BN);
          if (++stage == GF_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(GF_BM, GF_BN, 0, 0);
      GroupedTileIterF8 it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
      int stage = 0, e, mt, nt;
      uint32_t phase = 0, blk = 0;
      bool ok = true;
      while (ok && it.get(&e, &mt, &nt)) {
        for (int kb = 0; kb < num_kb; ++kb, ++blk) {
          const int buf = blk & 1;
          if (!mbar_wait_bounded(&acc_empty[buf], ((blk >> 1) & 1) ^ 1, abort_flag, err) ||
              !mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * GF_STAGE);
          const uint64_t da = umma_desc_k128(sA), db = umma_desc_k128(sA + GF_BM * GF_BK);
#pragma unroll
          for (int k = 0; k < GF_BK / 32; ++k)
            umma_f8(tmem_base + buf * GF_BN, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          umma_commit(&acc_full[buf]);
          if (++stage == GF_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // promotion + epilogue: 8 warps, each thread owns one row and 64 columns of the tile
    const int quarter = warp & 3;
    const int col_half = (warp - 2) >> 2;
    const int n_blocks = (N + 127) / 128;  // weight scale blocks along N per expert
    GroupedTileIterF8 it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
    int e, mt, nt;
    uint32_t blk = 0;
    bool alive = true;
    while (alive && it.get(&e, &mt, &nt)) {
      const int row = offsets[e] + mt * GF_BM + quarter * 32 + lane;
      const bool row_ok = row < offsets[e + 1];
      const float* sa_row = sa + static_cast<size_t>(row_ok ? row : 0) * sa_stride;
      const float* sw_row = sw + (static_cast<size_t>(e) * n_blocks + nt) * num_kb;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb, ++blk) {
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
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * GF_BN + col_half * 64;
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
      if (row_ok) {
        const int col_base = nt * GF_BN + col_half * 64;
        __nv_bfloat16* crow = C + static_cast<size_t>(row) * ldc;
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
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * GF_BN);
  }
}

// One warp per (row, 128 outputs): a = SiLU(gate) * up in fp32, amax over the 128 -> scale = amax / 448, q = a / scale.
// x: [T, 2 I] bf16 (gate columns then up columns), q: [T, I] e4m3, scales: [T, I / 128] fp32.
__global__ void silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_fp8_e4m3* __restrict__ q,
                                      int ldq, float* __restrict__ scales, int T, int I) {
  const int groups = I >> 7;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= T * groups) return;
  const int t = gw / groups, g = gw - t * groups;
  const __nv_bfloat16* gp = x + static_cast<size_t>(t) * ldx + g * 128 + lane * 4;
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + 2));
  const float2 u0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + I));
  const float2 u1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gp + I + 2));
  // the product is rounded to bf16 first, exactly what the unfused SiLU * mul kernel hands to the quantiser
  const float a0 = __bfloat162float(__float2bfloat16(g0.x / (1.f + __expf(-g0.x)) * u0.x));
  const float a1 = __bfloat162float(__float2bfloat16(g0.y / (1.f + __expf(-g0.y)) * u0.y));
  const float a2 = __bfloat162float(__float2bfloat16(g1.x / (1.f + __expf(-g1.x)) * u1.x));
  const float a3 = __bfloat162float(__float2bfloat16(g1.y / (1.f + __expf(-g1.y)) * u1.y));
  float amax = fmaxf(fmaxf(fabsf(a0), fabsf(a1)), fmaxf(fabsf(a2), fabsf(a3)));
  amax = fmaxf(warp_max(amax), 1e-10f);
  const float inv = 448.f / amax;
  __nv_fp8_e4m3 o[4] = {__nv_fp8_e4m3(a0 * inv), __nv_fp8_e4m3(a1 * inv), __nv_fp8_e4m3(a2 * inv),
                        __nv_fp8_e4m3(a3 * inv)};
  *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * ldq + g * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) scales[static_cast<size_t>(t) * groups + g] = amax / 448.f;
}

}  // namespace ksana

using namespace ksana;

// C[sorted rows, N] (bf16) = block-scaled A8[sorted rows, K] * W8[e]^T per expert.
// A8: [max_rows, K] e4m3 with row pitch lda bytes (a multiple of 16), sa: fp32 scales, K / 128 per row, rows
// sa_stride floats apart (rows that carry their scales behind their values pass lda = K + K / 32 and
// sa = A8 + K); W8: [E, N, K] e4m3 contiguous, sw: [E, ceil(N / 128), K / 128] fp32; offsets: [E + 1] device ints
// (rows of expert e are [offsets[e], offsets[e + 1])). K % 128 == 0, N % 8 == 0.
KSANA_API int ksana_moe_grouped_gemm_fp8(const void* A8, int lda, const float* sa, int sa_stride, const void* W8,
                                         const float* sw, void* C, const int* offsets, int E, int max_rows, int N,
                                         int K, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if ((K & 127) || (N & 7) || (lda & 15) || lda < K || sa_stride < K / 128) return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, max_rows, K, lda, GF_BM, GF_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, static_cast<uint64_t>(E) * N, K, K, GF_BN, GF_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (KSANA_SMEM_ONCE(moe_grouped_gemm_fp8_kernel, GF_SMEM) != 0) return -4;
  moe_grouped_gemm_fp8_kernel<<<sm_count(), GF_THREADS, GF_SMEM, stream>>>(
      tmA, tmB, sa, sw, reinterpret_cast<__nv_bfloat16*>(C), offsets, E, N, K, N, sa_stride, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// x: [T, 2 I] bf16 (row pitch ldx) -> q [T, I] e4m3 (row pitch ldq bytes) + scales [T, I / 128]. I % 128 == 0.
KSANA_API int ksana_silu_mul_quant_fp8(const void* x, int ldx, void* q, int ldq, float* scales, int T, int I,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((I & 127) || (ldx & 3) || (ldq & 3)) return -1;
  const long long warps = static_cast<long long>(T) * (I / 128);
  silu_mul_quant_kernel<<<static_cast<unsigned int>((warps + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_fp8_e4m3*>(q), ldq, scales, T, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
