// ONE kernel for a row-parallel linear layer under tensor parallelism:
//   tcgen05 GEMM (this rank's K-slice)  ->  reduce-scatter over NVLink  ->  residual add + RMSNorm  ->  all-gather.
//
// It replaces the reference's sequence "cuBLAS GEMM into reduce_buffer -> custom / NCCL / TokenWeave all-reduce ->
// fused add + RMSNorm kernel" (src/ksana_llm/modules/attention/common_attention.cpp:64-75,
// modules/ffn/two_layered_ffn.cpp:108-118, modules/basic/all_reduce_fused_norm_add.cpp:30-53,
// layers/nvidia/custom_all_reduce_sum_layer.cpp:124-176) and is the fused compute + collective path of the engine.
//
// Grid = G GEMM CTAs + C communication CTAs, all resident at once (G + C <= SM count, one CTA per SM).
//  * GEMM CTAs run the persistent TMA -> tcgen05 -> TMEM pipeline of gemm_bf16.cu over 128 x 128 tiles in row-major
//    tile order, so the rows owned by rank 0 finish first, then rank 1's, ... The epilogue does NOT write a local
//    result: each thread stores its row's 128 bf16 straight into the OWNER rank's receive buffer
//    recv[owner][source = this rank][row - owner_first_row][col] with 16-byte peer stores (row r is owned by rank
//    r / rows_per), then the tile is published with a system-scope release add on the owner's arrival counter of
//    that 128-row band.
//  * Communication CTAs of the owner poll those counters (bounded wait). As soon as a band has all
//    world_size x (N / 128) tile contributions they sum the per-source slots in fixed rank order (deterministic),
//    add the owner's slice of the residual stream, apply RMSNorm and broadcast the normalised rows into every
//    rank's activation buffer (multimem.st through the NVSwitch when a multicast mapping exists, else peer
//    stores). NVLink transfers of early bands therefore overlap the tensor-core work on later bands.
//  * End of call: the last communication CTA resets the counters, tells every peer "my rows are out" and waits for
//    the same message from all of them, so when the kernel ends the full normalised activation is local.
// No TMA touches peer memory (tiles are pushed with ordinary stores), every wait is bounded.
#include "comm.cuh"
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int FR_BM = 128, FR_BN = 128, FR_BK = 64, FR_STAGES = 6;
constexpr int FR_A_BYTES = FR_BM * FR_BK * 2, FR_B_BYTES = FR_BN * FR_BK * 2, FR_STAGE = FR_A_BYTES + FR_B_BYTES;
constexpr int FR_BAR = FR_STAGES * FR_STAGE;
constexpr int FR_SMEM = FR_BAR + 256 + 1024;
constexpr int FR_MAX_RANKS = 8;
constexpr int FR_SIG_BAND = 5000;   // [64] arrival counters per 128-row band (in the owner's signal buffer)
constexpr int FR_SIG_DONE = 5100;   // [8] end-of-call flags
constexpr int FR_SIG_LOCAL = 5120;  // local counter of finished communication CTAs
constexpr int FR_VPT = 6;           // 192 threads x 6 x 8 = 9216 >= H

struct FusedRsCtx {
  int rank, ws;
  __nv_bfloat16* recv[FR_MAX_RANKS];  // each rank's receive buffer [ws][rows_cap][H]
  __nv_bfloat16* hbuf[FR_MAX_RANKS];  // each rank's activation buffer [T, H]
  uint32_t* sig[FR_MAX_RANKS];
  __nv_bfloat16* hbuf_mc;             // multicast view of hbuf or nullptr
  int rows_cap;                       // row capacity of one source slot in recv
};

__global__ void __launch_bounds__(192, 1)
gemm_rs_norm_ag_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, FusedRsCtx ctx,
                       int M, int N, int K, __nv_bfloat16* __restrict__ residual,
                       const __nv_bfloat16* __restrict__ norm_w, float eps, uint32_t epoch, int gemm_ctas, int mode,
                       unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + FR_BM - 1) / FR_BM;
  const int tiles_n = N / FR_BN;
  const int rank = ctx.rank, ws = ctx.ws;
  const int rows_per = (M + ws - 1) / ws;

  if (static_cast<int>(blockIdx.x) >= gemm_ctas) {
    // ======================= communication CTA (owner side) =======================
    const int c_idx = blockIdx.x - gemm_ctas;
    const int c_num = gridDim.x - gemm_ctas;
    uint32_t* my_sig = ctx.sig[rank];
    const int row_lo = rank * rows_per;
    const int row_hi = min(M, row_lo + rows_per);
    __shared__ float red[6];
    __shared__ int s_ok;
    const int tid = threadIdx.x;
    if (row_lo < row_hi) {
      const int band_lo = row_lo / FR_BM, band_hi = (row_hi - 1) / FR_BM;
      for (int band = band_lo + c_idx; band <= band_hi; band += c_num) {
        if (tid == 0) s_ok = wait_flag_ge(my_sig + FR_SIG_BAND + band, static_cast<uint32_t>(ws * tiles_n), err) ? 1 : 0;
        __syncthreads();
        const bool ok = s_ok != 0;
        __syncthreads();
        if (!ok) break;
        const int r0 = max(row_lo, band * FR_BM), r1 = min(row_hi, (band + 1) * FR_BM);
        for (int row = r0; row < r1; ++row) {
          const int lrow = row - row_lo;
          float v[FR_VPT][8];
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < FR_VPT; ++i) {
            const int c = (i * 192 + tid) * 8;
            if (c < N) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
              for (int p = 0; p < ws; ++p) {
                float t[8];
                // pushed by peers with system-scope stores: bypass L1
                unpack8(ld_peer16(ctx.recv[rank] + (static_cast<size_t>(p) * ctx.rows_cap + lrow) * N + c), t);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] += t[j];
              }
              const size_t off = static_cast<size_t>(row) * N + c;
              if (mode & 2) {
                float r[8];
                unpack8(*reinterpret_cast<const uint4*>(residual + off), r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] += r[j];
                const uint4 packed = pack8(v[i]);
                *reinterpret_cast<uint4*>(residual + off) = packed;
                unpack8(packed, v[i]);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
            }
          }
          float inv = 1.f;
          if (mode & 1) {
            ss = warp_sum(ss);
            __syncthreads();
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < 6; ++i) tot += red[i];
            inv = rsqrtf(tot / static_cast<float>(N) + eps);
          }
#pragma unroll
          for (int i = 0; i < FR_VPT; ++i) {
            const int c = (i * 192 + tid) * 8;
            if (c < N) {
              const size_t off = static_cast<size_t>(row) * N + c;
              float o[8];
              if (mode & 1) {
                float g[8];
                unpack8(*reinterpret_cast<const uint4*>(norm_w + c), g);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * g[j];
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[i][j];
              }
              const uint4 packed = pack8(o);
              if (ctx.hbuf_mc != nullptr) {
                multimem_st16(ctx.hbuf_mc + off, packed);
              } else {
                for (int p = 0; p < ws; ++p) st_peer16(ctx.hbuf[p] + off, packed);
              }
            }
          }
        }
        if (tid == 0) my_sig[FR_SIG_BAND + band] = 0;  // consumed: ready for the next call
      }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (tid == 0) {
      const uint32_t prev = atomicAdd(my_sig + FR_SIG_LOCAL, 1u);
      s_last = (prev == static_cast<uint32_t>(c_num - 1));
      if (s_last) my_sig[FR_SIG_LOCAL] = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence_system();
      if (tid < ws) st_release_sys(ctx.sig[tid] + FR_SIG_DONE + rank, epoch);
      if (tid < ws) wait_flag_ge(my_sig + FR_SIG_DONE + tid, epoch, err);
    }
    return;
  }

  // ======================= GEMM CTA =======================
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + FR_BAR);
  uint64_t* empty_bar = full_bar + FR_STAGES;
  uint64_t* acc_full = empty_bar + FR_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int num_kb = (K + FR_BK - 1) / FR_BK;
  const int total_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < FR_STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 2 * FR_BN);
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gemm_ctas) {
        const int m_idx = tile / tiles_n, n_idx = tile - m_idx * tiles_n;  // row-major: low rows complete first
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * FR_STAGE;
          mbar_expect_tx(&full_bar[stage], FR_STAGE);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * FR_BK, m_idx * FR_BM);
          tma_load_2d(sa + FR_A_BYTES, &tmB, &full_bar[stage], kb * FR_BK, n_idx * FR_BN);
          if (++stage == FR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FR_BM, FR_BN, 1, 1);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gemm_ctas, ++it) {
        const int as = it & 1;
        if (!mbar_wait_bounded(&acc_empty[as], ((it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * FR_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + FR_A_BYTES);
#pragma unroll
          for (int k = 0; k < FR_BK / 16; ++k)
            umma_f16(tmem_base + as * FR_BN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == FR_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
      }
    }
  } else {
    // epilogue: push the tile to the owners of its rows, then publish it
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gemm_ctas, ++it) {
      const int m_idx = tile / tiles_n, n_idx = tile - m_idx * tiles_n;
      const int as = it & 1;
      uint32_t ok_in = mbar_wait_bounded(&acc_full[as], (it >> 1) & 1, abort_flag, err) ? 1u : 0u, ok_all;
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
      const int row = m_idx * FR_BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const int owner = row_ok ? row / rows_per : 0;
      const int lrow = row_ok ? row - owner * rows_per : 0;
      __nv_bfloat16* drow = ctx.recv[owner] + (static_cast<size_t>(rank) * ctx.rows_cap + lrow) * N + n_idx * FR_BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * FR_BN;
#pragma unroll 1
      for (int c = 0; c < FR_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            o.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            o.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            o.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            st_peer16(drow + c * 32 + j, o);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      __threadfence_system();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int first_row = m_idx * FR_BM;
        const int last_row = min(M, first_row + FR_BM) - 1;
        for (int o = first_row / rows_per; o <= last_row / rows_per; ++o)
          red_release_sys_add(ctx.sig[o] + FR_SIG_BAND + m_idx, 1u);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * FR_BN);
  }
}

}  // namespace ksana

using namespace ksana;

// y = AllGather(RMSNorm(residual_slice += ReduceScatter(A * W^T)) * norm_w) in one launch.
// A: [M, K] bf16 (pitch lda), W: [N, K] bf16 (pitch ldw); recv/hbuf/sig: per-rank symmetric buffer pointers
// (recv: [ws][rows_cap][N] bf16, hbuf: [>= M][N] bf16, sig: >= 8192 uint32, zero-initialised once).
// N % 128 == 0, N <= 9216, M <= 64 * 128. mode bit0: RMSNorm, bit1: residual add (residual [M, N], row-sharded).
KSANA_API int ksana_gemm_rs_norm_ag(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank,
                                    int ws, void* const* recv, void* const* hbuf, void* const* sig, void* hbuf_mc,
                                    int rows_cap, void* residual, const void* norm_w, float eps, unsigned int epoch,
                                    int mode, int comm_ctas, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (ws < 1 || ws > FR_MAX_RANKS || (N % FR_BN) || N > 192 * FR_VPT * 8 || (K & 7) || (lda & 7) || (ldw & 7) ||
      M > 64 * FR_BM || (M + ws - 1) / ws > rows_cap)
    return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, FR_BM, FR_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, FR_BN, FR_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  FusedRsCtx ctx;
  ctx.rank = rank;
  ctx.ws = ws;
  for (int i = 0; i < FR_MAX_RANKS; ++i) {
    ctx.recv[i] = i < ws ? reinterpret_cast<__nv_bfloat16*>(recv[i]) : nullptr;
    ctx.hbuf[i] = i < ws ? reinterpret_cast<__nv_bfloat16*>(hbuf[i]) : nullptr;
    ctx.sig[i] = i < ws ? reinterpret_cast<uint32_t*>(sig[i]) : nullptr;
  }
  ctx.hbuf_mc = reinterpret_cast<__nv_bfloat16*>(hbuf_mc);
  ctx.rows_cap = rows_cap;
  static bool once = false;
  if (!once) {
    if (cudaFuncSetAttribute(gemm_rs_norm_ag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FR_SMEM) != cudaSuccess)
      return -4;
    once = true;
  }
  const int sms = sm_count();
  if (comm_ctas <= 0) comm_ctas = 16;
  const int rows_per = (M + ws - 1) / ws;
  const int my_bands = (rows_per + FR_BM - 1) / FR_BM + 1;
  if (comm_ctas > my_bands) comm_ctas = my_bands;
  if (comm_ctas < 1) comm_ctas = 1;
  const int tiles = ((M + FR_BM - 1) / FR_BM) * (N / FR_BN);
  int gemm_ctas = sms - comm_ctas;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  if (gemm_ctas < 1) return -1;
  gemm_rs_norm_ag_kernel<<<gemm_ctas + comm_ctas, 192, FR_SMEM, stream>>>(
      tmA, tmB, ctx, M, N, K, reinterpret_cast<__nv_bfloat16*>(residual),
      reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, epoch, gemm_ctas, mode, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
