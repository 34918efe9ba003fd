// All-gather -> GEMM in one kernel: C[T, N] = concat_r(A_r)[T, K] * W[N, K]^T where A_r (rows_per rows) lives in rank
// r's symmetric buffer. Every CTA carries 8 communication warps next to its 6 GEMM warps. The communication warps of
// all CTAs deal the remote rows among themselves, pull each row ONCE over NVLink (peer loads) into a local staging
// buffer and bump the row band's arrival counter; the TMA producer walks the tiles starting with the local rows (so
// the tensor cores are busy while remote rows are still in flight), and waits for a band's counter before its first
// load from that band. Remote rows therefore cross NVLink once and every re-read by other column tiles hits local L2
// (reading A tiles straight from peer memory re-crosses the link for each of the N / 256 column tiles: measured 4-5x
// slower than all-gather + GEMM). The last CTA to finish tells every peer that this rank is done reading, which is
// what lets the owners overwrite their rows for the next call.
// The reference all-gathers with NCCL and then runs cuBLAS (src/ksana_llm/layers/nvidia/nccl_all_gather_layer.cpp:15-58
// followed by matmul_layer.cpp); TokenWeave's fused_rs_ln_ag kernel (3rdparty/LLM_kernels/csrc/kernels/nvidia/others/
// tokenweave) gathers inside the norm kernel instead.
// Pipeline: same warp-specialised tcgen05 main loop as gemm_bf16.cu (128 x 256 tiles, 4 stages, double-buffered TMEM).
#include "comm.cuh"
#include "host_common.h"

namespace ksana {

constexpr int AG_BM = 128, AG_BN = 256, AG_BK = 64, AG_STAGES = 4, AG_MAX_RANKS = 8;
constexpr int AG_A_BYTES = AG_BM * AG_BK * 2, AG_B_BYTES = AG_BN * AG_BK * 2, AG_STAGE = AG_A_BYTES + AG_B_BYTES;
constexpr int AG_BAR = AG_STAGES * AG_STAGE;
constexpr int AG_SMEM = AG_BAR + 256 + 1024;

struct AgMaps {
  CUtensorMap a[AG_MAX_RANKS];
};
constexpr int AG_COMM_WARPS = 8, AG_THREADS = 192 + 32 * AG_COMM_WARPS, AG_MAX_BANDS = 64;
struct AgCtx {
  int rank, ws;
  uint32_t* flags[AG_MAX_RANKS];          // per rank: ready[ws] | done[ws] | arrival counter | band counters
  const __nv_bfloat16* a[AG_MAX_RANKS];   // every rank's rows
  __nv_bfloat16* staged;                  // local [ws * rows_per, K] copy of the remote rows
};

__global__ void __launch_bounds__(AG_THREADS, 1)
gemm_ag_kernel(const __grid_constant__ AgMaps maps, const __grid_constant__ CUtensorMap tmB, AgCtx ctx,
               __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int rows_per, int T, int N, int K,
               int lda, int ldc, uint32_t epoch, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + AG_BAR);
  uint64_t* empty_bar = full_bar + AG_STAGES;
  uint64_t* acc_full = empty_bar + AG_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_r = (rows_per + AG_BM - 1) / AG_BM;   // row tiles per rank segment
  const int tiles_n = (N + AG_BN - 1) / AG_BN;
  const int per_seg = tiles_r * tiles_n;
  const int total_units = ctx.ws * per_seg;
  const int num_kb = (K + AG_BK - 1) / AG_BK;
  uint32_t* band_cnt = ctx.flags[ctx.rank] + 2 * ctx.ws + 1;  // [ws][tiles_r] rows staged so far

  if (threadIdx.x == 0) {
    for (int s = 0; s < AG_STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 2 * AG_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // unit -> (source rank, row tile inside its segment, column tile): local segment first, then the ranks after us
  auto decode = [&](int unit, int* src, int* m_local, int* n_idx) {
    const int seg = unit / per_seg, rem = unit - seg * per_seg;
    *src = (ctx.rank + seg) % ctx.ws;
    *m_local = rem % tiles_r;
    *n_idx = rem / tiles_r;
  };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int seen_src = -1, seen_band = -1;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        int src, m_local, n_idx;
        decode(unit, &src, &m_local, &n_idx);
        if (src != ctx.rank && (src != seen_src || m_local != seen_band)) {
          // rows of this band staged by the communication warps (local rows were written earlier on this stream)
          const int rows_in_band = min(AG_BM, rows_per - m_local * AG_BM);
          if (!wait_flag_ge(band_cnt + src * tiles_r + m_local, static_cast<uint32_t>(rows_in_band), err)) {
            *abort_flag = 1;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");  // the TMA reads below come after the acquire
          seen_src = src;
          seen_band = m_local;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * AG_STAGE;
          mbar_expect_tx(&full_bar[stage], AG_STAGE);
          tma_load_2d(sa, &maps.a[src], &full_bar[stage], kb * AG_BK, m_local * AG_BM);
          tma_load_2d(sa + AG_A_BYTES, &tmB, &full_bar[stage], kb * AG_BK, n_idx * AG_BN);
          if (++stage == AG_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(AG_BM, AG_BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * AG_BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * AG_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + AG_A_BYTES);
#pragma unroll
          for (int k = 0; k < AG_BK / 16; ++k) umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == AG_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
      }
    }
  } else if (warp >= 6) {
    // ---------------- communication warps: stage remote rows locally, one row per warp at a time ----------------
    const int gw = blockIdx.x * AG_COMM_WARPS + (warp - 6), nw = gridDim.x * AG_COMM_WARPS;
    const uint32_t* my_flags = ctx.flags[ctx.rank];
    const int remote_rows = (ctx.ws - 1) * rows_per;
    unsigned ready_mask = 0;
    for (int i = gw; i < remote_rows; i += nw) {
      const int seg = 1 + i / rows_per, row = i - (seg - 1) * rows_per;
      const int src = (ctx.rank + seg) % ctx.ws;
      if (src * rows_per + row >= T) {  // padding rows still count towards the band
        if (lane == 0) red_release_gpu_add(band_cnt + src * tiles_r + row / AG_BM, 1u);
        continue;
      }
      if (!((ready_mask >> src) & 1u)) {
        int ok = 1;
        if (lane == 0) ok = wait_flag_ge(my_flags + src, epoch, err) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          *abort_flag = 1;
          break;
        }
        ready_mask |= 1u << src;
      }
      const __nv_bfloat16* from = ctx.a[src] + static_cast<size_t>(row) * lda;
      __nv_bfloat16* to = ctx.staged + (static_cast<size_t>(src) * rows_per + row) * K;
      for (int c = lane * 8; c < K; c += 1024) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + u * 256 < K) v[u] = ld_peer16(from + c + u * 256);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + u * 256 < K) *reinterpret_cast<uint4*>(to + c + u * 256) = v[u];
      }
      __syncwarp();
      if (lane == 0) red_release_gpu_add(band_cnt + src * tiles_r + row / AG_BM, 1u);
    }
  } else {
    const int quarter = warp & 3;
    int it = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++it) {
      int src, m_local, n_idx;
      decode(unit, &src, &m_local, &n_idx);
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      {
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
      const int row_local = m_local * AG_BM + quarter * 32 + lane;
      const int row = src * rows_per + row_local;
      const bool row_ok = row_local < rows_per && row < T;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * AG_BN;
      __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc;
#pragma unroll 1
      for (int c = 0; c < AG_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = n_idx * AG_BN + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (row_ok && col0 + j < N) {
            float v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              v[q] = __uint_as_float(r[j + q]);
              if (bias != nullptr) v[q] += __bfloat162float(bias[col0 + j + q]);
            }
            *reinterpret_cast<uint4*>(crow + col0 + j) = pack8(v);
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
    tmem_dealloc(tmem_base, 2 * AG_BN);
  }
  // the last CTA of this rank tells every peer that their rows are no longer being read here
  if (threadIdx.x == 0) {
    uint32_t* mine = ctx.flags[ctx.rank];
    __threadfence();
    const unsigned prev = atomicAdd(mine + 2 * ctx.ws, 1u);
    if (prev == gridDim.x - 1) {
      mine[2 * ctx.ws] = 0;
      for (int i = 0; i < ctx.ws * tiles_r; ++i) band_cnt[i] = 0;
      __threadfence_system();
      for (int d = 0; d < ctx.ws; ++d) st_release_sys(ctx.flags[d] + ctx.ws + ctx.rank, epoch);
    }
  }
}

// Publishes "my rows of this epoch are written" to every rank (the rows were produced by earlier work on the stream).
__global__ void ag_publish_kernel(AgCtx ctx, uint32_t epoch) {
  if (threadIdx.x < ctx.ws) {
    __threadfence_system();
    st_release_sys(ctx.flags[threadIdx.x] + ctx.rank, epoch);
  }
}
// Blocks the stream until every rank has finished reading this rank's rows of `epoch` (call before overwriting them).
__global__ void ag_wait_readers_kernel(const uint32_t* done, int ws, uint32_t epoch, unsigned int* err) {
  if (threadIdx.x < ws) wait_flag_ge(done + threadIdx.x, epoch, err);
}

static int ag_ctx(AgCtx* ctx, int rank, int ws, void* const* flags) {
  if (ws < 1 || ws > AG_MAX_RANKS || rank < 0 || rank >= ws) return -1;
  ctx->rank = rank;
  ctx->ws = ws;
  for (int i = 0; i < AG_MAX_RANKS; ++i) {
    ctx->flags[i] = i < ws ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
    ctx->a[i] = nullptr;
  }
  ctx->staged = nullptr;
  return 0;
}

}  // namespace ksana

using namespace ksana;

KSANA_API int ksana_ag_wait_readers(int rank, int ws, void* const* flags, unsigned int epoch, cudaStream_t stream) {
  AgCtx ctx;
  if (ag_ctx(&ctx, rank, ws, flags)) return -1;
  ag_wait_readers_kernel<<<1, 32, 0, stream>>>(ctx.flags[rank] + ws, ws, epoch, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// a_bufs[r]: rank r's [rows_per, K] bf16 rows (row stride lda elements) in symmetric memory; flags[r]: rank r's flag
// words (2 * ws + 1 + ws * 64 uint32, zero-initialised); staged: local scratch of ws * rows_per * K bf16.
// C: [T, N] bf16 with T <= ws * rows_per (global row = r * rows_per + i).
KSANA_API int ksana_gemm_allgather(int rank, int ws, void* const* a_bufs, void* const* flags, void* staged,
                                   const void* W, const void* bias, void* C, int rows_per, int T, int N, int K,
                                   int lda, int ldw, int ldc, unsigned int epoch, cudaStream_t stream) {
  AgCtx ctx;
  if (ag_ctx(&ctx, rank, ws, flags)) return -1;
  if (rows_per <= 0 || T <= 0 || T > ws * rows_per || (N & 7) || (K & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return -1;
  if ((rows_per + AG_BM - 1) / AG_BM > AG_MAX_BANDS || staged == nullptr) return -1;
  ctx.staged = reinterpret_cast<__nv_bfloat16*>(staged);
  for (int r = 0; r < ws; ++r) ctx.a[r] = reinterpret_cast<const __nv_bfloat16*>(a_bufs[r]);
  AgMaps maps;
  for (int r = 0; r < AG_MAX_RANKS; ++r) {
    // own rows are read in place, remote rows from their slot of the staging buffer
    const int rr = r < ws ? r : 0;
    const void* base = rr == rank ? a_bufs[rank]
                                  : static_cast<const void*>(ctx.staged + static_cast<size_t>(rr) * rows_per * K);
    if (make_tmap_2d(&maps.a[r], base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_per, K, rr == rank ? lda : K, AG_BM,
                     AG_BK, CU_TENSOR_MAP_SWIZZLE_128B))
      return -2;
  }
  CUtensorMap tmB;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, AG_BN, AG_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (KSANA_SMEM_ONCE(gemm_ag_kernel, AG_SMEM) != 0) return -4;
  ag_publish_kernel<<<1, 32, 0, stream>>>(ctx, epoch);
  const int tiles = ws * ((rows_per + AG_BM - 1) / AG_BM) * ((N + AG_BN - 1) / AG_BN);
  int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_ag_kernel<<<grid, AG_THREADS, AG_SMEM, stream>>>(maps, tmB, ctx, reinterpret_cast<__nv_bfloat16*>(C),
                                                       reinterpret_cast<const __nv_bfloat16*>(bias), rows_per, T, N, K,
                                                       lda, ldc, epoch, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
