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

constexpr int FR_BM = 128, FR_BN = 256, FR_BK = 64, FR_STAGES = 4;
constexpr int FR_A_BYTES = FR_BM * FR_BK * 2, FR_B_BYTES = FR_BN * FR_BK * 2, FR_STAGE = FR_A_BYTES + FR_B_BYTES;
constexpr int FR_STG_COLS = 64;                            // the epilogue ships the tile in 64-column slabs
constexpr int FR_STG_PITCH = FR_STG_COLS * 2 + 16;         // bytes per staged row (16-byte pad against bank conflicts)
constexpr int FR_STG = FR_STAGES * FR_STAGE;               // offset of the epilogue staging tile
constexpr int FR_BAR = FR_STG + FR_BM * FR_STG_PITCH;
constexpr int FR_SMEM = FR_BAR + 256 + 1024;
constexpr int FR_MAX_RANKS = 8;
constexpr int FR_MAX_SLOTS = 32;  // world_size x k-splits contributions per output element
constexpr int FR_SIG_BAND = 5000;   // [64] arrival counters per 128-row band (in the owner's signal buffer)
constexpr int FR_SIG_DONE = 5100;   // [8] end-of-call flags
constexpr int FR_SIG_LOCAL = 5120;  // local counter of finished communication CTAs
constexpr int FR_COMM_WARPS = 8;    // communication warps living next to the 6 GEMM warps in every CTA
constexpr int FR_THREADS = 192 + FR_COMM_WARPS * 32;

// Tile order: bands of FR_GROUP_M consecutive 128-row tiles are finished one after the other (low rows first, so
// their owners can start reducing early); inside a band group the order is column-major over (n, m) so that the
// CTAs running at the same time share W tiles and A tiles in L2.
constexpr int FR_GROUP_M = 8;
__device__ __forceinline__ void fused_tile_coords(int t, int tiles_m, int tiles_n, int* m_idx, int* n_idx) {
  const int per_group = FR_GROUP_M * tiles_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m0 = g * FR_GROUP_M;
  const int gm = min(FR_GROUP_M, tiles_m - m0);
  *n_idx = r / gm;
  *m_idx = m0 + (r - (*n_idx) * gm);
}

struct FusedRsCtx {
  int rank, ws;
  __nv_bfloat16* recv[FR_MAX_RANKS];  // each rank's receive buffer [ws][rows_cap][H]
  __nv_bfloat16* hbuf[FR_MAX_RANKS];  // each rank's activation buffer [T, H]
  uint32_t* sig[FR_MAX_RANKS];
  __nv_bfloat16* hbuf_mc;             // multicast view of hbuf or nullptr
  int slot_rows;                      // row capacity of one (source rank, k-split) slot in recv
};

__global__ void __launch_bounds__(FR_THREADS, 1)
gemm_rs_norm_ag_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, FusedRsCtx ctx,
                       int M, int N, int K, __nv_bfloat16* __restrict__ residual,
                       const __nv_bfloat16* __restrict__ norm_w, float eps, uint32_t epoch, int gemm_ctas, int mode,
                       int splits, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + FR_BM - 1) / FR_BM;
  const int tiles_n = N / FR_BN;
  const int rank = ctx.rank, ws = ctx.ws;
  const int rows_per = (M + ws - 1) / ws;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + FR_BAR);
  uint64_t* empty_bar = full_bar + FR_STAGES;
  uint64_t* acc_full = empty_bar + FR_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* s_last_p = const_cast<int*>(abort_flag) + 1;
  const int num_kb = (K + FR_BK - 1) / FR_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_tiles = tiles_m * tiles_n * splits;  // work units: (tile, k-split)
  uint8_t* stg = smem + FR_STG;
  const bool has_gemm_work = static_cast<int>(blockIdx.x) < gemm_ctas;

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

  if (warp >= 6) {
    // ======================= communication warps (owner side) =======================
    // One warp per row: all communication warps of the rank wait for a band's arrival counter, then take the
    // band's rows round-robin. Two passes per row keep the register footprint independent of H: pass 1 sums the
    // per-source slots (+ residual) into the residual stream (or, without a residual, into the local activation
    // row) and accumulates the square sum; pass 2 re-reads that row, normalises and broadcasts it.
    uint32_t* my_sig = ctx.sig[rank];
    const int row_lo = rank * rows_per;
    const int row_hi = min(M, row_lo + rows_per);
    const int tid = threadIdx.x - 192;
    const int gwarp = blockIdx.x * FR_COMM_WARPS + (warp - 6), nwarps = gridDim.x * FR_COMM_WARPS;
    const int nvec = N >> 3;
    const __nv_bfloat16* my_recv = ctx.recv[rank];
    const int nslots = ws * splits;
    float* s_red = reinterpret_cast<float*>(s_last_p + 4);  // [8] partial square sums (row-per-CTA mode)
    if (row_lo < row_hi && rows_per <= static_cast<int>(gridDim.x)) {
      // ---- few rows (decode): one row per CTA, its 256 communication threads split the columns, so the whole
      // row is one round of loads instead of a serial chain inside one warp ----
      int ready_band = -1;
      bool ok = true;
      for (int row = row_lo + blockIdx.x; row < row_hi && ok; row += gridDim.x) {
        const int band = row / FR_BM;
        if (band != ready_band) {
          if (tid == 0)
            s_last_p[1] = wait_flag_ge(my_sig + FR_SIG_BAND + band, static_cast<uint32_t>(ws * tiles_n * splits), err) ? 1 : 0;
          asm volatile("bar.sync 3, 256;" ::: "memory");
          ok = s_last_p[1] != 0;
          if (!ok) break;
          __threadfence();
          ready_band = band;
        }
        const int lrow = row - row_lo;
        __nv_bfloat16* acc_row = (mode & 2) ? residual + static_cast<size_t>(row) * N
                                            : ctx.hbuf[rank] + static_cast<size_t>(row) * N;
        float ss = 0.f;
        for (int v0 = tid; v0 < nvec; v0 += 256) {
          float acc[8];
          if (mode & 2) {
            unpack8(*reinterpret_cast<const uint4*>(acc_row + (v0 << 3)), acc);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          }
          for (int pb = 0; pb < nslots; pb += 8) {
            uint4 raw[8];
#pragma unroll
            for (int p = 0; p < 8; ++p)
              if (pb + p < nslots)
                raw[p] = __ldcg(reinterpret_cast<const uint4*>(
                    my_recv + (static_cast<size_t>(pb + p) * ctx.slot_rows + lrow) * N + (v0 << 3)));
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              if (pb + p < nslots) {
                float t[8];
                unpack8(raw[p], t);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += t[j];
              }
            }
          }
          const uint4 packed = pack8(acc);
          *reinterpret_cast<uint4*>(acc_row + (v0 << 3)) = packed;
          float v[8];
          unpack8(packed, v);
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
        }
        float inv = 1.f;
        if (mode & 1) {
          ss = warp_sum(ss);
          if (lane == 0) s_red[warp - 6] = ss;
          asm volatile("bar.sync 3, 256;" ::: "memory");
          float tot = 0.f;
#pragma unroll
          for (int i = 0; i < FR_COMM_WARPS; ++i) tot += s_red[i];
          inv = rsqrtf(tot / static_cast<float>(N) + eps);
        }
        for (int v0 = tid; v0 < nvec; v0 += 256) {
          float v[8], o[8];
          unpack8(*reinterpret_cast<const uint4*>(acc_row + (v0 << 3)), v);  // written by this thread above
          if (mode & 1) {
            float g[8];
            unpack8(*reinterpret_cast<const uint4*>(norm_w + (v0 << 3)), g);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[j] * inv * g[j];
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[j];
          }
          const uint4 packed = pack8(o);
          const size_t off = static_cast<size_t>(row) * N + (v0 << 3);
          if (ctx.hbuf_mc != nullptr) {
            multimem_st16(ctx.hbuf_mc + off, packed);
          } else {
            for (int p = 0; p < ws; ++p) st_peer16(ctx.hbuf[p] + off, packed);
          }
        }
        asm volatile("bar.sync 3, 256;" ::: "memory");  // s_red / s_last_p[1] are reused by the next row
      }
    } else if (row_lo < row_hi) {
      // rows are dealt round-robin over ALL communication warps of the rank, so different warps wait on different
      // 128-row bands and many bands are reduced concurrently; each warp meets its bands in increasing order
      bool ok = true;
      int ready_band = -1;
      for (int row = row_lo + gwarp; row < row_hi && ok; row += nwarps) {
        const int band = row / FR_BM;
        if (band != ready_band) {
          // one lane polls (a whole warp of system-scope acquire loads on one word only adds traffic)
          int okw = 1;
          if (lane == 0)
            okw = wait_flag_ge(my_sig + FR_SIG_BAND + band, static_cast<uint32_t>(ws * tiles_n * splits), err) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, okw, 0) != 0;
          if (!ok) break;
          __threadfence();  // order this lane's reads of the band after the acquire observed by lane 0
          ready_band = band;
        }
        {
          const int lrow = row - row_lo;
          __nv_bfloat16* acc_row = (mode & 2) ? residual + static_cast<size_t>(row) * N
                                              : ctx.hbuf[rank] + static_cast<size_t>(row) * N;
          float ss = 0.f;
          // 4 vectors per lane per iteration, contribution slots in groups of 8: up to 32 (+ 4 residual) loads are
          // in flight together; slots are summed in fixed order, so the result does not depend on arrival order
          for (int v0 = lane; v0 < nvec; v0 += 128) {
            float acc[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vi = v0 + u * 32;
              if ((mode & 2) && vi < nvec) {
                unpack8(*reinterpret_cast<const uint4*>(acc_row + (vi << 3)), acc[u]);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
              }
            }
            for (int pb = 0; pb < nslots; pb += 4) {
              uint4 raw[4][4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int vi = v0 + u * 32;
                if (vi < nvec) {
#pragma unroll
                  for (int p = 0; p < 4; ++p)
                    if (pb + p < nslots)
                      raw[u][p] = __ldcg(reinterpret_cast<const uint4*>(
                          my_recv + (static_cast<size_t>(pb + p) * ctx.slot_rows + lrow) * N + (vi << 3)));
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int vi = v0 + u * 32;
                if (vi < nvec) {
#pragma unroll
                  for (int p = 0; p < 4; ++p) {
                    if (pb + p < nslots) {
                      float t[8];
                      unpack8(raw[u][p], t);
#pragma unroll
                      for (int j = 0; j < 8; ++j) acc[u][j] += t[j];
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vi = v0 + u * 32;
              if (vi < nvec) {
                const uint4 packed = pack8(acc[u]);
                *reinterpret_cast<uint4*>(acc_row + (vi << 3)) = packed;
                float v[8];
                unpack8(packed, v);  // the norm sees the bf16-rounded sum, like the unfused kernels
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
              }
            }
          }
          float inv = 1.f;
          if (mode & 1) inv = rsqrtf(warp_sum(ss) / static_cast<float>(N) + eps);
          __syncwarp();
          for (int v0 = lane; v0 < nvec; v0 += 128) {
            uint4 rv[4], gv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vi = v0 + u * 32;
              if (vi < nvec) {
                rv[u] = *reinterpret_cast<const uint4*>(acc_row + (vi << 3));  // written by this lane in pass 1
                if (mode & 1) gv[u] = *reinterpret_cast<const uint4*>(norm_w + (vi << 3));
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int vi = v0 + u * 32;
              if (vi < nvec) {
                const int c = vi << 3;
                float v[8], o[8];
                unpack8(rv[u], v);
                if (mode & 1) {
                  float g[8];
                  unpack8(gv[u], g);
#pragma unroll
                  for (int j = 0; j < 8; ++j) o[j] = v[j] * inv * g[j];
                } else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) o[j] = v[j];
                }
                const uint4 packed = pack8(o);
                const size_t off = static_cast<size_t>(row) * N + c;
                if (ctx.hbuf_mc != nullptr) {
                  multimem_st16(ctx.hbuf_mc + off, packed);
                } else {
                  for (int p = 0; p < ws; ++p) st_peer16(ctx.hbuf[p] + off, packed);
                }
              }
            }
          }
        }
      }
    }
    __threadfence_system();
    asm volatile("bar.sync 3, 256;" ::: "memory");
    if (tid == 0) {
      const uint32_t prev = atomicAdd(my_sig + FR_SIG_LOCAL, 1u);
      const int last = (prev == gridDim.x - 1);
      if (last) my_sig[FR_SIG_LOCAL] = 0;
      *s_last_p = last;
    }
    asm volatile("bar.sync 3, 256;" ::: "memory");
    if (*s_last_p) {
      // every communication warp of this rank is done: counters back to zero, then the end-of-call handshake
      if (row_lo < row_hi)
        for (int band = row_lo / FR_BM + tid; band <= (row_hi - 1) / FR_BM; band += 256)
          my_sig[FR_SIG_BAND + band] = 0;
      __threadfence_system();
      asm volatile("bar.sync 3, 256;" ::: "memory");
      if (tid < ws) st_release_sys(ctx.sig[tid] + FR_SIG_DONE + rank, epoch);
      if (tid < ws) wait_flag_ge(my_sig + FR_SIG_DONE + tid, epoch, err);
    }
  } else if (!has_gemm_work) {
    // this CTA only contributes communication warps
  } else if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gemm_ctas) {
        const int t2 = tile / splits, split = tile - t2 * splits;
        int m_idx, n_idx;
        fused_tile_coords(t2, tiles_m, tiles_n, &m_idx, &n_idx);
        const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
        for (int kb = kb0; kb < kb1; ++kb) {
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
        const int split = tile % splits;
        const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
        if (!mbar_wait_bounded(&acc_empty[as], ((it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * FR_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + FR_A_BYTES);
#pragma unroll
          for (int k = 0; k < FR_BK / 16; ++k)
            umma_f16(tmem_base + as * FR_BN, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
      const int t2 = tile / splits, split = tile - t2 * splits;
      int m_idx, n_idx;
      fused_tile_coords(t2, tiles_m, tiles_n, &m_idx, &n_idx);
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
      // TMEM -> registers -> 64-column staging slab in shared memory (row per thread) -> coalesced peer stores
      const int trow = quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * FR_BN;
      const int et = threadIdx.x - 64;
      const int seg = et & 7;
#pragma unroll 1
      for (int slab = 0; slab < FR_BN / FR_STG_COLS; ++slab) {
#pragma unroll
        for (int c = 0; c < FR_STG_COLS / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + slab * FR_STG_COLS + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            o.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            o.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            o.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(stg + trow * FR_STG_PITCH + (c * 32 + j) * 2) = o;
          }
        }
        if (slab == FR_BN / FR_STG_COLS - 1) {
          tc_fence_before();
          mbar_arrive(&acc_empty[as]);  // the tensor core may refill this accumulator while the tile is shipped
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        // 8 threads move one 128-byte row segment, 16 rows per pass
#pragma unroll 4
        for (int pass = 0; pass < FR_BM / 16; ++pass) {
          const int lr = pass * 16 + (et >> 3);
          const int row = m_idx * FR_BM + lr;
          if (row < M) {
            const int owner = row / rows_per;
            const int lrow = row - owner * rows_per;
            const uint4 val = *reinterpret_cast<const uint4*>(stg + lr * FR_STG_PITCH + seg * 16);
            __nv_bfloat16* dst = ctx.recv[owner] +
                                 (static_cast<size_t>(rank * splits + split) * ctx.slot_rows + lrow) * N +
                                 n_idx * FR_BN + slab * FR_STG_COLS;
            st_peer16(dst + seg * 8, val);
          }
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
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
// N % 256 == 0, N <= 9216, M <= 64 * 128. mode bit0: RMSNorm, bit1: residual add (residual [M, N], row-sharded).
KSANA_API int ksana_gemm_rs_norm_ag(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank,
                                    int ws, void* const* recv, void* const* hbuf, void* const* sig, void* hbuf_mc,
                                    int rows_cap, void* residual, const void* norm_w, float eps, unsigned int epoch,
                                    int mode, int comm_ctas, int force_splits, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (ws < 1 || ws > FR_MAX_RANKS || (N % FR_BN) || N > 16384 || (K & 7) || (lda & 7) || (ldw & 7) ||
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

  if (KSANA_SMEM_ONCE(gemm_rs_norm_ag_kernel, FR_SMEM) != 0) return -4;
  const int sms = sm_count();
  const int tiles = ((M + FR_BM - 1) / FR_BM) * (N / FR_BN);
  const int rows_per = (M + ws - 1) / ws;
  (void)comm_ctas;
  // small M: weight streaming needs every SM pulling, so K is split and each split is one more contribution slot
  const int num_kb = (K + FR_BK - 1) / FR_BK;
  int splits = 1;
  if (force_splits > 0) splits = force_splits;
  else if (tiles * 2 <= sms && num_kb >= 16) {
    splits = sms / tiles;
    if (splits > 4) splits = 4;
  }
  while (splits > 1 && (ws * splits > FR_MAX_SLOTS || rows_per * splits > rows_cap ||
                        ((num_kb + splits - 1) / splits) * (splits - 1) >= num_kb))
    --splits;
  ctx.slot_rows = rows_cap / splits;
  int gemm_ctas = sms;
  if (gemm_ctas > tiles * splits) gemm_ctas = tiles * splits;
  // CTAs without GEMM work still contribute their communication warps (one warp normalises one row at a time)
  int grid = gemm_ctas;
  const int want = rows_per < sms ? rows_per : sms;
  if (grid < want) grid = want;
  gemm_rs_norm_ag_kernel<<<grid, FR_THREADS, FR_SMEM, stream>>>(
      tmA, tmB, ctx, M, N, K, reinterpret_cast<__nv_bfloat16*>(residual),
      reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, epoch, gemm_ctas, mode, splits, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
