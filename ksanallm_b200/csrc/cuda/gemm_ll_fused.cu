// Latency-optimised row-parallel block for decode-sized steps under tensor parallelism, ONE kernel:
//   tcgen05 GEMM (this rank's K slice, cluster split-K)  ->  reduce-scatter  ->  residual add + RMSNorm  ->  all-gather.
//
// Small-M counterpart of gemm_fused_rs.cu. It replaces the reference's small-message paths: the one-shot "lamport"
// all-reduce (3rdparty/LLM_kernels/csrc/kernels/nvidia/others/tensorrt-llm/main/communication_kernels/
// trtllm_all_reduce.cu:381-506) and the 1-stage P2P reduce (all_reduce/custom_all_reduce.cu:196-265, thresholds in
// src/ksana_llm/layers/nvidia/custom_all_reduce_sum_layer.cpp:124-176), each followed by the fused add + RMSNorm.
//
// A decode step's row-parallel block moves little data; its cost is the chain of NVLink round trips. This kernel
// shortens the chain:
//   hop 1  The GEMM epilogue sends every finished accumulator slice straight to the rank that OWNS the row, as
//          8-byte words {2 x bf16, epoch}. The receiver polls the words themselves: data and "it is there" arrive in
//          the same store, so there is no fence and no flag round trip, and a slice travels while later tiles are
//          still being multiplied. Words of an earlier call carry an older epoch and are never mistaken for data.
//   owner  One CTA per owned row sums the per-source words in rank order (deterministic), adds the row of the
//          residual stream, applies RMSNorm ...
//   hop 2  ... and sends the normalised row to every rank, again as flagged words (multimem.st through the switch or
//          plain peer stores): no fence, no flag round trip here either.
//   end    Every rank polls the words of all rows and unpacks them into its activation buffer: when the kernel ends
//          the full activation is local, in the plain layout the next GEMM's TMA loads read.
// With two ranks there is no second hop: each rank sends its slices to both ranks, both reduce every row (the
// traffic is the same as reduce-scatter + all-gather, the chain is one NVLink trip shorter) and keep the whole
// residual stream; the word buffer is double-buffered by call parity because no hop-2 wait orders the calls.
// The same two hops without a GEMM (a partial sum that is already in memory, e.g. an expert layer's output) are the
// second entry point below.
//
// Buffer reuse needs no extra handshake: a rank starts call e + 1 only after it has seen every row of call e, so
// every owner had finished reading call e's words, and an owner sends rows of call e + 1 to a peer only after that
// peer's words of call e + 1 arrived, i.e. after the peer has unpacked call e. All CTAs are resident (grid <= SM count, one CTA per SM); every wait is bounded by wall time.
#include "comm.cuh"
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int LL_BM = 128, LL_BN = 128, LL_BK = 64, LL_STAGES = 4;
constexpr int LL_A_BYTES = LL_BM * LL_BK * 2, LL_B_BYTES = LL_BN * LL_BK * 2, LL_STAGE = LL_A_BYTES + LL_B_BYTES;
constexpr int LL_PITCH = LL_BN + 4;
constexpr int LL_STG = LL_STAGES * LL_STAGE;
constexpr int LL_BAR = LL_STG + LL_BM * LL_PITCH * 4;
constexpr int LL_SMEM = LL_BAR + 256 + 1024;
constexpr int LL_THREADS = 192;
constexpr int LL_MAX_RANKS = 8;
constexpr int LL_MAX_H = 8192;
constexpr int LL_MAX_GROUPS = (LL_MAX_H / 8 + LL_THREADS - 1) / LL_THREADS;  // 8-column groups per thread and row

struct LlCtx {
  int rank, ws;
  uint2* recv[LL_MAX_RANKS];   // each rank's hop-1 word buffer [ws][rows_cap][H / 2] of {bf16x2, epoch}
  uint2* recv2[LL_MAX_RANKS];  // each rank's hop-2 word buffer [>= M][H / 2] (unused with one_shot)
  uint2* recv2_mc;             // multicast view of recv2, or nullptr (plain peer stores)
  __nv_bfloat16* hbuf;         // this rank's activation buffer [>= M][H]
  int rows_cap;                // rows of one source slot in recv
  int one_shot;                // every rank receives and reduces every row; no hop 2
};

__device__ __forceinline__ int ll_owner(const LlCtx& ctx, int rows_per, int row) { return row / rows_per; }

// Optional timeline of CTA 0 (nanoseconds of the global timer), switched on by ksana_ll_set_trace: [0] entry,
// [1] set-up done, [2] first operands landed, [3] last MMA committed, [4] first slice sent, [5] GEMM phase over,
// [6] first owned row complete, [7] first owned row broadcast, [8] all row flags seen.
__device__ unsigned long long* g_ll_trace = nullptr;
__device__ __forceinline__ void ll_stamp(int i) {
  if (g_ll_trace != nullptr && blockIdx.x == 0) g_ll_trace[i] = global_timer_ns();
}

__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Sends 4 consecutive columns of one row to the row's owner: two words in one 16-byte store.
__device__ __forceinline__ void ll_send4(const LlCtx& ctx, int rows_per, int row, int col, int H, float a, float b,
                                         float c, float d, uint32_t epoch) {
  uint4 w;
  w.x = pack_bf16(a, b);
  w.y = epoch;
  w.z = pack_bf16(c, d);
  w.w = epoch;
  if (ctx.one_shot) {
    const size_t off = (static_cast<size_t>(ctx.rank) * ctx.rows_cap + row) * (H >> 1) + (col >> 1);
    for (int p = 0; p < ctx.ws; ++p) st_peer16(ctx.recv[p] + off, w);
    return;
  }
  const int owner = row / rows_per;
  const int lrow = row - owner * rows_per;
  st_peer16(ctx.recv[owner] + (static_cast<size_t>(ctx.rank) * ctx.rows_cap + lrow) * (H >> 1) + (col >> 1), w);
}

// Polls two 16-byte word pairs (8 columns of one row from one source) until they carry `epoch`.
__device__ __forceinline__ bool ll_poll8(const uint2* p, uint32_t epoch, uint4* wa, uint4* wb, bool* alive,
                                         unsigned int* err) {
  *wa = ld_volatile16(p);
  *wb = ld_volatile16(p + 2);
  if (wa->y == epoch && wa->w == epoch && wb->y == epoch && wb->w == epoch) return true;
  const unsigned long long t0 = global_timer_ns();
  while (*alive) {
    *wa = ld_volatile16(p);
    *wb = ld_volatile16(p + 2);
    if (wa->y == epoch && wa->w == epoch && wb->y == epoch && wb->w == epoch) return true;
    const unsigned long long dt = global_timer_ns() - t0;
    // after a millisecond: give up at once if an earlier wait on this GPU has already expired (the host has not yet
    // read the status word), otherwise keep waiting up to the full bound
    if (dt > KSANA_PEER_TIMEOUT_NS ||
        (dt > KSANA_PEER_TIMEOUT_AFTER_FAILURE_NS &&
         (*reinterpret_cast<volatile unsigned int*>(err) & KERR_PEER_TIMEOUT) != 0u)) {
      atomicOr(err, KERR_PEER_TIMEOUT);
      *alive = false;
    }
  }
  return false;
}

// Owner side + hop 2 + unpack; called by all threads of every CTA once its own sends are issued.
// MAXR: upper bound of the rank count (sizes the register arrays), GB: 8-column groups whose words are requested
// together (MAXR * GB * 2 loads of 16 bytes in flight per thread before the first one is looked at).
template <int MAXR, int GB>
__device__ __forceinline__ void ll_reduce_norm_gather(const LlCtx& ctx, int M, int H, __nv_bfloat16* residual,
                                                      const __nv_bfloat16* norm_w, float eps, uint32_t epoch, int mode,
                                                      float* s_red, unsigned int* err) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int rank = ctx.rank, ws = ctx.ws;
  const int rows_per = ctx.one_shot ? M : (M + ws - 1) / ws;
  const int row_lo = ctx.one_shot ? 0 : rank * rows_per, row_hi = min(M, row_lo + rows_per);
  const int ngroups = H >> 3;
  const uint2* my_recv = ctx.recv[rank];
  bool alive = true;
  bool first_row = true;
  for (int row = row_lo + static_cast<int>(blockIdx.x); row < row_hi; row += gridDim.x) {
    const int lrow = row - row_lo;
    float v[LL_MAX_GROUPS][8];
    float ss = 0.f;
#pragma unroll
    for (int gb = 0; gb < LL_MAX_GROUPS; gb += GB) {
      uint4 wa[GB][MAXR], wb[GB][MAXR];
#pragma unroll
      for (int u = 0; u < GB; ++u) {
        const int g = tid + (gb + u) * nthr;
        if (gb + u < LL_MAX_GROUPS && g < ngroups) {
#pragma unroll
          for (int s = 0; s < MAXR; ++s) {
            if (s < ws) {
              const uint2* p = my_recv + (static_cast<size_t>(s) * ctx.rows_cap + lrow) * (H >> 1) + (g << 2);
              wa[u][s] = ld_volatile16(p);
              wb[u][s] = ld_volatile16(p + 2);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < GB; ++u) {
        const int gi = gb + u;
        const int g = tid + gi * nthr;
        if (gi < LL_MAX_GROUPS && g < ngroups) {
          float acc[8];
          if (mode & 2) {
            unpack8(*reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * H + (g << 3)), acc);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          }
#pragma unroll
          for (int s = 0; s < MAXR; ++s) {
            if (s < ws) {
              if (wa[u][s].y != epoch || wa[u][s].w != epoch || wb[u][s].y != epoch || wb[u][s].w != epoch)
                ll_poll8(my_recv + (static_cast<size_t>(s) * ctx.rows_cap + lrow) * (H >> 1) + (g << 2), epoch,
                         &wa[u][s], &wb[u][s], &alive, err);
              const uint32_t d[4] = {wa[u][s].x, wa[u][s].z, wb[u][s].x, wb[u][s].z};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d[j]));
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
              }
            }
          }
          if (mode & 2) {
            const uint4 packed = pack8(acc);
            *reinterpret_cast<uint4*>(residual + static_cast<size_t>(row) * H + (g << 3)) = packed;
            unpack8(packed, acc);  // the norm sees the bf16-rounded residual, like the unfused kernels
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[gi][j] = acc[j];
            ss += acc[j] * acc[j];
          }
        }
      }
    }
    if (first_row && tid == 0) ll_stamp(6);
    float inv = 1.f;
    if (mode & 1) {
      ss = warp_sum(ss);
      __syncthreads();  // s_red of the previous row has been read by everybody
      if ((tid & 31) == 0) s_red[tid >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int i = 0; i < (nthr >> 5); ++i) tot += s_red[i];
      inv = rsqrtf(tot / static_cast<float>(H) + eps);
    }
#pragma unroll
    for (int gi = 0; gi < LL_MAX_GROUPS; ++gi) {
      const int g = tid + gi * nthr;
      if (g < ngroups) {
        float o[8];
        if (mode & 1) {
          float gw[8];
          unpack8(*reinterpret_cast<const uint4*>(norm_w + (g << 3)), gw);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[gi][j] * inv * gw[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = v[gi][j];
        }
        const uint4 packed = pack8(o);
        if (ctx.one_shot) {
          *reinterpret_cast<uint4*>(ctx.hbuf + static_cast<size_t>(row) * H + (g << 3)) = packed;
        } else if (alive) {  // a failed wait sends nothing: the peers time out too instead of reading garbage
          const size_t woff = static_cast<size_t>(row) * (H >> 1) + (g << 2);
          const uint4 w0 = make_uint4(packed.x, epoch, packed.y, epoch), w1 = make_uint4(packed.z, epoch, packed.w, epoch);
          if (ctx.recv2_mc != nullptr) {
            multimem_st16(ctx.recv2_mc + woff, w0);
            multimem_st16(ctx.recv2_mc + woff + 2, w1);
          } else {
            for (int p = 0; p < ws; ++p) {
              st_peer16(ctx.recv2[p] + woff, w0);
              st_peer16(ctx.recv2[p] + woff + 2, w1);
            }
          }
        }
      }
    }
    if (first_row && tid == 0) ll_stamp(7);
    first_row = false;
  }
  if (!ctx.one_shot) {
    // every row of every owner: words -> plain activation rows
    const uint2* my_recv2 = ctx.recv2[rank];
    for (int row = static_cast<int>(blockIdx.x); row < M; row += gridDim.x) {
#pragma unroll
      for (int gi = 0; gi < LL_MAX_GROUPS; ++gi) {
        const int g = tid + gi * nthr;
        if (g < ngroups) {
          uint4 wa, wb;
          if (ll_poll8(my_recv2 + static_cast<size_t>(row) * (H >> 1) + (g << 2), epoch, &wa, &wb, &alive, err))
            *reinterpret_cast<uint4*>(ctx.hbuf + static_cast<size_t>(row) * H + (g << 3)) =
                make_uint4(wa.x, wa.z, wb.x, wb.z);
        }
      }
    }
  }
  __syncthreads();
  if (tid == 0) ll_stamp(8);
}

// ---- GEMM + the two hops ----------------------------------------------------------------------------------
template <int MAXR, int GB>
__global__ void __launch_bounds__(LL_THREADS, 1)
gemm_ll_reduce_norm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, LlCtx ctx,
                           int M, int N, int K, __nv_bfloat16* __restrict__ residual,
                           const __nv_bfloat16* __restrict__ norm_w, float eps, uint32_t epoch, int mode, int splits,
                           unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* stg = reinterpret_cast<float*>(smem + LL_STG);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + LL_BAR);
  uint64_t* empty_bar = full_bar + LL_STAGES;
  uint64_t* acc_full = empty_bar + LL_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* part_ready = acc_empty + 2;
  uint64_t* stg_free = part_ready + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(stg_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* s_red = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 2);  // [8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + LL_BM - 1) / LL_BM;
  const int tiles_n = N / LL_BN;
  const int num_kb = (K + LL_BK - 1) / LL_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_tiles = tiles_m * tiles_n;
  const int split = static_cast<int>(cluster_ctarank());
  const int cluster_id = blockIdx.x / splits;
  const int num_clusters = gridDim.x / splits;
  const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);
  const int rows_per = (M + ctx.ws - 1) / ctx.ws;
  if (threadIdx.x == 0) ll_stamp(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < LL_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 128);
    }
    mbar_init(part_ready, splits);
    mbar_init(stg_free, splits);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * LL_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();
  const uint32_t tmem_base = *tmem_holder;
  if (threadIdx.x == 0) ll_stamp(1);

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters) {
        const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * LL_STAGE;
          mbar_expect_tx(&full_bar[stage], LL_STAGE);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * LL_BK, m_idx * LL_BM);
          tma_load_2d(sa + LL_A_BYTES, &tmB, &full_bar[stage], kb * LL_BK, n_idx * LL_BN);
          if (++stage == LL_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(LL_BM, LL_BN, 1, 1);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < total_tiles && ok; tile += num_clusters, ++it) {
        const int as = it & 1;
        if (!mbar_wait_bounded(&acc_empty[as], ((it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (it == 0 && kb == kb0) ll_stamp(2);
          const uint32_t sa = smem_u32(smem + stage * LL_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + LL_A_BYTES);
#pragma unroll
          for (int k = 0; k < LL_BK / 16; ++k)
            umma_f16(tmem_base + as * LL_BN, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == LL_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
        if (it == 0) ll_stamp(3);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127
    int it = 0;
    for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++it) {
      const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
      const int as = it & 1;
      const uint32_t ph = it & 1;
      uint32_t ok_in = (mbar_wait_bounded(&acc_full[as], (it >> 1) & 1, abort_flag, err) &&
                        mbar_wait_cluster_bounded(stg_free, ph ^ 1, abort_flag, err)) ? 1u : 0u, ok_all;
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
      // 1. my fp32 partial tile -> my shared memory (row per thread)
      const int trow = quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * LL_BN;
      const int rows_valid = min(LL_BM, M - m_idx * LL_BM);  // rows of this tile that exist in the matrix
      if (quarter * 32 < rows_valid) {
#pragma unroll 2
        for (int c = 0; c < LL_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(stg + trow * LL_PITCH + c * 32 + j) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                            __uint_as_float(r[j + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      // 2. publish to every CTA of the cluster, 3. wait for all partial tiles
      if (et < splits) mbar_arrive_remote(mapa_u32(smem_u32(part_ready), et));
      ok_in = mbar_wait_cluster_bounded(part_ready, ph, abort_flag, err) ? 1u : 0u;
      asm volatile(
          "{\n\t.reg .pred pin, pout;\n\t"
          "setp.ne.u32 pin, %1, 0;\n\t"
          "bar.red.and.pred pout, 1, 128, pin;\n\t"
          "selp.u32 %0, 1, 0, pout;\n\t}"
          : "=r"(ok_all)
          : "r"(ok_in)
          : "memory");
      if (!ok_all) break;
      // 4. reduce my slice of the tile's rows over the cluster in rank order and send it to the rows' owners
      const uint32_t stg_addr = smem_u32(stg);
      const int rows_slice = (rows_valid + splits - 1) / splits;
      const int r0 = split * rows_slice;
      const int n_items = max(min(rows_valid, r0 + rows_slice) - r0, 0) * (LL_BN / 4);
      for (int i0 = et; i0 < n_items; i0 += 128 * 4) {
        float4 acc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
          if (p < splits) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i = i0 + u * 128;
              if (i < n_items) {
                const int lr = r0 + i / (LL_BN / 4), c4 = (i % (LL_BN / 4)) * 4;
                const float4 v = ld_cluster_f4(mapa_u32(stg_addr + (lr * LL_PITCH + c4) * 4, p));
                acc[u].x += v.x;
                acc[u].y += v.y;
                acc[u].z += v.z;
                acc[u].w += v.w;
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * 128;
          if (i < n_items) {
            const int lr = r0 + i / (LL_BN / 4), c4 = (i % (LL_BN / 4)) * 4;
            ll_send4(ctx, rows_per, m_idx * LL_BM + lr, n_idx * LL_BN + c4, N, acc[u].x, acc[u].y, acc[u].z,
                     acc[u].w, epoch);
          }
        }
      }
      if (it == 0 && et == 0) ll_stamp(4);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (et < splits) mbar_arrive_remote(mapa_u32(smem_u32(stg_free), et));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody reads a peer's shared memory past this point
  if (threadIdx.x == 0) ll_stamp(5);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * LL_BN);
  }
  if (*abort_flag) return;  // a wait inside the GEMM gave up: the status word is set, peers time out on their own
  ll_reduce_norm_gather<MAXR, GB>(ctx, M, N, residual, norm_w, eps, epoch, mode, s_red, err);
}

// ---- the two hops for a partial sum that is already in memory ---------------------------------------------------
template <int MAXR, int GB>
__global__ void __launch_bounds__(LL_THREADS)
ll_reduce_norm_kernel(LlCtx ctx, const __nv_bfloat16* __restrict__ partial, int ldp, int M, int H,
                      __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ norm_w, float eps,
                      uint32_t epoch, int mode, unsigned int* err) {
  __shared__ float s_red[8];
  const int rows_per = (M + ctx.ws - 1) / ctx.ws;
  const int nq = H >> 2;  // 4-column pieces per row
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * nq; i += gridDim.x * blockDim.x) {
    const int row = i / nq, col = (i - row * nq) << 2;
    const uint2 raw = *reinterpret_cast<const uint2*>(partial + static_cast<size_t>(row) * ldp + col);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    ll_send4(ctx, rows_per, row, col, H, a.x, a.y, b.x, b.y, epoch);
  }
  ll_reduce_norm_gather<MAXR, GB>(ctx, M, H, residual, norm_w, eps, epoch, mode, s_red, err);
}

// recv_off: word offset added to every rank's hop-1 buffer (the parity half of the one-shot double buffer).
static int fill_ctx(LlCtx* ctx, int rank, int ws, void* const* recv, long long recv_off, void* const* recv2,
                    void* recv2_mc, void* hbuf, int rows_cap, int one_shot, int M) {
  if (ws < 1 || ws > LL_MAX_RANKS || rank < 0 || rank >= ws) return -1;
  if (one_shot ? M > rows_cap : (M + ws - 1) / ws > rows_cap) return -1;
  ctx->rank = rank;
  ctx->ws = ws;
  for (int i = 0; i < LL_MAX_RANKS; ++i) {
    ctx->recv[i] = i < ws ? reinterpret_cast<uint2*>(recv[i]) + recv_off : nullptr;
    ctx->recv2[i] = (i < ws && recv2 != nullptr) ? reinterpret_cast<uint2*>(recv2[i]) : nullptr;
  }
  if (!one_shot && recv2 == nullptr) return -1;
  ctx->recv2_mc = reinterpret_cast<uint2*>(recv2_mc);
  ctx->hbuf = reinterpret_cast<__nv_bfloat16*>(hbuf);
  ctx->rows_cap = rows_cap;
  ctx->one_shot = one_shot;
  return 0;
}

}  // namespace ksana

using namespace ksana;

// The kernels are instantiated for up to 2, 4 and 8 ranks (register array sizes, loads in flight). With fewer GPUs than
// 8 at hand, a test can ask for a larger instantiation than the rank count needs: the 8-rank code then runs on 2 or 4.
static int g_ll_kernel_ranks = 0;
KSANA_API void ksana_ll_set_kernel_ranks(int ranks) { g_ll_kernel_ranks = ranks; }

// y = AllGather(RMSNorm(residual_slice += ReduceScatter(A * W^T)) * norm_w) in one launch, for small M.
// A: [M, K] bf16 (pitch lda), W: [N, K] bf16 (pitch ldw); hbuf: this rank's activation buffer [>= M][N] bf16.
// Per-rank symmetric buffers of 8-byte words, zero-initialised once (arrays indexed by rank):
//   two hops (one_shot = 0): recv [ws][rows_cap][N / 2] with rows_cap >= ceil(M / ws); recv2 [>= M][N / 2]
//                            (recv2_mc: its multicast view or null); only the owner's rows of `residual` change;
//   one hop (one_shot = 1):  recv [ws][rows_cap][N / 2] with rows_cap >= M, starting recv_off words into each rank's
//                            buffer - the caller alternates between two such halves from call to call; recv2 unused;
//                            every row of `residual` changes on every rank.
// N % 128 == 0, N <= 8192; epoch != 0 and different from the epochs of earlier calls on these buffers.
// mode bit0: RMSNorm, bit1: residual add (residual [M, N]).
KSANA_API int ksana_gemm_ll_reduce_norm(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank,
                                        int ws, void* const* recv, long long recv_off, void* const* recv2,
                                        void* recv2_mc, void* hbuf, int rows_cap, int one_shot, void* residual,
                                        const void* norm_w, float eps, unsigned int epoch, int mode, int force_splits,
                                        cudaStream_t stream) {
  if (M <= 0) return 0;
  LlCtx ctx;
  if (fill_ctx(&ctx, rank, ws, recv, recv_off, recv2, recv2_mc, hbuf, rows_cap, one_shot, M)) return -1;
  if ((N % LL_BN) || N > LL_MAX_H || (K & 7) || (lda & 7) || (ldw & 7) || epoch == 0) return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, LL_BM, LL_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, LL_BN, LL_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  const int kws = g_ll_kernel_ranks > ws ? g_ll_kernel_ranks : ws;  // which instantiation (tests: see the setter)
  auto kern = kws <= 2 ? gemm_ll_reduce_norm_kernel<2, 6> : kws <= 4 ? gemm_ll_reduce_norm_kernel<4, 3>
                                                                     : gemm_ll_reduce_norm_kernel<8, 2>;
  if (kws <= 2) {
    if (KSANA_SMEM_ONCE((gemm_ll_reduce_norm_kernel<2, 6>), LL_SMEM) != 0) return -4;
  } else if (kws <= 4) {
    if (KSANA_SMEM_ONCE((gemm_ll_reduce_norm_kernel<4, 3>), LL_SMEM) != 0) return -4;
  } else {
    if (KSANA_SMEM_ONCE((gemm_ll_reduce_norm_kernel<8, 2>), LL_SMEM) != 0) return -4;
  }
  const int sms = sm_count();
  const int tiles = ((M + LL_BM - 1) / LL_BM) * (N / LL_BN);
  const int num_kb = (K + LL_BK - 1) / LL_BK;
  int splits = 1;
  if (force_splits == 1 || force_splits == 2 || force_splits == 4 || force_splits == 8) {
    splits = force_splits;
  } else {
    splits = 8;
    while (splits > 1 && (splits * tiles > sms || num_kb / splits < 2)) splits >>= 1;
  }
  while (splits > 1 && ((num_kb + splits - 1) / splits) * (splits - 1) >= num_kb) splits >>= 1;
  int clusters = sms / splits;
  if (clusters > tiles) clusters = tiles;
  if (clusters < 1) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * splits);
  cfg.blockDim = dim3(LL_THREADS);
  cfg.dynamicSmemBytes = LL_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  __nv_bfloat16* res = reinterpret_cast<__nv_bfloat16*>(residual);
  const __nv_bfloat16* nw = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  unsigned int* e = error_word();
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, ctx, M, N, K, res, nw, eps, epoch, mode, splits, e) != cudaSuccess)
    return -5;
  return 0;
}

// Debug aid: device buffer of 16 uint64 that receives the timeline of CTA 0 of subsequent launches (nullptr: off).
KSANA_API int ksana_ll_set_trace(void* buf) {
  unsigned long long* p = reinterpret_cast<unsigned long long*>(buf);
  return cudaMemcpyToSymbol(g_ll_trace, &p, sizeof(p)) == cudaSuccess ? 0 : -5;
}

// The same reduction for a partial sum in memory (partial: [M, H] bf16 with pitch ldp, H % 8 == 0, H <= 8192).
KSANA_API int ksana_ll_reduce_norm(const void* partial, int ldp, int M, int H, int rank, int ws, void* const* recv,
                                   long long recv_off, void* const* recv2, void* recv2_mc, void* hbuf, int rows_cap,
                                   int one_shot, void* residual, const void* norm_w, float eps, unsigned int epoch,
                                   int mode, cudaStream_t stream) {
  if (M <= 0) return 0;
  LlCtx ctx;
  if (fill_ctx(&ctx, rank, ws, recv, recv_off, recv2, recv2_mc, hbuf, rows_cap, one_shot, M)) return -1;
  if ((H & 7) || H > LL_MAX_H || (ldp & 3) || epoch == 0) return -1;
  const int rows_per = one_shot ? M : (M + ws - 1) / ws;
  int grid = sm_count();
  const int want = rows_per > (M * (H >> 2) + LL_THREADS - 1) / LL_THREADS ? rows_per
                                                                             : (M * (H >> 2) + LL_THREADS - 1) / LL_THREADS;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  const int kws = g_ll_kernel_ranks > ws ? g_ll_kernel_ranks : ws;
  auto kern = kws <= 2 ? ll_reduce_norm_kernel<2, 6> : kws <= 4 ? ll_reduce_norm_kernel<4, 3> : ll_reduce_norm_kernel<8, 2>;
  kern<<<grid, LL_THREADS, 0, stream>>>(ctx, reinterpret_cast<const __nv_bfloat16*>(partial), ldp, M, H,
                                        reinterpret_cast<__nv_bfloat16*>(residual),
                                        reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, epoch, mode, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
