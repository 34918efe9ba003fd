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
//   hop 2  ... and writes the normalised row into every rank's activation buffer (multimem.st through the switch
//          or plain peer stores), fences, and raises that row's flag on every rank.
//   end    Every rank waits for the flags of all rows: when the kernel ends the full activation is local.
// The same two hops without a GEMM (a partial sum that is already in memory, e.g. an expert layer's output) are the
// second entry point below.
//
// Buffer reuse needs no extra handshake: a rank starts call e + 1 only after it has seen every row of call e, so
// every owner had finished reading call e's words, and an owner writes rows of call e + 1 to a peer only after that
// peer's words of call e + 1 arrived, i.e. after the peer's earlier kernels (the readers of the activation buffer)
// are over. All CTAs are resident (grid <= SM count, one CTA per SM); every wait is bounded by wall time.
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
  uint2* recv[LL_MAX_RANKS];          // each rank's word buffer [ws][rows_cap][H / 2] of {bf16x2, epoch}
  __nv_bfloat16* hbuf[LL_MAX_RANKS];  // each rank's activation buffer [>= M][H]
  uint32_t* flags[LL_MAX_RANKS];      // each rank's row flags [>= M]
  __nv_bfloat16* hbuf_mc;             // multicast view of hbuf, or nullptr (plain peer stores)
  int rows_cap;                       // rows of one source slot in recv
};

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
  const int owner = row / rows_per;
  const int lrow = row - owner * rows_per;
  uint2* dst = ctx.recv[owner] + (static_cast<size_t>(ctx.rank) * ctx.rows_cap + lrow) * (H >> 1) + (col >> 1);
  uint4 w;
  w.x = pack_bf16(a, b);
  w.y = epoch;
  w.z = pack_bf16(c, d);
  w.w = epoch;
  st_peer16(dst, w);
}

// Owner side + hop 2 + final wait; called by all threads of every CTA once its own sends are issued.
__device__ __forceinline__ void ll_reduce_norm_gather(const LlCtx& ctx, int M, int H, __nv_bfloat16* residual,
                                                      const __nv_bfloat16* norm_w, float eps, uint32_t epoch, int mode,
                                                      float* s_red, int* s_flag, unsigned int* err) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int rank = ctx.rank, ws = ctx.ws;
  const int rows_per = (M + ws - 1) / ws;
  const int row_lo = rank * rows_per, row_hi = min(M, row_lo + rows_per);
  const int ngroups = H >> 3;
  const uint2* my_recv = ctx.recv[rank];
  bool alive = true;
  for (int row = row_lo + static_cast<int>(blockIdx.x); row < row_hi; row += gridDim.x) {
    const int lrow = row - row_lo;
    float v[LL_MAX_GROUPS][8];
    float ss = 0.f;
    int ok = 1;
#pragma unroll
    for (int gi = 0; gi < LL_MAX_GROUPS; ++gi) {
      const int g = tid + gi * nthr;
      if (g < ngroups) {
        float acc[8];
        if (mode & 2) {
          unpack8(*reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * H + (g << 3)), acc);
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        uint4 wa[LL_MAX_RANKS], wb[LL_MAX_RANKS];
#pragma unroll
        for (int s = 0; s < LL_MAX_RANKS; ++s) {
          if (s < ws) {
            const uint2* p = my_recv + (static_cast<size_t>(s) * ctx.rows_cap + lrow) * (H >> 1) + (g << 2);
            wa[s] = ld_volatile16(p);
            wb[s] = ld_volatile16(p + 2);
          }
        }
#pragma unroll
        for (int s = 0; s < LL_MAX_RANKS; ++s) {
          if (s < ws) {
            if (wa[s].y != epoch || wa[s].w != epoch || wb[s].y != epoch || wb[s].w != epoch) {
              // not there yet: poll this source's words (bounded by wall time)
              const uint2* p = my_recv + (static_cast<size_t>(s) * ctx.rows_cap + lrow) * (H >> 1) + (g << 2);
              const unsigned long long t0 = global_timer_ns();
              while (alive) {
                wa[s] = ld_volatile16(p);
                wb[s] = ld_volatile16(p + 2);
                if (wa[s].y == epoch && wa[s].w == epoch && wb[s].y == epoch && wb[s].w == epoch) break;
                if (global_timer_ns() - t0 > KSANA_PEER_TIMEOUT_NS) {
                  atomicOr(err, KERR_PEER_TIMEOUT);
                  alive = false;
                }
              }
              if (!alive) ok = 0;
            }
            const uint32_t d[4] = {wa[s].x, wa[s].z, wb[s].x, wb[s].z};
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
    float inv = 1.f;
    if (mode & 1) {
      ss = warp_sum(ss);
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
        const size_t off = static_cast<size_t>(row) * H + (g << 3);
        if (ctx.hbuf_mc != nullptr) {
          multimem_st16(ctx.hbuf_mc + off, packed);
        } else {
          for (int p = 0; p < ws; ++p) st_peer16(ctx.hbuf[p] + off, packed);
        }
      }
    }
    // the row is out: fence, then raise its flag on every rank (a failed wait raises nothing: peers time out too)
    __threadfence_system();
    if (tid == 0) *s_flag = 1;
    __syncthreads();
    if (!ok) *s_flag = 0;
    __syncthreads();
    if (*s_flag && tid < ws) st_release_sys(ctx.flags[tid] + row, epoch);
    __syncthreads();  // s_red / s_flag are reused by the next row
  }
  // all rows of all owners have landed here
  const uint32_t* my_flags = ctx.flags[rank];
  for (int r = static_cast<int>(blockIdx.x) * nthr + tid; r < M; r += gridDim.x * nthr) wait_flag_ge(my_flags + r, epoch, err);
}

// ---- GEMM + the two hops ----------------------------------------------------------------------------------
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
  int* s_flag = const_cast<int*>(abort_flag) + 1;
  float* s_red = reinterpret_cast<float*>(s_flag + 1);  // [8]

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
      }
    }
  } else {
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127
    const int rows_slice = LL_BM / splits;
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
#pragma unroll 1
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
      // 4. reduce my slice of rows over the cluster in rank order and send it to the rows' owners
      const uint32_t stg_addr = smem_u32(stg);
#pragma unroll 4
      for (int i = et; i < rows_slice * (LL_BN / 4); i += 128) {
        const int lr = split * rows_slice + i / (LL_BN / 4);
        const int c4 = (i % (LL_BN / 4)) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < splits; ++p) {
          const float4 v = ld_cluster_f4(mapa_u32(stg_addr + (lr * LL_PITCH + c4) * 4, p));
          acc.x += v.x;
          acc.y += v.y;
          acc.z += v.z;
          acc.w += v.w;
        }
        const int row = m_idx * LL_BM + lr;
        if (row < M) ll_send4(ctx, rows_per, row, n_idx * LL_BN + c4, N, acc.x, acc.y, acc.z, acc.w, epoch);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (et < splits) mbar_arrive_remote(mapa_u32(smem_u32(stg_free), et));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody reads a peer's shared memory past this point
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * LL_BN);
  }
  if (*abort_flag) return;  // a wait inside the GEMM gave up: the status word is set, peers time out on their own
  ll_reduce_norm_gather(ctx, M, N, residual, norm_w, eps, epoch, mode, s_red, s_flag, err);
}

// ---- the two hops for a partial sum that is already in memory ---------------------------------------------------
__global__ void __launch_bounds__(LL_THREADS)
ll_reduce_norm_kernel(LlCtx ctx, const __nv_bfloat16* __restrict__ partial, int ldp, int M, int H,
                      __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ norm_w, float eps,
                      uint32_t epoch, int mode, unsigned int* err) {
  __shared__ float s_red[8];
  __shared__ int s_flag;
  const int rows_per = (M + ctx.ws - 1) / ctx.ws;
  const int nq = H >> 2;  // 4-column pieces per row
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < M * nq; i += gridDim.x * blockDim.x) {
    const int row = i / nq, col = (i - row * nq) << 2;
    const uint2 raw = *reinterpret_cast<const uint2*>(partial + static_cast<size_t>(row) * ldp + col);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    ll_send4(ctx, rows_per, row, col, H, a.x, a.y, b.x, b.y, epoch);
  }
  ll_reduce_norm_gather(ctx, M, H, residual, norm_w, eps, epoch, mode, s_red, &s_flag, err);
}

static int fill_ctx(LlCtx* ctx, int rank, int ws, void* const* recv, void* const* hbuf, void* const* flags,
                    void* hbuf_mc, int rows_cap) {
  if (ws < 1 || ws > LL_MAX_RANKS || rank < 0 || rank >= ws) return -1;
  ctx->rank = rank;
  ctx->ws = ws;
  for (int i = 0; i < LL_MAX_RANKS; ++i) {
    ctx->recv[i] = i < ws ? reinterpret_cast<uint2*>(recv[i]) : nullptr;
    ctx->hbuf[i] = i < ws ? reinterpret_cast<__nv_bfloat16*>(hbuf[i]) : nullptr;
    ctx->flags[i] = i < ws ? reinterpret_cast<uint32_t*>(flags[i]) : nullptr;
  }
  ctx->hbuf_mc = reinterpret_cast<__nv_bfloat16*>(hbuf_mc);
  ctx->rows_cap = rows_cap;
  return 0;
}

}  // namespace ksana

using namespace ksana;

// y = AllGather(RMSNorm(residual_slice += ReduceScatter(A * W^T)) * norm_w) in one launch, for small M.
// A: [M, K] bf16 (pitch lda), W: [N, K] bf16 (pitch ldw). Per-rank symmetric buffers (index = rank):
// recv [ws][rows_cap][N / 2] 8-byte words (zero-initialised once), hbuf [>= M][N] bf16, flags [>= M] uint32
// (zero-initialised once). N % 128 == 0, N <= 8192, M <= ws * rows_cap, epoch != 0 and growing by one per call on
// these buffers. mode bit0: RMSNorm, bit1: residual add (residual [M, N], only the owner's rows are touched).
KSANA_API int ksana_gemm_ll_reduce_norm(const void* A, const void* W, int M, int N, int K, int lda, int ldw, int rank,
                                        int ws, void* const* recv, void* const* hbuf, void* const* flags, void* hbuf_mc,
                                        int rows_cap, void* residual, const void* norm_w, float eps, unsigned int epoch,
                                        int mode, int force_splits, cudaStream_t stream) {
  if (M <= 0) return 0;
  LlCtx ctx;
  if (fill_ctx(&ctx, rank, ws, recv, hbuf, flags, hbuf_mc, rows_cap)) return -1;
  if ((N % LL_BN) || N > LL_MAX_H || (K & 7) || (lda & 7) || (ldw & 7) || (M + ws - 1) / ws > rows_cap || epoch == 0)
    return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, LL_BM, LL_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, LL_BN, LL_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (KSANA_SMEM_ONCE(gemm_ll_reduce_norm_kernel, LL_SMEM) != 0) return -4;
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
  if (cudaLaunchKernelEx(&cfg, gemm_ll_reduce_norm_kernel, tmA, tmB, ctx, M, N, K, res, nw, eps, epoch, mode, splits,
                         e) != cudaSuccess)
    return -5;
  return 0;
}

// The same reduction for a partial sum in memory (partial: [M, H] bf16 with pitch ldp, H % 8 == 0, H <= 8192).
KSANA_API int ksana_ll_reduce_norm(const void* partial, int ldp, int M, int H, int rank, int ws, void* const* recv,
                                   void* const* hbuf, void* const* flags, void* hbuf_mc, int rows_cap, void* residual,
                                   const void* norm_w, float eps, unsigned int epoch, int mode, cudaStream_t stream) {
  if (M <= 0) return 0;
  LlCtx ctx;
  if (fill_ctx(&ctx, rank, ws, recv, hbuf, flags, hbuf_mc, rows_cap)) return -1;
  if ((H & 7) || H > LL_MAX_H || (ldp & 3) || (M + ws - 1) / ws > rows_cap || epoch == 0) return -1;
  const int rows_per = (M + ws - 1) / ws;
  int grid = sm_count();
  const int want = rows_per > (M * (H >> 2) + LL_THREADS - 1) / LL_THREADS ? rows_per
                                                                             : (M * (H >> 2) + LL_THREADS - 1) / LL_THREADS;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  ll_reduce_norm_kernel<<<grid, LL_THREADS, 0, stream>>>(ctx, reinterpret_cast<const __nv_bfloat16*>(partial), ldp, M, H,
                                                         reinterpret_cast<__nv_bfloat16*>(residual),
                                                         reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, epoch,
                                                         mode, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
