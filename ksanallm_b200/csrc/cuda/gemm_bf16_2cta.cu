// bf16 GEMM on CTA pairs for sm_100a: C[M, N] = A[M, K] * W[N, K]^T (+ bias), one tcgen05.mma spanning two SMs.
//
// The large-M (prefill) counterpart of gemm_bf16.cu; same role as the reference's cuBLASLt path
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/gemm_wrapper/gemm_wrapper.cu:70-285).
//
// Why pairs: a single-CTA 128 x 256 x 16 MMA reads 12 KB of operands from shared memory per 128 tensor-core cycles
// while TMA refills the same amount, which is more than one SM's shared-memory port sustains, so the tensor pipe
// idles ~20 % of the time. With cta_group::2 the pair computes a 256 x BN tile: each CTA stages only ITS 128 rows
// of A and ITS half of the W rows (8 KB per MMA per SM), the hardware exchanges the W halves between the two SMs.
//
// Launch: clusters of 2 CTAs, one cluster per TPC, persistent over 256 x BN output tiles in a grouped order. Full
// waves of tiles are dealt round-robin (pairs running at the same time work on neighbouring tiles and share their
// operand panels in L2). The tiles of the last, partial wave are split stream-K fashion: their (tile, k-block)
// iterations form one sequence that is cut into equal contiguous ranges, one per CTA pair, so every SM pair
// streams operands for the same time whatever the tile count. A range that ends inside a tile leaves a partial
// tile: the pair that owns the tile's FIRST k-blocks (it reaches them last) finishes the tile; the pairs that own
// later k-blocks (they reach them first) park their fp32 partial in a workspace slot, raise a flag and move on. So
// nobody ever waits for work that has not started, and a pair parks at most one partial. Per CTA, 6 warps:
//   warp 0      TMA producer (both CTAs): own A rows and own W half of every k-block; the byte counts of BOTH
//               CTAs are credited to the LEADER's "full" barrier (plain tiled loads, no cluster fan-out).
//   warp 1      allocates TMEM (both CTAs); in the leader one lane issues tcgen05.mma.cta_group::2 and commits to
//               the stage's "empty" barrier of both CTAs and, after the last k-block, to both "accumulator full".
//   warps 2..5  epilogue (both CTAs): own 128 accumulator rows x BN columns from TMEM (+ the parked partials of the
//               other contributors), bias / SwiGLU, 16-byte global stores - or the partial to the workspace; arrive
//               on the leader's "accumulator empty" barrier. The accumulator is double-buffered.
// Every wait is bounded; on expiry the status word is set and the kernel leaves through its normal teardown.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int P_BM = 128;  // rows per CTA, 256 per pair
constexpr int P_BK = 64;

template <int BN>
struct PairCfg {
  static constexpr int HALF_N = BN / 2;
  static constexpr int A_BYTES = P_BM * P_BK * 2;
  static constexpr int B_BYTES = HALF_N * P_BK * 2;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 6 : 8;
  static constexpr int BAR = STAGES * STAGE;
  static constexpr int SMEM = BAR + 512 + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

constexpr int P_GROUP_M = 8;  // tile order: groups of 8 row tiles, column-major inside a group
__device__ __forceinline__ void pair_tile_coords(int t, int tiles_m, int tiles_n, int* m_idx, int* n_idx) {
  const int per_group = P_GROUP_M * tiles_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m0 = g * P_GROUP_M;
  const int gm = min(P_GROUP_M, tiles_m - m0);
  *n_idx = r / gm;
  *m_idx = m0 + (r - (*n_idx) * gm);
}

// Work list of one CTA pair: its tiles of the full waves, then its range of the stream-K tail.
struct PairSched {
  int pair, num_pairs, num_kb, dp_waves, sk_tile0;
  long long sk_total, per, I, I_end;
  int wave;
  int total_tiles;
  __device__ PairSched(int pair_, int num_pairs_, int total_tiles_, int num_kb_) {
    pair = pair_;
    num_pairs = num_pairs_;
    num_kb = num_kb_;
    total_tiles = total_tiles_;
    dp_waves = total_tiles / num_pairs;
    // After many full waves an idle tail costs a few percent, less than the fix-up of the partial tiles: the tail
    // is then one more round-robin wave. With few waves it is split by k-blocks, at most ~4 ranges per tile.
    if (dp_waves >= 8) dp_waves = (total_tiles + num_pairs - 1) / num_pairs;
    sk_tile0 = min(total_tiles, dp_waves * num_pairs);
    sk_total = static_cast<long long>(total_tiles - sk_tile0) * num_kb;
    per = (sk_total + num_pairs - 1) / num_pairs;
    const long long floor_per = num_kb < 8 ? num_kb : max(8, (num_kb + 3) / 4);
    if (per < floor_per) per = floor_per;
    I = min(sk_total, per * pair);
    I_end = min(sk_total, per * (pair + 1));
    wave = 0;
  }
  // next segment: tile, k-block range [kb0, kb1). Returns false when the list is exhausted.
  __device__ bool next(int* tile, int* kb0, int* kb1) {
    if (wave < dp_waves) {
      *tile = pair + wave * num_pairs;
      ++wave;
      if (*tile < total_tiles) {
        *kb0 = 0;
        *kb1 = num_kb;
        return true;
      }
    }
    if (I >= I_end) return false;
    const int t = static_cast<int>(I / num_kb);
    *tile = sk_tile0 + t;
    *kb0 = static_cast<int>(I - static_cast<long long>(t) * num_kb);
    *kb1 = static_cast<int>(min(static_cast<long long>(num_kb), *kb0 + (I_end - I)));
    I += *kb1 - *kb0;
    return true;
  }
  // last pair that holds k-blocks of stream-K tile `tile` (the pairs after the finisher up to this one park partials)
  __device__ int last_contributor(int tile) const {
    const long long tile_end = static_cast<long long>(tile - sk_tile0 + 1) * num_kb;
    return static_cast<int>((tile_end - 1) / per);
  }
};

// EPI 0: C = acc (+ bias).  EPI 1: gated activation. The W rows are interleaved in groups of 16 (16 gate rows, then
// the 16 up rows of the same features), so every 32 accumulator columns hold 16 (gate, up) pairs:
// C[row, col / 2 + j] = silu(acc[col + j]) * acc[col + 16 + j]; C is [M, N / 2].
template <int BN, int EPI, typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      OutT* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc,
                      float* __restrict__ part, uint32_t* __restrict__ part_flags, uint32_t seq, unsigned int* err) {
  using L = PairCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR);
  uint64_t* empty_bar = full_bar + L::STAGES;
  uint64_t* acc_full = empty_bar + L::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: leader (issues the MMAs), 1: peer
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + P_BK - 1) / P_BK;
  const int total_tiles = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // used in the leader only: its producer's arrive + both CTAs' bytes
      mbar_init(&empty_bar[s], 1);  // one commit from the leader's MMA lane
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);  // used in the leader only: 4 epilogue warps x 2 CTAs
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, L::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them remotely
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ---------------- producer (both CTAs) ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairSched sched(pair, num_pairs, total_tiles, num_kb);
      int tile, kb0, kb1;
      while (ok && sched.next(&tile, &kb0, &kb1)) {
        int m_idx, n_idx;
        pair_tile_coords(tile, tiles_m, tiles_n, &m_idx, &n_idx);
        const int row0 = m_idx * 2 * P_BM + static_cast<int>(cta) * P_BM;
        const int wrow0 = n_idx * BN + static_cast<int>(cta) * L::HALF_N;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::STAGE;
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE);
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tmA, leader_full, kb * P_BK, row0);
          tma_load_2d_pair(sa + L::A_BYTES, &tmB, leader_full, kb * P_BK, wrow0);
          if (++stage == L::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only) ----------------
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = umma_idesc(2 * P_BM, BN, 1, 1);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairSched sched(pair, num_pairs, total_tiles, num_kb);
      int tile, kb0, kb1;
      for (; ok && sched.next(&tile, &kb0, &kb1); ++it) {
        const int as = it & 1;
        if (!mbar_wait_cluster_bounded(&acc_empty[as], ((it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_cluster_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < P_BK / 16; ++k)
            umma_f16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(eb);               // my producer may refill the stage
          umma_commit_pair(mapa_u32(eb, 1));  // and so may the peer's
          if (++stage == L::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t fb = smem_u32(&acc_full[as]);
          umma_commit_pair(fb);
          umma_commit_pair(mapa_u32(fb, 1));
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127
    int it = 0;
    PairSched sched(pair, num_pairs, total_tiles, num_kb);
    int tile, kb0, kb1;
    for (; sched.next(&tile, &kb0, &kb1); ++it) {
      int m_idx, n_idx;
      pair_tile_coords(tile, tiles_m, tiles_n, &m_idx, &n_idx);
      const int as = it & 1;
      // tcgen05.ld is warp-collective: the lanes of a warp must agree on the outcome of the bounded wait
      const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[as], (it >> 1) & 1, abort_flag, err));
      if (!ok) break;
      tc_fence_after();
      const int trow = quarter * 32 + lane;  // row inside this CTA's half of the tile
      const int row = m_idx * 2 * P_BM + static_cast<int>(cta) * P_BM + trow;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN;
      if (kb0 != 0) {
        // ---- later k-blocks of a tile somebody else finishes: park the partial, raise the flag, move on ----
        // slot layout [BN / 4 column quads][128 rows] of float4: the 32 lanes of a warp (32 rows) touch 512
        // contiguous bytes per access
        float4* slot = reinterpret_cast<float4*>(part) + (static_cast<size_t>(pair) * 2 + cta) * (P_BM * BN / 4) + trow;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            __stcg(slot + static_cast<size_t>(c * 8 + (j >> 2)) * P_BM,
                   make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                               __uint_as_float(r[j + 3])));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&acc_empty[as]), 0));
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(part_flags + pair * 2 + cta), "r"(seq) : "memory");
        }
        continue;
      }
      // ---- this pair owns the tile's first k-blocks: collect the partials of the pairs that own the rest ----
      int q_first = pair + 1, q_last = pair;  // contributors [q_first, q_last]
      if (kb1 < num_kb) {
        q_last = sched.last_contributor(tile);
        bool got = true;
        if (lane == 0) {
          for (int q = q_first; q <= q_last && got; ++q) {
            const uint32_t* f = part_flags + q * 2 + cta;
            uint32_t v = 0;
            for (uint32_t spin = 0; spin < KSANA_MBAR_SPIN_LIMIT; ++spin) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
              if (v == seq || *abort_flag) break;
              if ((spin & 15u) == 15u) __nanosleep(100);
            }
            if (v != seq) {
              got = false;
              *abort_flag = 1;
              atomicOr(err, KERR_FLAG_TIMEOUT);
            }
          }
        }
        got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!got) break;
      }
      OutT* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        for (int q = q_first; q <= q_last; ++q) {  // fixed order: the result does not depend on timing
          const float4* src = reinterpret_cast<const float4*>(part) + (static_cast<size_t>(q) * 2 + cta) * (P_BM * BN / 4) +
                              static_cast<size_t>(c * 8) * P_BM + trow;
          float4 p4[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) p4[j] = __ldcg(src + static_cast<size_t>(j) * P_BM);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[4 * j] += p4[j].x;
            v[4 * j + 1] += p4[j].y;
            v[4 * j + 2] += p4[j].z;
            v[4 * j + 3] += p4[j].w;
          }
        }
        const int col0 = n_idx * BN + c * 32;
        if (bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < N) v[j] += __bfloat162float(bias[col0 + j]);
        }
        if constexpr (EPI == 1) {
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = v[j] / (1.f + __expf(-v[j])) * v[16 + j];
          if (row_ok && col0 < N) {
            OutT* dst = crow + (col0 >> 1);
            if constexpr (sizeof(OutT) == 2) {
#pragma unroll
              for (int j = 0; j < 16; j += 8) {
                uint4 u;
                u.x = pack_bf16(o[j], o[j + 1]);
                u.y = pack_bf16(o[j + 2], o[j + 3]);
                u.z = pack_bf16(o[j + 4], o[j + 5]);
                u.w = pack_bf16(o[j + 6], o[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = u;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
            }
          }
        } else if constexpr (sizeof(OutT) == 2) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (row_ok && col0 + j < N) {
              uint4 u;
              u.x = pack_bf16(v[j], v[j + 1]);
              u.y = pack_bf16(v[j + 2], v[j + 3]);
              u.z = pack_bf16(v[j + 4], v[j + 5]);
              u.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(crow + col0 + j) = u;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            if (row_ok && col0 + j < N)
              *reinterpret_cast<float4*>(crow + col0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          }
        }
      }
      // this warp's accumulator rows are drained: one arrival per warp on the leader's barrier
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa_u32(smem_u32(&acc_empty[as]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or leaves while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
  }
}

// Parking space for partial tiles: one slot of 2 x 128 x 256 floats and two flags per SM pair, per device,
// allocated on first use and kept. `seq` tags the flags of one launch (launches on a device are assumed to be
// ordered on one stream, like every other user of the library's scratch buffers).
struct PairScratch {
  float* part = nullptr;
  uint32_t* flags = nullptr;
  uint32_t seq = 0;
};
static PairScratch g_pair_scratch[64][2];
// Which of the two scratch sets the calling thread's next launches use: launches that may run at the same time (two
// streams of one device) must not share parked partials and flags.
static thread_local int g_pair_lane = 0;

static PairScratch* pair_scratch(int pairs) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  PairScratch* s = &g_pair_scratch[dev][g_pair_lane & 1];
  if (s->part == nullptr) {
    const size_t bytes = static_cast<size_t>(128) * 2 * P_BM * 256 * sizeof(float);  // up to 128 pairs
    if (cudaMalloc(&s->part, bytes) != cudaSuccess) return nullptr;
    if (cudaMalloc(&s->flags, 1024) != cudaSuccess) return nullptr;
    cudaMemset(s->flags, 0, 1024);
  }
  return pairs <= 128 ? s : nullptr;
}

template <int BN, int EPI, typename OutT>
static int launch_pair(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw,
                       int ldc, cudaStream_t stream) {
  using L = PairCfg<BN>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, P_BM, P_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, L::HALF_N, P_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  auto kern = gemm_bf16_pair_kernel<BN, EPI, OutT>;
  if (KSANA_SMEM_ONCE(kern, L::SMEM) != 0) return -4;
  const int tiles = ((M + 2 * P_BM - 1) / (2 * P_BM)) * ((N + BN - 1) / BN);
  const int num_kb = (K + P_BK - 1) / P_BK;
  int pairs = sm_count() / 2;
  // never more pairs than 4-k-block ranges of work
  const long long total_iters = static_cast<long long>(tiles) * num_kb;
  if (pairs > (total_iters + 3) / 4) pairs = static_cast<int>((total_iters + 3) / 4);
  if (pairs < 1) pairs = 1;
  PairScratch* scratch = pair_scratch(pairs);
  if (scratch == nullptr) return -6;
  if (++scratch->seq == 0) scratch->seq = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = L::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  OutT* c = reinterpret_cast<OutT*>(C);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(bias);
  unsigned int* e = error_word();
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, c, b, M, N, K, ldc, scratch->part, scratch->flags, scratch->seq, e) !=
      cudaSuccess)
    return -5;
  return 0;
}

void gemm_pair_set_lane(int lane) { g_pair_lane = lane & 1; }

// epi 0: plain (+ bias); epi 1: gated SiLU over 16-row interleaved W (C is [M, N / 2], N % 32 == 0).
// bn: 128 or 256. Same argument rules as ksana_gemm_bf16.
int gemm_bf16_pair(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw,
                   int ldc, int out_fp32, int bn, int epi, cudaStream_t stream) {
  if (epi == 1 && (N & 31)) return -1;
#define KSANA_PAIR_CASE(BN_, EPI_)                                                                       \
  return out_fp32 ? launch_pair<BN_, EPI_, float>(A, W, C, bias, M, N, K, lda, ldw, ldc, stream)         \
                  : launch_pair<BN_, EPI_, __nv_bfloat16>(A, W, C, bias, M, N, K, lda, ldw, ldc, stream)
  if (bn == 128) {
    if (epi == 1) { KSANA_PAIR_CASE(128, 1); }
    KSANA_PAIR_CASE(128, 0);
  }
  if (epi == 1) { KSANA_PAIR_CASE(256, 1); }
  KSANA_PAIR_CASE(256, 0);
#undef KSANA_PAIR_CASE
}

}  // namespace ksana
