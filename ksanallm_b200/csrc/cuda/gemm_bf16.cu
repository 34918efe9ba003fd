// bf16 GEMM for sm_100a: C[M, N] = A[M, K] * W[N, K]^T (+ bias), fp32 accumulation in TMEM.
//
// Replaces the reference's cuBLAS/cuBLASLt path (3rdparty/LLM_kernels/csrc/kernels/nvidia/gemm_wrapper/
// gemm_wrapper.cu:70-285, wrapper InvokeMatMul src/ksana_llm/kernels/nvidia/basic_kernel_wrapper.cpp:363-378)
// for every un-quantised linear layer.
//
// Design: persistent, warp-specialised CTA of 6 warps.
//   warp 0      TMA producer: 128 x 64 A tile and BN x 64 W tile per stage (128-byte swizzle), mbarrier tx.
//   warp 1      allocates TMEM, issues tcgen05.mma (128 x BN x 16 per instruction, cta_group::1), commits
//               to the stage's "empty" barrier and, after the last k-block, to the accumulator's "full" one.
//   warps 2..5  epilogue: tcgen05.ld of their TMEM lane quarter, bias, convert, 16-byte global stores. The
//               accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps
//               the main loop of tile i + 1.
// Split-K (small M: decode) spreads one output tile over several CTAs; partials go to an fp32 workspace
// and the CTA that arrives last on the tile's counter reduces them in split order (deterministic) and
// resets the counter. No CTA ever waits for another one.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int BM = 128;
constexpr int BK = 64;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // + barriers + alignment slack
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* __restrict__ C,
                 const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc, int splits,
                 float* __restrict__ ws, unsigned int* __restrict__ counters, unsigned int* err,
                 unsigned long long* trace) {
  using L = GemmSmem<BN, STAGES>;
  // optional timeline of CTA 0 (nanoseconds of the global timer): [0] entry, [1] set-up done, [2] first operands
  // landed, [3] last MMA committed, [4] accumulator visible to the epilogue, [5] epilogue done
  auto stamp = [&](int i) {
    if (trace != nullptr && blockIdx.x == 0) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      trace[i] = t;
    }
  };
  if (threadIdx.x == 0) stamp(0);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_units = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
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
    tmem_alloc(tmem_holder, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (threadIdx.x == 0) stamp(1);

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
        const int kb0 = split * kb_per;
        const int kb1 = min(kb0 + kb_per, num_kb);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m_idx * BM);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * BK, n_idx * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x, ++it) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int kb0 = split * kb_per;
        const int kb1 = min(kb0 + kb_per, num_kb);
        const int as = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (it == 0 && kb == kb0) stamp(2);
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint64_t da = umma_desc_k128(sa);
          const uint64_t db = umma_desc_k128(sa + L::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
        if (it == 0) stamp(3);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;
    int it = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x, ++it) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
      const int as = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      // the 128 epilogue threads agree on the outcome of the bounded wait, so that none of them can be
      // left alone at the named barrier below
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
      if (it == 0 && threadIdx.x == 64) stamp(4);
      const int row = m_idx * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN;
      bool reduce_here = true;
      if (splits > 1) {
        // write fp32 partial, then find out whether this CTA is the last one of the tile
        float* wrow = ws + (static_cast<size_t>(split) * M + row) * N + n_idx * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int col = n_idx * BN + c * 32 + j;
              if (col < N) {
                *reinterpret_cast<float4*>(wrow + c * 32 + j) =
                    make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                __uint_as_float(r[j + 3]));
              }
            }
          }
        }
        __threadfence();
        // named barrier over the 128 epilogue threads
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          unsigned int prev = atomicAdd(&counters[tile], 1u);
          int last = (prev == static_cast<unsigned int>(splits - 1));
          if (last) counters[tile] = 0;
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        reduce_here = (*last_flag != 0);
        __threadfence();
      }
      // tcgen05.ld is warp-collective (.sync.aligned): every lane executes the loads, only the global
      // stores are predicated on the row being inside the matrix.
      const bool row_ok = row < M;
      if (reduce_here) {
        OutT* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          if (splits > 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
            for (int s = 0; s < splits; ++s) {
              const float* wrow = ws + (static_cast<size_t>(s) * M + (row_ok ? row : 0)) * N + n_idx * BN + c * 32;
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                if (row_ok && n_idx * BN + c * 32 + j < N) {
                  float4 p = __ldcg(reinterpret_cast<const float4*>(wrow + j));
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
          const int col0 = n_idx * BN + c * 32;
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) v[j] += __bfloat162float(bias[col0 + j]);
          }
          if constexpr (sizeof(OutT) == 2) {
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
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (row_ok && col0 + j < N) {
                *reinterpret_cast<float4*>(crow + col0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      if (it == 0 && threadIdx.x == 64) stamp(5);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0) stamp(6);
}

template <int BN, int STAGES, typename OutT>
static int launch_gemm(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw,
                       int ldc, int splits, float* ws, unsigned int* counters, int max_ctas, cudaStream_t stream,
                       unsigned long long* trace = nullptr) {
  using L = GemmSmem<BN, STAGES>;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return -3;
  auto kern = gemm_bf16_kernel<BN, STAGES, OutT>;
  if (KSANA_SMEM_ONCE(kern, L::TOTAL) != 0) return -4;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles * splits;
  if (grid > max_ctas) grid = max_ctas;
  kern<<<grid, 192, L::TOTAL, stream>>>(tmA, tmB, reinterpret_cast<OutT*>(C),
                                        reinterpret_cast<const __nv_bfloat16*>(bias), M, N, K, ldc, splits, ws, counters,
                                        error_word(), trace);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ksana

namespace ksana {
int gemm_bf16_cluster_splitk(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda,
                             int ldw, int ldc, int out_fp32, int splits, cudaStream_t stream);
int gemm_bf16_pair(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda, int ldw,
                   int ldc, int out_fp32, int bn, int epi, cudaStream_t stream);
void gemm_pair_set_lane(int lane);
}

// GEMM launches of the calling thread that may overlap on the device (two streams) must use different lanes (0 / 1):
// a lane owns its own parking space for partial tiles. Default lane 0.
KSANA_API void ksana_gemm_set_lane(int lane) { ksana::gemm_pair_set_lane(lane); }

// Gated FFN in one kernel: C[M, N / 2] = SiLU(A Wg^T) * (A Wu^T), for a weight whose gate and up rows are interleaved
// in groups of 16 (rows [32 b, 32 b + 16) = gate rows of features 16 b .. 16 b + 15, the next 16 rows their up rows),
// so every 32 accumulator columns of the CTA-pair GEMM hold 16 (gate, up) pairs and the activation never goes through
// memory as a [M, N] intermediate. N = 2 x features, N % 32 == 0; otherwise the rules of ksana_gemm_bf16. The
// reference's counterpart is its fused gated GEMM (3rdparty/LLM_kernels/csrc/kernels/nvidia/asymmetric_gemm/
// fused_gated_gemm/).
KSANA_API int ksana_gemm_bf16_swiglu(const void* A, const void* W_interleaved, void* C, int M, int N, int K, int lda,
                                     int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 31) || (K & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return -1;
  return ksana::gemm_bf16_pair(A, W_interleaved, C, nullptr, M, N, K, lda, ldw, ldc, 0, 256, 1, stream);
}

static unsigned long long* g_gemm_trace = nullptr;
// Debug aid: device buffer of 8 uint64 that receives the timeline of CTA 0 of subsequent GEMM launches (nullptr: off).
KSANA_API void ksana_gemm_set_trace(void* buf) { g_gemm_trace = reinterpret_cast<unsigned long long*>(buf); }

// C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]). A, W bf16 with row pitches lda / ldw (elements, multiples of 8,
// base pointers 16-byte aligned); C bf16 (out_fp32 = 0) or fp32 (out_fp32 = 1) with row pitch ldc; N % 8 == 0.
// ws: fp32 workspace of at least splits * M * N floats and counters: zero-initialised uint32 per output tile
// (both only read when the launcher decides to split K; pass ws_floats = 0 to forbid splitting).
// bn: 0 = choose; 64 / 128 / 256 = single-CTA kernel with that tile width; 1128 / 1256 = CTA-pair kernel
// (gemm_bf16_2cta.cu) with 256 x 128 / 256 x 256 tiles. Returns 0 on success.
KSANA_API int ksana_gemm_bf16(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda,
                              int ldw, int ldc, int out_fp32, int bn, int force_splits, float* ws, long long ws_floats,
                              unsigned int* counters, int num_counters, cudaStream_t stream) {
  using namespace ksana;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldw & 7) || (ldc & 3)) return -1;
  const int sms = sm_count();
  const int tiles_m = (M + BM - 1) / BM;
  if (bn == 1128 || bn == 1256)
    return gemm_bf16_pair(A, W, C, bias, M, N, K, lda, ldw, ldc, out_fp32, bn - 1000, 0, stream);
  if (bn == 0 && force_splits == 0 && M >= 384 && N >= 256)
    // prefill-sized M: CTA pairs with 256 x 256 tiles (the 256 x 128 pair tile runs the tensor cores at half rate
    // and is only for narrow outputs); measured at or above the library GEMM from M = 512 up, while for M <= 256
    // the single-CTA tiles and the cluster split-K path below stay ahead
    return gemm_bf16_pair(A, W, C, bias, M, N, K, lda, ldw, ldc, out_fp32, 256, 0, stream);
  if (bn == 0) {
    // A CTA's K loop is latency-bound (~0.3 us per 64-wide k-block whatever the tile width), so the cost of a
    // launch is (number of waves) x (k-blocks) with a ~15 % surcharge for the wider tile: pick the cheaper one.
    const int t256 = tiles_m * ((N + 255) / 256);
    const int t128 = tiles_m * ((N + 127) / 128);
    const float c128 = static_cast<float>((t128 + sms - 1) / sms);
    const float c256 = 1.15f * static_cast<float>((t256 + sms - 1) / sms);
    bn = (c256 < c128) ? 256 : 128;
    if (t128 * 2 <= sms) bn = 128;  // few tiles: the cluster split-K path below takes over
    if (N <= 64) bn = 64;
  }
  const int num_kb = (K + BK - 1) / BK;
  // ---- small M: K-splits of a tile run as one thread-block cluster and reduce through distributed shared memory.
  // force_splits > 0 requests that many splits (2 / 4 / 8 take the cluster path), force_splits < 0 requests
  // |force_splits| splits through the global-workspace reduction below.
  {
    const int tiles128 = tiles_m * ((N + 127) / 128);
    int cs = 0;
    if (force_splits == 2 || force_splits == 4 || force_splits == 8) {
      cs = force_splits;
    } else if (force_splits == 0 && (bn == 128 || bn == 64) && tiles128 * 2 <= sms && num_kb >= 8) {
      cs = 8;
      while (cs > 1 && (cs * tiles128 > sms + tiles128 / 2 || num_kb / cs < 4)) cs >>= 1;
    }
    if (cs >= 2 && (bn == 0 || bn == 128 || force_splits == 0) && ((num_kb + cs - 1) / cs) * (cs - 1) < num_kb &&
        cs <= sms)
      return gemm_bf16_cluster_splitk(A, W, C, bias, M, N, K, lda, ldw, ldc, out_fp32, cs, stream);
  }
  if (force_splits < 0) force_splits = -force_splits;
  const int tiles = tiles_m * ((N + bn - 1) / bn);
  // the global-workspace reduction runs on request only (the automatic choice for small M is the cluster path above)
  int splits = force_splits > 1 ? force_splits : 1;
  if (splits > 16) splits = 16;
  // every split must own at least one k-block
  while (splits > 1 && ((num_kb + splits - 1) / splits) * (splits - 1) >= num_kb) --splits;
  if (splits > 1 && (ws == nullptr || counters == nullptr || static_cast<long long>(splits) * M * N > ws_floats ||
                     tiles > num_counters))
    splits = 1;
#define KSANA_GEMM_CASE(BN_, ST_)                                                                                   \
  return out_fp32 ? launch_gemm<BN_, ST_, float>(A, W, C, bias, M, N, K, lda, ldw, ldc, splits, ws, counters, sms, \
                                                 stream, g_gemm_trace)                                              \
                  : launch_gemm<BN_, ST_, __nv_bfloat16>(A, W, C, bias, M, N, K, lda, ldw, ldc, splits, ws,        \
                                                         counters, sms, stream, g_gemm_trace)
  if (bn == 64) { KSANA_GEMM_CASE(64, 8); }
  if (bn == 256) { KSANA_GEMM_CASE(256, 4); }
  KSANA_GEMM_CASE(128, 6);
#undef KSANA_GEMM_CASE
}
