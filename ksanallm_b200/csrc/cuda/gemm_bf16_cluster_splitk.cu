// Split-K bf16 GEMM for small M (decode): the K-splits of one 128 x 128 output tile run as ONE thread-block cluster
// and are reduced through distributed shared memory - no global workspace, no atomics, no memory fences.
//
// Why: a decode GEMM is a weight stream. One CTA keeps at most ~200 KB of TMA loads in flight, so the stream only
// approaches HBM speed when (nearly) all 148 SMs pull at once; with few output tiles that means splitting K. The
// global-workspace reduction of gemm_bf16.cu costs ~13 us per tile (scattered fp32 stores, fence, atomic, re-read);
// here each CTA parks its fp32 partial tile in its own shared memory, the cluster synchronises through remote
// mbarrier arrivals, and every CTA reduces a 128/splits-row slice of the tile by reading the peers' tiles with
// ld.shared::cluster, then writes the final bf16 rows with coalesced stores.
//
// Pipeline per CTA as in gemm_bf16.cu: warp 0 TMA producer, warp 1 tcgen05 issuer, warps 2-5 epilogue.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int CS_BM = 128, CS_BN = 128, CS_BK = 64, CS_STAGES = 4;
constexpr int CS_A_BYTES = CS_BM * CS_BK * 2, CS_B_BYTES = CS_BN * CS_BK * 2, CS_STAGE = CS_A_BYTES + CS_B_BYTES;
constexpr int CS_PITCH = CS_BN + 4;                       // floats per staged row (+4: bank-conflict padding)
constexpr int CS_STG = CS_STAGES * CS_STAGE;              // fp32 partial tile
constexpr int CS_BAR = CS_STG + CS_BM * CS_PITCH * 4;
constexpr int CS_SMEM = CS_BAR + 256 + 1024;

template <typename OutT>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_cluster_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                OutT* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                                int ldc, int splits, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* stg = reinterpret_cast<float*>(smem + CS_STG);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + CS_BAR);
  uint64_t* empty_bar = full_bar + CS_STAGES;
  uint64_t* acc_full = empty_bar + CS_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* part_ready = acc_empty + 2;  // every CTA of the cluster arrives once per tile: partial tiles are in place
  uint64_t* stg_free = part_ready + 1;   // every CTA arrives once per tile: it has finished reading my partial tile
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(stg_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + CS_BM - 1) / CS_BM;
  const int tiles_n = (N + CS_BN - 1) / CS_BN;
  const int num_kb = (K + CS_BK - 1) / CS_BK;
  const int kb_per = (num_kb + splits - 1) / splits;
  const int total_tiles = tiles_m * tiles_n;
  const int split = static_cast<int>(cluster_ctarank());
  const int cluster_id = blockIdx.x / splits;
  const int num_clusters = gridDim.x / splits;
  const int kb0 = split * kb_per, kb1 = min(kb0 + kb_per, num_kb);

  if (threadIdx.x == 0) {
    for (int s = 0; s < CS_STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 2 * CS_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();  // peers' barriers are initialised before anybody arrives on them remotely
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
          uint8_t* sa = smem + stage * CS_STAGE;
          mbar_expect_tx(&full_bar[stage], CS_STAGE);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * CS_BK, m_idx * CS_BM);
          tma_load_2d(sa + CS_A_BYTES, &tmB, &full_bar[stage], kb * CS_BK, n_idx * CS_BN);
          if (++stage == CS_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(CS_BM, CS_BN, 1, 1);
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
          const uint32_t sa = smem_u32(smem + stage * CS_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + CS_A_BYTES);
#pragma unroll
          for (int k = 0; k < CS_BK / 16; ++k)
            umma_f16(tmem_base + as * CS_BN, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == CS_STAGES) {
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
    int it = 0;
    for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++it) {
      const int m_idx = tile % tiles_m, n_idx = tile / tiles_m;
      const int as = it & 1;
      const uint32_t ph = it & 1;
      // all 128 epilogue threads agree on every bounded wait (nobody is left alone at a named barrier)
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
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * CS_BN;
      const int rows_valid = min(CS_BM, M - m_idx * CS_BM);  // rows of this tile that exist in the matrix
      if (quarter * 32 < rows_valid) {
#pragma unroll 2
        for (int c = 0; c < CS_BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(stg + trow * CS_PITCH + c * 32 + j) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                            __uint_as_float(r[j + 3]));
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      // 2. publish to every CTA of the cluster (including myself)
      if (et < splits) mbar_arrive_remote(mapa_u32(smem_u32(part_ready), et));
      // 3. wait until all partial tiles of the cluster are in place
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
      // 4. reduce my slice of the tile's rows over all CTAs, in rank order (deterministic), and write the final rows
      const uint32_t stg_addr = smem_u32(stg);
      const int rows_slice = (rows_valid + splits - 1) / splits;
      const int r0 = split * rows_slice;
      const int n_items = max(min(rows_valid, r0 + rows_slice) - r0, 0) * (CS_BN / 4);
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
                const int lr = r0 + i / (CS_BN / 4), c4 = (i % (CS_BN / 4)) * 4;
                const float4 v = ld_cluster_f4(mapa_u32(stg_addr + (lr * CS_PITCH + c4) * 4, p));
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
          const int lr = r0 + i / (CS_BN / 4), c4 = (i % (CS_BN / 4)) * 4;
          const int row = m_idx * CS_BM + lr, col = n_idx * CS_BN + c4;
          if (i < n_items && col < N) {
            float4 a = acc[u];
            if (bias != nullptr) {
              a.x += __bfloat162float(bias[col]);
              a.y += __bfloat162float(bias[col + 1]);
              a.z += __bfloat162float(bias[col + 2]);
              a.w += __bfloat162float(bias[col + 3]);
            }
            OutT* dst = C + static_cast<size_t>(row) * ldc + col;
            if constexpr (sizeof(OutT) == 2) {
              uint2 o;
              o.x = pack_bf16(a.x, a.y);
              o.y = pack_bf16(a.z, a.w);
              *reinterpret_cast<uint2*>(dst) = o;
            } else {
              *reinterpret_cast<float4*>(dst) = a;
            }
          }
        }
      }
      // 5. tell every CTA that I am done reading its tile
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (et < splits) mbar_arrive_remote(mapa_u32(smem_u32(stg_free), et));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * CS_BN);
  }
}

template <typename OutT>
static int launch_cluster_splitk(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda,
                                 int ldw, int ldc, int splits, int sms, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, CS_BM, CS_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, CS_BN, CS_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  auto kern = gemm_bf16_cluster_splitk_kernel<OutT>;
  if (KSANA_SMEM_ONCE(kern, CS_SMEM) != 0) return -4;
  const int tiles = ((M + CS_BM - 1) / CS_BM) * ((N + CS_BN - 1) / CS_BN);
  int clusters = sms / splits;
  if (clusters > tiles) clusters = tiles;
  if (clusters < 1) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(clusters * splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = CS_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  OutT* c = reinterpret_cast<OutT*>(C);
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(bias);
  unsigned int* e = error_word();
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, c, b, M, N, K, ldc, splits, e) != cudaSuccess) return -5;
  return 0;
}

// splits must be 2, 4 or 8 and every split must own at least one k-block.
int gemm_bf16_cluster_splitk(const void* A, const void* W, void* C, const void* bias, int M, int N, int K, int lda,
                             int ldw, int ldc, int out_fp32, int splits, cudaStream_t stream) {
  const int sms = sm_count();
  return out_fp32 ? launch_cluster_splitk<float>(A, W, C, bias, M, N, K, lda, ldw, ldc, splits, sms, stream)
                  : launch_cluster_splitk<__nv_bfloat16>(A, W, C, bias, M, N, K, lda, ldw, ldc, splits, sms, stream);
}

}  // namespace ksana
