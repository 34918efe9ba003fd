// fp8 GEMM with the scales applied by the tensor core (tcgen05.mma kind::mxf8f6f4.block_scale) for sm_100a:
//   C[M, N] = sum_kb 2^(ea[m, kb] + eb[n, kb]) * (A8[m, kb] . W8[n, kb])  (+ bias),  kb = 128-wide K blocks
// with e4m3 activations and weights whose scales are powers of two (UE8M0 bytes, value 2^(e - 127)).
//
// The block-scaled kernel in gemm_fp8_block.cu takes arbitrary fp32 scales and therefore folds every 128-wide K block
// into register accumulators on the CUDA cores ("promotion"), which caps it at about a quarter of the fp8 tensor rate.
// When both scale sets are powers of two the tensor core multiplies them in itself: the whole K loop accumulates in
// TMEM like a bf16 GEMM, at the fp8 rate, and the epilogue only converts. Weights get power-of-two block scales when
// they are quantised at load time (models/loader.py); activations are quantised with power-of-two 1 x 128 group
// scales by the kernels at the end of this file. The reference reaches the same point on Hopper with DeepGEMM /
// CUTLASS fp32-scale kernels (src/ksana_llm/layers/nvidia/blockwise_matmul_layer.cpp:71-301); Blackwell's scaled MMA
// has no counterpart there.
//
// Tile 128 x 192 x 128 per stage, one CTA per SM, persistent:
//   warp 0   TMA: A tile (128 x 128 B), W tile (192 x 128 B), 512 B of A scales, 1024 B of W scales per stage
//   warp 1   tcgen05.cp of the scales into TMEM, then 4 scaled MMAs (K = 32 each) per stage
//   warps 2-5 epilogue: TMEM -> bf16 -> global, overlapped with the next tile's K loop (two accumulators in TMEM)
// TMEM columns: [0, 192) and [192, 384) accumulators, then four sets of 4 columns of A scales + 8 of W scales.
//
// Scale layouts in global memory. The hardware keeps 4 scale bytes per row in one 32-bit TMEM word and an MMA picks one
// of them; here the 4 bytes are the scales of 4 CONSECUTIVE 128-wide K groups, so one 512-byte block serves 4 stages
// (copying scales into TMEM every stage costs ~10 % of the GEMM, measured):
//   sfa: [ceil(M / 128)][ceil(K / 512)][512]   byte (r % 32) * 16 + (r / 32) * 4 + c: row r of the 128-row group,
//                                              K group 4 q + c of the q-th block
//   sfb: [ceil(K / 512)][ceil(N / 192)][2][512] the same 512-byte pattern for rows nt * 192 + j * 128 + r of W (j < 2)
// which is the order tcgen05.cp (32 x 128 bit, replicated to the four lane groups) expects in shared memory, so the
// scales arrive with one plain bulk copy each in every fourth stage.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int MX_BM = 128, MX_BN = 192, MX_BK = 128, MX_STAGES = 5;
constexpr int MX_A_BYTES = MX_BM * MX_BK, MX_B_BYTES = MX_BN * MX_BK;
constexpr int MX_SFA_BYTES = 512, MX_SFB_BYTES = 1024;
constexpr int MX_STAGE = MX_A_BYTES + MX_B_BYTES + MX_SFA_BYTES + MX_SFB_BYTES;  // 42496, a multiple of 1024 + 1536
constexpr int MX_STAGE_PITCH = 43008;                                           // next multiple of 1024
constexpr int MX_BAR = MX_STAGES * MX_STAGE_PITCH;
constexpr int MX_SMEM = MX_BAR + 256 + 1024;
// four sets of scale columns, used in turn: the copy for the next stage does not wait for the MMAs that still read
// the previous stage's scales
constexpr int MX_TMEM_SFA = 2 * MX_BN, MX_TMEM_SFB = 2 * MX_BN + 4, MX_TMEM_SF_SET = 12, MX_SF_SETS = 4;

__global__ void __launch_bounds__(192, 1)
gemm_mxf8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, __nv_bfloat16* __restrict__ C,
                 const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc, unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + MX_BAR);
  uint64_t* empty_bar = full_bar + MX_STAGES;
  uint64_t* acc_full = empty_bar + MX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + MX_BM - 1) / MX_BM;
  const int tiles_n = (N + MX_BN - 1) / MX_BN;
  const int num_kb = K / MX_BK;
  const int total = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MX_STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 512);
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
        const int mt = tile % tiles_m, nt = tile / tiles_m;
        const int num_q = (num_kb + 3) >> 2;
        const uint8_t* sfa_t = sfa + static_cast<size_t>(mt) * num_q * MX_SFA_BYTES;
        const uint8_t* sfb_t = sfb + static_cast<size_t>(nt) * MX_SFB_BYTES;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * MX_STAGE_PITCH;
          const bool sf = (kb & 3) == 0;  // this stage also carries the scales of k blocks kb .. kb + 3
          mbar_expect_tx(&full_bar[stage], sf ? MX_STAGE : MX_A_BYTES + MX_B_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * MX_BK, mt * MX_BM);
          tma_load_2d(sa + MX_A_BYTES, &tmB, &full_bar[stage], kb * MX_BK, nt * MX_BN);
          if (sf) {
            bulk_load(sa + MX_A_BYTES + MX_B_BYTES, sfa_t + static_cast<size_t>(kb >> 2) * MX_SFA_BYTES, MX_SFA_BYTES,
                      &full_bar[stage]);
            bulk_load(sa + MX_A_BYTES + MX_B_BYTES + MX_SFA_BYTES,
                      sfb_t + static_cast<size_t>(kb >> 2) * tiles_n * MX_SFB_BYTES, MX_SFB_BYTES, &full_bar[stage]);
          }
          if (++stage == MX_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, n_it = 0;
      uint32_t phase = 0, sf_set = 0;
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
          const uint32_t sa = smem_u32(smem + stage * MX_STAGE_PITCH);
          const uint32_t ssf = sa + MX_A_BYTES + MX_B_BYTES;
          if ((kb & 3) == 0) {
            sf_set = (sf_set + 1) & (MX_SF_SETS - 1);
            const uint32_t t = tmem_base + sf_set * MX_TMEM_SF_SET;
            tmem_cp_sf(t + MX_TMEM_SFA, umma_desc_sf(ssf));
            tmem_cp_sf(t + MX_TMEM_SFB, umma_desc_sf(ssf + MX_SFA_BYTES));
            tmem_cp_sf(t + MX_TMEM_SFB + 4, umma_desc_sf(ssf + MX_SFA_BYTES + 512));
          }
          const uint32_t t_sfa = tmem_base + MX_TMEM_SFA + sf_set * MX_TMEM_SF_SET;
          const uint32_t t_sfb = tmem_base + MX_TMEM_SFB + sf_set * MX_TMEM_SF_SET;
          const int sf_id = kb & 3;
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + MX_A_BYTES);
          const uint32_t idesc = umma_idesc_block_scaled(MX_BM, MX_BN, 0, 0, sf_id, sf_id);
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k)
            umma_mxf8(tmem_base + as * MX_BN, da + 2 * k, db + 2 * k, idesc, t_sfa, t_sfb, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == MX_STAGES) {
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
      const int mt = tile % tiles_m, nt = tile / tiles_m;
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
      const int row = mt * MX_BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * MX_BN;
      const int col0 = nt * MX_BN;
      __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc + col0;
#pragma unroll 1
      for (int c = 0; c < MX_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(t_row + c * 32, rr);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const int col = col0 + c * 32 + j;
            if (col < N) {  // N % 8 == 0: a group of 8 columns is inside or outside as a whole
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(rr[j + i]);
              if (bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += __bfloat162float(bias[col + i]);
              }
              uint4 o;
              o.x = pack_bf16(v[0], v[1]);
              o.y = pack_bf16(v[2], v[3]);
              o.z = pack_bf16(v[4], v[5]);
              o.w = pack_bf16(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + c * 32 + j) = o;
            }
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
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- the same GEMM on CTA pairs (tcgen05 cta_group::2): a 256 x 192 tile over two SMs -------------------------------
// Each CTA stages its own 128 rows of A, its half (96 rows) of the W tile, its A scales and all of the tile's W scales;
// 30 KB per stage instead of 41.5, so 7 stages fit and the L2 -> SM traffic per FLOP drops by 29 %. (It measures no
// faster than the single-CTA kernel: neither L2 traffic nor load latency is what holds that one at ~2 PFLOP/s.) One lane of the
// leader issues the scale copies and the MMAs for both CTAs; every byte count is credited to the leader's "full"
// barrier (tiled loads in their pair form, also for the scale bytes, which are read through tensor maps here).
constexpr int MP_STAGES = 7;
constexpr int MP_HALF_N = MX_BN / 2;
constexpr int MP_B_BYTES = MP_HALF_N * MX_BK;
constexpr int MP_SF_OFF = MX_A_BYTES + MP_B_BYTES;                        // 28672
constexpr int MP_STAGE = MP_SF_OFF + MX_SFA_BYTES + MX_SFB_BYTES;         // 30208 bytes arrive per CTA per stage
constexpr int MP_STAGE_PITCH = 30720;
constexpr int MP_BAR = MP_STAGES * MP_STAGE_PITCH;
constexpr int MP_SMEM = MP_BAR + 512 + 1024;
constexpr int MP_GROUP_M = 8;

__device__ __forceinline__ void mp_tile_coords(int t, int tiles_m, int tiles_n, int* m_idx, int* n_idx) {
  const int per_group = MP_GROUP_M * tiles_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m0 = g * MP_GROUP_M;
  const int gm = min(MP_GROUP_M, tiles_m - m0);
  *n_idx = r / gm;
  *m_idx = m0 + (r - (*n_idx) * gm);
}

__global__ void __launch_bounds__(192, 1)
gemm_mxf8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                      __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, int ldc,
                      unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + MP_BAR);
  uint64_t* empty_bar = full_bar + MP_STAGES;
  uint64_t* acc_full = empty_bar + MP_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * MX_BM - 1) / (2 * MX_BM);
  const int tiles_n = (N + MX_BN - 1) / MX_BN;
  const int num_kb = K / MX_BK;
  const int total = tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MP_STAGES; ++s) {
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
    tmem_alloc_pair(tmem_holder, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them remotely
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmSFA);
      tma_prefetch_desc(&tmSFB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += num_pairs) {
        int mt, nt;
        mp_tile_coords(tile, tiles_m, tiles_n, &mt, &nt);
        const int atom = mt * 2 + static_cast<int>(cta);
        const int row0 = atom * MX_BM;
        const int wrow0 = nt * MX_BN + static_cast<int>(cta) * MP_HALF_N;
        const int num_q = (num_kb + 3) >> 2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * MP_STAGE_PITCH;
          const bool sf = (kb & 3) == 0;  // this stage also carries the scales of k blocks kb .. kb + 3
          if (cta == 0) mbar_expect_tx(&full_bar[stage], 2 * (sf ? MP_STAGE : MP_SF_OFF));
          const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
          tma_load_2d_pair(sa, &tmA, leader_full, kb * MX_BK, row0);
          tma_load_2d_pair(sa + MX_A_BYTES, &tmB, leader_full, kb * MX_BK, wrow0);
          if (sf) {
            tma_load_2d_pair(sa + MP_SF_OFF, &tmSFA, leader_full, 0, atom * num_q + (kb >> 2));
            tma_load_2d_pair(sa + MP_SF_OFF + MX_SFA_BYTES, &tmSFB, leader_full, 0, (kb >> 2) * tiles_n + nt);
          }
          if (++stage == MP_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      int stage = 0, n_it = 0;
      uint32_t phase = 0, sf_set = 0;
      bool ok = true;
      for (int tile = pair; tile < total && ok; tile += num_pairs, ++n_it) {
        const int as = n_it & 1;
        if (!mbar_wait_cluster_bounded(&acc_empty[as], ((n_it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_cluster_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * MP_STAGE_PITCH);
          const uint32_t ssf = sa + MP_SF_OFF;
          if ((kb & 3) == 0) {
            sf_set = (sf_set + 1) & (MX_SF_SETS - 1);
            const uint32_t t = tmem_base + sf_set * MX_TMEM_SF_SET;
            tmem_cp_sf_pair(t + MX_TMEM_SFA, umma_desc_sf(ssf));
            tmem_cp_sf_pair(t + MX_TMEM_SFB, umma_desc_sf(ssf + MX_SFA_BYTES));
            tmem_cp_sf_pair(t + MX_TMEM_SFB + 4, umma_desc_sf(ssf + MX_SFA_BYTES + 512));
          }
          const uint32_t t_sfa = tmem_base + MX_TMEM_SFA + sf_set * MX_TMEM_SF_SET;
          const uint32_t t_sfb = tmem_base + MX_TMEM_SFB + sf_set * MX_TMEM_SF_SET;
          const uint32_t idesc = umma_idesc_block_scaled(2 * MX_BM, MX_BN, 0, 0, kb & 3, kb & 3);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + MX_A_BYTES);
#pragma unroll
          for (int k = 0; k < MX_BK / 32; ++k)
            umma_mxf8_pair(tmem_base + as * MX_BN, da + 2 * k, db + 2 * k, idesc, t_sfa, t_sfb,
                           (kb > 0 || k > 0) ? 1u : 0u);
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(eb);               // my producer may refill the stage
          umma_commit_pair(mapa_u32(eb, 1));  // and so may the peer's
          if (++stage == MP_STAGES) {
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
    const int quarter = warp & 3;
    int n_it = 0;
    for (int tile = pair; tile < total; tile += num_pairs, ++n_it) {
      int mt, nt;
      mp_tile_coords(tile, tiles_m, tiles_n, &mt, &nt);
      const int as = n_it & 1;
      // tcgen05.ld is warp-collective: the lanes of a warp must agree on the outcome of the bounded wait
      const bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[as], (n_it >> 1) & 1, abort_flag, err));
      if (!ok) break;
      tc_fence_after();
      const int row = (mt * 2 + static_cast<int>(cta)) * MX_BM + quarter * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * MX_BN;
      const int col0 = nt * MX_BN;
      __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc + col0;
#pragma unroll 1
      for (int c = 0; c < MX_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(t_row + c * 32, rr);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const int col = col0 + c * 32 + j;
            if (col < N) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(rr[j + i]);
              if (bias != nullptr) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += __bfloat162float(bias[col + i]);
              }
              uint4 o;
              o.x = pack_bf16(v[0], v[1]);
              o.y = pack_bf16(v[2], v[3]);
              o.z = pack_bf16(v[4], v[5]);
              o.w = pack_bf16(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + c * 32 + j) = o;
            }
          }
        }
      }
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
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// UE8M0 byte of the smallest power of two >= amax / 448 (so that amax / scale <= 448), and its reciprocal.
__device__ __forceinline__ uint32_t ue8m0_scale(float amax, float* inv) {
  const float s = fmaxf(amax, 1e-30f) * (1.f / 448.f);
  const uint32_t bits = __float_as_uint(s);
  uint32_t e = (bits >> 23) & 0xFFu;
  if (bits & 0x7FFFFFu) ++e;
  e = min(max(e, 1u), 254u);
  *inv = __uint_as_float((254u - e) << 23);  // 2^(127 - e)
  return e;
}

// where the scale byte of (row, K group g) lives in the packed A-scale layout
__device__ __forceinline__ size_t sfa_offset(int row, int g, int groups) {
  const int r = row & 127;
  return (static_cast<size_t>(row >> 7) * ((groups + 3) >> 2) + (g >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (g & 3);
}

__device__ __forceinline__ void store_scale(uint32_t e, int t, int g, int groups, float* scales, uint8_t* sfa) {
  if (scales != nullptr) scales[static_cast<size_t>(t) * groups + g] = __uint_as_float(e << 23);
  if (sfa != nullptr) sfa[sfa_offset(t, g, groups)] = static_cast<uint8_t>(e);
}

// max over the 8 lanes that share a 128-column group
__device__ __forceinline__ float group8_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
}

__device__ __forceinline__ void unpack16(const uint4& lo, const uint4& hi, float* v) {
  const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// 16 values -> 16 e4m3 bytes
__device__ __forceinline__ uint4 to_e4m3x16(const float* v, float inv) {
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_fp8_e4m3 b[4] = {__nv_fp8_e4m3(v[4 * i] * inv), __nv_fp8_e4m3(v[4 * i + 1] * inv),
                          __nv_fp8_e4m3(v[4 * i + 2] * inv), __nv_fp8_e4m3(v[4 * i + 3] * inv)};
    o[i] = *reinterpret_cast<uint32_t*>(b);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Eight lanes per (row, 128-column group), 16 values (two 16-byte loads) per lane, rows up to the next multiple of
// 128: q = x / 2^e in e4m3 with 2^e >= amax / 448. The scale goes out as fp32 ([T, K / 128], for the kernels that take
// fp32 scales) and / or as packed bytes for the scaled GEMM; the padding rows of the last 128-row group get the byte
// of 1.0. ldx / ldq multiples of 8 / 16.
__global__ void __launch_bounds__(256)
quant_fp8_ue8m0_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_fp8_e4m3* __restrict__ q, int ldq,
                       float* __restrict__ scales, uint8_t* __restrict__ sfa, int T, int T_pad, int K) {
  const int groups = K >> 7;
  const long long gi = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const bool in_range = gi < static_cast<long long>(T_pad) * groups;
  const int t = in_range ? static_cast<int>(gi / groups) : 0;
  const int g = in_range ? static_cast<int>(gi - static_cast<long long>(t) * groups) : 0;
  const bool real = in_range && t < T;
  float v[16];
  if (real) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx + g * 128 + sub * 16);
    const uint4 lo = __ldg(src), hi = __ldg(src + 1);
    unpack16(lo, hi, v);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = group8_max(amax);
  if (!in_range) return;
  if (!real) {
    if (sub == 0 && sfa != nullptr) sfa[sfa_offset(t, g, groups)] = 127;
    return;
  }
  float inv;
  const uint32_t e = ue8m0_scale(amax, &inv);
  *reinterpret_cast<uint4*>(q + static_cast<size_t>(t) * ldq + g * 128 + sub * 16) = to_e4m3x16(v, inv);
  if (sub == 0) store_scale(e, t, g, groups, scales, sfa);
}

// The same for the gated FFN's activation: a = SiLU(gate) * up (rounded to bf16 as the unfused kernel would hand it
// over), x: [T, 2 I] gate columns then up columns.
__global__ void __launch_bounds__(256)
silu_mul_quant_ue8m0_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_fp8_e4m3* __restrict__ q, int ldq,
                            float* __restrict__ scales, uint8_t* __restrict__ sfa, int T, int T_pad, int I) {
  const int groups = I >> 7;
  const long long gi = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  const bool in_range = gi < static_cast<long long>(T_pad) * groups;
  const int t = in_range ? static_cast<int>(gi / groups) : 0;
  const int g = in_range ? static_cast<int>(gi - static_cast<long long>(t) * groups) : 0;
  const bool real = in_range && t < T;
  float v[16];
  if (real) {
    const uint4* gp = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx + g * 128 + sub * 16);
    const uint4* up = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx + I + g * 128 + sub * 16);
    const uint4 g0 = __ldg(gp), g1 = __ldg(gp + 1), u0 = __ldg(up), u1 = __ldg(up + 1);
    float u[16];
    unpack16(g0, g1, v);
    unpack16(u0, u1, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __bfloat162float(__float2bfloat16(v[i] / (1.f + __expf(-v[i])) * u[i]));
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = group8_max(amax);
  if (!in_range) return;
  if (!real) {
    if (sub == 0 && sfa != nullptr) sfa[sfa_offset(t, g, groups)] = 127;
    return;
  }
  float inv;
  const uint32_t e = ue8m0_scale(amax, &inv);
  *reinterpret_cast<uint4*>(q + static_cast<size_t>(t) * ldq + g * 128 + sub * 16) = to_e4m3x16(v, inv);
  if (sub == 0) store_scale(e, t, g, groups, scales, sfa);
}

// Packs power-of-two 128 x 128 block scales (fp32 [ceil(N / 128), K / 128]) into the per-tile byte layout of
// gemm_mxf8_kernel. One thread per (k block, n tile, atom, row).
__global__ void pack_sfb_kernel(const float* __restrict__ sw, uint8_t* __restrict__ sfb, int N, int K, int tiles_n,
                                int* __restrict__ bad) {
  const int groups = K >> 7;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(groups) * tiles_n * 256) return;
  const int r = static_cast<int>(i & 127), j = static_cast<int>((i >> 7) & 1);
  const int nt = static_cast<int>((i >> 8) % tiles_n), kb = static_cast<int>((i >> 8) / tiles_n);
  const int n = nt * MX_BN + j * 128 + r;
  uint32_t e = 127u;
  if (n < N && j * 128 + r < MX_BN) {
    const uint32_t bits = __float_as_uint(sw[static_cast<size_t>(n >> 7) * groups + kb]);
    e = (bits >> 23) & 0xFFu;
    if ((bits & 0x807FFFFFu) != 0u || e == 0u || e == 255u) atomicExch(bad, 1);  // not a positive power of two
  }
  sfb[(static_cast<size_t>(kb >> 2) * tiles_n + nt) * MX_SFB_BYTES + j * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] =
      static_cast<uint8_t>(e);
}

}  // namespace ksana

using namespace ksana;

// Bytes of the packed scale arrays for an [M, K] activation / [N, K] weight.
KSANA_API long long ksana_mxf8_sfa_bytes(int M, int K) {
  return static_cast<long long>((M + 127) / 128) * ((K / 128 + 3) / 4) * MX_SFA_BYTES;
}
KSANA_API long long ksana_mxf8_sfb_bytes(int N, int K) {
  return static_cast<long long>((N + MX_BN - 1) / MX_BN) * ((K / 128 + 3) / 4) * MX_SFB_BYTES;
}

// sw: fp32 [ceil(N / 128), K / 128], every entry a power of two -> sfb (ksana_mxf8_sfb_bytes(N, K) bytes).
// *bad_dev (device int, zeroed by the caller) is set to 1 if an entry is not a positive normal power of two.
KSANA_API int ksana_mxf8_pack_sfb(const float* sw, void* sfb, int N, int K, int* bad_dev, cudaStream_t stream) {
  if (N <= 0 || (K & 127)) return -1;
  const int tiles_n = (N + MX_BN - 1) / MX_BN;
  const long long n = static_cast<long long>(K / 128) * tiles_n * 256;
  pack_sfb_kernel<<<static_cast<unsigned int>((n + 255) / 256), 256, 0, stream>>>(sw, reinterpret_cast<uint8_t*>(sfb), N,
                                                                                 K, tiles_n, bad_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// x: [T, K] bf16 -> q: [T, K] e4m3 with power-of-two 1 x 128 group scales; scales (fp32 [T, K / 128]) and sfa (packed
// bytes, ksana_mxf8_sfa_bytes(T, K)) may each be null.
KSANA_API int ksana_quant_fp8_ue8m0(const void* x, int ldx, void* q, int ldq, float* scales, void* sfa, int T, int K,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 127) || (ldx & 7) || (ldq & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15))
    return -1;
  const int T_pad = sfa != nullptr ? (T + 127) / 128 * 128 : T;
  const long long groups = static_cast<long long>(T_pad) * (K / 128);  // 32 groups per block of 256 threads
  quant_fp8_ue8m0_kernel<<<static_cast<unsigned int>((groups + 31) / 32), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_fp8_e4m3*>(q), ldq, scales,
      reinterpret_cast<uint8_t*>(sfa), T, T_pad, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_silu_mul_quant_ue8m0(const void* x, int ldx, void* q, int ldq, float* scales, void* sfa, int T,
                                         int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((I & 127) || (ldx & 7) || (ldq & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 15))
    return -1;
  const int T_pad = sfa != nullptr ? (T + 127) / 128 * 128 : T;
  const long long groups = static_cast<long long>(T_pad) * (I / 128);
  silu_mul_quant_ue8m0_kernel<<<static_cast<unsigned int>((groups + 31) / 32), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<__nv_fp8_e4m3*>(q), ldq, scales,
      reinterpret_cast<uint8_t*>(sfa), T, T_pad, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// C[M, N] (bf16, row pitch ldc) = A8[M, K] (e4m3, row pitch lda bytes) x W8[N, K]^T (row pitch ldw) with the packed
// power-of-two scales sfa / sfb (layouts at the top of this file). K % 128 == 0, N % 8 == 0, lda / ldw % 16 == 0.
// variant 0 or 1: one CTA per tile; 2: the CTA-pair kernel (measured within 5 % of each other at every size, the
// single-CTA kernel slightly ahead, so it is the default).
KSANA_API int ksana_gemm_mxf8(const void* A8, const void* sfa, const void* W8, const void* sfb, void* C,
                              const void* bias, int M, int N, int K, int lda, int ldw, int ldc, int variant,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 127) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7) || (reinterpret_cast<uintptr_t>(sfa) & 15) ||
      (reinterpret_cast<uintptr_t>(sfb) & 15) || (reinterpret_cast<uintptr_t>(C) & 15))
    return -1;
  const int tiles_n = (N + MX_BN - 1) / MX_BN, num_kb = K / MX_BK;
  const bool pair = variant == 2;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, MX_BM, MX_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldw, pair ? MP_HALF_N : MX_BN, MX_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  auto c = reinterpret_cast<__nv_bfloat16*>(C);
  auto b = reinterpret_cast<const __nv_bfloat16*>(bias);
  if (!pair) {
    if (KSANA_SMEM_ONCE(gemm_mxf8_kernel, MX_SMEM) != 0) return -4;
    const int total = ((M + MX_BM - 1) / MX_BM) * tiles_n;
    int grid = sm_count();
    if (grid > total) grid = total;
    gemm_mxf8_kernel<<<grid, 192, MX_SMEM, stream>>>(tmA, tmB, reinterpret_cast<const uint8_t*>(sfa),
                                                     reinterpret_cast<const uint8_t*>(sfb), c, b, M, N, K, ldc,
                                                     error_word());
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
  }
  // the scale arrays as 2-d tensors of 32-bit words: one row per (128-row group, k block) / (k block, n tile)
  CUtensorMap tmSFA, tmSFB;
  const uint64_t m_atoms = (M + MX_BM - 1) / MX_BM;
  const uint64_t num_q = (num_kb + 3) / 4;
  if (make_tmap_2d(&tmSFA, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, m_atoms * num_q, MX_SFA_BYTES / 4, MX_SFA_BYTES / 4, 1,
                   MX_SFA_BYTES / 4, CU_TENSOR_MAP_SWIZZLE_NONE))
    return -2;
  if (make_tmap_2d(&tmSFB, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, num_q * tiles_n,
                   MX_SFB_BYTES / 4, MX_SFB_BYTES / 4, 1, MX_SFB_BYTES / 4, CU_TENSOR_MAP_SWIZZLE_NONE))
    return -3;
  if (KSANA_SMEM_ONCE(gemm_mxf8_pair_kernel, MP_SMEM) != 0) return -4;
  const int total = ((M + 2 * MX_BM - 1) / (2 * MX_BM)) * tiles_n;
  int pairs = sm_count() / 2;
  if (pairs > total) pairs = total;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = MP_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  unsigned int* e = error_word();
  if (cudaLaunchKernelEx(&cfg, gemm_mxf8_pair_kernel, tmA, tmB, tmSFA, tmSFB, c, b, M, N, K, ldc, e) != cudaSuccess)
    return -5;
  return 0;
}
