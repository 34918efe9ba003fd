// Mixture-of-experts kernels for sm_100a: router (softmax / sigmoid + correction bias + group-limited top-k),
// device-side counting sort of (token, slot) pairs by expert, row gather, grouped expert GEMM on tcgen05, and the
// weighted combine. Everything is sized on the device: no host synchronisation between routing and the GEMMs.
//
// Reference kernels replaced: FusedDSV3GroupedTopkKernel / BasicSoftmaxTopkKernel
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/grouped_topk/grouped_topk.cu:560-752), moe_align_block_size /
// token sort (moe_utils/moe_utils.cu:713-754), the ahead-of-time compiled Triton fused_moe_kernel
// (moe/fused_moe/fused_moe.py, driver InvokeFusedMoe src/ksana_llm/kernels/nvidia/moe_kernel_wrapper.cpp:463-655),
// silu_and_mul / moe_sum helpers (moe_utils.cu:795-860).
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

// ---- router -------------------------------------------------------------------------------------------------------
// One CTA per token, one thread per expert (E <= 512, k <= 16, n_group <= 32).
// scoring: 0 softmax, 1 sigmoid. Selection runs on (score + bias) restricted to the topk_group best groups
// (group score = sum of its two largest biased scores when a bias is given, else its maximum); the returned
// weights are the UNBIASED scores of the selected experts, optionally renormalised, times routed_scale.
__global__ void __launch_bounds__(512)
moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int E, int k, int scoring,
                 int norm_topk, int n_group, int topk_group, float routed_scale, int* __restrict__ ids,
                 float* __restrict__ weights) {
  __shared__ float s_score[512];
  __shared__ float s_choice[512];
  __shared__ float s_red[32];
  __shared__ int s_redi[32];
  __shared__ float s_group[32];
  __shared__ int s_sel_i[16];
  __shared__ float s_sel_w[16];
  const int t = blockIdx.x, e = threadIdx.x;
  const int lane = e & 31, warp = e >> 5, nwarps = (blockDim.x + 31) >> 5;
  const float x = e < E ? logits[static_cast<size_t>(t) * ld + e] : -INFINITY;
  float score;
  if (scoring == 1) {
    score = e < E ? 1.f / (1.f + __expf(-x)) : 0.f;
  } else {
    float m = warp_max(x);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = -INFINITY;
    for (int i = 0; i < nwarps; ++i) m = fmaxf(m, s_red[i]);
    __syncthreads();
    const float ex = e < E ? __expf(x - m) : 0.f;
    float s = warp_sum(ex);
    if (lane == 0) s_red[warp] = s;
    __syncthreads();
    s = 0.f;
    for (int i = 0; i < nwarps; ++i) s += s_red[i];
    __syncthreads();
    score = ex / s;
  }
  if (e < 512) {
    s_score[e] = score;
    s_choice[e] = e < E ? score + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  __syncthreads();
  if (n_group > 1) {
    const int gs = E / n_group;
    if (e < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = s_choice[e * gs + i];
        if (v > a) {
          b = a;
          a = v;
        } else if (v > b) {
          b = v;
        }
      }
      s_group[e] = bias ? a + b : a;
    }
    __syncthreads();
    if (e == 0) {
      // keep the topk_group best groups (ties: lowest index), mark the others
      for (int r = 0; r < topk_group; ++r) {
        int best = -1;
        float bv = -INFINITY;
        for (int g = 0; g < n_group; ++g) {
          const float v = s_group[g];
          if (v != INFINITY && (best < 0 || v > bv)) {
            best = g;
            bv = v;
          }
        }
        if (best >= 0) s_group[best] = INFINITY;  // selected marker
      }
    }
    __syncthreads();
    if (e < E && s_group[e / gs] != INFINITY) s_choice[e] = -INFINITY;
    __syncthreads();
  }
  // k rounds of block arg-max (ties: lowest expert index)
  for (int r = 0; r < k; ++r) {
    float v = e < E ? s_choice[e] : -INFINITY;
    int vi = e < E ? e : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, vi, o);
      if (ov > v || (ov == v && oi < vi)) {
        v = ov;
        vi = oi;
      }
    }
    if (lane == 0) {
      s_red[warp] = v;
      s_redi[warp] = vi;
    }
    __syncthreads();
    if (e == 0) {
      float bv = s_red[0];
      int bi = s_redi[0];
      for (int i = 1; i < nwarps; ++i)
        if (s_red[i] > bv || (s_red[i] == bv && s_redi[i] < bi)) {
          bv = s_red[i];
          bi = s_redi[i];
        }
      if (bi == 0x7FFFFFFF || bi >= E) bi = 0;
      s_sel_i[r] = bi;
      s_sel_w[r] = s_score[bi];
      s_choice[bi] = -INFINITY;
    }
    __syncthreads();
  }
  if (e == 0) {
    float tot = 0.f;
    for (int r = 0; r < k; ++r) tot += s_sel_w[r];
    const float inv = norm_topk ? 1.f / fmaxf(tot, 1e-20f) : 1.f;
    for (int r = 0; r < k; ++r) {
      ids[static_cast<size_t>(t) * k + r] = s_sel_i[r];
      weights[static_cast<size_t>(t) * k + r] = s_sel_w[r] * inv * routed_scale;
    }
  }
}

// ---- counting sort by expert -----------------------------------------------------------------------------------------
// counts[E_local] must be zero on entry (the scan kernel re-zeroes it for the next call through `cursor`).
__global__ void moe_count_kernel(const int* __restrict__ ids, int n, int expert_offset, int E_local,
                                 int* __restrict__ counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i] - expert_offset;
  if (e >= 0 && e < E_local) atomicAdd(&counts[e], 1);
}
// offsets[e] = exclusive prefix sum of counts, offsets[E_local] = total; cursor[e] = 0; counts[e] = 0.
__global__ void moe_scan_kernel(int* __restrict__ counts, int E_local, int* __restrict__ offsets,
                                int* __restrict__ cursor) {
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E_local; ++e) {
      offsets[e] = acc;
      acc += counts[e];
      counts[e] = 0;
      cursor[e] = 0;
    }
    offsets[E_local] = acc;
  }
}
// pos[i] = sorted row of pair i (or -1 when its expert lives elsewhere).
__global__ void moe_scatter_kernel(const int* __restrict__ ids, int n, int expert_offset, int E_local,
                                   const int* __restrict__ offsets, int* __restrict__ cursor, int* __restrict__ pos,
                                   int* __restrict__ row_src) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i] - expert_offset;
  if (e < 0 || e >= E_local) {
    pos[i] = -1;
    return;
  }
  const int p = offsets[e] + atomicAdd(&cursor[e], 1);
  pos[i] = p;
  row_src[p] = i;
}
// xs[p] = x[row_src[p] / k] for the first offsets[E_local] rows.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ row_src, int k,
                                  const int* __restrict__ offsets, int E_local, __nv_bfloat16* __restrict__ xs, int H) {
  const int p = blockIdx.y;
  if (p >= offsets[E_local]) return;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  const int t = row_src[p] / k;
  *reinterpret_cast<uint4*>(xs + static_cast<size_t>(p) * H + c) =
      *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx + c);
}
// out[t] = sum_j weights[t, j] * y[pos[t, j]] (pairs with pos < 0 contribute nothing).
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ weights, int k, __nv_bfloat16* __restrict__ out, int H) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int j = 0; j < k; ++j) {
    const int p = pos[t * k + j];
    if (p < 0) continue;
    const float w = weights[t * k + j];
    const uint4 u = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(p) * H + c);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc[2 * i] += w * f.x;
      acc[2 * i + 1] += w * f.y;
    }
  }
  uint4 o;
  o.x = pack_bf16(acc[0], acc[1]);
  o.y = pack_bf16(acc[2], acc[3]);
  o.z = pack_bf16(acc[4], acc[5]);
  o.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) = o;
}

// ---- grouped expert GEMM (bf16, tcgen05) -----------------------------------------------------------------------------
// C[rows of expert e, N] = A[rows of expert e, K] * W[e][N, K]^T for every local expert, rows given by offsets[].
// Same pipeline as gemm_bf16_kernel (TMA producer warp / MMA warp / 4 epilogue warps, double-buffered TMEM
// accumulator); the persistent tile loop walks (expert, m-tile, n-tile) using the device-side offsets, so ragged and
// empty experts cost nothing. A tile's trailing rows may belong to the next expert: they are computed and dropped.
constexpr int G_BM = 128, G_BN = 128, G_BK = 64, G_STAGES = 6;
constexpr int G_A_BYTES = G_BM * G_BK * 2, G_B_BYTES = G_BN * G_BK * 2, G_STAGE = G_A_BYTES + G_B_BYTES;
constexpr int G_BAR = G_STAGES * G_STAGE;
constexpr int G_SMEM = G_BAR + 256 + 1024;

struct GroupedTileIter {
  const int* offsets;
  int E, tiles_n, stride, next;  // next: global tile index this CTA wants
  int e, base;                   // current expert and the global index of its first tile
  __device__ GroupedTileIter(const int* off, int E_, int tiles_n_, int first, int stride_)
      : offsets(off), E(E_), tiles_n(tiles_n_), stride(stride_), next(first), e(0), base(0) {}
  // Returns false when no tile is left; otherwise fills (expert, m-tile, n-tile).
  __device__ bool get(int* expert, int* mt, int* nt) {
    while (e < E) {
      const int rows = offsets[e + 1] - offsets[e];
      const int tiles = ((rows + G_BM - 1) / G_BM) * tiles_n;
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

__global__ void __launch_bounds__(192, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        __nv_bfloat16* __restrict__ C, const int* __restrict__ offsets, int E, int N, int K, int ldc,
                        unsigned int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + G_BAR);
  uint64_t* empty_bar = full_bar + G_STAGES;
  uint64_t* acc_full = empty_bar + G_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + G_BN - 1) / G_BN;
  const int num_kb = (K + G_BK - 1) / G_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G_STAGES; ++s) {
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
    tmem_alloc(tmem_holder, 2 * G_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      GroupedTileIter it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
      int stage = 0, e, mt, nt;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && it.get(&e, &mt, &nt)) {
        const int row0 = offsets[e] + mt * G_BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, err)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * G_STAGE;
          mbar_expect_tx(&full_bar[stage], G_STAGE);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * G_BK, row0);
          tma_load_2d(sa + G_A_BYTES, &tmB, &full_bar[stage], kb * G_BK, e * N + nt * G_BN);
          if (++stage == G_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(G_BM, G_BN, 1, 1);
      GroupedTileIter it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
      int stage = 0, e, mt, nt, n_it = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && it.get(&e, &mt, &nt)) {
        const int as = n_it & 1;
        if (!mbar_wait_bounded(&acc_empty[as], ((n_it >> 1) & 1) ^ 1, abort_flag, err)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, err)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * G_STAGE);
          const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + G_A_BYTES);
#pragma unroll
          for (int k = 0; k < G_BK / 16; ++k)
            umma_f16(tmem_base + as * G_BN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == G_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[as]);
        ++n_it;
      }
    }
  } else {
    const int quarter = warp & 3;
    GroupedTileIter it(offsets, E, tiles_n, blockIdx.x, gridDim.x);
    int e, mt, nt, n_it = 0;
    while (it.get(&e, &mt, &nt)) {
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
      const int row = offsets[e] + mt * G_BM + quarter * 32 + lane;
      const bool row_ok = row < offsets[e + 1];
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * G_BN;
      __nv_bfloat16* crow = C + static_cast<size_t>(row_ok ? row : 0) * ldc;
#pragma unroll 1
      for (int c = 0; c < G_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(t_row + c * 32, r);
        tmem_wait_ld();
        const int col0 = nt * G_BN + c * 32;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (row_ok && col0 + j < N) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            o.y = pack_bf16(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            o.z = pack_bf16(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            o.w = pack_bf16(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(crow + col0 + j) = o;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[as]);
      ++n_it;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * G_BN);
  }
}

}  // namespace ksana

using namespace ksana;

KSANA_API int ksana_moe_route(const float* logits, int ld, const float* bias, int T, int E, int k, int scoring,
                              int norm_topk, int n_group, int topk_group, float routed_scale, int* ids, float* weights,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 512 || k > 16 || k < 1 || n_group > 32 || n_group < 1 || E % n_group) return -1;
  const int threads = ((E + 31) / 32) * 32;
  moe_route_kernel<<<T, threads, 0, stream>>>(logits, ld, bias, E, k, scoring, norm_topk, n_group, topk_group,
                                              routed_scale, ids, weights);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Sorts the T*k (token, slot) pairs by local expert. meta: int workspace of at least 3 * E_local + 2 ints laid out as
// counts[E_local] (zero on first use, kept zero by the kernel) | offsets[E_local + 1] | cursor[E_local].
// pos: [T*k] sorted row or -1; row_src: [T*k]; xs: [T*k, H] gathered rows (only the first offsets[E_local] are valid).
KSANA_API int ksana_moe_permute(const void* x, int ldx, const int* ids, int T, int k, int H, int expert_offset,
                                int E_local, int* meta, int* pos, int* row_src, void* xs, cudaStream_t stream) {
  const int n = T * k;
  if (n <= 0) return 0;
  if (H & 7) return -1;
  int* counts = meta;
  int* offsets = meta + E_local;
  int* cursor = offsets + E_local + 1;
  moe_count_kernel<<<(n + 255) / 256, 256, 0, stream>>>(ids, n, expert_offset, E_local, counts);
  moe_scan_kernel<<<1, 32, 0, stream>>>(counts, E_local, offsets, cursor);
  moe_scatter_kernel<<<(n + 255) / 256, 256, 0, stream>>>(ids, n, expert_offset, E_local, offsets, cursor, pos, row_src);
  dim3 grid((H / 8 + 255) / 256, n);
  moe_gather_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, row_src, k, offsets,
                                              E_local, reinterpret_cast<__nv_bfloat16*>(xs), H);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// C[sorted rows, N] = A[sorted rows, K] * W[e]^T per expert. W: [E, N, K] bf16 contiguous; max_rows = rows of A.
KSANA_API int ksana_moe_grouped_gemm(const void* A, const void* W, void* C, const int* offsets, int E, int max_rows,
                                     int N, int K, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if ((N % G_BN) || (K & 7)) return -1;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, max_rows, K, K, G_BM, G_BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -2;
  if (make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, static_cast<uint64_t>(E) * N, K, K, G_BN, G_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (KSANA_SMEM_ONCE(moe_grouped_gemm_kernel, G_SMEM) != 0) return -4;
  moe_grouped_gemm_kernel<<<sm_count(), 192, G_SMEM, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(C), offsets, E,
                                                              N, K, N, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_moe_combine(const void* y, const int* pos, const float* weights, int T, int k, int H, void* out,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  dim3 grid((H / 8 + 255) / 256, T);
  moe_combine_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y), pos, weights, k,
                                               reinterpret_cast<__nv_bfloat16*>(out), H);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
