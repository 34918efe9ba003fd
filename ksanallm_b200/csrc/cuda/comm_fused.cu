// Tensor-parallel reduction fused with residual add + RMSNorm + all-gather, over NVLink peer memory.
//
// Replaces, in one kernel, the reference's chain "custom P2P all-reduce / NCCL all-reduce -> fused add + RMSNorm"
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/all_reduce/custom_all_reduce.cu:196-265,
//  src/ksana_llm/layers/nvidia/custom_all_reduce_sum_layer.cpp:124-176,
//  src/ksana_llm/modules/basic/all_reduce_fused_norm_add.cpp:30-53) and its NVLS "TokenWeave" variant
// (others/vllm/main/tokenweave/tokenweave_fused_kernels.cu:46-174), without the extra D2D copy out of the
// multicast buffer: activations live in the symmetric heap and the next GEMM reads them in place.
//
// Data flow per call (every rank runs the same kernel on its own GPU, one process per GPU):
//   partial[r]   each rank's un-reduced GEMM output [T, H] bf16 in ITS symmetric buffer (written by the GEMM)
//   rank r owns rows [r * rows_per, (r + 1) * rows_per): it sums those rows over all ranks - in the NVSwitch
//   with multimem.ld_reduce when a multicast mapping exists, else with plain peer loads in rank order - adds its
//   slice of the residual stream (the residual is row-sharded between calls: only the owner keeps it), applies
//   RMSNorm and writes the normalised rows into every rank's `hbuf` (multimem.st / peer stores).
// Cross-rank ordering uses epoch-stamped flag words (st.release.sys / ld.acquire.sys) in a symmetric signal
// buffer; every wait is bounded and reports KERR_PEER_TIMEOUT instead of hanging. No TMA is involved here.
#include "host_common.h"
#include "sm100.cuh"
#include "comm.cuh"

namespace ksana {

constexpr int MAX_RANKS = 8;
constexpr int SIG_START = 0;     // [MAX_CTAS][MAX_RANKS] start-barrier slots
constexpr int SIG_DONE = 4096;   // [MAX_RANKS] end-of-call slots
constexpr int SIG_LOCAL = 4160;  // local CTA counter
constexpr int COMM_MAX_CTAS = 256;

struct CommCtx {
  int rank, ws;
  __nv_bfloat16* partial[MAX_RANKS];
  __nv_bfloat16* hbuf[MAX_RANKS];
  uint32_t* sig[MAX_RANKS];
  __nv_bfloat16* partial_mc;  // multicast view of `partial` (nullptr: plain peer loads)
  __nv_bfloat16* hbuf_mc;     // multicast view of `hbuf` (nullptr: plain peer stores)
};

// One CTA per owned row (grid-stride). THREADS * VPT * 8 >= H.
// mode bit0: apply RMSNorm (else plain sum -> all-reduce); bit1: add residual.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rs_norm_ag_kernel(CommCtx ctx, int T, int H, __nv_bfloat16* __restrict__ residual,
                  const __nv_bfloat16* __restrict__ norm_w, float eps, uint32_t epoch, int mode, unsigned int* err) {
  const int rank = ctx.rank, ws = ctx.ws;
  const int tid = threadIdx.x;
  uint32_t* my_sig = ctx.sig[rank];
  __shared__ int s_ok;
  __shared__ float red[THREADS / 32];

  // ---- start barrier: every rank's partial is complete (its GEMM ran earlier on its stream) ----
  if (tid < ws) st_release_sys(ctx.sig[tid] + SIG_START + blockIdx.x * MAX_RANKS + rank, epoch);
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < ws) {
    if (!wait_flag_ge(my_sig + SIG_START + blockIdx.x * MAX_RANKS + tid, epoch, err)) s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;

  const int rows_per = (T + ws - 1) / ws;
  const int row_begin = rank * rows_per;
  const int row_end = min(T, row_begin + rows_per);
  if (ok) {
    for (int row = row_begin + blockIdx.x; row < row_end; row += gridDim.x) {
      float v[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = (i * THREADS + tid) * 8;
        if (c < H) {
          const size_t off = static_cast<size_t>(row) * H + c;
          if (ctx.partial_mc != nullptr) {
            unpack8(multimem_ld_reduce_bf16x8(ctx.partial_mc + off), v[i]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
            for (int p = 0; p < ws; ++p) {
              float t[8];
              unpack8(ld_peer16(ctx.partial[p] + off), t);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[i][j] += t[j];
            }
          }
          if (mode & 2) {
            float r[8];
            unpack8(*reinterpret_cast<const uint4*>(residual + off), r);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] += r[j];
            const uint4 packed = pack8(v[i]);
            *reinterpret_cast<uint4*>(residual + off) = packed;
            unpack8(packed, v[i]);  // the norm sees the bf16-rounded residual, like the unfused kernel
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        }
      }
      float inv = 1.f;
      if (mode & 1) {
        ss = warp_sum(ss);
        __syncthreads();
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < THREADS / 32; ++i) tot += red[i];
        inv = rsqrtf(tot / static_cast<float>(H) + eps);
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = (i * THREADS + tid) * 8;
        if (c < H) {
          const size_t off = static_cast<size_t>(row) * H + c;
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
  }
  // ---- end of call: after the last local CTA has finished its stores, tell every peer; then wait for all ----
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (tid == 0) {
    const uint32_t prev = atomicAdd(my_sig + SIG_LOCAL, 1u);
    s_last = (prev == gridDim.x - 1);
    if (s_last) my_sig[SIG_LOCAL] = 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < ws) st_release_sys(ctx.sig[tid] + SIG_DONE + rank, epoch);
    if (tid < ws) wait_flag_ge(my_sig + SIG_DONE + tid, epoch, err);
  }
}

// Bounded wait on a flag nobody sets: exercises the time-out path without faulting or hanging the GPU.
__global__ void flag_timeout_probe_kernel(const uint32_t* flag, uint32_t want, unsigned int* err, int* result) {
  if (threadIdx.x == 0) *result = wait_flag_ge(flag, want, err, 300000000ull) ? 1 : 0;  // 0.3 s
}

}  // namespace ksana

using namespace ksana;

// ptrs: partial[ws], hbuf[ws], sig[ws] device pointers of every rank's symmetric buffers (index = rank).
KSANA_API int ksana_rs_norm_ag(int rank, int ws, void* const* partial, void* const* hbuf, void* const* sig,
                               void* partial_mc, void* hbuf_mc, int T, int H, void* residual, const void* norm_w,
                               float eps, unsigned int epoch, int mode, int max_ctas, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (ws < 1 || ws > MAX_RANKS || (H & 7)) return -1;
  CommCtx ctx;
  ctx.rank = rank;
  ctx.ws = ws;
  for (int i = 0; i < MAX_RANKS; ++i) {
    ctx.partial[i] = i < ws ? reinterpret_cast<__nv_bfloat16*>(partial[i]) : nullptr;
    ctx.hbuf[i] = i < ws ? reinterpret_cast<__nv_bfloat16*>(hbuf[i]) : nullptr;
    ctx.sig[i] = i < ws ? reinterpret_cast<uint32_t*>(sig[i]) : nullptr;
  }
  ctx.partial_mc = reinterpret_cast<__nv_bfloat16*>(partial_mc);
  ctx.hbuf_mc = reinterpret_cast<__nv_bfloat16*>(hbuf_mc);
  const int rows_per = (T + ws - 1) / ws;
  int grid = rows_per < 1 ? 1 : rows_per;
  if (max_ctas <= 0 || max_ctas > COMM_MAX_CTAS) max_ctas = COMM_MAX_CTAS;
  if (grid > max_ctas) grid = max_ctas;
  auto R = reinterpret_cast<__nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(norm_w);
  unsigned int* err = error_word();
  if (H <= 2048) rs_norm_ag_kernel<256, 1><<<grid, 256, 0, stream>>>(ctx, T, H, R, W, eps, epoch, mode, err);
  else if (H <= 4096) rs_norm_ag_kernel<256, 2><<<grid, 256, 0, stream>>>(ctx, T, H, R, W, eps, epoch, mode, err);
  else if (H <= 8192) rs_norm_ag_kernel<512, 2><<<grid, 512, 0, stream>>>(ctx, T, H, R, W, eps, epoch, mode, err);
  else if (H <= 16384) rs_norm_ag_kernel<1024, 2><<<grid, 1024, 0, stream>>>(ctx, T, H, R, W, eps, epoch, mode, err);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Runs the bounded wait on `flag` (device memory holding a value < want) and returns 1 if it was satisfied,
// 0 if it timed out (the status word then carries KERR_PEER_TIMEOUT). Synchronous.
KSANA_API int ksana_flag_timeout_probe(const void* flag, unsigned int want, int* result_dev, cudaStream_t stream) {
  flag_timeout_probe_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(flag), want, error_word(),
                                                  result_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
