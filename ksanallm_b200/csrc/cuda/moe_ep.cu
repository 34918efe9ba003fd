// Expert-parallel token exchange over NVLink peer memory: dispatch (token rows -> the ranks that host their experts)
// and combine (weighted expert outputs -> the rank that owns the token), each ONE kernel that does its local
// gather / weighted sum and the all-to-all stores together. The reference delegates this to DeepEP running in a
// separate process driven through shared-memory flags and CUDA IPC (src/ksana_llm/data_hub/
// expert_parallel_deepep_wrapper.cpp, tools/deepep_wrapper), or skips it (replicated tokens + all-reduce).
//
// Every rank owns T_local tokens of the step (T_stride = the largest T_local of any rank, known to every host).
// Rank r's symmetric buffer holds, for every source rank s, T_stride row slots:
//   recv_x  [ws * T_stride, H]  bf16   token rows sent here (slot s * T_stride + t)
//   recv_ids[ws * T_stride, k]  int32  the token's expert ids that live on this rank, -1 elsewhere (ALWAYS written)
//   recv_w  [ws * T_stride, k]  fp32   routing weights
//   ret     [ws * T_stride, H]  bf16   combine results coming back: slot d * T_stride + t from expert rank d
//   flags   [2 * ws + 2]        u32    dispatch-done / combine-done epochs per peer + two local arrival counters
// A token is sent ONCE per destination rank however many of its experts live there; the destination's own
// permute -> grouped GEMM pipeline runs on (recv_x, recv_ids, recv_w), the combine kernel folds the local experts'
// outputs with their weights and stores one row per (token, expert rank) straight into the owner's `ret`; the owner
// sums at most ws rows in rank order (deterministic). Slots are fixed by (source rank, token), so there are no remote
// atomics and no receive-side compaction. Flags carry the call's epoch; every wait is bounded by wall time.
#include "comm.cuh"
#include "host_common.h"

namespace ksana {

constexpr int EP_MAX_RANKS = 8;

struct EpCtx {
  int rank, ws;
  uint8_t* base[EP_MAX_RANKS];
  long long off_x, off_ret, off_ids, off_w, off_flags;
};

__device__ __forceinline__ void ep_signal_all(const EpCtx& ctx, int flag_base, int counter_idx, uint32_t epoch) {
  // last CTA to arrive publishes the epoch to every rank (itself included)
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* local = reinterpret_cast<uint32_t*>(ctx.base[ctx.rank] + ctx.off_flags);
    __threadfence_system();
    const unsigned prev = atomicAdd(local + 2 * ctx.ws + counter_idx, 1u);
    if (prev == gridDim.x * gridDim.y - 1) {
      local[2 * ctx.ws + counter_idx] = 0;
      __threadfence_system();
      for (int d = 0; d < ctx.ws; ++d)
        st_release_sys(reinterpret_cast<uint32_t*>(ctx.base[d] + ctx.off_flags) + flag_base + ctx.rank, epoch);
    }
  }
}

// One warp per (token slot, destination rank).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpCtx ctx, const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ ids,
                   const float* __restrict__ w, int T_local, int T_stride, int k, int H, int E_local,
                   uint32_t epoch) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int total = T_stride * ctx.ws;
  for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < total; p += warps) {
    const int t = p / ctx.ws, d = p - t * ctx.ws;
    const size_t slot = static_cast<size_t>(ctx.rank) * T_stride + t;
    int idv = -1;
    float wv = 0.f;
    if (t < T_local && lane < k) {
      const int e = ids[t * k + lane];
      if (e >= d * E_local && e < (d + 1) * E_local) {
        idv = e;
        wv = w[t * k + lane];
      }
    }
    const unsigned any = __ballot_sync(0xffffffffu, idv >= 0);
    uint8_t* dst = ctx.base[d];
    if (lane < k) {
      reinterpret_cast<int*>(dst + ctx.off_ids)[slot * k + lane] = idv;
      reinterpret_cast<float*>(dst + ctx.off_w)[slot * k + lane] = wv;
    }
    if (any) {
      const __nv_bfloat16* src = x + static_cast<size_t>(t) * ldx;
      __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(dst + ctx.off_x) + slot * H;
      for (int c = lane * 8; c < H; c += 256) st_peer16(row + c, *reinterpret_cast<const uint4*>(src + c));
    }
  }
  ep_signal_all(ctx, 0, 0, epoch);
}

// Blocks the stream until every listed flag reached the epoch (one lane per peer).
__global__ void ep_wait_kernel(const uint32_t* flags, int n, uint32_t epoch, unsigned int* err) {
  if (threadIdx.x < n) wait_flag_ge(flags + threadIdx.x, epoch, err);
}

// Row R = (source rank s, token t) of the local pipeline: out = sum_j recv_w[R, j] * y[pos[R, j]] over the experts
// hosted here, stored into rank s's ret slot (rank, t). grid = (H chunks, ws * T_stride).
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpCtx ctx, const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, int T_stride, int k,
                  int H, uint32_t epoch) {
  const int R = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const float* w = reinterpret_cast<const float*>(ctx.base[ctx.rank] + ctx.off_w) + static_cast<size_t>(R) * k;
  if (c < H) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    bool any = false;
    for (int j = 0; j < k; ++j) {
      const int p = pos[R * k + j];
      if (p < 0) continue;
      any = true;
      const float wj = w[j];
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(y + static_cast<size_t>(p) * H + c), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += wj * f[i];
    }
    if (any) {
      const int s = R / T_stride, t = R - s * T_stride;
      __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(ctx.base[s] + ctx.off_ret) +
                           (static_cast<size_t>(ctx.rank) * T_stride + t) * H;
      st_peer16(row + c, pack8(acc));
    }
  }
  ep_signal_all(ctx, ctx.ws, 1, epoch);
}

// out[t] = add[t] + sum over the expert ranks d that received token t of ret[d * T_stride + t]. grid = (H chunks, T).
__global__ void __launch_bounds__(256)
ep_finish_kernel(EpCtx ctx, const int* __restrict__ ids, int T_stride, int k, int H, int E_local,
                 const __nv_bfloat16* __restrict__ add, int ld_add, __nv_bfloat16* __restrict__ out, int ldo,
                 uint32_t epoch, unsigned int* err) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < ctx.ws) {
    const uint32_t* flags = reinterpret_cast<const uint32_t*>(ctx.base[ctx.rank] + ctx.off_flags) + ctx.ws;
    if (!wait_flag_ge(flags + threadIdx.x, epoch, err)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  unsigned mask = 0;
  for (int j = 0; j < k; ++j) {
    const int e = ids[t * k + j];
    if (e >= 0) mask |= 1u << (e / E_local);
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (add != nullptr) unpack8(*reinterpret_cast<const uint4*>(add + static_cast<size_t>(t) * ld_add + c), acc);
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(ctx.base[ctx.rank] + ctx.off_ret);
  for (int d = 0; d < ctx.ws; ++d) {
    if (!((mask >> d) & 1u)) continue;
    float f[8];
    unpack8(ld_peer16(ret + (static_cast<size_t>(d) * T_stride + t) * H + c), f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
  }
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ldo + c) = pack8(acc);
}

static int ep_fill(EpCtx* ctx, int rank, int ws, void* const* bufs, const long long* offs) {
  if (ws < 1 || ws > EP_MAX_RANKS || rank < 0 || rank >= ws) return -1;
  ctx->rank = rank;
  ctx->ws = ws;
  for (int i = 0; i < EP_MAX_RANKS; ++i) ctx->base[i] = i < ws ? reinterpret_cast<uint8_t*>(bufs[i]) : nullptr;
  ctx->off_x = offs[0];
  ctx->off_ret = offs[1];
  ctx->off_ids = offs[2];
  ctx->off_w = offs[3];
  ctx->off_flags = offs[4];
  return 0;
}

}  // namespace ksana

using namespace ksana;

// bufs: every rank's symmetric buffer (index = rank); offs: byte offsets {recv_x, ret, recv_ids, recv_w, flags}.
// Sends this rank's token rows and then waits (on the stream) until every rank's rows for this epoch have landed
// here, so the kernels that follow may read recv_x / recv_ids / recv_w of the local buffer.
KSANA_API int ksana_ep_dispatch(int rank, int ws, void* const* bufs, const long long* offs, const void* x, int ldx,
                                const int* ids, const float* w, int T_local, int T_stride, int k, int H, int E_local,
                                unsigned int epoch, cudaStream_t stream) {
  EpCtx ctx;
  if (ep_fill(&ctx, rank, ws, bufs, offs)) return -1;
  if (T_stride <= 0 || T_local > T_stride || k < 1 || k > 32 || (H & 7) || (ldx & 7)) return -1;
  const int warps = T_stride * ws;
  int grid = (warps + 7) / 8;
  const int cap = 2 * sm_count();
  if (grid > cap) grid = cap;
  ep_dispatch_kernel<<<grid, 256, 0, stream>>>(ctx, reinterpret_cast<const __nv_bfloat16*>(x), ldx, ids, w, T_local,
                                               T_stride, k, H, E_local, epoch);
  ep_wait_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(ctx.base[rank] + ctx.off_flags), ws, epoch,
                                       error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// y: the local pipeline's sorted expert outputs; pos: [ws * T_stride * k] sorted row of each (slot, j) pair or -1.
KSANA_API int ksana_ep_combine(int rank, int ws, void* const* bufs, const long long* offs, const void* y,
                               const int* pos, int T_stride, int k, int H, unsigned int epoch, cudaStream_t stream) {
  EpCtx ctx;
  if (ep_fill(&ctx, rank, ws, bufs, offs)) return -1;
  if (T_stride <= 0 || (H & 7)) return -1;
  dim3 grid((H / 8 + 255) / 256, ws * T_stride);
  ep_combine_kernel<<<grid, 256, 0, stream>>>(ctx, reinterpret_cast<const __nv_bfloat16*>(y), pos, T_stride, k, H,
                                              epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// out[t] = (add ? add[t] : 0) + the combined expert outputs of this rank's T_local tokens. ids: the same [T_local, k]
// global expert ids given to ksana_ep_dispatch.
KSANA_API int ksana_ep_finish(int rank, int ws, void* const* bufs, const long long* offs, const int* ids, int T_local,
                              int T_stride, int k, int H, int E_local, const void* add, int ld_add, void* out, int ldo,
                              unsigned int epoch, cudaStream_t stream) {
  EpCtx ctx;
  if (ep_fill(&ctx, rank, ws, bufs, offs)) return -1;
  if ((H & 7) || (ldo & 7) || (ld_add & 7)) return -1;
  if (T_local <= 0) {
    // still consume the epoch so the flags stay in step
    ep_wait_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const uint32_t*>(ctx.base[rank] + ctx.off_flags) + ws, ws,
                                         epoch, error_word());
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
  }
  dim3 grid((H / 8 + 255) / 256, T_local);
  ep_finish_kernel<<<grid, 256, 0, stream>>>(ctx, ids, T_stride, k, H, E_local,
                                             reinterpret_cast<const __nv_bfloat16*>(add), ld_add,
                                             reinterpret_cast<__nv_bfloat16*>(out), ldo, epoch, error_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
