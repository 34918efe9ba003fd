// Paged flash-decode for sm_100a: split-KV attention of a few query tokens (q_len = 1 .. MTP verify length)
// per sequence over the paged cache, all query heads of one KV head per CTA (GQA).
//
// Replaces vLLM-style paged_attention_v1/v2 (+ reduce) of the reference
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/paged_attention/paged_attention.cu:393-436, partition 512) and the
// RoPE + CachePosCopy preamble of InvokePagedAttention (src/ksana_llm/kernels/nvidia/attention_kernel_wrapper.cpp:
// 500-650), which here has already run as one fused kernel.
//
// Decode attention is a pure HBM stream (every K/V byte is used once for at most `group * q_len` rows), so the
// kernel is organised around 16-byte coalesced page reads: cache layout [block][2][hk][block_size][d] makes one
// (block, head) K or V page a contiguous block_size * d * 2 bytes. Each warp owns whole pages; two lanes share a
// token for QK^T (64 dims each), four output dims per lane for PV. Warps of a CTA and CTAs of a split are merged
// with log-sum-exp weights; the cross-split merge is a second tiny kernel over an fp32 workspace.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

constexpr int DEC_WARPS = 4;

template <int D, int BS, int RMAX, typename CacheT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const CacheT* __restrict__ cache,
                    const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                    const int* __restrict__ kv_lens, int seq_base, int h, int hk, float scale_log2,
                    const float* __restrict__ alibi, float k_scale, float v_scale, __nv_bfloat16* __restrict__ out,
                    int ldo, float* __restrict__ part_o, float* __restrict__ part_lse, int splits, int pages_per_split,
                    int max_rows) {
  static_assert(D == 128 && BS == 16, "layout below assumes 16-token pages of 128-dim heads");
  const int b = blockIdx.x + seq_base;
  const int kh = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = h / hk;
  const int q0 = cu_q[b];
  const int q_len = cu_q[b + 1] - q0;
  const int L = kv_lens[b];
  const int n_pages = (L + BS - 1) / BS;
  const int page_begin = split * pages_per_split;
  const int page_end = min(page_begin + pages_per_split, n_pages);
  const int R_total = q_len * group;

  extern __shared__ float sm[];
  float* q_s = sm;                               // [RMAX][D]
  float* red_o = q_s + RMAX * D;                 // [DEC_WARPS][RMAX][D]
  float* red_m = red_o + DEC_WARPS * RMAX * D;   // [DEC_WARPS][RMAX]
  float* red_l = red_m + DEC_WARPS * RMAX;       // [DEC_WARPS][RMAX]

  for (int r_base = 0; r_base < R_total; r_base += RMAX) {
    const int R = min(RMAX, R_total - r_base);
    __syncthreads();
    // stage the query rows (row r = j * group + g: query token j, head kh * group + g)
    for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
      const int r = i / D, c = i - r * D;
      const int rr = r_base + r;
      const int j = rr / group, g = rr - j * group;
      q_s[r * D + c] = __bfloat162float(q[static_cast<size_t>(q0 + j) * ldq + (kh * group + g) * D + c]);
    }
    __syncthreads();

    float m[RMAX], l[RMAX], acc[RMAX][4];
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      m[r] = -INFINITY;
      l[r] = 0.f;
      acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    }
    const int tk = lane >> 1, half = lane & 1;
    for (int pg = page_begin + warp; pg < page_end; pg += DEC_WARPS) {
      const int blk = block_tables[static_cast<size_t>(b) * max_blocks + pg];
      const CacheT* kpage = cache + ((static_cast<size_t>(blk) * 2 + 0) * hk + kh) * (BS * D);
      const CacheT* vpage = cache + ((static_cast<size_t>(blk) * 2 + 1) * hk + kh) * (BS * D);
      // ---- K: this lane's 64 dims of token tk ----
      float kf[64];
      if constexpr (sizeof(CacheT) == 2) {
        const uint4* kp = reinterpret_cast<const uint4*>(kpage + tk * D + half * 64);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint4 u = __ldg(kp + i);
          const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(hp[e]);
            kf[i * 8 + 2 * e] = f.x;
            kf[i * 8 + 2 * e + 1] = f.y;
          }
        }
      } else {
        const uint4* kp = reinterpret_cast<const uint4*>(kpage + tk * D + half * 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 u = __ldg(kp + i);
          const __nv_fp8_e4m3* bp = reinterpret_cast<const __nv_fp8_e4m3*>(&u);
#pragma unroll
          for (int e = 0; e < 16; ++e) kf[i * 16 + e] = static_cast<float>(bp[e]) * k_scale;
        }
      }
      // ---- V: 4 output dims per lane for each of the 16 tokens (issued early, consumed after the softmax) ----
      float vf[BS][4];
      if constexpr (sizeof(CacheT) == 2) {
#pragma unroll
        for (int t = 0; t < BS; ++t) {
          uint2 u = __ldg(reinterpret_cast<const uint2*>(vpage + t * D + lane * 4));
          const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&u);
          float2 a = __bfloat1622float2(hp[0]), c = __bfloat1622float2(hp[1]);
          vf[t][0] = a.x; vf[t][1] = a.y; vf[t][2] = c.x; vf[t][3] = c.y;
        }
      } else {
#pragma unroll
        for (int t = 0; t < BS; ++t) {
          uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(vpage + t * D + lane * 4));
          const __nv_fp8_e4m3* bp = reinterpret_cast<const __nv_fp8_e4m3*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) vf[t][e] = static_cast<float>(bp[e]) * v_scale;
        }
      }
      const int kpos = pg * BS + tk;
#pragma unroll
      for (int r = 0; r < RMAX; ++r) {
        if (r < R) {
          const float* qr = q_s + r * D + half * 64;
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            float4 qq = *reinterpret_cast<const float4*>(qr + i);
            s += kf[i] * qq.x + kf[i + 1] * qq.y + kf[i + 2] * qq.z + kf[i + 3] * qq.w;
          }
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          const int rr = r_base + r;
          const int j = rr / group;
          const int qpos = L - q_len + j;
          s *= scale_log2;
          if (alibi != nullptr) s += alibi[kh * group + (rr - j * group)] * 1.4426950408889634f * (kpos - qpos);
          if (kpos > qpos || kpos >= L) s = -INFINITY;
          float mx = warp_max(s);
          const float m_new = fmaxf(m[r], mx);
          float p = 0.f, corr = 1.f;
          if (m_new > -INFINITY) {
            p = exp2f(s - m_new);
            corr = exp2f(m[r] - m_new);
          }
          // each token's p is held by two lanes: count it once
          float psum = warp_sum(half == 0 ? p : 0.f);
          l[r] = l[r] * corr + psum;
          m[r] = m_new;
          acc[r][0] *= corr; acc[r][1] *= corr; acc[r][2] *= corr; acc[r][3] *= corr;
#pragma unroll
          for (int t = 0; t < BS; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t * 2);
            acc[r][0] += pt * vf[t][0];
            acc[r][1] += pt * vf[t][1];
            acc[r][2] += pt * vf[t][2];
            acc[r][3] += pt * vf[t][3];
          }
        }
      }
    }
    // ---- merge the warps of this CTA ----
#pragma unroll
    for (int r = 0; r < RMAX; ++r) {
      if (r < R) {
        float* o = red_o + (warp * RMAX + r) * D + lane * 4;
        o[0] = acc[r][0]; o[1] = acc[r][1]; o[2] = acc[r][2]; o[3] = acc[r][3];
        if (lane == 0) {
          red_m[warp * RMAX + r] = m[r];
          red_l[warp * RMAX + r] = l[r];
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
      const int r = i / D, c = i - r * D;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w * RMAX + r]);
      float ll = 0.f, oo = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float mw = red_m[w * RMAX + r];
        const float f = mw > -INFINITY ? exp2f(mw - mm) : 0.f;
        ll += red_l[w * RMAX + r] * f;
        oo += red_o[(w * RMAX + r) * D + c] * f;
      }
      const int rr = r_base + r;
      const int j = rr / group, g = rr - j * group;
      const int head = kh * group + g;
      const float o_norm = ll > 0.f ? oo / ll : 0.f;
      if (splits == 1) {
        out[static_cast<size_t>(q0 + j) * ldo + head * D + c] = __float2bfloat16(o_norm);
      } else {
        const size_t prow = (static_cast<size_t>(blockIdx.x) * max_rows + (j * h + head)) * splits + split;
        part_o[prow * D + c] = o_norm;
        if (c == 0) part_lse[prow] = ll > 0.f ? mm + log2f(ll) : -INFINITY;
      }
    }
  }
}

// Merge of the per-split partial results: one warp per (sequence, query token, head) row.
template <int D>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                      const int* __restrict__ cu_q, int seq_base, int h, int splits, int max_rows,
                                      __nv_bfloat16* __restrict__ out, int ldo) {
  const int bi = blockIdx.x;
  const int b = bi + seq_base;
  const int q0 = cu_q[b];
  const int rows = (cu_q[b + 1] - q0) * h;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += gridDim.y * (blockDim.x >> 5)) {
    const size_t base = (static_cast<size_t>(bi) * max_rows + row) * splits;
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_lse[base + s]);
    float den = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
      const float lse = part_lse[base + s];
      if (lse == -INFINITY) continue;
      const float w = exp2f(lse - mm);
      den += w;
      const float4 v = *reinterpret_cast<const float4*>(part_o + (base + s) * D + lane * 4);
      o[0] += w * v.x; o[1] += w * v.y; o[2] += w * v.z; o[3] += w * v.w;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const int j = row / h, head = row - j * h;
    __nv_bfloat16* dst = out + static_cast<size_t>(q0 + j) * ldo + head * D + lane * 4;
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(o[0] * inv, o[1] * inv);
    *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(o[2] * inv, o[3] * inv);
  }
}

// The merge step for other kernels that write partials in this layout (attention_decode_gqa.cu).
int launch_decode_combine(const float* part_o, const float* part_lse, const int* cu_q, int seq_base, int h, int splits,
                          int max_rows, int num_seqs, void* out, int ldo, cudaStream_t stream) {
  dim3 cgrid(num_seqs, (max_rows + 3) / 4);
  decode_combine_kernel<128><<<cgrid, 128, 0, stream>>>(part_o, part_lse, cu_q, seq_base, h, splits, max_rows,
                                                        reinterpret_cast<__nv_bfloat16*>(out), ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace ksana

using namespace ksana;

// Decode attention for sequences [seq_base, seq_base + num_seqs) of the step.
// q: [T, h, d] bf16 with token pitch ldq; cache: one layer [blocks][2][hk][16][128] (bf16: cache_kind 0, e4m3: 1);
// out: [T, h, d] bf16 with token pitch ldo. max_q_len bounds q_len over these sequences, max_kv_len bounds kv_len.
// workspace (fp32) is needed when KV is split: num_seqs * max_q_len * h * splits * (d + 1) floats.
// Returns 0, or a negative code (-1 unsupported shape, -6 workspace too small).
KSANA_API int ksana_paged_decode(const void* q, int ldq, const void* cache, int cache_kind, const int* block_tables,
                                 int max_blocks, const int* cu_q, const int* kv_lens, int seq_base, int num_seqs,
                                 int max_q_len, int max_kv_len, int h, int hk, int d, int block_size, float scale,
                                 const float* alibi, float k_scale, float v_scale, void* out, int ldo, float* workspace,
                                 long long workspace_floats, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (d != 128 || block_size != 16 || h % hk != 0) return -1;
  const int n_pages = (max_kv_len + block_size - 1) / block_size;
  const int sms = sm_count();
  int splits = 1;
  const int base_ctas = num_seqs * hk;
  if (base_ctas < 4 * sms) {
    splits = (4 * sms + base_ctas - 1) / base_ctas;
    const int max_splits = (n_pages + 2 * DEC_WARPS - 1) / (2 * DEC_WARPS);  // at least 2 pages per warp
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
  }
  int pages_per_split = (n_pages + splits - 1) / splits;
  if (pages_per_split < 1) pages_per_split = 1;
  splits = (n_pages + pages_per_split - 1) / pages_per_split;
  if (splits < 1) splits = 1;
  const int max_rows = max_q_len * h;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    const long long rows = static_cast<long long>(num_seqs) * max_rows * splits;
    if (workspace == nullptr || rows * (d + 1) > workspace_floats) return -6;
    part_o = workspace;
    part_lse = workspace + rows * d;
  }
  dim3 grid(num_seqs, hk, splits);
  const float scale_log2 = scale * 1.4426950408889634f;
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  const int rows_per_cta = max_q_len * (h / hk);
#define KSANA_DECODE_LAUNCH(RM, CT)                                                                                  \
  {                                                                                                                  \
    auto kern = paged_decode_kernel<128, 16, RM, CT>;                                                                \
    const size_t smem = (RM * 128 + DEC_WARPS * RM * 128 + 2 * DEC_WARPS * RM) * sizeof(float);                      \
    if (KSANA_SMEM_ONCE(kern, static_cast<int>(smem)) != 0) return -4;                                               \
    kern<<<grid, DEC_WARPS * 32, smem, stream>>>(Q, ldq, reinterpret_cast<const CT*>(cache), block_tables,           \
                                                 max_blocks, cu_q, kv_lens, seq_base, h, hk, scale_log2, alibi,      \
                                                 k_scale, v_scale, O, ldo, part_o, part_lse, splits,                 \
                                                 pages_per_split, max_rows);                                         \
  }
  if (cache_kind == 0) {
    if (rows_per_cta <= 1) KSANA_DECODE_LAUNCH(1, __nv_bfloat16)
    else if (rows_per_cta <= 4) KSANA_DECODE_LAUNCH(4, __nv_bfloat16)
    else if (rows_per_cta <= 8) KSANA_DECODE_LAUNCH(8, __nv_bfloat16)
    else KSANA_DECODE_LAUNCH(16, __nv_bfloat16)
  } else {
    if (rows_per_cta <= 1) KSANA_DECODE_LAUNCH(1, __nv_fp8_e4m3)
    else if (rows_per_cta <= 4) KSANA_DECODE_LAUNCH(4, __nv_fp8_e4m3)
    else if (rows_per_cta <= 8) KSANA_DECODE_LAUNCH(8, __nv_fp8_e4m3)
    else KSANA_DECODE_LAUNCH(16, __nv_fp8_e4m3)
  }
#undef KSANA_DECODE_LAUNCH
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (splits > 1) {
    dim3 cgrid(num_seqs, (max_rows + 3) / 4);
    decode_combine_kernel<128><<<cgrid, 128, 0, stream>>>(part_o, part_lse, cu_q, seq_base, h, splits, max_rows, O, ldo);
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention that allocates nothing (see attention_decode.h for who needs it and why).
//
// The split-KV partial results live in a fixed array that is part of the loaded library image instead of a
// caller-provided workspace. In host code `g_decode_static_scratch` is only a handle for the runtime, not a
// device address, so the address is resolved once per device with cudaGetSymbolAddress (on the first call made
// while that device is current) and handed to the kernels as an ordinary pointer.
// ---------------------------------------------------------------------------------------------------------------
namespace ksana {
constexpr long long kDecodeStaticScratchFloats = 2ll << 20;  // 8 MiB, held by every GPU that loads the library
static __device__ __align__(256) float g_decode_static_scratch[kDecodeStaticScratchFloats];
static float* g_decode_static_scratch_ptr[64] = {nullptr};
}  // namespace ksana

KSANA_API long long ksana_paged_decode_static_scratch_floats() { return ksana::kDecodeStaticScratchFloats; }

KSANA_API const char* ksana_paged_decode_static_error(int code) {
  switch (code) {
    case 0: return "ok";
    case -1: return "unsupported shape: needs head_dim 128, block_size 16 and h divisible by hk";
    case -5: return "kernel launch failed";
    case -7: return "problem too large for the built-in scratch array: num_seqs * max_q_len * h * kv_splits * 129 "
                    "floats exceed ksana_paged_decode_static_scratch_floats(); use ksana_paged_decode with a "
                    "caller-provided workspace instead";
    case -8: return "could not resolve the device address of the built-in scratch array (cudaGetSymbolAddress)";
    case -9: return "device index out of range";
    default: return "unknown error";
  }
}

KSANA_API int ksana_paged_decode_static(const void* q, int ldq, const void* cache, int cache_kind,
                                        const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens,
                                        int seq_base, int num_seqs, int max_q_len, int max_kv_len, int h, int hk, int d,
                                        int block_size, float scale, const float* alibi, float k_scale, float v_scale,
                                        void* out, int ldo, cudaStream_t stream) {
  using namespace ksana;
  if (num_seqs <= 0) return 0;
  if (d != 128 || block_size != 16 || hk <= 0 || h % hk != 0) return -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -9;
  if (g_decode_static_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_static_scratch) != cudaSuccess || p == nullptr)
      return -8;
    g_decode_static_scratch_ptr[dev] = p;
  }
  float* scratch = g_decode_static_scratch_ptr[dev];
  // same KV split policy as ksana_paged_decode
  const int n_pages = (max_kv_len + block_size - 1) / block_size;
  int sms = 148;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  int splits = 1;
  const int base_ctas = num_seqs * hk;
  if (base_ctas < 4 * sms) {
    splits = (4 * sms + base_ctas - 1) / base_ctas;
    const int max_splits = (n_pages + 2 * DEC_WARPS - 1) / (2 * DEC_WARPS);
    if (splits > max_splits) splits = max_splits;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
  }
  int pages_per_split = (n_pages + splits - 1) / splits;
  if (pages_per_split < 1) pages_per_split = 1;
  splits = (n_pages + pages_per_split - 1) / pages_per_split;
  if (splits < 1) splits = 1;
  const int max_rows = max_q_len * h;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    const long long rows = static_cast<long long>(num_seqs) * max_rows * splits;
    if (rows * (d + 1) > kDecodeStaticScratchFloats) return -7;
    part_o = scratch;
    part_lse = scratch + rows * d;
  }
  dim3 grid(num_seqs, hk, splits);
  const float scale_log2 = scale * 1.4426950408889634f;
  auto Q = reinterpret_cast<const __nv_bfloat16*>(q);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  const int rows_per_cta = max_q_len * (h / hk);
#define KSANA_DECODE_STATIC_LAUNCH(RM, CT)                                                                          \
  {                                                                                                                  \
    auto kern = paged_decode_kernel<128, 16, RM, CT>;                                                                \
    const size_t smem = (RM * 128 + DEC_WARPS * RM * 128 + 2 * DEC_WARPS * RM) * sizeof(float);                      \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));                 \
    kern<<<grid, DEC_WARPS * 32, smem, stream>>>(Q, ldq, reinterpret_cast<const CT*>(cache), block_tables,           \
                                                 max_blocks, cu_q, kv_lens, seq_base, h, hk, scale_log2, alibi,      \
                                                 k_scale, v_scale, O, ldo, part_o, part_lse, splits,                 \
                                                 pages_per_split, max_rows);                                         \
  }
  if (cache_kind == 0) {
    if (rows_per_cta <= 1) KSANA_DECODE_STATIC_LAUNCH(1, __nv_bfloat16)
    else if (rows_per_cta <= 4) KSANA_DECODE_STATIC_LAUNCH(4, __nv_bfloat16)
    else if (rows_per_cta <= 8) KSANA_DECODE_STATIC_LAUNCH(8, __nv_bfloat16)
    else KSANA_DECODE_STATIC_LAUNCH(16, __nv_bfloat16)
  } else {
    if (rows_per_cta <= 1) KSANA_DECODE_STATIC_LAUNCH(1, __nv_fp8_e4m3)
    else if (rows_per_cta <= 4) KSANA_DECODE_STATIC_LAUNCH(4, __nv_fp8_e4m3)
    else if (rows_per_cta <= 8) KSANA_DECODE_STATIC_LAUNCH(8, __nv_fp8_e4m3)
    else KSANA_DECODE_STATIC_LAUNCH(16, __nv_fp8_e4m3)
  }
#undef KSANA_DECODE_STATIC_LAUNCH
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (splits > 1) {
    dim3 cgrid(num_seqs, (max_rows + 3) / 4);
    decode_combine_kernel<128><<<cgrid, 128, 0, stream>>>(part_o, part_lse, cu_q, seq_base, h, splits, max_rows, O, ldo);
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}
