// Token selection kernels: arg-max and batched temperature / top-k / top-p sampling.
//
// Reference kernels replaced: LocalArgMaxReduceKernel / WarpArgMaxReduceKernel
// (3rdparty/LLM_kernels/csrc/kernels/nvidia/samplers/greedy.cu:240-424) and the TRT-LLM two-stage top-k sampler with
// its separate temperature-softmax pass (samplers/sampling_topk_kernels.cu:150-250). Here one CTA handles one
// logits row end to end with per-row parameters: 4-pass radix select of the k-th largest logit, compaction of the
// <= 1024 survivors into shared memory, bitonic sort, softmax restricted to the survivors (the full-vocabulary
// softmax is never needed: only ratios inside the top-k set matter), top-p cut inside the top-k set and an
// inverse-CDF draw from one uniform number.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

__device__ __forceinline__ uint32_t f2key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(u);
}

// One CTA per row. Ties resolve to the lowest index (same as torch.argmax).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int ld, int V,
                                                      int* __restrict__ out) {
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  float best = -INFINITY;
  int bi = 0x7FFFFFFF;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  if (bi == 0x7FFFFFFF) bi = threadIdx.x < V ? threadIdx.x : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  __shared__ float sv[32];
  __shared__ int si[32];
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
  }
}

constexpr int SAMP_THREADS = 1024;
constexpr int SAMP_CAP = 1024;

__global__ void __launch_bounds__(SAMP_THREADS)
topk_topp_sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
                        const int* __restrict__ top_k, const float* __restrict__ top_p,
                        const float* __restrict__ uniform, int* __restrict__ out) {
  const int rowi = blockIdx.x;
  const float* row = logits + static_cast<size_t>(rowi) * ld;
  const int tid = threadIdx.x;
  int k = top_k[rowi];
  k = k < 1 ? 1 : (k > SAMP_CAP ? SAMP_CAP : k);
  if (k > V) k = V;
  const float inv_t = 1.f / fmaxf(temperature[rowi], 1e-6f);
  const float tp = fminf(fmaxf(top_p[rowi], 0.f), 1.f);

  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need, s_cnt_gt, s_cnt_eq;
  __shared__ uint32_t keys[SAMP_CAP];
  __shared__ int idxs[SAMP_CAP];
  __shared__ float cum[SAMP_CAP];
  __shared__ float wsum[32];
  __shared__ int s_kept, s_pick;

  // ---- radix select: key of the k-th largest element ----
  if (tid == 0) {
    s_prefix = 0;
    s_need = k;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t pmask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += SAMP_THREADS) {
      const uint32_t key = f2key(row[i]);
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t need = s_need, acc = 0;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (acc + hist[bin] >= need) break;
        acc += hist[bin];
      }
      s_need = need - acc;
      s_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  const uint32_t need_eq = s_need;  // how many elements equal to kth belong to the top-k set
  if (tid == 0) {
    s_cnt_gt = 0;
    s_cnt_eq = 0;
  }
  for (int i = tid; i < SAMP_CAP; i += SAMP_THREADS) {
    keys[i] = 0;
    idxs[i] = 0x7FFFFFFF;
  }
  __syncthreads();
  const uint32_t n_gt = k - need_eq;
  for (int i = tid; i < V; i += SAMP_THREADS) {
    const uint32_t key = f2key(row[i]);
    if (key > kth) {
      const uint32_t s = atomicAdd(&s_cnt_gt, 1u);
      if (s < SAMP_CAP) {
        keys[s] = key;
        idxs[s] = i;
      }
    } else if (key == kth) {
      const uint32_t s = atomicAdd(&s_cnt_eq, 1u);
      if (s < need_eq) {
        keys[n_gt + s] = key;
        idxs[n_gt + s] = i;
      }
    }
  }
  __syncthreads();
  // ---- bitonic sort, descending by key, ascending by index among equal keys ----
  for (int size = 2; size <= SAMP_CAP; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid;
      const int j = i ^ stride;
      if (j > i) {
        const bool desc = (i & size) == 0;
        const uint32_t ki = keys[i], kj = keys[j];
        const int ii = idxs[i], ij = idxs[j];
        const bool i_before_j = (ki > kj) || (ki == kj && ii < ij);
        if (desc != i_before_j) {
          keys[i] = kj;
          keys[j] = ki;
          idxs[i] = ij;
          idxs[j] = ii;
        }
      }
      __syncthreads();
    }
  }
  // ---- softmax over the survivors + inclusive scan ----
  const float v0 = key2f(keys[0]);
  float p = 0.f;
  if (tid < k) p = __expf((key2f(keys[tid]) - v0) * inv_t);
  float x = p;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float y = __shfl_up_sync(0xffffffffu, x, o);
    if ((tid & 31) >= o) x += y;
  }
  if ((tid & 31) == 31) wsum[tid >> 5] = x;
  __syncthreads();
  if (tid < 32) {
    float w = wsum[tid];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, w, o);
      if (tid >= o) w += y;
    }
    wsum[tid] = w;
  }
  __syncthreads();
  const float c_incl = x + ((tid >> 5) > 0 ? wsum[(tid >> 5) - 1] : 0.f);
  cum[tid] = c_incl;
  if (tid == 0) {
    s_kept = 0;
    s_pick = 0;
  }
  __syncthreads();
  const float mass = cum[k - 1];
  // kept prefix: elements whose preceding mass is still below top_p * mass (always at least one)
  const int keep_me = (tid < k) && (tid == 0 || (c_incl - p) < tp * mass);
  const int kept_w = __popc(__ballot_sync(0xffffffffu, keep_me));
  if ((tid & 31) == 0 && kept_w) atomicAdd(&s_kept, kept_w);
  __syncthreads();
  const int kept = s_kept;
  const float target = fminf(fmaxf(uniform[rowi], 0.f), 0.99999994f) * cum[kept - 1];
  const int below = (tid < kept) && (c_incl <= target);
  const int below_w = __popc(__ballot_sync(0xffffffffu, below));
  if ((tid & 31) == 0 && below_w) atomicAdd(&s_pick, below_w);
  __syncthreads();
  if (tid == 0) {
    int pick = s_pick;
    if (pick > kept - 1) pick = kept - 1;
    out[rowi] = idxs[pick];
  }
}


// ---- batched logits processing -----------------------------------------------------------------------------------
// One CTA per logits row applies, on the device, what the reference does in per-request host loops on rank 0
// (src/ksana_llm/samplers/sampler.cpp:90-217, 371-434): repetition penalty over prompt + output tokens (once per
// distinct token: positive logits divided, negative ones multiplied), presence / frequency penalties over the output
// tokens, the three no-repeat-n-gram rules, additive edits (logit bias), bans (min_tokens) and the grammar bitmask.
// hist: the rows' token histories back to back (prompt then output), row r = hist[row_off[r] .. row_off[r + 1]) with
// prompt_len[r] prompt tokens. fparams[r] = {repetition, presence, frequency}; iparams[r] = {no_repeat_ngram,
// encoder_no_repeat_ngram, decoder_no_repeat_ngram, has_bitmask}. edits / bans: (row, token[, value]) triples sorted by
// row with CSR offsets. A V-bit map in shared memory marks the tokens already handled.
__global__ void __launch_bounds__(512)
logits_process_kernel(float* __restrict__ x, int ld, int V, const int* __restrict__ hist,
                      const int* __restrict__ row_off, const int* __restrict__ prompt_len,
                      const float* __restrict__ fparams, const int* __restrict__ iparams,
                      const int* __restrict__ edit_off, const int* __restrict__ edit_tok,
                      const float* __restrict__ edit_val, const int* __restrict__ ban_off,
                      const int* __restrict__ ban_tok, const int* __restrict__ bitmask, int mask_words) {
  extern __shared__ unsigned int seen[];  // ceil(V / 32) words
  const int r = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
  float* xr = x + static_cast<size_t>(r) * ld;
  const int* h = hist + row_off[r];
  const int n = row_off[r + 1] - row_off[r];
  const int np = min(prompt_len[r], n);
  const float rep = fparams[3 * r], pres = fparams[3 * r + 1], freq = fparams[3 * r + 2];
  const int words = (V + 31) >> 5;
  if (rep != 1.f) {
    for (int i = tid; i < words; i += nthr) seen[i] = 0u;
    __syncthreads();
    for (int i = tid; i < n; i += nthr) {
      const int t = h[i];
      if (t < 0 || t >= V) continue;
      const unsigned int bit = 1u << (t & 31);
      if (!(atomicOr(&seen[t >> 5], bit) & bit)) {  // first occurrence: this thread alone touches the logit
        const float v = xr[t];
        xr[t] = v > 0.f ? v / rep : v * rep;
      }
    }
    __syncthreads();
  }
  if (pres != 0.f || freq != 0.f) {
    for (int i = tid; i < words; i += nthr) seen[i] = 0u;
    __syncthreads();
    for (int i = np + tid; i < n; i += nthr) {
      const int t = h[i];
      if (t < 0 || t >= V) continue;
      const unsigned int bit = 1u << (t & 31);
      float d = -freq;
      if (!(atomicOr(&seen[t >> 5], bit) & bit)) d -= pres;
      atomicAdd(&xr[t], d);
    }
    __syncthreads();
  }
  for (int i = edit_off[r] + tid; i < edit_off[r + 1]; i += nthr) {
    const int t = edit_tok[i];
    if (t >= 0 && t < V) atomicAdd(&xr[t], edit_val[i]);
  }
  __syncthreads();
  // n-gram rules: a window of the source that equals the last (size - 1) tokens of the suffix source bans its next token
  const int sizes[3] = {iparams[4 * r], iparams[4 * r + 1], iparams[4 * r + 2]};
#pragma unroll
  for (int rule = 0; rule < 3; ++rule) {
    const int g = sizes[rule];
    if (g <= 0) continue;
    // rule 0: windows and suffix over prompt + output; rule 1: windows over the prompt, suffix of the output;
    // rule 2: windows and suffix over the output
    const int* win = rule == 2 ? h + np : h;
    const int nwin = rule == 0 ? n : (rule == 1 ? np : n - np);
    const int* suf = rule == 0 ? h : h + np;
    const int nsuf = rule == 0 ? n : n - np;
    if (nsuf < g - 1 || nwin < g) continue;
    const int* tail = suf + nsuf - (g - 1);
    for (int i = tid; i + g <= nwin; i += nthr) {
      bool same = true;
      for (int j = 0; j < g - 1 && same; ++j) same = win[i + j] == tail[j];
      if (same) {
        const int t = win[i + g - 1];
        if (t >= 0 && t < V) xr[t] = -INFINITY;
      }
    }
  }
  for (int i = ban_off[r] + tid; i < ban_off[r + 1]; i += nthr) {
    const int t = ban_tok[i];
    if (t >= 0 && t < V) xr[t] = -INFINITY;
  }
  if (iparams[4 * r + 3] && bitmask != nullptr) {
    __syncthreads();
    const int* bm = bitmask + static_cast<size_t>(r) * mask_words;
    for (int t = tid; t < V; t += nthr) {
      const int w = t >> 5;
      const unsigned int bits = w < mask_words ? static_cast<unsigned int>(bm[w]) : 0xFFFFFFFFu;
      if (!((bits >> (t & 31)) & 1u)) xr[t] = -INFINITY;
    }
  }
}

}  // namespace ksana

using namespace ksana;

KSANA_API int ksana_argmax(const float* logits, int ld, int rows, int V, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, 1024, 0, stream>>>(logits, ld, V, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_sample(const float* logits, int ld, int rows, int V, const float* temperature, const int* top_k,
                           const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  topk_topp_sample_kernel<<<rows, SAMP_THREADS, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, uniform, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// In-place processing of fp32 logits [rows, V] (row pitch ld); see logits_process_kernel for the arguments. All
// arrays are device memory; edit_* / ban_* / bitmask may be null when their offsets are all zero / no row has a mask.
KSANA_API int ksana_logits_process(float* logits, int ld, int rows, int V, const int* hist, const int* row_off,
                                   const int* prompt_len, const float* fparams, const int* iparams,
                                   const int* edit_off, const int* edit_tok, const float* edit_val, const int* ban_off,
                                   const int* ban_tok, const int* bitmask, int mask_words, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int smem = ((V + 31) / 32) * 4;
  if (smem > 200 * 1024) return -1;
  if (KSANA_SMEM_ONCE(logits_process_kernel, 200 * 1024) != 0) return -4;
  logits_process_kernel<<<rows, 512, smem, stream>>>(logits, ld, V, hist, row_off, prompt_len, fparams, iparams, edit_off,
                                                     edit_tok, edit_val, ban_off, ban_tok, bitmask, mask_words);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
