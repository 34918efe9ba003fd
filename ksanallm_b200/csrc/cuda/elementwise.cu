// Bandwidth-bound kernels: RMSNorm (+ residual add), SiLU*mul, embedding gather, fused
// QK-RMSNorm + RoPE + paged KV-cache append, and the 1 x 128 fp8 activation quantiser.
//
// Reference kernels replaced: flashinfer RMSNorm / FusedAddRMSNorm (csrc/kernels/nvidia/layernorm/
// layernorm.cu:564-568, fused_add_norm/fused_add_norm.cu:17-27), RowBasedActivationKernel
// (activation/activation.cu:210-577), LookupFusedEmbeddingKernelWithCSRKernel (embedding/embedding.cu:205-208),
// rotary_embedding.cu:237-431 + paged_attention/cache_copy.cu (CachePosCopy) + layernorm.cu:838-848
// (fused QKV RMSNorm), per_token_group_quant_fp8_kernel (others/sglang/.../per_token_group_quant.cu:265-269).
// All of them are pure HBM streams: one 16-byte vector per thread per access, one pass over the data.
#include "host_common.h"
#include "sm100.cuh"

namespace ksana {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) {
  bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) {
  bf16x8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = r;
}

// ---- RMSNorm ----------------------------------------------------------------------------------------------
// One CTA per row; each thread keeps up to VPT 8-element vectors in registers: the row is read once.
template <int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* __restrict__ residual, int ldr,
                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, int ldo, int H, float eps) {
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  __nv_bfloat16* rr = residual ? residual + static_cast<size_t>(row) * ldr : nullptr;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = (i * THREADS + threadIdx.x) * 8;
    if (c < H) {
      load8(xr + c, v[i]);
      if (rr) {
        float r[8];
        load8(rr + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        // the residual stream keeps the bf16-rounded sum; the norm uses the same rounded values
        bf16x8 t;
#pragma unroll
        for (int j = 0; j < 4; ++j) t.v[j] = __floats2bfloat162_rn(v[i][2 * j], v[i][2 * j + 1]);
        *reinterpret_cast<bf16x8*>(rr + c) = t;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(t.v[j]);
          v[i][2 * j] = f.x;
          v[i][2 * j + 1] = f.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  __shared__ float red[THREADS / 32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
  __nv_bfloat16* orow = out + static_cast<size_t>(row) * ldo;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = (i * THREADS + threadIdx.x) * 8;
    if (c < H) {
      float g[8], o[8];
      load8(w + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[i][j] * inv * g[j];
      store8(orow + c, o);
    }
  }
}

// ---- SiLU(gate) * up ------------------------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* __restrict__ out, int ldo,
                                int I) {
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= I) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  float g[8], u[8], o[8];
  load8(xr + c, g);
  load8(xr + I + c, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  store8(out + static_cast<size_t>(row) * ldo + c, o);
}

// ---- embedding gather -------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int H, int vocab, float scale) {
  const int row = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  float f[8];
  load8(table + static_cast<size_t>(id) * H + c, f);
  if (scale != 1.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= scale;
  }
  store8(out + static_cast<size_t>(row) * H + c, f);
}

// ---- QK-RMSNorm + RoPE + KV cache append --------------------------------------------------------------------------
// One warp per (token, head). Heads 0..h-1 are query heads (normalised + rotated in place), h..h+hk-1 key heads
// (normalised + rotated in place and written to the cache), h+hk..h+2hk-1 value heads (written to the cache).
// Cache layout [block][2][hk][block_size][d]. Pairs are (i, i + rd/2) (neox) or (2i, 2i+1) (interleaved).
template <typename CacheT>
__global__ void rope_cache_kernel(__nv_bfloat16* __restrict__ q, int ldq, __nv_bfloat16* __restrict__ k, int ldk,
                                  const __nv_bfloat16* __restrict__ v, int ldv, const int* __restrict__ positions,
                                  const float* __restrict__ cos_sin, const int* __restrict__ slots,
                                  CacheT* __restrict__ cache, const __nv_bfloat16* __restrict__ qw,
                                  const __nv_bfloat16* __restrict__ kw, float eps, int T, int h, int hk, int d, int rd,
                                  int interleaved, int block_size, float k_inv_scale, float v_inv_scale) {
  const int warps_per_block = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = h + 2 * hk;
  if (gw >= T * heads) return;
  const int t = gw / heads, hh = gw - t * heads;
  const int slot = slots[t];
  const int blk = slot / block_size, off = slot - blk * block_size;
  if (hh >= h + hk) {
    // value head: straight copy into the cache
    const int kh = hh - h - hk;
    const __nv_bfloat16* src = v + static_cast<size_t>(t) * ldv + kh * d;
    CacheT* dst = cache + ((static_cast<size_t>(blk) * 2 + 1) * hk + kh) * block_size * d + static_cast<size_t>(off) * d;
    for (int i = lane * 2; i < d; i += 64) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
      if constexpr (sizeof(CacheT) == 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(f.x, f.y);
      } else {
        dst[i] = CacheT(f.x * v_inv_scale);
        dst[i + 1] = CacheT(f.y * v_inv_scale);
      }
    }
    return;
  }
  const bool is_q = hh < h;
  __nv_bfloat16* p = is_q ? q + static_cast<size_t>(t) * ldq + hh * d : k + static_cast<size_t>(t) * ldk + (hh - h) * d;
  const __nv_bfloat16* nw = is_q ? qw : kw;
  float inv = 1.f;
  const bool fast = d == 128 && rd == 128 && !interleaved;
  if (nw != nullptr && !fast) {
    float ss = 0.f;
    for (int i = lane * 2; i < d; i += 64) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
      ss += f.x * f.x + f.y * f.y;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / static_cast<float>(d) + eps);
  }
  CacheT* dst = nullptr;
  if (!is_q) {
    const int kh = hh - h;
    dst = cache + ((static_cast<size_t>(blk) * 2 + 0) * hk + kh) * block_size * d + static_cast<size_t>(off) * d;
  }
  const int half = rd >> 1;
  const float* cs = cos_sin ? cos_sin + static_cast<size_t>(positions[t]) * rd : nullptr;
  if (fast) {
    // the common head: every lane owns elements (2l, 2l + 1) of the low half and their partners in the high half, so
    // each access of the warp is one full 128-byte line
    const int e = lane * 2;
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + e));
    float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 64 + e));
    if (nw != nullptr) {
      const float inv2 = rsqrtf(warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y) / 128.f + eps);
      const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + e));
      const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(nw + 64 + e));
      a = __bfloat1622float2(__floats2bfloat162_rn(a.x * inv2 * wa.x, a.y * inv2 * wa.y));
      b = __bfloat1622float2(__floats2bfloat162_rn(b.x * inv2 * wb.x, b.y * inv2 * wb.y));
    }
    float2 ra = a, rb = b;
    if (cs != nullptr) {
      const float2 c = *reinterpret_cast<const float2*>(cs + e), sn = *reinterpret_cast<const float2*>(cs + 64 + e);
      ra = make_float2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
      rb = make_float2(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
    }
    const __nv_bfloat162 oa = __floats2bfloat162_rn(ra.x, ra.y), ob = __floats2bfloat162_rn(rb.x, rb.y);
    *reinterpret_cast<__nv_bfloat162*>(p + e) = oa;
    *reinterpret_cast<__nv_bfloat162*>(p + 64 + e) = ob;
    if (dst != nullptr) {
      if constexpr (sizeof(CacheT) == 2) {
        *reinterpret_cast<__nv_bfloat162*>(dst + e) = oa;
        *reinterpret_cast<__nv_bfloat162*>(dst + 64 + e) = ob;
      } else {
        const float2 fa = __bfloat1622float2(oa), fb = __bfloat1622float2(ob);
        dst[e] = CacheT(fa.x * k_inv_scale);
        dst[e + 1] = CacheT(fa.y * k_inv_scale);
        dst[64 + e] = CacheT(fb.x * k_inv_scale);
        dst[64 + e + 1] = CacheT(fb.y * k_inv_scale);
      }
    }
    return;
  }
  // rotated part
  for (int i = lane; i < half; i += 32) {
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + half;
    float a = __bfloat162float(p[i0]), b = __bfloat162float(p[i1]);
    if (nw != nullptr) {
      a = __bfloat162float(__float2bfloat16(a * inv * __bfloat162float(nw[i0])));
      b = __bfloat162float(__float2bfloat16(b * inv * __bfloat162float(nw[i1])));
    }
    float ra = a, rb = b;
    if (cs != nullptr) {
      const float c = cs[i], s = cs[half + i];
      ra = a * c - b * s;
      rb = b * c + a * s;
    }
    const __nv_bfloat16 oa = __float2bfloat16(ra), ob = __float2bfloat16(rb);
    p[i0] = oa;
    p[i1] = ob;
    if (dst != nullptr) {
      if constexpr (sizeof(CacheT) == 2) {
        dst[i0] = oa;
        dst[i1] = ob;
      } else {
        dst[i0] = CacheT(__bfloat162float(oa) * k_inv_scale);
        dst[i1] = CacheT(__bfloat162float(ob) * k_inv_scale);
      }
    }
  }
  // pass-through part (partial rotary)
  for (int i = rd + lane; i < d; i += 32) {
    float a = __bfloat162float(p[i]);
    if (nw != nullptr) a = a * inv * __bfloat162float(nw[i]);
    const __nv_bfloat16 oa = __float2bfloat16(a);
    p[i] = oa;
    if (dst != nullptr) {
      if constexpr (sizeof(CacheT) == 2) dst[i] = oa;
      else dst[i] = CacheT(__bfloat162float(oa) * k_inv_scale);
    }
  }
}

// ---- 1 x 128 dynamic e4m3 activation quantisation ---------------------------------------------------------------------
// One warp per (row, 128-column group): amax -> scale = amax / 448 -> q = x / scale. Scales are stored
// [T, K/128] row-major fp32.
__global__ void quant_fp8_group_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_fp8_e4m3* __restrict__ q,
                                       int ldq, float* __restrict__ scales, int T, int K) {
  const int groups = K >> 7;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= T * groups) return;
  const int t = gw / groups, g = gw - t * groups;
  const __nv_bfloat16* src = x + static_cast<size_t>(t) * ldx + g * 128 + lane * 4;
  float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
  float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + 2));
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = fmaxf(warp_max(amax), 1e-10f);
  const float scale = amax / 448.f;
  const float inv = 448.f / amax;
  __nv_fp8_e4m3 o[4] = {__nv_fp8_e4m3(a.x * inv), __nv_fp8_e4m3(a.y * inv), __nv_fp8_e4m3(b.x * inv),
                        __nv_fp8_e4m3(b.y * inv)};
  *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * ldq + g * 128 + lane * 4) = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) scales[static_cast<size_t>(t) * groups + g] = scale;
}

// ---- KV block mover ---------------------------------------------------------------------------------------------------
// Copies whole cache blocks, for every layer at once: pairs[i] = (source block, destination block). Source and
// destination layers may be device memory or pinned host memory mapped into the device's address space, so the same
// kernel serves swap-out (device -> host), swap-in (host -> device) and copy-on-write forks (device -> device)
// without a host-side gather / scatter or a blocking copy. The reference moves blocks with per-block cudaMemcpyAsync
// calls (src/ksana_llm/cache_manager/block_allocator/, prefix_cache_manager.cpp swap paths).
__global__ void __launch_bounds__(256)
block_copy_kernel(const uint4* const* __restrict__ src_layers, uint4* const* __restrict__ dst_layers,
                  const int* __restrict__ pairs, long long block_vec16) {
  const int pair = blockIdx.x, layer = blockIdx.y;
  const uint4* src = src_layers[layer] + static_cast<size_t>(pairs[2 * pair]) * block_vec16;
  uint4* dst = dst_layers[layer] + static_cast<size_t>(pairs[2 * pair + 1]) * block_vec16;
  for (long long i = static_cast<long long>(blockIdx.z) * blockDim.x + threadIdx.x; i < block_vec16;
       i += static_cast<long long>(gridDim.z) * blockDim.x)
    dst[i] = src[i];
}

}  // namespace ksana

using namespace ksana;

// src_layers / dst_layers: device arrays of n_layers base pointers; pairs: device int array [n_pairs][2];
// block_bytes: bytes of one block of one layer (a multiple of 16).
KSANA_API int ksana_block_copy(const void* src_layers, const void* dst_layers, int n_layers, const int* pairs,
                               int n_pairs, long long block_bytes, cudaStream_t stream) {
  if (n_pairs <= 0 || n_layers <= 0) return 0;
  if (block_bytes & 15) return -1;
  const long long vec = block_bytes / 16;
  int z = static_cast<int>((vec + 256 * 8 - 1) / (256 * 8));
  if (z < 1) z = 1;
  if (z > 16) z = 16;
  dim3 grid(n_pairs, n_layers, z);
  block_copy_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint4* const*>(src_layers),
                                              reinterpret_cast<uint4* const*>(dst_layers), pairs, vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_rms_norm(const void* x, int ldx, void* residual, int ldr, const void* w, void* out, int ldo, int T,
                             int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || (ldx & 7) || (ldo & 7) || (residual && (ldr & 7))) return -1;
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<__nv_bfloat16*>(residual);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
  if (H <= 1024) rms_norm_kernel<128, 1><<<T, 128, 0, stream>>>(X, ldx, R, ldr, W, O, ldo, H, eps);
  else if (H <= 2048) rms_norm_kernel<256, 1><<<T, 256, 0, stream>>>(X, ldx, R, ldr, W, O, ldo, H, eps);
  else if (H <= 4096) rms_norm_kernel<256, 2><<<T, 256, 0, stream>>>(X, ldx, R, ldr, W, O, ldo, H, eps);
  else if (H <= 8192) rms_norm_kernel<512, 2><<<T, 512, 0, stream>>>(X, ldx, R, ldr, W, O, ldo, H, eps);
  else if (H <= 16384) rms_norm_kernel<1024, 2><<<T, 1024, 0, stream>>>(X, ldx, R, ldr, W, O, ldo, H, eps);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_silu_mul(const void* x, int ldx, void* out, int ldo, int T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((I & 7) || (ldx & 7) || (ldo & 7)) return -1;
  dim3 grid((I / 8 + 255) / 256, T);
  silu_mul_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                            reinterpret_cast<__nv_bfloat16*>(out), ldo, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_embedding(const int* ids, const void* table, void* out, int T, int H, int vocab, float scale,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  dim3 grid((H / 8 + 255) / 256, T);
  embedding_kernel<<<grid, 256, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                             reinterpret_cast<__nv_bfloat16*>(out), H, vocab, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// cache_kind: 0 = bf16 cache, 1 = fp8 e4m3 cache (values stored as x / scale).
KSANA_API int ksana_rope_cache(void* q, int ldq, void* k, int ldk, const void* v, int ldv, const int* positions,
                               const float* cos_sin, const int* slots, void* cache, const void* qw, const void* kw,
                               float eps, int T, int h, int hk, int d, int rd, int interleaved, int block_size,
                               int cache_kind, float k_scale, float v_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((d & 1) || (rd & 1) || rd > d) return -1;
  const int warps = T * (h + 2 * hk);
  const int wpb = 8;
  const int grid = (warps + wpb - 1) / wpb;
  auto Q = reinterpret_cast<__nv_bfloat16*>(q);
  auto K = reinterpret_cast<__nv_bfloat16*>(k);
  auto V = reinterpret_cast<const __nv_bfloat16*>(v);
  auto QW = reinterpret_cast<const __nv_bfloat16*>(qw);
  auto KW = reinterpret_cast<const __nv_bfloat16*>(kw);
  if (cache_kind == 0) {
    rope_cache_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>(Q, ldq, K, ldk, V, ldv, positions, cos_sin, slots,
                                                                    reinterpret_cast<__nv_bfloat16*>(cache), QW, KW, eps,
                                                                    T, h, hk, d, rd, interleaved, block_size, 1.f, 1.f);
  } else {
    rope_cache_kernel<__nv_fp8_e4m3><<<grid, wpb * 32, 0, stream>>>(
        Q, ldq, K, ldk, V, ldv, positions, cos_sin, slots, reinterpret_cast<__nv_fp8_e4m3*>(cache), QW, KW, eps, T, h,
        hk, d, rd, interleaved, block_size, 1.f / k_scale, 1.f / v_scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

KSANA_API int ksana_quant_fp8_group(const void* x, int ldx, void* q, int ldq, float* scales, int T, int K,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 127) || (ldx & 3) || (ldq & 3)) return -1;
  const int warps = T * (K / 128);
  quant_fp8_group_kernel<<<(warps + 7) / 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                              reinterpret_cast<__nv_fp8_e4m3*>(q), ldq, scales, T, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
