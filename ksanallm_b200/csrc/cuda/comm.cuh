// Device-side primitives for kernels that talk to other GPUs over NVLink: system-scope release/acquire flag
// accesses, peer loads/stores, NVLS multimem load-reduce / store, bounded flag waits.
#pragma once
#include "sm100.cuh"

namespace ksana {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer16(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// sum of 8 bf16 over all ranks, performed by the switch, fp32 accumulation
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#ifndef KSANA_PEER_TIMEOUT_NS
#define KSANA_PEER_TIMEOUT_NS 8000000000ull  // ranks may be skewed by host work; a lost peer still ends the wait
#endif
#ifndef KSANA_PEER_TIMEOUT_AFTER_FAILURE_NS
#define KSANA_PEER_TIMEOUT_AFTER_FAILURE_NS 1000000ull  // once a peer wait has expired on this GPU: 1 ms per wait
#endif
// Waits until *p >= want (epochs / counters only grow within a call). Bounded by wall time: returns false and
// records KERR_PEER_TIMEOUT on expiry, so a missing peer can never hang the GPU. The full bound is paid once: while
// the status word carries KERR_PEER_TIMEOUT (until the host has read and cleared it) every further wait gives up
// after a millisecond, so the kernels queued behind a lost peer drain in milliseconds instead of 8 s each.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t want, unsigned int* err,
                                             unsigned long long timeout_ns = KSANA_PEER_TIMEOUT_NS) {
  for (int it = 0; it < 64; ++it)
    if (static_cast<int32_t>(ld_acquire_sys(p) - want) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned int polls = 0;
  while (true) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - want) >= 0) return true;
    __nanosleep(400);
    if (err != nullptr && (++polls & 255u) == 0u && timeout_ns > KSANA_PEER_TIMEOUT_AFTER_FAILURE_NS &&
        (*reinterpret_cast<volatile unsigned int*>(err) & KERR_PEER_TIMEOUT) != 0u)
      timeout_ns = KSANA_PEER_TIMEOUT_AFTER_FAILURE_NS;
    if (global_timer_ns() - t0 > timeout_ns) break;
  }
  if (err) atomicOr(err, KERR_PEER_TIMEOUT);
  return false;
}

__device__ __forceinline__ void unpack8(uint4 u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  return u;
}


__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

}  // namespace ksana
