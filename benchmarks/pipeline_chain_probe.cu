// Latency probes of the building blocks of a tcgen05 pipeline (128 threads per CTA; 1, 2 or 4 CTAs per SM):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Iksanallm_b200/csrc/cuda \
//        -o pipeline_chain_probe benchmarks/pipeline_chain_probe.cu && ./pipeline_chain_probe
//  mode 0: [tcgen05.st x32 by 128 threads -> wait::st -> fence -> bar -> 4 ts-MMAs (N=16) -> commit -> all wait mbarrier] per iter
//  mode 1: [TMA bulk 4 KB -> mbarrier wait] per iter (dependent)
//  mode 2: [4 ts-MMAs -> commit -> wait] per iter (thread 0 only, no st)
//  mode 3: [global ld 2 x uint4 per thread dependent on previous iter? no: independent stream, 1 in flight]
#include <cstdio>
#include <cuda_runtime.h>
#include "sm100.cuh"
using namespace ksana;

__global__ void __launch_bounds__(128, 1) probe(int mode, int reps, const uint8_t* gsrc, long long* out, unsigned int* err) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar, bar2;
  __shared__ uint32_t holder;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (32 * 1024) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (tid == 0) { mbar_init(&bar, 1); mbar_init(&bar2, 1); abort_flag = 0; fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&holder, 128); tmem_relinquish(); }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = holder;
  const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;
  long long t0 = clock64();
  constexpr uint32_t idesc = umma_idesc(128, 16, 1, 1);
  uint32_t v[32];
  for (int i = 0; i < 32; ++i) v[i] = tid + i;
  uint4 acc = make_uint4(0, 0, 0, 0);
  for (int r = 0; r < reps; ++r) {
    if (mode == 0) {
      tmem_st32(tb + 64 + lane_off, v);
      tmem_wait_st();
      tc_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after();
        for (int k = 0; k < 4; ++k) umma_f16_ts(tb, tb + 64 + k * 8, umma_desc_k128(smem_u32(smem) + k * 32), idesc, 1u);
        umma_commit(&bar);
      }
      mbar_wait_bounded(&bar, r & 1, &abort_flag, err);
      tc_fence_after();
    } else if (mode == 1) {
      if (tid == 0) {
        mbar_expect_tx(&bar, 4096);
        bulk_load(smem + 8192, gsrc + (static_cast<size_t>(blockIdx.x) * reps + r) * 4096, 4096, &bar);
      }
      mbar_wait_bounded(&bar, r & 1, &abort_flag, err);
    } else if (mode == 2) {
      if (tid == 0) {
        for (int k = 0; k < 4; ++k) umma_f16_ts(tb, tb + 64 + k * 8, umma_desc_k128(smem_u32(smem) + k * 32), idesc, 1u);
        umma_commit(&bar);
        mbar_wait_bounded(&bar, r & 1, &abort_flag, err);
      }
    } else if (mode == 3) {
      const uint4* p = reinterpret_cast<const uint4*>(gsrc + (static_cast<size_t>(blockIdx.x) * reps + r) * 4096) + tid * 2;
      uint4 a = __ldg(p), b = __ldg(p + 1);
      acc.x += a.x + b.y;  // consumed immediately: one k-block in flight
      if (acc.x == 0x12345678u) v[0]++;
    }
  }
  __syncthreads();
  long long t1 = clock64();
  if (tid == 0 && blockIdx.x == 0) out[0] = t1 - t0;
  if (acc.x == 0xdeadbeefu) out[1] = v[0];
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tb, 128); }
}

int main() {
  long long* d; unsigned int* e; uint8_t* g;
  const int reps = 1000;
  cudaMalloc(&d, 16); cudaMalloc(&e, 4); cudaMemset(e, 0, 4);
  cudaMalloc(&g, size_t(148) * reps * 4096); cudaMemset(g, 1, size_t(148) * reps * 4096);
  cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024);
  const char* names[4] = {"st->MMAx4->commit->wait", "bulk 4KB -> wait", "MMAx4->commit->wait", "ldg 32B/thread dependent"};
  for (int grid : {148, 296, 592})
    for (int mode = 0; mode < 3; mode += 2) {
      probe<<<grid, 128, 40 * 1024>>>(mode, reps, g, d, e);
      probe<<<grid, 128, 40 * 1024>>>(mode, reps, g, d, e);
      cudaError_t st = cudaDeviceSynchronize();
      long long h = 0; unsigned int he = 0;
      cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost); cudaMemcpy(&he, e, 4, cudaMemcpyDeviceToHost);
      printf("grid %3d %-28s %.0f cycles/iter (err %u %s)\n", grid, names[mode], double(h) / reps, he, cudaGetErrorString(st));
    }
  return 0;
}
