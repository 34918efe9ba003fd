// Issue-rate probe for tcgen05.mma (M = 128, K = 16, bf16): cycles per instruction against N and the A operand's source
// (shared memory or TMEM). Zero-filled operands, bounded waits; nothing here can fault.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Iksanallm_b200/csrc/cuda \
//        -o tcgen05_rate_probe benchmarks/tcgen05_rate_probe.cu && ./tcgen05_rate_probe
#include <cstdio>
#include <cuda_runtime.h>
#include "sm100.cuh"
using namespace ksana;

template <int N, int MODE>  // MODE 0: A smem, 1: A tmem
__global__ void __launch_bounds__(128, 1) rate_kernel(long long* out, int reps, unsigned int* err) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t holder;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (64 * 1024) / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (tid == 0) { mbar_init(&bar, 1); abort_flag = 0; fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&holder, 512); tmem_relinquish(); }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = holder;
  long long t0 = 0, t1 = 0;
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc(128, N, 1, 1);
    t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      const uint32_t a = smem_u32(smem) + (r & 3) * 32 + ((r >> 2) & 1) * 16384;
      const uint32_t b = smem_u32(smem) + 32768 + (r & 3) * 32;
      if (MODE == 0) umma_f16(tb, umma_desc_k128(a), umma_desc_k128(b), idesc, 1u);
      else umma_f16_ts(tb, tb + 256 + (r & 3) * 8, umma_desc_k128(b), idesc, 1u);
    }
    umma_commit(&bar);
  }
  mbar_wait_bounded(&bar, 0, &abort_flag, err);
  if (tid == 0) { t1 = clock64(); if (blockIdx.x == 0) out[0] = t1 - t0; }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int N, int MODE> void run(const char* name, int grid) {
  long long* d; unsigned int* e;
  cudaMalloc(&d, 8); cudaMalloc(&e, 4); cudaMemset(e, 0, 4);
  auto k = rate_kernel<N, MODE>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 66 * 1024);
  const int reps = 4000;
  for (int i = 0; i < 2; ++i) k<<<grid, 128, 66 * 1024>>>(d, reps, e);
  cudaError_t st = cudaDeviceSynchronize();
  long long h = 0; unsigned int he = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost); cudaMemcpy(&he, e, 4, cudaMemcpyDeviceToHost);
  printf("%s N=%d grid=%d: %.1f cycles/mma (err %u, %s)\n", name, N, grid, double(h) / reps, he, cudaGetErrorString(st));
  cudaFree(d); cudaFree(e);
}

int main() {
  for (int grid : {1, 148}) {
    run<32, 0>("A=smem", grid); run<64, 0>("A=smem", grid); run<128, 0>("A=smem", grid); run<256, 0>("A=smem", grid);
    run<32, 1>("A=tmem", grid); run<64, 1>("A=tmem", grid); run<128, 1>("A=tmem", grid); run<256, 1>("A=tmem", grid);
  }
  return 0;
}
