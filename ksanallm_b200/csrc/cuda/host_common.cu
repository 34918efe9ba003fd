#include "host_common.h"

#include <mutex>

namespace ksana {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int make_tmap_nd(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = enc(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld_elems * static_cast<uint64_t>(elem_bytes)};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tmap_nd(out, base, dt, 2, dims, strides, box, swz);
}

static unsigned int* g_err[64] = {nullptr};
static int g_sms[64] = {0};

unsigned int* error_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!g_err[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_err[dev] = p;
  }
  return g_err[dev];
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!g_sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

int set_max_smem_once(unsigned long long* done_mask, const void* kernel, int bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  const unsigned long long bit = 1ull << (dev & 63);
  if (__atomic_load_n(done_mask, __ATOMIC_ACQUIRE) & bit) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -4;
  __atomic_fetch_or(done_mask, bit, __ATOMIC_RELEASE);
  return 0;
}

}  // namespace ksana

// Reads and clears the status word of the current device. 0 = no kernel reported a problem.
KSANA_API unsigned int ksana_read_error(int clear) {
  unsigned int* p = ksana::error_word();
  if (!p) return 0xFFFFFFFFu;
  unsigned int v = 0;
  cudaMemcpy(&v, p, sizeof(v), cudaMemcpyDeviceToHost);
  if (clear && v) cudaMemset(p, 0, sizeof(v));
  return v;
}

KSANA_API int ksana_sm_count() { return ksana::sm_count(); }
