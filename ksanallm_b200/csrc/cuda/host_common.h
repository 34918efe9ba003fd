// Host-side helpers shared by all launchers: TMA descriptor creation (through the runtime's driver entry
// point lookup, so the library does not link libcuda), the per-device kernel status word, SM count cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define KSANA_API extern "C" __attribute__((visibility("default")))

namespace ksana {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled();

// 2D row-major tensor [rows, cols] of `elem_bytes` elements with row pitch `ld_elems`; box = [box_rows, box_cols].
// Returns 0 on success.
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz);

// General N-d (rank <= 5): dims/strides innermost first; strides in bytes for dims 1..rank-1.
int make_tmap_nd(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz);

// Device-resident status word of the current device (allocated on first use; never freed).
unsigned int* error_word();
int sm_count();

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute and a process may drive several devices:
// `done_mask` (one static word per call site) keeps one bit per device ordinal. Returns 0 on success.
int set_max_smem_once(unsigned long long* done_mask, const void* kernel, int bytes);
#define KSANA_SMEM_ONCE(kern, bytes)                                                                \
  ([&]() -> int {                                                                                   \
    static unsigned long long mask__ = 0;                                                           \
    return ::ksana::set_max_smem_once(&mask__, reinterpret_cast<const void*>(kern), (bytes));       \
  }())

}  // namespace ksana
