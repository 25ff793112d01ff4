// Host-side helpers shared by the C-ABI translation units: error reporting, the device
// status word, driver entry points for tensor-map encoding.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/mosaicist_sm100a.h"

namespace msc {

// Sets the thread-local message msc_last_error() returns and hands `code` back.
int fail(int code, const char* fmt, ...);

// Device pointer of the current device's status word (lazily resolved, one per device).
int* status_word();

// cuTensorMapEncodeTiled, resolved through the runtime so libcuda is not a link-time
// dependency.  Returns nullptr (and sets the error message) if it cannot be resolved.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// 2-D byte tensor [rows][row_bytes] with a [box_rows][128 B] box and 128-byte swizzle.
int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                       uint32_t box_rows);

// 2-D bf16 tensor [rows][cols] with a [box_rows][64 columns = 128 B] box and 128-byte swizzle
// (the epilogue's store map).
int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint32_t box_rows);

// 2-D byte tensor [rows][128 B] with a [box_rows][128 B] box, no swizzle: scale-factor chunks
// (each 512-byte chunk is four such rows).
int make_tmap_sf_2d(CUtensorMap* map, const void* base, uint64_t rows128, uint32_t box_rows);

// 2-D byte tensor [rows][row_bytes] with a [box_rows][32 B] box, no swizzle (packed int4
// weights: 64 K-elements of box_rows rows).
int make_tmap_narrow_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint32_t box_rows);


// 2-D byte tensor [rows][row_bytes] whose rows are `pitch_bytes` apart, with a
// [box_rows][128 B] box and 128-byte swizzle (operands and outputs of the dense GEMM, where a
// shard of a larger matrix keeps the parent's pitch).
int make_tmap_pitched_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                         uint64_t pitch_bytes, uint32_t box_rows);

// Forgets every cached tensor map (msc_shutdown).
void clear_tmap_cache();

int num_sms();

// Scale re-tiling (quantize.cu): (groups, mn, kwords * 4) row-major bytes to the 128-row MMA
// tiling; rows_used (device, may be null, one group only) bounds the tiles that are written.
int launch_sf_swizzle(const void* sf_rowmajor, void* sf_tiled, int groups, int mn, int kwords,
                      const int* rows_used, cudaStream_t stream);

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device); safe to call from
// several host threads.
int allow_dynamic_smem(const void* kernel, int bytes);

// Launch configuration with programmatic stream serialization: the kernel's set-up may overlap
// the tail of its predecessor in the stream; the kernel calls grid_dependency_wait() before it
// touches global memory.  `attr` must outlive the launch call.
inline cudaLaunchConfig_t pdl_launch_config(int grid, int threads, int smem, cudaStream_t stream,
                                            cudaLaunchAttribute* attr) {
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(threads);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  return lc;
}

#define MSC_CUDA_OK(expr)                                                              \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ::msc::fail(MSC_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__));      \
  } while (0)

}  // namespace msc
