// Host-side helpers shared by the entry points: error reporting, TMA descriptor creation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/sqattn_b200.h"

namespace sq {

inline char* err_buf() {
  static thread_local char buf[512] = "";
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}
#define SQ_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (expr);                                                                       \
    if (e_ != cudaSuccess) return sq::fail(SQATTN_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library links without libcuda.
inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 4-D map over a [B, H, N, D] 16-bit tensor given by element strides; box = 64 elements (128 bytes,
// 128-byte swizzle) x box_rows sequence positions.  Rows past `n` read as zero.
inline int make_tmap_bhnd(CUtensorMap* out, const void* ptr, int dtype, int64_t sb, int64_t sh, int64_t sn, int b,
                          int h, int n, int d, int box_rows, const char* name) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(SQATTN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return fail(SQATTN_ERR_INVALID_ARG, "%s: pointer must be 16-byte aligned", name);
  // a dimension of extent 1 never contributes to an address; give it a harmless stride
  if (b == 1) sb = static_cast<int64_t>(h) * n * d;
  if (h == 1) sh = static_cast<int64_t>(n) * d;
  if ((sb * 2) % 16 || (sh * 2) % 16 || (sn * 2) % 16 || sn <= 0 || sh <= 0 || sb <= 0)
    return fail(SQATTN_ERR_INVALID_ARG, "%s: strides must be positive multiples of 8 elements", name);
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(b)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(sn) * 2, static_cast<cuuint64_t>(sh) * 2,
                           static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dtype == SQATTN_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SQATTN_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", name, static_cast<int>(r));
  return SQATTN_OK;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace sq
