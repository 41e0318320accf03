// Host-side plumbing of the C ABI: version, error text, tensor-map encoding, device queries.
#include "host.h"

#include <mutex>

namespace b200 {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    (void)cudaGetLastError();
  });
  return fn;
}

int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                       const char* what) {
  EncodeTiledFn fn = encoder();
  if (!fn) return fail(B200_E_DRIVER, "%s: cuTensorMapEncodeTiled is not available", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_bytes & 15) || row_bytes < 128 || rows == 0)
    return fail(B200_E_ALIGN, "%s: tensor base / row pitch must be 16-byte aligned and rows >= 1", what);
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_E_ARG, "%s: cuTensorMapEncodeTiled failed (%d)", what, static_cast<int>(r));
  return 0;
}

int make_tmap_f32_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                     const char* what) {
  EncodeTiledFn fn = encoder();
  if (!fn) return fail(B200_E_DRIVER, "%s: cuTensorMapEncodeTiled is not available", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols & 3) || cols < 32 || rows == 0)
    return fail(B200_E_ALIGN, "%s: tensor base must be 16-byte aligned, cols a multiple of 4 and >= 32", what);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 4};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_E_ARG, "%s: cuTensorMapEncodeTiled failed (%d)", what, static_cast<int>(r));
  return 0;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool pdl_enabled() {
  static const bool on = getenv("B200_NO_PDL") == nullptr;
  return on;
}

}  // namespace b200

extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }
extern "C" const char* b200_last_error(void) { return b200::last_error_buffer(); }
