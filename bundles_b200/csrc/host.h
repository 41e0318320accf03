// Host-side helpers shared by the C-ABI translation units: error reporting, the device view of the
// routing lists, and the TMA tensor-map encoder (looked up through the runtime so that the library
// loads on a machine without a CUDA driver).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <mutex>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/b200nodes.h"

namespace b200 {

struct MoeLists {
  int32_t* counts;
  int32_t* offsets;
  int32_t* row_of_pair;
  int32_t* slot_of_row;
  float* wt_of_row;
  int32_t* blk_expert;
  int32_t* blk_row0;
  int32_t* blk_rows;
  int32_t* nblocks;
};

char* last_error_buffer();  // thread-local, 512 bytes

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int launch_status(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return 0;
  return fail(static_cast<int>(e), "%s: launch failed: %s", what, cudaGetErrorString(e));
}

// 2-D tensor map over a row-major byte matrix [rows, row_bytes] (element type uint8), box
// [box_rows, 128 bytes], 128-byte swizzle, zero fill outside the matrix.
int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows,
                       const char* what);

// 2-D tensor map over a row-major fp32 matrix [rows, cols], box [box_rows, 32 floats], 128-byte swizzle
int make_tmap_f32_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                     const char* what);

void b200_quant_rows_f8_launch(const void* x, int T, int H, uint8_t* xq, float* xs, cudaStream_t st);

int sm_count();  // SMs of the current device (cached per device)

// One-time set-up per device (kernel attributes): `run(fn)` calls fn once for the current device, whichever
// host thread gets there first.
struct DeviceOnce {
  std::once_flag flags[64];
  template <typename F>
  void run(F fn) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
      fn();
      return;
    }
    std::call_once(flags[dev], fn);
  }
};

// writers of each translation unit's copy of the device-side wait budget
int set_wait_budget_router(unsigned long long ns);
int set_wait_budget_moe(unsigned long long ns);
int set_wait_budget_moe_fp8(unsigned long long ns);
int set_wait_budget_attn(unsigned long long ns);
int set_wait_budget_attn_verify(unsigned long long ns);
int set_wait_budget_gdn(unsigned long long ns);
int set_wait_budget_ep(unsigned long long ns);

// Whether kernels are launched with programmatic stream serialization (on unless B200_NO_PDL is set in the
// environment).  Every kernel of the library then starts while its predecessor in the stream drains: it does
// its set-up, executes griddepcontrol.wait before the first access to memory that the predecessor writes
// (and before its own first global write), and only then griddepcontrol.launch_dependents, so a kernel's
// part before the wait may read what kernels two or more launches back have written (routing lists,
// for the GEMMs' weight prefetch).
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200
