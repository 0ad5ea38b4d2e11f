// Host-side helpers shared by the launchers: error reporting, device checks, TMA tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace tb {
namespace host {

// Record `msg` as the calling thread's last error and return `code`.
int fail(int code, const char* msg);
// Record the pending CUDA error (cudaGetLastError) prefixed by `what`; returns TYBOK_ERR_CUDA.
int fail_cuda(const char* what);

int current_device();
int sm_count();
// TYBOK_OK when the current device is compute capability 10.x, TYBOK_ERR_ARCH otherwise.
int require_sm100();

bool pdl_enabled();
void count_launch();
// Tuning aid: device buffer that kernels fill with per-CTA clock samples (NULL = off).
long long* trace_buffer();
// Debugging aid: device int array [16 kernels][8 stages] that kernels bump at their stage boundaries (NULL = off).
int* counter_buffer();
// Test aid: SM clocks the GEMM epilogue waits for its accumulator; 0 = the production limit.
long long epilogue_wait_limit();

// Encode a 2-D tiled tensor map with the 128-byte shared-memory swizzle.
//   dim0/dim1: extent in elements (dim0 innermost), pitch_bytes: distance between rows,
//   box0/box1: tile extent in elements; box0 * elem_bytes must be <= 128.
int tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                  uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1);

// 3-D variant: dim0 innermost; pitch1/pitch2 are the byte strides of dim1 and dim2.
int tensor_map_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                  uint64_t dim1, uint64_t dim2, uint64_t pitch1, uint64_t pitch2, uint32_t box0, uint32_t box1,
                  uint32_t box2);

}  // namespace host
}  // namespace tb
