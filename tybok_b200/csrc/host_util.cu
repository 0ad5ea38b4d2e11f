#include "host_util.h"

#include <atomic>
#include <cstdio>
#include <cstring>

#include "../../include/tybok_b200.h"

namespace tb {
namespace host {

static thread_local char g_err[512] = "";
static std::atomic<int> g_pdl{1};
static std::atomic<long long> g_launches{0};
static std::atomic<long long*> g_trace{nullptr};
static std::atomic<long long> g_epi_limit{0};
static std::atomic<int*> g_counters{nullptr};

int fail(int code, const char* msg) {
  std::snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}

int fail_cuda(const char* what) {
  const cudaError_t e = cudaGetLastError();
  std::snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  return TYBOK_ERR_CUDA;
}

const char* last_error() { return g_err; }

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  return dev;
}

struct DevInfo {
  bool known = false;
  int major = 0;
  int sms = 0;
};
static DevInfo g_dev[64];

static const DevInfo* dev_info() {
  const int dev = current_device();
  if (dev < 0 || dev >= 64) return nullptr;
  DevInfo& d = g_dev[dev];
  if (!d.known) {
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    d.major = major;
    d.sms = sms;
    d.known = true;
  }
  return &d;
}

int sm_count() {
  const DevInfo* d = dev_info();
  return d ? d->sms : 148;  // planning without a device (workspace sizing): assume a B200
}

int require_sm100() {
  const DevInfo* d = dev_info();
  if (!d) return fail_cuda("query device");
  if (d->major != 10) return fail(TYBOK_ERR_ARCH, "tybok_b200 kernels need an sm_100 (B200) device");
  return TYBOK_OK;
}

bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }
long long* trace_buffer() { return g_trace.load(std::memory_order_relaxed); }
int* counter_buffer() { return g_counters.load(std::memory_order_relaxed); }
long long epilogue_wait_limit() { return g_epi_limit.load(std::memory_order_relaxed); }
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

int tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                  uint64_t dim1, uint64_t pitch_bytes, uint32_t box0, uint32_t box1) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TYBOK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || box0 * elem_bytes > 128 || box1 > 256)
    return fail(TYBOK_ERR_ARG, "tensor map: base/pitch must be 16-byte aligned, box <= 128 bytes x 256 rows");
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, pitch %llu)",
                  static_cast<int>(r), static_cast<unsigned long long>(dim0), static_cast<unsigned long long>(dim1),
                  static_cast<unsigned long long>(pitch_bytes));
    return fail(TYBOK_ERR_CUDA, msg);
  }
  return TYBOK_OK;
}

int tensor_map_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t dim0,
                  uint64_t dim1, uint64_t dim2, uint64_t pitch1, uint64_t pitch2, uint32_t box0, uint32_t box1,
                  uint32_t box2) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TYBOK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch1 & 15) || (pitch2 & 15) || box0 * elem_bytes > 128 ||
      box1 > 256 || box2 > 256)
    return fail(TYBOK_ERR_ARG, "tensor map: base/pitches must be 16-byte aligned, box <= 128 bytes x 256 x 256");
  cuuint64_t dims[3] = {dim0, dim1, dim2};
  cuuint64_t strides[2] = {pitch1, pitch2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(out, dtype, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[160];
    std::snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled (3-D) failed with CUresult %d (dims %llu x %llu x %llu)",
                  static_cast<int>(r), static_cast<unsigned long long>(dim0), static_cast<unsigned long long>(dim1),
                  static_cast<unsigned long long>(dim2));
    return fail(TYBOK_ERR_CUDA, msg);
  }
  return TYBOK_OK;
}

}  // namespace host
}  // namespace tb

extern "C" {
int tybok_version(void) { return 100; }
const char* tybok_last_error(void) { return tb::host::last_error(); }
void tybok_set_pdl(int enabled) { tb::host::g_pdl.store(enabled ? 1 : 0); }
void tybok_debug_set_trace(void* device_buffer) { tb::host::g_trace.store(static_cast<long long*>(device_buffer)); }
void tybok_debug_set_counters(void* device_buffer) { tb::host::g_counters.store(static_cast<int*>(device_buffer)); }
void tybok_debug_set_epilogue_wait_limit(long long sm_clocks) { tb::host::g_epi_limit.store(sm_clocks > 0 ? sm_clocks : 0); }
long long tybok_launch_count(void) { return tb::host::g_launches.load(); }
}
