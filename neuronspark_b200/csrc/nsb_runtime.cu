// Host-side runtime shared by all entry points: status text, error records,
// device query, TMA descriptor encoding, tuning override, device error word.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "nsb_common.cuh"

namespace nsb {

namespace {
thread_local char g_err_text[256] = "no error";
thread_local LaunchInfo g_last_launch = {};
std::mutex g_mu;
Tuning g_tuning;
DeviceInfo g_dev_cache[16];
bool g_dev_cached[16] = {};
uint32_t* g_err_host = nullptr;
uint32_t* g_err_dev = nullptr;
constexpr unsigned long long kDefaultWaitNs = 2000000000ull;
std::atomic<unsigned long long> g_wait_ns{kDefaultWaitNs};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::atomic<EncodeTiledFn> g_encode{nullptr};
}  // namespace

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_err_text, sizeof g_err_text, "%s: %s (%s)", where, cudaGetErrorName(e),
           cudaGetErrorString(e));
}
void set_driver_error(int r, const char* where) {
  snprintf(g_err_text, sizeof g_err_text, "%s: CUresult %d", where, r);
}
LaunchInfo& last_launch() { return g_last_launch; }

Tuning get_tuning() {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_tuning;
}

int get_device_info(DeviceInfo* out) {
  int dev = 0;
  NSB_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  std::lock_guard<std::mutex> lk(g_mu);
  if (dev >= 0 && dev < 16 && g_dev_cached[dev]) {
    *out = g_dev_cache[dev];
    return NSB_OK;
  }
  DeviceInfo d;
  d.device = dev;
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev), "attr");
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev), "attr");
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev), "attr");
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev),
               "attr");
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev),
               "attr");
  NSB_CUDA_TRY(cudaDeviceGetAttribute(&d.reserved_smem_per_cta, cudaDevAttrReservedSharedMemoryPerBlock, dev),
               "attr");
  if (dev >= 0 && dev < 16) {
    g_dev_cache[dev] = d;
    g_dev_cached[dev] = true;
  }
  *out = d;
  return NSB_OK;
}

uint32_t* device_error_word_ptr() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_err_dev) return g_err_dev;
  void* h = nullptr;
  if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  memset(h, 0, 64);
  void* d = nullptr;
  if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(h);
    return nullptr;
  }
  g_err_host = static_cast<uint32_t*>(h);
  g_err_dev = static_cast<uint32_t*>(d);
  return g_err_dev;
}

int sticky_device_error() {
  // g_err_host is written once, under the mutex, before any kernel can set the word; a racing
  // first call sees nullptr and reports no error, which is true at that point.
  volatile uint32_t* w = g_err_host;
  return (w && *w) ? NSB_ERR_DEVICE_TIMEOUT : NSB_OK;
}

unsigned long long get_wait_limit_ns() { return g_wait_ns.load(std::memory_order_relaxed); }

namespace {
// One warp arms an mbarrier with bytes that no copy will ever deliver and waits for it with the
// library's bounded wait: the wait runs out, the error word is set (bit 31), the kernel returns.
// Nothing is in flight when it exits.
// A second warp waits, with the bounded wait of the chained backward launches, for a counter in
// global memory that nothing advances.
__device__ unsigned int g_selftest_counter = 0;

__global__ void wait_timeout_selftest_kernel(uint32_t* err, unsigned long long limit_ns) {
  if (threadIdx.x >= 32) {
    bool ok = true;
    if (threadIdx.x == 32) ok = counter_wait_bounded(&g_selftest_counter, 1u, err, 0x40000000u, limit_ns);
    (void)__all_sync(0xffffffffu, ok);
    return;
  }
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    mbar_init_fence();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_arrive_expect_tx(b, 16);
  __syncwarp();
  const bool ok = mbar_wait_bounded(b, 0, err, 0x80000000u, limit_ns);
  (void)__all_sync(0xffffffffu, ok);
  if (threadIdx.x == 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(b) : "memory");
}
}  // namespace

int make_tensor_map_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols,
                       uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = g_encode.load(std::memory_order_acquire);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
      if (e != cudaSuccess) set_cuda_error(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
      return NSB_ERR_UNSUPPORTED;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
    g_encode.store(fn, std::memory_order_release);
  }
  CUtensorMapDataType dt;
  size_t es;
  switch (dtype) {
    case NSB_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; es = 4; break;
    case NSB_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
    case NSB_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
    default: return NSB_ERR_INVALID_ARG;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A thread that has made no CUDA runtime call yet (seen: PyTorch's autograd thread when a
    // backward is the first thing it runs) has no context bound for driver entry points; a
    // runtime call binds the device's primary context, then the encode succeeds.
    cudaFree(nullptr);
    r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    set_driver_error(static_cast<int>(r), "cuTensorMapEncodeTiled");
    return NSB_ERR_CUDA;
  }
  return NSB_OK;
}

}  // namespace nsb

extern "C" {

int nsb_version(void) { return 100; }

const char* nsb_status_string(int s) {
  switch (s) {
    case NSB_OK: return "ok";
    case NSB_ERR_INVALID_ARG: return "invalid argument (null or misaligned pointer, bad size or enum)";
    case NSB_ERR_UNSUPPORTED: return "unsupported device or option (needs an sm_100 GPU)";
    case NSB_ERR_CUDA: return "CUDA call failed (see nsb_last_cuda_error)";
    case NSB_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case NSB_ERR_TOO_LARGE: return "size exceeds the documented maximum of this entry point";
    default: return "unknown status";
  }
}

const char* nsb_last_cuda_error(void) { return nsb::g_err_text; }

int nsb_device_error_word(uint32_t* out) {
  if (!out) return NSB_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lk(nsb::g_mu);
  if (!nsb::g_err_host) {
    *out = 0;
    return NSB_OK;
  }
  volatile uint32_t* w = nsb::g_err_host;
  *out = *w;
  *w = 0;
  return NSB_OK;
}

int nsb_set_wait_limit_ns(uint64_t ns) {
  nsb::g_wait_ns.store(ns ? ns : nsb::kDefaultWaitNs, std::memory_order_relaxed);
  return NSB_OK;
}

int nsb_selftest_wait_timeout(void* stream) {
  uint32_t* err = nsb::device_error_word_ptr();
  if (!err) return NSB_ERR_CUDA;
  nsb::wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(err, nsb::get_wait_limit_ns());
  NSB_CUDA_TRY(cudaGetLastError(), "launch wait_timeout_selftest_kernel");
  return NSB_OK;
}

int nsb_set_tuning(int warps_per_cta, int stages, int lanes_per_thread, int force_direct) {
  if (warps_per_cta > 16 || stages > 16 || force_direct < 0 || force_direct > 3 ||
      !(lanes_per_thread <= 0 || lanes_per_thread == 1 || lanes_per_thread == 2 ||
        lanes_per_thread == 4))
    return NSB_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lk(nsb::g_mu);
  nsb::g_tuning.warps_per_cta = warps_per_cta;
  nsb::g_tuning.stages = stages;
  nsb::g_tuning.lanes_per_thread = lanes_per_thread;
  nsb::g_tuning.force_direct = force_direct;
  return NSB_OK;
}

int nsb_last_launch_info(int32_t out[8]) {
  if (!out) return NSB_ERR_INVALID_ARG;
  const nsb::LaunchInfo& li = nsb::last_launch();
  out[0] = li.used_tma;
  out[1] = li.warps_per_cta;
  out[2] = li.stages;
  out[3] = li.lanes_per_thread;
  out[4] = li.grid;
  out[5] = li.smem_bytes;
  out[6] = li.tile_steps;
  out[7] = li.launches;
  return NSB_OK;
}

}  // extern "C"
