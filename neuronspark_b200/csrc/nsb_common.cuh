// Shared device/host helpers for the neuronspark_b200 kernels (sm_100a only).
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched at run time)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/neuronspark_b200.h"

namespace nsb {

// ------------------------------------------------------------------ host side

// Thread-local record of the last CUDA failure, and of the last launch shape.
void set_cuda_error(cudaError_t e, const char* where);
void set_driver_error(int cu_result, const char* where);
struct LaunchInfo {
  int used_tma, warps_per_cta, stages, lanes_per_thread, grid, smem_bytes, tile_steps, launches;
};
LaunchInfo& last_launch();

struct Tuning {
  int warps_per_cta = 0, stages = 0, lanes_per_thread = 0, force_direct = 0;
};
Tuning get_tuning();
// Adaptive surrogate slope from (sum, sum of squares) partials (nsb_surrogate.cu).
int launch_alpha_finalize(const double* partial, int nparts, long long n, int dtype, float alpha0, float sigma0,
                          float* alpha_out, cudaStream_t st);

// Device properties that the launch heuristics need (cached per device).
struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int max_smem_optin = 0;     // per CTA
  int smem_per_sm = 0;
  int reserved_smem_per_cta = 0;
};
int get_device_info(DeviceInfo* out);  // returns NSB status

// Pointer to the device-visible error word (mapped pinned host memory, one per
// process). Returns nullptr if it could not be set up.
uint32_t* device_error_word_ptr();
// NSB_ERR_DEVICE_TIMEOUT while the error word is non-zero (a plain host load, no
// synchronisation), NSB_OK otherwise. The word stays set until nsb_device_error_word reads it.
int sticky_device_error();
// Limit of every bounded device-side wait, in nanoseconds (nsb_set_wait_limit_ns; default 2 s).
unsigned long long get_wait_limit_ns();

// 2-D tiled tensor map over a row-major [rows, cols] tensor; box = [box_rows, box_cols].
// elem: NSB dtype, or 100 for raw fp32/uint32 words.
int make_tensor_map_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows,
                       uint64_t cols, uint32_t box_rows, uint32_t box_cols);

inline size_t dtype_size(int dt) { return dt == NSB_F32 ? 4 : 2; }

#define NSB_CUDA_TRY(expr, where)                 \
  do {                                            \
    cudaError_t _e = (expr);                      \
    if (_e != cudaSuccess) {                      \
      ::nsb::set_cuda_error(_e, where);           \
      return NSB_ERR_CUDA;                        \
    }                                             \
  } while (0)

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

// Element traits: widening to fp32 is exact; narrowing is round-to-nearest-even.
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kDtype = NSB_F32;
  __device__ static __forceinline__ float to_f32(float v) { return v; }
  __device__ static __forceinline__ float from_f32(float v) { return v; }
  __device__ static __forceinline__ float one() { return 1.0f; }
  __device__ static __forceinline__ float zero() { return 0.0f; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kDtype = NSB_BF16;
  __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) {
    return __uint_as_float(((uint32_t)__bfloat16_as_ushort(v)) << 16);
  }
  __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) {
    return __float2bfloat16_rn(v);
  }
  __device__ static __forceinline__ __nv_bfloat16 one() { return __ushort_as_bfloat16(0x3F80); }
  __device__ static __forceinline__ __nv_bfloat16 zero() { return __ushort_as_bfloat16(0); }
};
template <>
struct Elem<__half> {
  static constexpr int kDtype = NSB_F16;
  __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
  __device__ static __forceinline__ __half one() { return __ushort_as_half(0x3C00); }
  __device__ static __forceinline__ __half zero() { return __ushort_as_half(0); }
};

// A small aligned vector of N elements, moved with one load/store instruction.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void proxy_async_fence() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait on an mbarrier phase: gives up after `limit_ns` of wall time (or 2^28 polls,
// whichever comes first), records `code` in the error word and returns false. Never spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t* err_word,
                                                  uint32_t code, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 0x3F) == 0) {
      if (global_timer_ns() - t0 > limit_ns || it > (1u << 28)) {
        if (err_word) atomicOr(reinterpret_cast<unsigned int*>(err_word), code);
        return false;
      }
    }
  }
  return true;
}
// Bounded wait until a counter in global memory, which other CTAs of the same launch advance with
// counter_publish, has reached `want`. Same limits and error reporting as mbar_wait_bounded.
// A counter that reads kCounterPoisoned was abandoned by its writer (which gave up a wait of its own and
// has recorded why): the wait ends at once and reports failure, so that a chain of waiters does not
// run out one limit after the other.
constexpr unsigned int kCounterPoisoned = 0xffffffffu;
__device__ __forceinline__ bool counter_wait_bounded(const unsigned int* counter, unsigned int want,
                                                     uint32_t* err_word, uint32_t code,
                                                     unsigned long long limit_ns) {
  auto peek = [&] {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    return v;
  };
  unsigned int seen = peek();
  if (seen >= want) return seen != kCounterPoisoned;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  while ((seen = peek()) < want) {
    __nanosleep(200);
    if ((++it & 0x3F) == 0) {
      if (global_timer_ns() - t0 > limit_ns || it > (1u << 28)) {
        if (err_word) atomicOr(reinterpret_cast<unsigned int*>(err_word), code);
        return false;
      }
    }
  }
  return seen != kCounterPoisoned;
}
// The same on a word of shared memory that another warp of the CTA advances (smem_flag_publish): a
// plain polling loop, because the waiter sits on a serial chain and has to notice within tens of cycles
// (a suspended mbarrier wait took about a microsecond to resume, measured through a hand-off per 8 steps).
__device__ __forceinline__ bool smem_flag_wait_bounded(uint32_t flag, uint32_t want, uint32_t* err_word, uint32_t code,
                                                       unsigned long long limit_ns) {
  auto peek = [&] {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(flag) : "memory");
    return v;
  };
  if (peek() >= want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  while (peek() < want) {
    if ((++it & 0x3F) == 0) {
      if (global_timer_ns() - t0 > limit_ns || it > (1u << 28)) {
        if (err_word) atomicOr(reinterpret_cast<unsigned int*>(err_word), code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void smem_flag_publish(uint32_t flag, uint32_t value) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(flag), "r"(value) : "memory");
}

// Makes the calling thread's earlier global writes visible to a thread that then sees `value`.
__device__ __forceinline__ void counter_publish(unsigned int* counter, unsigned int value) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(counter), "r"(value) : "memory");
}

// ---- a launch that follows another on the same stream and reads what it wrote
// Launched with launch_dependent(), the second kernel's CTAs may become resident while the first still
// runs - as soon as every CTA of the first has called grid_dependents_may_launch() or exited - and must
// call grid_dependency_wait() before they touch anything the first wrote: it returns when the first grid
// has completed and its writes are visible. This takes the launch latency between the two (4-5 us) off
// pairs of launches that are short themselves. In a kernel launched the ordinary way both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// After a give-up: one shared allowance of `limit_ns` for all of a warp's stages whose loads may
// still be in flight, so that they can land before the CTA's shared memory is released.
__device__ __forceinline__ void mbar_drain(uint32_t bar0, int stages, int s_idx, uint32_t phase,
                                           unsigned long long limit_ns) {
  const uint64_t t0 = global_timer_ns();
  for (int s = 0; s < stages; ++s) {
    const uint64_t used = global_timer_ns() - t0;
    mbar_wait_bounded(bar0 + 8u * s, (s < s_idx) ? (phase ^ 1u) : phase, nullptr, 0u,
                      used < limit_ns ? limit_ns - used : 0ull);
  }
}

// One 2-D TMA tile load into this CTA's shared memory, completion counted in
// bytes on `bar`. x = innermost (column) coordinate, y = row (time) coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tm), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// One 2-D TMA tile store from this CTA's shared memory (bulk async group).
// Rows / columns of the box that fall outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm),
               "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until every committed bulk store of this thread has finished READING
// its shared-memory source (the source may then be overwritten).
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Same, but the most recently committed group may still be reading.
__device__ __forceinline__ void bulk_wait_read_keep1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// Waits until every committed bulk store of this thread has completed.
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

#endif  // __CUDACC__

}  // namespace nsb
