// Mixture-of-experts output combine: out[n, d] = shared[n, d] + sum_e experts[e, n, d] * w[n, e]
// and its backward (atomic_ops/moe_kernels.py:35-224).
//
// Pure streaming. Forward: one thread per VE consecutive channels of a row. Backward: one warp
// per row; for every expert it streams that expert's row once, writes grad_expert = g * w and
// reduces g . expert to grad_w[n, e] in the same pass (the reference runs two kernels and reads
// the gradient and the experts twice); the gradient row is re-read per expert from L1/L2, not DRAM.
// grad_shared is the incoming gradient itself, as in the reference.
#include "nsb_common.cuh"

namespace nsb {
namespace {

// EC > 0: the number of experts is the compile-time EC (all of a thread's loads are issued
// before the first use); EC == 0: any E.
template <typename T, int VE, int EC>
__global__ void moe_combine_fwd_kernel(const T* __restrict__ shared, const T* __restrict__ experts,
                                       const float* __restrict__ w, T* __restrict__ out, long long N,
                                       long long D, int E_rt) {
  const int E = EC > 0 ? EC : E_rt;
  const long long dv = D / VE;
  const long long total = N * dv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long n = idx / dv, d = (idx % dv) * VE;
    const Vec<T, VE> s = *reinterpret_cast<const Vec<T, VE>*>(shared + n * D + d);
    float acc[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) acc[j] = Elem<T>::to_f32(s.v[j]);
    if constexpr (EC > 0) {
      Vec<T, VE> x[EC];
      float we[EC];
#pragma unroll
      for (int e = 0; e < EC; ++e) {
        we[e] = w[n * EC + e];
        x[e] = *reinterpret_cast<const Vec<T, VE>*>(experts + ((long long)e * N + n) * D + d);
      }
#pragma unroll
      for (int e = 0; e < EC; ++e)
#pragma unroll
        for (int j = 0; j < VE; ++j) acc[j] = fmaf(Elem<T>::to_f32(x[e].v[j]), we[e], acc[j]);
    } else {
#pragma unroll 4
      for (int e = 0; e < E; ++e) {
        const float we = w[n * E + e];
        const Vec<T, VE> x = *reinterpret_cast<const Vec<T, VE>*>(experts + ((long long)e * N + n) * D + d);
#pragma unroll
        for (int j = 0; j < VE; ++j) acc[j] = fmaf(Elem<T>::to_f32(x.v[j]), we, acc[j]);
      }
    }
    Vec<T, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) o.v[j] = Elem<T>::from_f32(acc[j]);
    *reinterpret_cast<Vec<T, VE>*>(out + n * D + d) = o;
  }
}

template <typename T, int VE>
__global__ void moe_combine_bwd_kernel(const T* __restrict__ g_out, const T* __restrict__ experts,
                                       const float* __restrict__ w, T* __restrict__ g_experts,
                                       float* __restrict__ g_w, long long N, long long D, int E) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long n = warp; n < N; n += nwarps) {
    for (int e = 0; e < E; ++e) {
      const float we = w[n * E + e];
      const long long row = ((long long)e * N + n) * D;
      float dot = 0.0f;
      for (long long d = (long long)lane * VE; d < D; d += 32 * VE) {
        const Vec<T, VE> g = *reinterpret_cast<const Vec<T, VE>*>(g_out + n * D + d);
        Vec<T, VE> ge;
        if (g_w) {
          const Vec<T, VE> x = *reinterpret_cast<const Vec<T, VE>*>(experts + row + d);
#pragma unroll
          for (int j = 0; j < VE; ++j) dot = fmaf(Elem<T>::to_f32(g.v[j]), Elem<T>::to_f32(x.v[j]), dot);
        }
        if (g_experts) {
#pragma unroll
          for (int j = 0; j < VE; ++j) ge.v[j] = Elem<T>::from_f32(Elem<T>::to_f32(g.v[j]) * we);
          *reinterpret_cast<Vec<T, VE>*>(g_experts + row + d) = ge;
        }
      }
      if (g_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) g_w[n * E + e] = dot;
      }
    }
  }
}

template <typename T>
int pick_ve(long long D, std::initializer_list<const void*> ptrs) {
  for (int ve = 16 / (int)sizeof(T); ve > 1; ve >>= 1) {
    bool ok = D % ve == 0;
    for (const void* p : ptrs) ok = ok && reinterpret_cast<uintptr_t>(p) % (sizeof(T) * ve) == 0;
    if (ok) return ve;
  }
  return 1;
}

template <typename T>
int moe_fwd(const void* shared, const void* experts, const float* w, void* out, long long N, long long D, int E,
            cudaStream_t st) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  const int ve = pick_ve<T>(D, {shared, experts, out});
  const long long items = N * (D / ve);
  const int threads = 256;
  const int blocks = (int)std::max<long long>(1, std::min<long long>((items + threads - 1) / threads,
                                                                     (long long)dev.sm_count * 16));
#define NSB_GO_E(VE_, EC_)                                                                               \
  moe_combine_fwd_kernel<T, VE_, EC_><<<blocks, threads, 0, st>>>(static_cast<const T*>(shared),         \
                                                                  static_cast<const T*>(experts), w,     \
                                                                  static_cast<T*>(out), N, D, E)
#define NSB_GO(VE_)                                                                                      \
  do {                                                                                                   \
    if (E == 2) NSB_GO_E(VE_, 2);                                                                        \
    else if (E == 4) NSB_GO_E(VE_, 4);                                                                   \
    else if (E == 8) NSB_GO_E(VE_, 8);                                                                   \
    else NSB_GO_E(VE_, 0);                                                                               \
  } while (0)
  switch (ve) {
    case 8: NSB_GO((sizeof(T) == 2 ? 8 : 1)); break;
    case 4: NSB_GO(4); break;
    case 2: NSB_GO(2); break;
    default: NSB_GO(1); break;
  }
#undef NSB_GO
#undef NSB_GO_E
  NSB_CUDA_TRY(cudaGetLastError(), "launch moe_combine_fwd_kernel");
  return NSB_OK;
}

template <typename T>
int moe_bwd(const void* g_out, const void* experts, const float* w, void* g_experts, float* g_w, long long N,
            long long D, int E, cudaStream_t st) {
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  const int ve = pick_ve<T>(D, {g_out, experts, g_experts});
  const int threads = 256;  // 8 rows per CTA
  const int blocks = (int)std::max<long long>(1, std::min<long long>((N + 7) / 8, (long long)dev.sm_count * 8));
#define NSB_GO(VE_)                                                                                      \
  moe_combine_bwd_kernel<T, VE_><<<blocks, threads, 0, st>>>(static_cast<const T*>(g_out),               \
                                                             static_cast<const T*>(experts), w,          \
                                                             static_cast<T*>(g_experts), g_w, N, D, E)
  switch (ve) {
    case 8: NSB_GO((sizeof(T) == 2 ? 8 : 1)); break;
    case 4: NSB_GO(4); break;
    case 2: NSB_GO(2); break;
    default: NSB_GO(1); break;
  }
#undef NSB_GO
  NSB_CUDA_TRY(cudaGetLastError(), "launch moe_combine_bwd_kernel");
  return NSB_OK;
}

bool ok_dtype(int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; }

}  // namespace
}  // namespace nsb

using namespace nsb;

extern "C" int nsb_moe_combine_fwd(const void* shared, const void* experts, const float* weights, void* out,
                                   int64_t N, int64_t D, int E, int dtype, void* stream) {
  if (N < 0 || D < 0 || E < 0 || !ok_dtype(dtype)) return NSB_ERR_INVALID_ARG;
  if (N * D == 0) return NSB_OK;
  if (!shared || !out || (E > 0 && (!experts || !weights))) return NSB_ERR_INVALID_ARG;
  const size_t es = dtype_size(dtype);
  for (const void* p : {shared, experts, (const void*)out})
    if (reinterpret_cast<uintptr_t>(p) % es) return NSB_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(weights) & 3u) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NSB_F32: return moe_fwd<float>(shared, experts, weights, out, N, D, E, st);
    case NSB_BF16: return moe_fwd<__nv_bfloat16>(shared, experts, weights, out, N, D, E, st);
    default: return moe_fwd<__half>(shared, experts, weights, out, N, D, E, st);
  }
}

extern "C" int nsb_moe_combine_bwd(const void* g_out, const void* experts, const float* weights,
                                   void* g_experts, float* g_weights, int64_t N, int64_t D, int E, int dtype,
                                   void* stream) {
  if (N < 0 || D < 0 || E < 0 || !ok_dtype(dtype)) return NSB_ERR_INVALID_ARG;
  if (N * E == 0) return NSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (D == 0) {
    if (g_weights) NSB_CUDA_TRY(cudaMemsetAsync(g_weights, 0, sizeof(float) * N * E, st), "memset grad weights");
    return NSB_OK;
  }
  if (!g_out || !weights || (g_weights && !experts)) return NSB_ERR_INVALID_ARG;
  if (!g_experts && !g_weights) return NSB_OK;
  const size_t es = dtype_size(dtype);
  for (const void* p : {g_out, experts, (const void*)g_experts})
    if (reinterpret_cast<uintptr_t>(p) % es) return NSB_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(weights) & 3u) || (reinterpret_cast<uintptr_t>(g_weights) & 3u))
    return NSB_ERR_INVALID_ARG;
  switch (dtype) {
    case NSB_F32: return moe_bwd<float>(g_out, experts, weights, g_experts, g_weights, N, D, E, st);
    case NSB_BF16: return moe_bwd<__nv_bfloat16>(g_out, experts, weights, g_experts, g_weights, N, D, E, st);
    default: return moe_bwd<__half>(g_out, experts, weights, g_experts, g_weights, N, D, E, st);
  }
}
