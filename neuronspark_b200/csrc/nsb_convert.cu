// Element-type conversion of a contiguous array (fp32 / bf16 / fp16 in any pairing): widening is
// exact, narrowing rounds to nearest even, as torch's .to() does. The scan entry points stream
// every [T, cols] tensor of one call in one element type; a caller whose tensors differ in type
// (the reference widens each pointer on its own, atomic_ops/parallel_scan.py:223-225) brings them
// to a common one with this kernel instead of a framework op.
#include <algorithm>

#include "nsb_common.cuh"

namespace nsb {
namespace {

template <typename TI, typename TO, int VE>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, long long n) {
  const long long nv = n / VE;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const Vec<TI, VE> a = reinterpret_cast<const Vec<TI, VE>*>(in)[i];
    Vec<TO, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) o.v[j] = Elem<TO>::from_f32(Elem<TI>::to_f32(a.v[j]));
    reinterpret_cast<Vec<TO, VE>*>(out)[i] = o;
  }
  // the ragged tail (n not a multiple of VE)
  for (long long i = nv * VE + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = Elem<TO>::from_f32(Elem<TI>::to_f32(in[i]));
}

template <typename TI, typename TO>
int launch(const void* src, void* dst, long long n, cudaStream_t st) {
  if (reinterpret_cast<uintptr_t>(src) % sizeof(TI) || reinterpret_cast<uintptr_t>(dst) % sizeof(TO))
    return NSB_ERR_INVALID_ARG;
  DeviceInfo dev;
  if (int r = get_device_info(&dev); r != NSB_OK) return r;
  const bool v4 = reinterpret_cast<uintptr_t>(src) % (4 * sizeof(TI)) == 0 &&
                  reinterpret_cast<uintptr_t>(dst) % (4 * sizeof(TO)) == 0;
  const int threads = 256;
  const long long items = v4 ? (n + 3) / 4 : n;
  const int grid = (int)std::max(1LL, std::min((items + threads - 1) / threads, (long long)dev.sm_count * 16));
  if (v4)
    convert_kernel<TI, TO, 4><<<grid, threads, 0, st>>>(static_cast<const TI*>(src), static_cast<TO*>(dst), n);
  else
    convert_kernel<TI, TO, 1><<<grid, threads, 0, st>>>(static_cast<const TI*>(src), static_cast<TO*>(dst), n);
  NSB_CUDA_TRY(cudaGetLastError(), "launch convert_kernel");
  return NSB_OK;
}

template <typename TI>
int from(const void* src, void* dst, long long n, int dst_dtype, cudaStream_t st) {
  switch (dst_dtype) {
    case NSB_F32: return launch<TI, float>(src, dst, n, st);
    case NSB_BF16: return launch<TI, __nv_bfloat16>(src, dst, n, st);
    case NSB_F16: return launch<TI, __half>(src, dst, n, st);
    default: return NSB_ERR_INVALID_ARG;
  }
}

}  // namespace
}  // namespace nsb

extern "C" int nsb_convert(const void* src, void* dst, int64_t n, int src_dtype, int dst_dtype, void* stream) {
  if (n < 0) return NSB_ERR_INVALID_ARG;
  if (n == 0) return NSB_OK;
  if (!src || !dst) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (src_dtype) {
    case NSB_F32: return nsb::from<float>(src, dst, n, dst_dtype, st);
    case NSB_BF16: return nsb::from<__nv_bfloat16>(src, dst, n, dst_dtype, st);
    case NSB_F16: return nsb::from<__half>(src, dst, n, dst_dtype, st);
    default: return NSB_ERR_INVALID_ARG;
  }
}
