// Adaptive surrogate slope on the device.
//
// NeuronSpark's PLIFNode.get_surrogate (atomic_ops/plif_node.py:78-101) sets, before every scan,
//     alpha = clamp(alpha_0 * sigma_0 / max(std(u), 1e-6), 1, 20)
// with `u.std().item()`: a reduction followed by a device-to-host read that stalls the host once
// per scan call. Here the same number is produced into device memory; the backward entry points
// with the _dalpha suffix read it from there, so the host never waits.
//
// Two kernels, both with a fixed shape so that the summation order (and therefore the result) does
// not depend on anything but the data: kBlocks blocks accumulate sum and sum of squares (fp32
// within a 16-byte vector, double across vectors, threads and blocks), one warp finishes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "nsb_common.cuh"

namespace nsb {
namespace {

constexpr int kBlocks = 592;  // 4 per SM of a B200
constexpr int kThreads = 256;

template <typename T>
__global__ void moments_kernel(const T* __restrict__ u, long long n, double* __restrict__ partial) {
  constexpr int VE = 16 / (int)sizeof(T);
  double ds = 0.0, dq = 0.0;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const bool vec = (reinterpret_cast<uintptr_t>(u) & 15u) == 0;
  const long long nvec = vec ? n / VE : 0;
  // four independent 16-byte loads per thread and iteration keep ~64 KB per SM in flight
  constexpr int UN = 4;
  for (long long i0 = tid; i0 < nvec; i0 += nthreads * UN) {
    Vec<T, VE> x[UN];
#pragma unroll
    for (int r = 0; r < UN; ++r) {
      const long long i = i0 + r * nthreads;
      if (i < nvec) x[r] = *reinterpret_cast<const Vec<T, VE>*>(u + i * VE);
    }
#pragma unroll
    for (int r = 0; r < UN; ++r) {
      if (i0 + r * nthreads < nvec) {
        float s = 0.0f, q = 0.0f;
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float f = Elem<T>::to_f32(x[r].v[j]);
          s += f;
          q = fmaf(f, f, q);
        }
        ds += (double)s;
        dq += (double)q;
      }
    }
  }
  for (long long i = nvec * VE + tid; i < n; i += nthreads) {  // tail, or everything when unaligned
    const double f = (double)Elem<T>::to_f32(u[i]);
    ds += f;
    dq += f * f;
  }
  // fixed-order reduction: lanes of a warp, then the warps of the block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ds += __shfl_down_sync(0xffffffffu, ds, o);
    dq += __shfl_down_sync(0xffffffffu, dq, o);
  }
  __shared__ double sh[2][kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sh[0][warp] = ds;
    sh[1][warp] = dq;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0.0, b = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) {
      a += sh[0][w];
      b += sh[1][w];
    }
    partial[2 * blockIdx.x] = a;
    partial[2 * blockIdx.x + 1] = b;
  }
}

// rounds to the storage dtype, as `u.std()` of a low-precision tensor does
__device__ __forceinline__ double round_like(double x, int dtype) {
  if (dtype == NSB_BF16) return (double)__bfloat162float(__float2bfloat16_rn((float)x));
  if (dtype == NSB_F16) return (double)__half2float(__float2half_rn((float)x));
  return (double)(float)x;
}

__global__ void alpha_finalize_kernel(const double* __restrict__ partial, int nparts, long long n, int dtype,
                                      float alpha0, float sigma0, float* __restrict__ alpha_out) {
  const int lane = threadIdx.x;
  double s = 0.0, q = 0.0;
  for (int b = lane; b < nparts; b += 32) {
    s += partial[2 * b];
    q += partial[2 * b + 1];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_down_sync(0xffffffffu, s, o);
    q += __shfl_down_sync(0xffffffffu, q, o);
  }
  if (lane == 0) {
    double sd = 0.0;
    if (n > 1) {
      const double var = (q - s * s / (double)n) / (double)(n - 1);  // unbiased, as torch.std
      sd = var > 0.0 ? sqrt(var) : 0.0;
    }
    sd = round_like(sd, dtype);
    const double floor_ = round_like(1e-6, dtype);
    if (!(sd > floor_)) sd = floor_;
    double a = (double)alpha0 * (double)sigma0 / sd;
    a = a < 1.0 ? 1.0 : (a > 20.0 ? 20.0 : a);
    *alpha_out = (float)a;
  }
}

}  // namespace

// Slope from `nparts` (sum, sum of squares) pairs over n values; used by nsb_surrogate_alpha and by
// the modulated forward scan, which accumulates the moments of u = alpha*I while it streams.
int launch_alpha_finalize(const double* partial, int nparts, long long n, int dtype, float alpha0, float sigma0,
                          float* alpha_out, cudaStream_t st) {
  alpha_finalize_kernel<<<1, 32, 0, st>>>(partial, nparts, n, dtype, alpha0, sigma0, alpha_out);
  NSB_CUDA_TRY(cudaGetLastError(), "launch alpha_finalize_kernel");
  return NSB_OK;
}

}  // namespace nsb

using namespace nsb;

extern "C" int64_t nsb_surrogate_alpha_scratch_doubles(void) { return 2 * kBlocks; }

extern "C" int nsb_surrogate_alpha(const void* u, int64_t n, int dtype, float alpha0, float sigma0,
                                   double* scratch, float* alpha_out, void* stream) {
  if (n < 0 || (dtype != NSB_F32 && dtype != NSB_BF16 && dtype != NSB_F16) || !scratch || !alpha_out ||
      (n > 0 && !u))
    return NSB_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(scratch) & 7u) || (reinterpret_cast<uintptr_t>(alpha_out) & 3u) ||
      (reinterpret_cast<uintptr_t>(u) % dtype_size(dtype)))
    return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NSB_F32: moments_kernel<float><<<kBlocks, kThreads, 0, st>>>(static_cast<const float*>(u), n, scratch); break;
    case NSB_BF16:
      moments_kernel<__nv_bfloat16><<<kBlocks, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(u), n, scratch);
      break;
    default: moments_kernel<__half><<<kBlocks, kThreads, 0, st>>>(static_cast<const __half*>(u), n, scratch); break;
  }
  NSB_CUDA_TRY(cudaGetLastError(), "launch moments_kernel");
  return launch_alpha_finalize(scratch, kBlocks, n, dtype, alpha0, sigma0, alpha_out, st);
}
