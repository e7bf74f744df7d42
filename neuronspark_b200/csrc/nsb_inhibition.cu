// Lateral inhibition (divisive normalisation, = RMSNorm) forward and backward.
//
// out = x * rsqrt(mean(x^2) + eps) * gain over rows of D elements, fp32 math.
// One warp owns one row at a time and strides over the rows of the problem; a
// lane owns the fixed set of channels {lane*VE + 32*VE*i}, so the per-channel
// gain gradient of the backward can be accumulated privately (no atomics):
// each warp keeps a [D] fp32 accumulator row in shared memory, the warps of a
// CTA are summed in a fixed order into one partial row per CTA, and a second
// small kernel sums the partial rows in a fixed order. The result is therefore
// bit-reproducible from run to run.
#include <mutex>

#include "nsb_common.cuh"

namespace nsb {
namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, typename TG, int VE>
__global__ void li_fwd_kernel(const T* __restrict__ x, const TG* __restrict__ gain, T* __restrict__ out,
                              long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv_d = 1.0f / (float)D;
  for (long long r = warp; r < rows; r += nwarps) {
    const T* xr = x + r * D;
    float ss = 0.0f;
    for (int d = lane * VE; d < D; d += 32 * VE) {
      const Vec<T, VE> v = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
#pragma unroll
      for (int j = 0; j < VE; ++j) {
        const float f = Elem<T>::to_f32(v.v[j]);
        ss += f * f;
      }
    }
    ss = warp_sum(ss);
    const float rrms = 1.0f / sqrtf(ss * inv_d + eps);
    T* orow = out + r * D;
    for (int d = lane * VE; d < D; d += 32 * VE) {
      const Vec<T, VE> v = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
      const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
      Vec<T, VE> o;
#pragma unroll
      for (int j = 0; j < VE; ++j)
        o.v[j] = Elem<T>::from_f32(Elem<T>::to_f32(v.v[j]) * rrms * Elem<TG>::to_f32(g.v[j]));
      *reinterpret_cast<Vec<T, VE>*>(orow + d) = o;
    }
  }
}

// Backward, stage 1: g_x for every row, and one partial g_gain row per CTA.
template <typename T, typename TG, int VE>
__global__ void li_bwd_kernel(const T* __restrict__ g_out, const T* __restrict__ x,
                              const TG* __restrict__ gain, T* __restrict__ g_x,
                              float* __restrict__ partial, long long rows, int D, float eps) {
  extern __shared__ float acc_smem[];  // [warps][D]
  grid_dependents_may_launch();  // the reduction of the partial rows may take its places while this runs
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const long long warp = (long long)blockIdx.x * wpc + wib;
  const long long nwarps = (long long)gridDim.x * wpc;
  float* acc = acc_smem + (size_t)wib * D;
  for (int d = lane; d < D; d += 32) acc[d] = 0.0f;
  __syncwarp();
  const float inv_d = 1.0f / (float)D;
  for (long long r = warp; r < rows; r += nwarps) {
    const T* xr = x + r * D;
    const T* gr = g_out + r * D;
    float ss = 0.0f, dot = 0.0f;
    for (int d = lane * VE; d < D; d += 32 * VE) {
      const Vec<T, VE> v = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
      const Vec<T, VE> go = *reinterpret_cast<const Vec<T, VE>*>(gr + d);
      const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
#pragma unroll
      for (int j = 0; j < VE; ++j) {
        const float f = Elem<T>::to_f32(v.v[j]);
        ss += f * f;
        dot += Elem<T>::to_f32(go.v[j]) * Elem<TG>::to_f32(g.v[j]) * f;
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rrms = 1.0f / sqrtf(ss * inv_d + eps);
    // mean(dout*gain*x_hat) = rrms * sum(dout*gain*x) / D
    const float mean_dot = dot * rrms * inv_d;
    T* dxr = g_x + r * D;
    for (int d = lane * VE; d < D; d += 32 * VE) {
      const Vec<T, VE> v = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
      const Vec<T, VE> go = *reinterpret_cast<const Vec<T, VE>*>(gr + d);
      const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
      Vec<T, VE> o;
#pragma unroll
      for (int j = 0; j < VE; ++j) {
        const float xh = Elem<T>::to_f32(v.v[j]) * rrms;
        const float dout = Elem<T>::to_f32(go.v[j]);
        const float dg = dout * Elem<TG>::to_f32(g.v[j]);
        o.v[j] = Elem<T>::from_f32((dg - xh * mean_dot) * rrms);
        acc[d + j] += dout * xh;
      }
      *reinterpret_cast<Vec<T, VE>*>(dxr + d) = o;
    }
  }
  __syncthreads();
  float* prow = partial + (size_t)blockIdx.x * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = 0.0f;
    for (int w = 0; w < wpc; ++w) s += acc_smem[(size_t)w * D + d];
    prow[d] = s;
  }
}

// Register-resident variants for rows of at most 32*VE*NV elements: a lane keeps
// its NV vectors of the row (and of g_out in the backward) in registers, so the
// row is read from memory exactly once instead of once per pass.
template <typename T, typename TG, int VE, int NV>
__global__ void li_fwd_cached_kernel(const T* __restrict__ x, const TG* __restrict__ gain,
                                     T* __restrict__ out, long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const float inv_d = 1.0f / (float)D;
  // The next row of this warp is requested before the current one is reduced and written, so
  // that a warp always has loads in flight (a row is only 1.5 KB at D = 768).
  Vec<T, VE> xv[NV], xn[NV];
  auto load_row = [&](long long r, Vec<T, VE> (&dst)[NV]) {
    const T* xr = x + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) dst[i] = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
    }
  };
  if (warp < rows) load_row(warp, xv);
  for (long long r = warp; r < rows; r += nwarps) {
    if (r + nwarps < rows) load_row(r + nwarps, xn);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) {
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float f = Elem<T>::to_f32(xv[i].v[j]);
          ss += f * f;
        }
      }
    }
    ss = warp_sum(ss);
    const float rrms = 1.0f / sqrtf(ss * inv_d + eps);
    T* orow = out + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);  // stays in L1
        Vec<T, VE> o;
#pragma unroll
        for (int j = 0; j < VE; ++j)
          o.v[j] = Elem<T>::from_f32(Elem<T>::to_f32(xv[i].v[j]) * rrms * Elem<TG>::to_f32(g.v[j]));
        *reinterpret_cast<Vec<T, VE>*>(orow + d) = o;
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) xv[i] = xn[i];
  }
}

template <typename T, typename TG, int VE, int NV>
__global__ void __launch_bounds__(kWarpsPerCta * 32, NV <= 3 ? 2 : 1) li_bwd_cached_kernel(const T* __restrict__ g_out, const T* __restrict__ x,
                                     const TG* __restrict__ gain, T* __restrict__ g_x,
                                     float* __restrict__ partial, long long rows, int D, float eps) {
  extern __shared__ float acc_smem[];  // [warps][D], summed over the CTA's warps at the end
  grid_dependents_may_launch();
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int wpc = blockDim.x >> 5;
  const long long warp = (long long)blockIdx.x * wpc + wib;
  const long long nwarps = (long long)gridDim.x * wpc;
  const float inv_d = 1.0f / (float)D;
  float acc[NV][VE];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < VE; ++j) acc[i][j] = 0.0f;
  // next row requested before the current one is reduced (see the forward kernel)
  Vec<T, VE> xv[NV], gv[NV], xn[NV], gn[NV];
  auto load_row = [&](long long r, Vec<T, VE> (&dx)[NV], Vec<T, VE> (&dg)[NV]) {
    const T* xr = x + r * D;
    const T* gr = g_out + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) {
        dx[i] = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
        dg[i] = *reinterpret_cast<const Vec<T, VE>*>(gr + d);
      }
    }
  };
  if (warp < rows) load_row(warp, xv, gv);
  for (long long r = warp; r < rows; r += nwarps) {
    if (r + nwarps < rows) load_row(r + nwarps, xn, gn);
    float ss = 0.0f, dot = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);  // stays in L1
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float f = Elem<T>::to_f32(xv[i].v[j]);
          ss += f * f;
          dot += Elem<T>::to_f32(gv[i].v[j]) * Elem<TG>::to_f32(g.v[j]) * f;
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float rrms = 1.0f / sqrtf(ss * inv_d + eps);
    const float mean_dot = dot * rrms * inv_d;
    T* dxr = g_x + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = (lane + 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
        Vec<T, VE> o;
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float xh = Elem<T>::to_f32(xv[i].v[j]) * rrms;
          const float dout = Elem<T>::to_f32(gv[i].v[j]);
          o.v[j] = Elem<T>::from_f32((dout * Elem<TG>::to_f32(g.v[j]) - xh * mean_dot) * rrms);
          acc[i][j] += dout * xh;
        }
        *reinterpret_cast<Vec<T, VE>*>(dxr + d) = o;
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xv[i] = xn[i];
      gv[i] = gn[i];
    }
  }
  float* mine = acc_smem + (size_t)wib * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = (lane + 32 * i) * VE;
    if (d < D) {
#pragma unroll
      for (int j = 0; j < VE; ++j) mine[d + j] = acc[i][j];
    }
  }
  __syncthreads();
  float* prow = partial + (size_t)blockIdx.x * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = 0.0f;
    for (int w = 0; w < wpc; ++w) s += acc_smem[(size_t)w * D + d];
    prow[d] = s;
  }
}

constexpr int kCacheVecs = 8;  // vectors of 16 bytes a lane keeps per row in the cached kernels

// Wide rows (more than a warp can keep: 2048 elements of 16 bits, 1024 of 32): a CTA of 8 warps
// owns a row at a time, thread t keeps the 16-byte vectors t, t+256, ... (NV of them) of the row in
// registers, so the row is still read once. The row sums go through shared memory in a fixed order
// (warp sums, then the 8 of them), two buffers alternating between rows so that one barrier per
// row is enough. A thread owns the same channels in every row: the backward's gain gradient is
// accumulated in registers and written as this CTA's partial row without any reduction.
constexpr int kWideWarps = 8;

template <int NSUM>
__device__ __forceinline__ void block_sums(float (&v)[NSUM], float (*buf)[kWideWarps], int lane, int wib) {
#pragma unroll
  for (int q = 0; q < NSUM; ++q) {
    v[q] = warp_sum(v[q]);
    if (lane == 0) buf[q][wib] = v[q];
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < NSUM; ++q) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < kWideWarps; ++w) s += buf[q][w];
    v[q] = s;
  }
}

template <typename T, typename TG, int VE, int NV>
__global__ void __launch_bounds__(kWideWarps * 32)
li_fwd_wide_kernel(const T* __restrict__ x, const TG* __restrict__ gain, T* __restrict__ out, long long rows,
                   int D, float eps) {
  __shared__ float sums[2][1][kWideWarps];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const float inv_d = 1.0f / (float)D;
  Vec<T, VE> xv[NV], xn[NV];
  auto load_row = [&](long long r, Vec<T, VE> (&dst)[NV]) {
    const T* xr = x + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) dst[i] = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
    }
  };
  if (blockIdx.x < rows) load_row(blockIdx.x, xv);
  int par = 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x, par ^= 1) {
    if (r + gridDim.x < rows) load_row(r + gridDim.x, xn);
    float ss[1] = {0.0f};
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) {
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float f = Elem<T>::to_f32(xv[i].v[j]);
          ss[0] += f * f;
        }
      }
    }
    block_sums<1>(ss, sums[par], lane, wib);
    const float rrms = 1.0f / sqrtf(ss[0] * inv_d + eps);
    T* orow = out + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
        Vec<T, VE> o;
#pragma unroll
        for (int j = 0; j < VE; ++j)
          o.v[j] = Elem<T>::from_f32(Elem<T>::to_f32(xv[i].v[j]) * rrms * Elem<TG>::to_f32(g.v[j]));
        *reinterpret_cast<Vec<T, VE>*>(orow + d) = o;
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) xv[i] = xn[i];
  }
}

template <typename T, typename TG, int VE, int NV>
__global__ void __launch_bounds__(kWideWarps * 32)
li_bwd_wide_kernel(const T* __restrict__ g_out, const T* __restrict__ x, const TG* __restrict__ gain,
                   T* __restrict__ g_x, float* __restrict__ partial, long long rows, int D, float eps) {
  __shared__ float sums[2][2][kWideWarps];
  grid_dependents_may_launch();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const float inv_d = 1.0f / (float)D;
  float acc[NV][VE];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < VE; ++j) acc[i][j] = 0.0f;
  Vec<T, VE> xv[NV], gv[NV], xn[NV], gn[NV];
  auto load_row = [&](long long r, Vec<T, VE> (&dx)[NV], Vec<T, VE> (&dg)[NV]) {
    const T* xr = x + r * D;
    const T* gr = g_out + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) {
        dx[i] = *reinterpret_cast<const Vec<T, VE>*>(xr + d);
        dg[i] = *reinterpret_cast<const Vec<T, VE>*>(gr + d);
      }
    }
  };
  if (blockIdx.x < rows) load_row(blockIdx.x, xv, gv);
  int par = 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x, par ^= 1) {
    if (r + gridDim.x < rows) load_row(r + gridDim.x, xn, gn);
    float sd[2] = {0.0f, 0.0f};  // sum x^2, sum g_out*gain*x
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float f = Elem<T>::to_f32(xv[i].v[j]);
          sd[0] += f * f;
          sd[1] += Elem<T>::to_f32(gv[i].v[j]) * Elem<TG>::to_f32(g.v[j]) * f;
        }
      }
    }
    block_sums<2>(sd, sums[par], lane, wib);
    const float rrms = 1.0f / sqrtf(sd[0] * inv_d + eps);
    const float mean_dot = sd[1] * rrms * inv_d;
    T* dxr = g_x + r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
      if (d < D) {
        const Vec<TG, VE> g = *reinterpret_cast<const Vec<TG, VE>*>(gain + d);
        Vec<T, VE> o;
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          const float xh = Elem<T>::to_f32(xv[i].v[j]) * rrms;
          const float dout = Elem<T>::to_f32(gv[i].v[j]);
          o.v[j] = Elem<T>::from_f32((dout * Elem<TG>::to_f32(g.v[j]) - xh * mean_dot) * rrms);
          acc[i][j] += dout * xh;
        }
        *reinterpret_cast<Vec<T, VE>*>(dxr + d) = o;
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      xv[i] = xn[i];
      gv[i] = gn[i];
    }
  }
  float* prow = partial + (size_t)blockIdx.x * D;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = ((int)threadIdx.x + kWideWarps * 32 * i) * VE;
    if (d < D) {
#pragma unroll
      for (int j = 0; j < VE; ++j) prow[d + j] = acc[i][j];
    }
  }
}

constexpr int kWideVecs = 8;  // 16-byte vectors a thread of the wide kernels keeps per row at most

// Backward, stage 2: g_gain[d] = sum over the partial rows. A block covers 32 channels with
// 8 groups of threads; group g adds rows g, g+8, g+16, ... and the 8 group sums are then
// added in a fixed order, so the result does not depend on scheduling.
__global__ void li_bwd_reduce_kernel(const float* __restrict__ partial, float* __restrict__ g_gain,
                                     int nparts, int D) {
  __shared__ float part[8][33];
  const int c = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int d = blockIdx.x * 32 + c;
  grid_dependency_wait();  // the partial rows are the launch before's
  float s = 0.0f;
  if (d < D)
    for (int p = g; p < nparts; p += 8) s += partial[(size_t)p * D + d];
  part[g][c] = s;
  __syncthreads();
  if (g == 0 && d < D) {
    float t = 0.0f;
#pragma unroll
    for (int q = 0; q < 8; ++q) t += part[q][c];
    g_gain[d] = t;
  }
}

int bwd_grid(long long rows, int D, int* wpc_out) {
  DeviceInfo dev;
  if (get_device_info(&dev) != NSB_OK) return 0;
  int wpc = kWarpsPerCta;
  while (wpc > 1 && (size_t)wpc * D * sizeof(float) > (size_t)dev.max_smem_optin) wpc >>= 1;
  if ((size_t)wpc * D * sizeof(float) > (size_t)dev.max_smem_optin) return 0;
  long long g = (rows + wpc - 1) / wpc;
  const long long cap = (long long)dev.sm_count * 2;  // (3 per SM measured slower: 89 against 83 us at 65536 x 768, 93 against 72 us at 8192 x 6144)
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  if (wpc_out) *wpc_out = wpc;
  return (int)g;
}

bool dtype_ok(int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; }

template <typename F>
int with_dtype(int dtype, F&& f) {
  switch (dtype) {
    case NSB_F32: return f(float{});
    case NSB_BF16: return f(__nv_bfloat16{});
    case NSB_F16: return f(__half{});
    default: return NSB_ERR_INVALID_ARG;
  }
}

template <typename T, typename TG>
bool can_vec(int ve, long long D, std::initializer_list<const void*> tp, const void* gp) {
  if (D % ve) return false;
  for (const void* p : tp)
    if (reinterpret_cast<uintptr_t>(p) % (sizeof(T) * ve)) return false;
  return reinterpret_cast<uintptr_t>(gp) % (sizeof(TG) * ve) == 0;
}


// Launches both backward stages with the given partial-sum buffer and grid; shared by the
// entry point that takes scratch from the caller and the one with library-resident scratch,
// so that both run the same kernels and give bit-identical results for an equal grid.
template <typename T, typename TG>
int li_bwd_launch(const void* g_out, const void* x, const void* gain, void* g_x, float* g_gain,
                  float* partial, long long rows, long long D, float eps, int grid, int wpc,
                  cudaStream_t st) {
  if (!can_vec<T, TG>(1, D, {g_out, x, g_x}, gain)) return NSB_ERR_INVALID_ARG;
  const size_t smem = (size_t)wpc * D * sizeof(float);
  const T* gop = static_cast<const T*>(g_out);
  const T* xp = static_cast<const T*>(x);
  const TG* gp = static_cast<const TG*>(gain);
  T* gxp = static_cast<T*>(g_x);
#define NSB_LI_BWD(KERNEL_)                                                                       \
  {                                                                                               \
    auto k = KERNEL_;                                                                             \
    NSB_CUDA_TRY(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), \
                 "cudaFuncSetAttribute(li_bwd)");                                                 \
    k<<<grid, wpc * 32, smem, st>>>(gop, xp, gp, gxp, partial, rows, (int)D, eps);                \
  }
  constexpr int VMAX = 16 / (int)sizeof(T);  // elements in a 16-byte vector
  if (can_vec<T, TG>(VMAX, D, {g_out, x, g_x}, gain) && sizeof(TG) * VMAX <= 32 &&
      D <= 32 * VMAX * kCacheVecs) {
    if (D <= 32 * VMAX * 2)
      NSB_LI_BWD((li_bwd_cached_kernel<T, TG, VMAX, 2>))
    else if (D <= 32 * VMAX * 3)  // (768 channels of 16 bits: few enough registers for two CTAs per SM)
      NSB_LI_BWD((li_bwd_cached_kernel<T, TG, VMAX, 3>))
    else if (D <= 32 * VMAX * 4)
      NSB_LI_BWD((li_bwd_cached_kernel<T, TG, VMAX, 4>))
    else
      NSB_LI_BWD((li_bwd_cached_kernel<T, TG, VMAX, kCacheVecs>))
  } else if (can_vec<T, TG>(VMAX, D, {g_out, x, g_x}, gain) && sizeof(TG) * VMAX <= 32 &&
             D <= kWideWarps * 32 * VMAX * kWideVecs) {
    const long long per = (long long)kWideWarps * 32 * VMAX;
    const int nv = (int)((D + per - 1) / per);
#define NSB_LI_BWD_WIDE(NV_)                                                                             \
  li_bwd_wide_kernel<T, TG, VMAX, NV_><<<grid, kWideWarps * 32, 0, st>>>(gop, xp, gp, gxp, partial, rows, \
                                                                          (int)D, eps);
    if (nv <= 2) { NSB_LI_BWD_WIDE(2) }
    else if (nv <= 3) { NSB_LI_BWD_WIDE(3) }
    else if (nv <= 4) { NSB_LI_BWD_WIDE(4) }
    else if (nv <= 6) { NSB_LI_BWD_WIDE(6) }
    else { NSB_LI_BWD_WIDE(8) }
#undef NSB_LI_BWD_WIDE
  } else if (can_vec<T, TG>(4, D, {g_out, x, g_x}, gain))
    NSB_LI_BWD((li_bwd_kernel<T, TG, 4>))
  else if (can_vec<T, TG>(2, D, {g_out, x, g_x}, gain))
    NSB_LI_BWD((li_bwd_kernel<T, TG, 2>))
  else
    NSB_LI_BWD((li_bwd_kernel<T, TG, 1>))
#undef NSB_LI_BWD
  NSB_CUDA_TRY(cudaGetLastError(), "launch li_bwd_kernel");
  NSB_CUDA_TRY(launch_dependent(li_bwd_reduce_kernel, dim3((unsigned)((D + 31) / 32)), dim3(256), 0, st, partial, g_gain,
                                grid, (int)D),
               "launch li_bwd_reduce_kernel");
  return NSB_OK;
}

}  // namespace
}  // namespace nsb

using namespace nsb;

extern "C" {

int nsb_lateral_inhibition_fwd(const void* x, const void* gain, void* out, int64_t rows, int64_t D,
                               float eps, int dtype, int gain_dtype, void* stream) {
  if (rows < 0 || D < 0 || D >= (1ll << 31) || !dtype_ok(dtype) || !dtype_ok(gain_dtype))
    return NSB_ERR_INVALID_ARG;
  if (rows == 0 || D == 0) return NSB_OK;
  if (!x || !gain || !out) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceInfo dev;
  int r = get_device_info(&dev);
  if (r != NSB_OK) return r;
  long long grid = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  grid = std::min<long long>(grid, (long long)dev.sm_count * 8);
  return with_dtype(dtype, [&](auto t) {
    using T = decltype(t);
    return with_dtype(gain_dtype, [&](auto tg) {
      using TG = decltype(tg);
      if (!can_vec<T, TG>(1, D, {x, out}, gain)) return NSB_ERR_INVALID_ARG;
      const T* xp = static_cast<const T*>(x);
      const TG* gp = static_cast<const TG*>(gain);
      T* op = static_cast<T*>(out);
      constexpr int VMAX = 16 / (int)sizeof(T);  // elements in a 16-byte vector
      if (can_vec<T, TG>(VMAX, D, {x, out}, gain) && sizeof(TG) * VMAX <= 32 && D <= 32 * VMAX * kCacheVecs) {
        const int th = kWarpsPerCta * 32;
        // The warps stride over the rows, so every CTA of the grid does the same amount of work: no more
        // CTAs than are resident at once, or the ones that start late make the launch as long as two rounds.
        auto launch = [&](auto kern) {
          int per_sm = 0;
          if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, th, 0) != cudaSuccess || per_sm < 1)
            per_sm = 4;
          const int g = (int)std::min<long long>(grid, (long long)per_sm * dev.sm_count);
          kern<<<g, th, 0, st>>>(xp, gp, op, rows, (int)D, eps);
        };
        if (D <= 32 * VMAX * 2)
          launch(li_fwd_cached_kernel<T, TG, VMAX, 2>);
        else if (D <= 32 * VMAX * 3)  // (768 channels of 16 bits)
          launch(li_fwd_cached_kernel<T, TG, VMAX, 3>);
        else if (D <= 32 * VMAX * 4)
          launch(li_fwd_cached_kernel<T, TG, VMAX, 4>);
        else
          launch(li_fwd_cached_kernel<T, TG, VMAX, kCacheVecs>);
      } else if (can_vec<T, TG>(VMAX, D, {x, out}, gain) && sizeof(TG) * VMAX <= 32 &&
                 D <= kWideWarps * 32 * VMAX * kWideVecs) {
        const long long per = (long long)kWideWarps * 32 * VMAX;
        const int nv = (int)((D + per - 1) / per);
        const int g = (int)std::min<long long>(rows, (long long)dev.sm_count * 4);  // a CTA per row at a time
#define NSB_LI_FWD_WIDE(NV_) \
  li_fwd_wide_kernel<T, TG, VMAX, NV_><<<g, kWideWarps * 32, 0, st>>>(xp, gp, op, rows, (int)D, eps);
        if (nv <= 2) { NSB_LI_FWD_WIDE(2) }
        else if (nv <= 3) { NSB_LI_FWD_WIDE(3) }
        else if (nv <= 4) { NSB_LI_FWD_WIDE(4) }
        else if (nv <= 6) { NSB_LI_FWD_WIDE(6) }
        else { NSB_LI_FWD_WIDE(8) }
#undef NSB_LI_FWD_WIDE
      } else if (can_vec<T, TG>(4, D, {x, out}, gain))
        li_fwd_kernel<T, TG, 4><<<(int)grid, kWarpsPerCta * 32, 0, st>>>(xp, gp, op, rows, (int)D, eps);
      else if (can_vec<T, TG>(2, D, {x, out}, gain))
        li_fwd_kernel<T, TG, 2><<<(int)grid, kWarpsPerCta * 32, 0, st>>>(xp, gp, op, rows, (int)D, eps);
      else
        li_fwd_kernel<T, TG, 1><<<(int)grid, kWarpsPerCta * 32, 0, st>>>(xp, gp, op, rows, (int)D, eps);
      NSB_CUDA_TRY(cudaGetLastError(), "launch li_fwd_kernel");
      return NSB_OK;
    });
  });
}

int64_t nsb_li_bwd_scratch_floats(int64_t rows, int64_t D) {
  if (rows <= 0 || D <= 0 || D >= (1ll << 31)) return 0;
  const int g = bwd_grid(rows, (int)D, nullptr);
  return (int64_t)g * D;
}

int nsb_lateral_inhibition_bwd(const void* g_out, const void* x, const void* gain, void* g_x,
                               float* g_gain, float* partial, int64_t rows, int64_t D, float eps,
                               int dtype, int gain_dtype, void* stream) {
  if (rows < 0 || D < 0 || D >= (1ll << 31) || !dtype_ok(dtype) || !dtype_ok(gain_dtype))
    return NSB_ERR_INVALID_ARG;
  if (D == 0) return NSB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!g_gain || (reinterpret_cast<uintptr_t>(g_gain) & 3u)) return NSB_ERR_INVALID_ARG;
  if (rows == 0) {
    NSB_CUDA_TRY(cudaMemsetAsync(g_gain, 0, sizeof(float) * D, st), "memset g_gain");
    return NSB_OK;
  }
  if (!g_out || !x || !gain || !g_x || !partial || (reinterpret_cast<uintptr_t>(partial) & 3u))
    return NSB_ERR_INVALID_ARG;
  int wpc = 0;
  const int grid = bwd_grid(rows, (int)D, &wpc);
  if (grid == 0) return NSB_ERR_TOO_LARGE;
  return with_dtype(dtype, [&](auto t) {
    using T = decltype(t);
    return with_dtype(gain_dtype, [&](auto tg) {
      using TG = decltype(tg);
      return li_bwd_launch<T, TG>(g_out, x, gain, g_x, g_gain, partial, rows, D, eps, grid, wpc, st);
    });
  });
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Backward without any caller-provided or allocated scratch.
//
// Some hosts of this library may not allocate device memory at the point
// where they need the normaliser's backward: an inference/training server
// that handed the whole device to its own memory pool at start-up, a plugin
// that is only ever given input and output buffers, or a latency-critical
// loop in which cudaMalloc/cudaFree are banned because they synchronise the
// device. For them the per-CTA partial sums of grad_gain live in a fixed array
// that is part of the library image: kLiStaticFloats floats (2 MiB) of device
// memory on every GPU that loads the library, held until the process exits.
// ---------------------------------------------------------------------------
namespace nsb {
namespace {

constexpr long long kLiStaticFloats = 1LL << 19;  // 524 288 floats = 2 MiB
static __device__ __align__(256) float g_li_static_partial[kLiStaticFloats];

// In host code the name of a __device__ array is only a handle, not a device
// address; the address each device gave the array is looked up once per device.
std::mutex g_li_static_mu;
float* g_li_static_ptr[64] = {};

int li_static_scratch(float** out) {
  int dev = 0;
  NSB_CUDA_TRY(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= 64) return NSB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_li_static_mu);
  if (!g_li_static_ptr[dev]) {
    void* p = nullptr;
    NSB_CUDA_TRY(cudaGetSymbolAddress(&p, g_li_static_partial), "cudaGetSymbolAddress(li scratch)");
    if (!p) return NSB_ERR_CUDA;
    g_li_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_li_static_ptr[dev];
  return NSB_OK;
}

}  // namespace
}  // namespace nsb

extern "C" int nsb_lateral_inhibition_bwd_static(const void* g_out, const void* x, const void* gain,
                                                 void* g_x, float* g_gain, int64_t rows, int64_t D,
                                                 float eps, int dtype, int gain_dtype, void* stream) {
  if (rows < 0 || D < 0 || D >= (1ll << 31) || !dtype_ok(dtype) || !dtype_ok(gain_dtype))
    return NSB_ERR_INVALID_ARG;
  if (D == 0) return NSB_OK;
  if (D > kLiStaticFloats) return NSB_ERR_TOO_LARGE;  // not even one partial row fits
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!g_gain || (reinterpret_cast<uintptr_t>(g_gain) & 3u)) return NSB_ERR_INVALID_ARG;
  if (rows == 0) {
    NSB_CUDA_TRY(cudaMemsetAsync(g_gain, 0, sizeof(float) * D, st), "memset g_gain");
    return NSB_OK;
  }
  if (!g_out || !x || !gain || !g_x) return NSB_ERR_INVALID_ARG;
  float* partial = nullptr;
  int r = li_static_scratch(&partial);
  if (r != NSB_OK) return r;
  int wpc = 0;
  int grid = bwd_grid(rows, (int)D, &wpc);
  if (grid == 0) return NSB_ERR_TOO_LARGE;
  // one partial row of D floats per CTA has to fit the fixed array: use fewer CTAs if need be
  grid = (int)std::min<long long>(grid, kLiStaticFloats / D);
  return with_dtype(dtype, [&](auto t) {
    using T = decltype(t);
    return with_dtype(gain_dtype, [&](auto tg) {
      using TG = decltype(tg);
      return li_bwd_launch<T, TG>(g_out, x, gain, g_x, g_gain, partial, rows, D, eps, grid, wpc, st);
    });
  });
}
