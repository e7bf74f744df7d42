// FP16 boundary codec kernels: encode, decode (forward / backward), binary
// residual and the straight-through encode backward.
//
// Frames are [S*16, B, D] (frame s*16+k = bit 15-k of the IEEE half pattern of
// token s: sign, E4..E0, M9..M0), values are [B, S, D]. One thread owns VE
// consecutive channels of one (b, s) token (VE up to 16 bytes' worth); a warp therefore touches 32*VE
// consecutive elements of each of the 16 frame rows, so every access is a full
// coalesced line. The kernels are pure streaming: the 16 frame reads (or
// writes) of a thread are independent and all in flight together.
#include "nsb_common.cuh"
#include "nsb_codec.cuh"

namespace nsb {
namespace {

using codec::decode16;
using codec::half_bits_clamped;
using codec::round_through_bf16;
using codec::residual_half_bits;

template <typename TI, typename TO, int VE>
__global__ void encode_kernel(const TI* __restrict__ values, TO* __restrict__ frames, long long B,
                              long long S, long long D) {
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const Vec<TI, VE> in = *reinterpret_cast<const Vec<TI, VE>*>(values + (b * S + s) * D + d);
    uint32_t h[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) h[j] = half_bits_clamped(Elem<TI>::to_f32(in.v[j]));
    TO* out = frames + (s * 16 * B + b) * D + d;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      Vec<TO, VE> o;
#pragma unroll
      for (int j = 0; j < VE; ++j) o.v[j] = ((h[j] >> (15 - k)) & 1u) ? Elem<TO>::one() : Elem<TO>::zero();
      *reinterpret_cast<Vec<TO, VE>*>(out + k * frame_stride) = o;
    }
  }
}

template <typename T, int VE>
__global__ void decode_fwd_kernel(const T* __restrict__ frames, T* __restrict__ values, long long B,
                                  long long S, long long D) {
  constexpr bool EMU = Elem<T>::kDtype == NSB_BF16;
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const T* in = frames + (s * 16 * B + b) * D + d;
    Vec<T, VE> f[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) f[k] = *reinterpret_cast<const Vec<T, VE>*>(in + k * frame_stride);
    Vec<T, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      float bit[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) bit[k] = Elem<T>::to_f32(f[k].v[j]);
      o.v[j] = Elem<T>::from_f32(decode16<EMU>(bit));
    }
    *reinterpret_cast<Vec<T, VE>*>(values + (b * S + s) * D + d) = o;
  }
}

template <typename T, int VE>
__global__ void decode_bwd_kernel(const T* __restrict__ frames, const T* __restrict__ g_values,
                                  T* __restrict__ g_frames, long long B, long long S, long long D) {
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const T* in = frames + (s * 16 * B + b) * D + d;
    Vec<T, VE> f[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) f[k] = *reinterpret_cast<const Vec<T, VE>*>(in + k * frame_stride);
    const Vec<T, VE> gv = *reinterpret_cast<const Vec<T, VE>*>(g_values + (b * S + s) * D + d);
    Vec<T, VE> out[16];
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      float bit[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) bit[k] = Elem<T>::to_f32(f[k].v[j]);
      float gk[16];
      codec::decode16_bwd(bit, Elem<T>::to_f32(gv.v[j]), gk);
#pragma unroll
      for (int k = 0; k < 16; ++k) out[k].v[j] = Elem<T>::from_f32(gk[k]);
    }
    T* o = g_frames + (s * 16 * B + b) * D + d;
#pragma unroll
    for (int k = 0; k < 16; ++k) *reinterpret_cast<Vec<T, VE>*>(o + k * frame_stride) = out[k];
  }
}

template <typename T, int VE>
__global__ void residual_kernel(const T* __restrict__ fa, const T* __restrict__ fb, T* __restrict__ fo,
                                int compiled, long long B, long long S, long long D) {
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const long long base = (s * 16 * B + b) * D + d;
    Vec<T, VE> a[16], c[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      a[k] = *reinterpret_cast<const Vec<T, VE>*>(fa + base + k * frame_stride);
      c[k] = *reinterpret_cast<const Vec<T, VE>*>(fb + base + k * frame_stride);
    }
    uint32_t h[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      float ba[16], bb[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        ba[k] = Elem<T>::to_f32(a[k].v[j]);
        bb[k] = Elem<T>::to_f32(c[k].v[j]);
      }
      h[j] = residual_half_bits<Elem<T>::kDtype>(ba, bb, compiled != 0);
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      Vec<T, VE> o;
#pragma unroll
      for (int j = 0; j < VE; ++j) o.v[j] = ((h[j] >> (15 - k)) & 1u) ? Elem<T>::one() : Elem<T>::zero();
      *reinterpret_cast<Vec<T, VE>*>(fo + base + k * frame_stride) = o;
    }
  }
}

template <typename T, int VE>
__global__ void ste_bwd_kernel(const T* __restrict__ g_frames, T* __restrict__ g_values, long long B,
                               long long S, long long D) {
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const T* in = g_frames + (s * 16 * B + b) * D + d;
    Vec<T, VE> f[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) f[k] = *reinterpret_cast<const Vec<T, VE>*>(in + k * frame_stride);
    Vec<T, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      float acc = 0.0f;
#pragma unroll
      for (int k = 0; k < 16; ++k) acc += Elem<T>::to_f32(f[k].v[j]);
      o.v[j] = Elem<T>::from_f32(acc * 0.0625f);
    }
    *reinterpret_cast<Vec<T, VE>*>(g_values + (b * S + s) * D + d) = o;
  }
}

int grid_for(long long work_items, int threads) {
  DeviceInfo dev;
  if (get_device_info(&dev) != NSB_OK) return 0;
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)dev.sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

bool vec_ok(long long D, int ve, size_t elem, std::initializer_list<const void*> ptrs) {
  if (D % ve) return false;
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) % (elem * ve)) return false;
  return true;
}

bool dtype_ok(int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; }

// Widest vector (in elements) that D and every pointer allow, at most 16 bytes
// (MAXB = largest vector in bytes the kernel's register budget takes).
template <typename T>
int pick_ve(long long D, std::initializer_list<const void*> ptrs, int maxb) {
  for (int ve = maxb / (int)sizeof(T); ve > 1; ve >>= 1)
    if (vec_ok(D, ve, sizeof(T), ptrs)) return ve;
  return 1;
}

// Calls f.template operator()<T>() with the element type of `dtype`.
template <typename F>
int with_dtype(int dtype, F&& f) {
  switch (dtype) {
    case NSB_F32: return f(float{});
    case NSB_BF16: return f(__nv_bfloat16{});
    case NSB_F16: return f(__half{});
    default: return NSB_ERR_INVALID_ARG;
  }
}

constexpr int kThreads = 256;

}  // namespace
}  // namespace nsb

using namespace nsb;

extern "C" {

int nsb_fp16_encode(const void* values, void* frames, int64_t B, int64_t S, int64_t D, int dtype_in,
                    int dtype_out, void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype_in) || !dtype_ok(dtype_out)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!values || !frames) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return with_dtype(dtype_in, [&](auto ti) {
    using TI = decltype(ti);
    return with_dtype(dtype_out, [&](auto to) {
      using TO = decltype(to);
      if (reinterpret_cast<uintptr_t>(values) % sizeof(TI) || reinterpret_cast<uintptr_t>(frames) % sizeof(TO))
        return NSB_ERR_INVALID_ARG;
      int ve = 1;
      for (int c = 8; c > 1; c >>= 1) {
        if (c * sizeof(TI) > 16 || c * sizeof(TO) > 16) continue;
        if (D % c == 0 && reinterpret_cast<uintptr_t>(values) % (c * sizeof(TI)) == 0 &&
            reinterpret_cast<uintptr_t>(frames) % (c * sizeof(TO)) == 0) {
          ve = c;
          break;
        }
      }
      const long long items = (long long)B * S * (D / ve);
      const int grid = grid_for(items, kThreads);
      if (grid == 0) return NSB_ERR_CUDA;
      const TI* vp = static_cast<const TI*>(values);
      TO* fp = static_cast<TO*>(frames);
      switch (ve) {
        case 8: encode_kernel<TI, TO, (sizeof(TI) == 2 && sizeof(TO) == 2) ? 8 : 1><<<grid, kThreads, 0, st>>>(vp, fp, B, S, D); break;
        case 4: encode_kernel<TI, TO, 4><<<grid, kThreads, 0, st>>>(vp, fp, B, S, D); break;
        case 2: encode_kernel<TI, TO, 2><<<grid, kThreads, 0, st>>>(vp, fp, B, S, D); break;
        default: encode_kernel<TI, TO, 1><<<grid, kThreads, 0, st>>>(vp, fp, B, S, D); break;
      }
      NSB_CUDA_TRY(cudaGetLastError(), "launch encode_kernel");
      return NSB_OK;
    });
  });
}

#define NSB_CODEC_LAUNCH(KERNEL, WHERE, MAXB, PTRS, ...)                                   \
  return with_dtype(dtype, [&](auto t) {                                                   \
    using T = decltype(t);                                                                 \
    if (!vec_ok(D, 1, sizeof(T), PTRS)) return NSB_ERR_INVALID_ARG;                        \
    const int ve = pick_ve<T>(D, PTRS, MAXB);                                              \
    const long long items = (long long)B * S * (D / ve);                                   \
    const int grid = grid_for(items, kThreads);                                            \
    if (grid == 0) return NSB_ERR_CUDA;                                                    \
    switch (ve) {                                                                          \
      case 8: KERNEL<T, (sizeof(T) == 2 ? 8 : 1)><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D); break; \
      case 4: KERNEL<T, 4><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D); break;        \
      case 2: KERNEL<T, 2><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D); break;        \
      default: KERNEL<T, 1><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D); break;       \
    }                                                                                      \
    NSB_CUDA_TRY(cudaGetLastError(), WHERE);                                               \
    return NSB_OK;                                                                         \
  })

#define NSB_PTRS(...) std::initializer_list<const void*>{__VA_ARGS__}

int nsb_fp16_decode_fwd(const void* frames, void* values, int64_t B, int64_t S, int64_t D, int dtype,
                        void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!frames || !values) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_CODEC_LAUNCH(decode_fwd_kernel, "launch decode_fwd_kernel", 16, NSB_PTRS(frames, values),
                   static_cast<const T*>(frames), static_cast<T*>(values));
}

int nsb_fp16_decode_bwd(const void* frames, const void* g_values, void* g_frames, int64_t B, int64_t S,
                        int64_t D, int dtype, void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!frames || !g_values || !g_frames) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_CODEC_LAUNCH(decode_bwd_kernel, "launch decode_bwd_kernel", 8, NSB_PTRS(frames, g_values, g_frames),
                   static_cast<const T*>(frames), static_cast<const T*>(g_values),
                   static_cast<T*>(g_frames));
}

int nsb_binary_residual(const void* frames_a, const void* frames_b, void* frames_out, int64_t B,
                        int64_t S, int64_t D, int dtype, int rounding, void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype) ||
      (rounding != NSB_RESIDUAL_EAGER && rounding != NSB_RESIDUAL_COMPILED))
    return NSB_ERR_INVALID_ARG;
  const int compiled = rounding == NSB_RESIDUAL_COMPILED;
  if (B * S * D == 0) return NSB_OK;
  if (!frames_a || !frames_b || !frames_out) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_CODEC_LAUNCH(residual_kernel, "launch residual_kernel", 8, NSB_PTRS(frames_a, frames_b, frames_out),
                   static_cast<const T*>(frames_a), static_cast<const T*>(frames_b),
                   static_cast<T*>(frames_out), compiled);
}

int nsb_encode_ste_bwd(const void* g_frames, void* g_values, int64_t B, int64_t S, int64_t D, int dtype,
                       void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!g_frames || !g_values) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_CODEC_LAUNCH(ste_bwd_kernel, "launch ste_bwd_kernel", 16, NSB_PTRS(g_frames, g_values),
                   static_cast<const T*>(g_frames), static_cast<T*>(g_values));
}

}  // extern "C"
