// FP16 boundary codec on spikes packed in time: the 16 frames of a token and channel are one
// uint16, the IEEE half bit pattern they spell (frame 0 = sign = bit 15). Patterns are [S, B, D]
// (2 bytes per value where dense frames [S*16, B, D] take 16 elements), values are [B, S, D].
//
// A thread owns VE consecutive channels of one (s, b) token; a warp touches 32*VE consecutive
// elements of every row it reads or writes. All kernels are pure streaming.
#include <algorithm>
#include <initializer_list>

#include "nsb_codec.cuh"
#include "nsb_common.cuh"

namespace nsb {
namespace {

using codec::decode16;
using codec::pattern_to_bits;

constexpr int kThreads = 256;

int grid_for(long long items) {
  DeviceInfo dev;
  if (get_device_info(&dev) != NSB_OK) return 0;
  long long blocks = (items + kThreads - 1) / kThreads;
  const long long cap = (long long)dev.sm_count * 16;
  return (int)std::max(1LL, std::min(blocks, cap));
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

// 4 channels per thread when D and every pointer allow 4-element accesses, else 1
template <typename T>
int pick_ve(long long D, std::initializer_list<const void*> elems, std::initializer_list<const void*> pats) {
  if (D % 4) return 1;
  for (const void* p : elems)
    if (reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T))) return 1;
  for (const void* p : pats)
    if (reinterpret_cast<uintptr_t>(p) % 8) return 1;
  return 4;
}

struct Tok {
  long long s, b, d;
};
__device__ __forceinline__ Tok token_of(long long idx, long long B, long long dv, int ve) {
  Tok t;
  t.d = (idx % dv) * ve;
  const long long sb = idx / dv;
  t.b = sb % B;
  t.s = sb / B;
  return t;
}

// frames {0,1} -> patterns (a frame counts as set when it is >= 0.5)
template <typename T, int VE>
__global__ void pack_kernel(const T* __restrict__ frames, uint16_t* __restrict__ pats, long long B, long long S,
                            long long D) {
  const long long dv = D / VE, total = S * B * dv, fs = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const Tok t = token_of(idx, B, dv, VE);
    const T* in = frames + (t.s * 16 * B + t.b) * D + t.d;
    Vec<T, VE> f[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) f[k] = *reinterpret_cast<const Vec<T, VE>*>(in + k * fs);
    Vec<uint16_t, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      uint32_t h = 0;
#pragma unroll
      for (int k = 0; k < 16; ++k) h |= (Elem<T>::to_f32(f[k].v[j]) >= 0.5f ? 1u : 0u) << (15 - k);
      o.v[j] = (uint16_t)h;
    }
    *reinterpret_cast<Vec<uint16_t, VE>*>(pats + (t.s * B + t.b) * D + t.d) = o;
  }
}

template <typename T, int VE>
__global__ void unpack_kernel(const uint16_t* __restrict__ pats, T* __restrict__ frames, long long B, long long S,
                              long long D) {
  const long long dv = D / VE, total = S * B * dv, fs = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const Tok t = token_of(idx, B, dv, VE);
    const Vec<uint16_t, VE> p = *reinterpret_cast<const Vec<uint16_t, VE>*>(pats + (t.s * B + t.b) * D + t.d);
    T* out = frames + (t.s * 16 * B + t.b) * D + t.d;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      Vec<T, VE> o;
#pragma unroll
      for (int j = 0; j < VE; ++j) o.v[j] = ((p.v[j] >> (15 - k)) & 1u) ? Elem<T>::one() : Elem<T>::zero();
      *reinterpret_cast<Vec<T, VE>*>(out + k * fs) = o;
    }
  }
}

// patterns -> values with the roundings fp16_decode performs on frames stored as T
template <typename T, int VE>
__global__ void decode_packed_fwd_kernel(const uint16_t* __restrict__ pats, T* __restrict__ values, long long B,
                                         long long S, long long D) {
  constexpr bool EMU = Elem<T>::kDtype == NSB_BF16;
  const long long dv = D / VE, total = S * B * dv;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const Tok t = token_of(idx, B, dv, VE);
    const Vec<uint16_t, VE> p = *reinterpret_cast<const Vec<uint16_t, VE>*>(pats + (t.s * B + t.b) * D + t.d);
    Vec<T, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      if constexpr (EMU) {  // bf16 frames decode with bf16 intermediates (the reference calls fp16_decode eagerly)
        float bit[16];
        pattern_to_bits(p.v[j], bit);
        o.v[j] = Elem<T>::from_f32(decode16<true>(bit));
      } else {
        o.v[j] = Elem<T>::from_f32(codec::decode_pattern_exact(p.v[j]));
      }
    }
    *reinterpret_cast<Vec<T, VE>*>(values + (t.b * S + t.s) * D + t.d) = o;
  }
}

// value gradients [B,S,D] -> the 16 frame gradients of every value, dense [S*16,B,D]
template <typename T, int VE>
__global__ void decode_packed_bwd_kernel(const uint16_t* __restrict__ pats, const T* __restrict__ g_values,
                                         T* __restrict__ g_frames, long long B, long long S, long long D) {
  const long long dv = D / VE, total = S * B * dv, fs = B * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const Tok t = token_of(idx, B, dv, VE);
    const Vec<uint16_t, VE> p = *reinterpret_cast<const Vec<uint16_t, VE>*>(pats + (t.s * B + t.b) * D + t.d);
    const Vec<T, VE> gv = *reinterpret_cast<const Vec<T, VE>*>(g_values + (t.b * S + t.s) * D + t.d);
    Vec<T, VE> out[16];
#pragma unroll
    for (int j = 0; j < VE; ++j) {
      float bit[16], gk[16];
      pattern_to_bits(p.v[j], bit);
      codec::decode16_bwd(bit, Elem<T>::to_f32(gv.v[j]), gk);
#pragma unroll
      for (int k = 0; k < 16; ++k) out[k].v[j] = Elem<T>::from_f32(gk[k]);
    }
    T* o = g_frames + (t.s * 16 * B + t.b) * D + t.d;
#pragma unroll
    for (int k = 0; k < 16; ++k) *reinterpret_cast<Vec<T, VE>*>(o + k * fs) = out[k];
  }
}

template <int VE>
__global__ void residual_packed_kernel(const uint16_t* __restrict__ pa, const uint16_t* __restrict__ pb,
                                       uint16_t* __restrict__ po, long long n, int frame_dtype, int compiled) {
  const long long nv = n / VE;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < nv;
       idx += (long long)gridDim.x * blockDim.x) {
    const Vec<uint16_t, VE> a = reinterpret_cast<const Vec<uint16_t, VE>*>(pa)[idx];
    const Vec<uint16_t, VE> b = reinterpret_cast<const Vec<uint16_t, VE>*>(pb)[idx];
    Vec<uint16_t, VE> o;
#pragma unroll
    for (int j = 0; j < VE; ++j)
      o.v[j] = (uint16_t)codec::residual_of_patterns(a.v[j], b.v[j], frame_dtype, compiled != 0);
    reinterpret_cast<Vec<uint16_t, VE>*>(po)[idx] = o;
  }
}

}  // namespace
}  // namespace nsb

using namespace nsb;

#define NSB_PACKED_LAUNCH(KERNEL, WHERE, ELEMS, PATS, ...)                                  \
  return with_dtype(dtype, [&](auto t) {                                                    \
    using T = decltype(t);                                                                  \
    for (const void* q : ELEMS)                                                             \
      if (reinterpret_cast<uintptr_t>(q) % sizeof(T)) return NSB_ERR_INVALID_ARG;           \
    for (const void* q : PATS)                                                              \
      if (reinterpret_cast<uintptr_t>(q) % 2) return NSB_ERR_INVALID_ARG;                   \
    const int ve = pick_ve<T>(D, ELEMS, PATS);                                              \
    const int grid = grid_for((long long)B * S * (D / ve));                                 \
    if (grid == 0) return NSB_ERR_CUDA;                                                     \
    if (ve == 4)                                                                            \
      KERNEL<T, 4><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D);                        \
    else                                                                                    \
      KERNEL<T, 1><<<grid, kThreads, 0, st>>>(__VA_ARGS__, B, S, D);                        \
    NSB_CUDA_TRY(cudaGetLastError(), WHERE);                                                \
    return NSB_OK;                                                                          \
  })

#define NSB_LIST(...) std::initializer_list<const void*>{__VA_ARGS__}

extern "C" {

int nsb_frames_pack(const void* frames, uint16_t* patterns, int64_t B, int64_t S, int64_t D, int dtype,
                    void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!frames || !patterns) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_PACKED_LAUNCH(pack_kernel, "launch pack_kernel", NSB_LIST(frames), NSB_LIST(patterns),
                    static_cast<const T*>(frames), patterns);
}

int nsb_frames_unpack(const uint16_t* patterns, void* frames, int64_t B, int64_t S, int64_t D, int dtype,
                      void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!frames || !patterns) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_PACKED_LAUNCH(unpack_kernel, "launch unpack_kernel", NSB_LIST(frames), NSB_LIST(patterns), patterns,
                    static_cast<T*>(frames));
}

int nsb_fp16_decode_packed_fwd(const uint16_t* patterns, void* values, int64_t B, int64_t S, int64_t D,
                               int dtype, void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!values || !patterns) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_PACKED_LAUNCH(decode_packed_fwd_kernel, "launch decode_packed_fwd_kernel", NSB_LIST(values),
                    NSB_LIST(patterns), patterns, static_cast<T*>(values));
}

int nsb_fp16_decode_packed_bwd(const uint16_t* patterns, const void* g_values, void* g_frames, int64_t B,
                               int64_t S, int64_t D, int dtype, void* stream) {
  if (B < 0 || S < 0 || D < 0 || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!g_values || !g_frames || !patterns) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NSB_PACKED_LAUNCH(decode_packed_bwd_kernel, "launch decode_packed_bwd_kernel", NSB_LIST(g_values, g_frames),
                    NSB_LIST(patterns), patterns, static_cast<const T*>(g_values), static_cast<T*>(g_frames));
}

int nsb_binary_residual_packed(const uint16_t* patterns_a, const uint16_t* patterns_b, uint16_t* patterns_out,
                               int64_t n, int frame_dtype, int rounding, void* stream) {
  if (n < 0 || !dtype_ok(frame_dtype) || (rounding != NSB_RESIDUAL_EAGER && rounding != NSB_RESIDUAL_COMPILED))
    return NSB_ERR_INVALID_ARG;
  if (n == 0) return NSB_OK;
  if (!patterns_a || !patterns_b || !patterns_out) return NSB_ERR_INVALID_ARG;
  const void* ps[] = {patterns_a, patterns_b, patterns_out};
  bool v4 = n % 4 == 0;
  for (const void* q : ps) {
    if (reinterpret_cast<uintptr_t>(q) % 2) return NSB_ERR_INVALID_ARG;
    v4 = v4 && reinterpret_cast<uintptr_t>(q) % 8 == 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int compiled = rounding == NSB_RESIDUAL_COMPILED;
  const int grid = grid_for(v4 ? n / 4 : n);
  if (grid == 0) return NSB_ERR_CUDA;
  if (v4)
    residual_packed_kernel<4><<<grid, kThreads, 0, st>>>(patterns_a, patterns_b, patterns_out, n, frame_dtype, compiled);
  else
    residual_packed_kernel<1><<<grid, kThreads, 0, st>>>(patterns_a, patterns_b, patterns_out, n, frame_dtype, compiled);
  NSB_CUDA_TRY(cudaGetLastError(), "launch residual_packed_kernel");
  return NSB_OK;
}

}  // extern "C"
