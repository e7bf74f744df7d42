// Expert merge of the mixture-of-experts SNN FFN in the frame domain, one kernel each way.
//
// NeuronSpark's MoESNNFFN merges its experts per token in value space and re-encodes
// (atomic_ops/moe_snn_ffn.py:377-393):
//     shared_val  = fp16_decode(shared_out)            expert_vals[e] = fp16_decode(expert_spikes[e])
//     combined    = shared_val + (expert_vals * w).sum(dim=0)          w = full_weights[t, b, e]
//     total       = combined + fp16_decode(spike_in)
//     out         = binary_encode_ste(total)
// which is E+2 decode launches, a stack, a multiply, a sum, two adds and an encode, every one a pass
// over [B, T, D] values or their 16x larger frame tensors. Here the forward reads the 16 frames of
// every stream of a value, does the arithmetic in registers with the reference's roundings
// (products, the sum over experts, both additions each rounded to the frame dtype) and writes the
// 16 output frames: nothing but frames moves. An expert whose weight is exactly 0 for a token is
// not read at all - its product is a signed zero and cannot change the sum - which with top-k
// routing is most of them.
//
// The backward takes dL/d(out frames), forms the straight-through gradient of `total` (mean over
// the 16 frames, atomic_ops/fp16_codec.py:222-226), and pushes it through every decode: the
// gradients of the shared and residual frames, of each expert's frames (scaled by its weight), and
// grad_w[t, b, e] = sum_d g_total * expert_val[e], reduced per token inside the CTA in a fixed order.
#include "nsb_codec.cuh"
#include "nsb_common.cuh"

namespace nsb {
namespace {

using codec::decode16;
using codec::decode16_bwd;
using codec::half_bits_clamped;

template <typename T>
__device__ __forceinline__ float round_like(float x) {
  return Elem<T>::to_f32(Elem<T>::from_f32(x));
}

// 16 frames of VE channels of one token: element (k, j) is frame k, channel j
template <typename T, int VE>
struct FrameBlock {
  Vec<T, VE> f[16];
  __device__ __forceinline__ void load(const T* p, long long frame_stride) {
#pragma unroll
    for (int k = 0; k < 16; ++k) f[k] = *reinterpret_cast<const Vec<T, VE>*>(p + k * frame_stride);
  }
  __device__ __forceinline__ void store(T* p, long long frame_stride) const {
#pragma unroll
    for (int k = 0; k < 16; ++k) *reinterpret_cast<Vec<T, VE>*>(p + k * frame_stride) = f[k];
  }
  __device__ __forceinline__ void bits(int j, float (&bit)[16]) const {
#pragma unroll
    for (int k = 0; k < 16; ++k) bit[k] = Elem<T>::to_f32(f[k].v[j]);
  }
  // the decoded value of channel j, rounded to the frame dtype as fp16_decode's output is
  __device__ __forceinline__ float value(int j) const {
    float bit[16];
    bits(j, bit);
    return round_like<T>(decode16<Elem<T>::kDtype == NSB_BF16>(bit));
  }
};

template <typename T, int VE>
__global__ void __maxnreg__(80) frames_combine_fwd_kernel(const T* __restrict__ shared, const T* __restrict__ experts,
                                          const T* __restrict__ weights, const T* __restrict__ residual,
                                          T* __restrict__ out, long long B, long long S, long long D, int E) {
  const long long dv = D / VE;
  const long long total = B * S * dv;
  const long long frame_stride = B * D;
  const long long expert_stride = S * 16 * frame_stride;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long d = (idx % dv) * VE;
    const long long bs = idx / dv;
    const long long s = bs % S, b = bs / S;
    const long long base = (s * 16 * B + b) * D + d;
    FrameBlock<T, VE> blk;
    float sum[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) sum[j] = 0.0f;
    const T* wrow = weights + (s * B + b) * E;
    for (int e = 0; e < E; ++e) {
      const float w = Elem<T>::to_f32(wrow[e]);
      if (w == 0.0f) continue;  // product +-0: leaves the sum as it is
      blk.load(experts + e * expert_stride + base, frame_stride);
#pragma unroll
      for (int j = 0; j < VE; ++j) sum[j] += round_like<T>(blk.value(j) * w);
    }
    float tot[VE];
    blk.load(shared + base, frame_stride);
#pragma unroll
    for (int j = 0; j < VE; ++j) tot[j] = round_like<T>(blk.value(j) + round_like<T>(sum[j]));
    blk.load(residual + base, frame_stride);
    uint32_t h[VE];
#pragma unroll
    for (int j = 0; j < VE; ++j) h[j] = half_bits_clamped(round_like<T>(tot[j] + blk.value(j)));
#pragma unroll
    for (int k = 0; k < 16; ++k)
#pragma unroll
      for (int j = 0; j < VE; ++j) blk.f[k].v[j] = ((h[j] >> (15 - k)) & 1u) ? Elem<T>::one() : Elem<T>::zero();
    blk.store(out + base, frame_stride);
  }
}

constexpr int kMaxExperts = 16;
constexpr int kMaxWarps = 32;

// One CTA per token at a time (grid-stride over tokens); its threads cover the channels.
template <typename T, int VE>
__global__ void __maxnreg__(96) frames_combine_bwd_kernel(const T* __restrict__ g_out, const T* __restrict__ shared,
                                          const T* __restrict__ experts, const T* __restrict__ weights,
                                          const T* __restrict__ residual, T* __restrict__ g_shared,
                                          T* __restrict__ g_experts, T* __restrict__ g_weights,
                                          T* __restrict__ g_residual, long long B, long long S, long long D,
                                          int E) {
  __shared__ float part[kMaxExperts][kMaxWarps];
  const long long dv = D / VE;
  const long long frame_stride = B * D;
  const long long expert_stride = S * 16 * frame_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (long long tok = blockIdx.x; tok < B * S; tok += gridDim.x) {
    const long long s = tok % S, b = tok / S;
    const T* wrow = weights + (s * B + b) * E;
    float dot[kMaxExperts];
#pragma unroll
    for (int e = 0; e < kMaxExperts; ++e) dot[e] = 0.0f;
    for (long long v = threadIdx.x; v < dv; v += blockDim.x) {
      const long long base = (s * 16 * B + b) * D + v * VE;
      FrameBlock<T, VE> blk, gblk;
      blk.load(g_out + base, frame_stride);
      float gt[VE];  // straight-through gradient of `total`: mean over the 16 frames, in the frame dtype
#pragma unroll
      for (int j = 0; j < VE; ++j) {
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < 16; ++k) acc += Elem<T>::to_f32(blk.f[k].v[j]);
        gt[j] = round_like<T>(acc * 0.0625f);
      }
      auto through_decode = [&](const T* frames, T* g_frames, float scale, float* dots) {
        blk.load(frames + base, frame_stride);
#pragma unroll
        for (int j = 0; j < VE; ++j) {
          float bit[16], gk[16];
          blk.bits(j, bit);
          if (dots) *dots = fmaf(gt[j], round_like<T>(decode16<Elem<T>::kDtype == NSB_BF16>(bit)), *dots);
          decode16_bwd(bit, dots ? round_like<T>(gt[j] * scale) : gt[j], gk);
#pragma unroll
          for (int k = 0; k < 16; ++k) gblk.f[k].v[j] = Elem<T>::from_f32(gk[k]);
        }
        if (g_frames) gblk.store(g_frames + base, frame_stride);
      };
      if (g_shared) through_decode(shared, g_shared, 1.0f, nullptr);
      if (g_residual) through_decode(residual, g_residual, 1.0f, nullptr);
#pragma unroll
      for (int e = 0; e < kMaxExperts; ++e)
        if (e < E)
          through_decode(experts + e * expert_stride, g_experts ? g_experts + e * expert_stride : nullptr,
                         Elem<T>::to_f32(wrow[e]), &dot[e]);
    }
    if (g_weights) {
#pragma unroll
      for (int e = 0; e < kMaxExperts; ++e) {
        if (e < E) {
          float x = dot[e];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
          if (lane == 0) part[e][warp] = x;
        }
      }
      __syncthreads();
      if (threadIdx.x < E) {
        float x = 0.0f;
        for (int wi = 0; wi < nwarps; ++wi) x += part[threadIdx.x][wi];
        g_weights[(s * B + b) * E + threadIdx.x] = Elem<T>::from_f32(x);
      }
      __syncthreads();
    }
  }
}

bool ptr_ok(const void* p, size_t align) { return reinterpret_cast<uintptr_t>(p) % align == 0; }

template <typename T>
int pick_ve(long long D, std::initializer_list<const void*> ptrs, int max_bytes) {
  for (int ve = max_bytes / (int)sizeof(T); ve > 1; ve >>= 1) {
    bool ok = D % ve == 0;
    for (const void* p : ptrs) ok = ok && (!p || ptr_ok(p, sizeof(T) * ve));
    if (ok) return ve;
  }
  return 1;
}

template <typename T>
int launch_fwd(const void* shared, const void* experts, const void* weights, const void* residual, void* out,
               long long B, long long S, long long D, int E, cudaStream_t st) {
  const int ve = pick_ve<T>(D, {shared, experts, residual, out}, 8);  // 16-byte vectors measured 20 % slower
  DeviceInfo dev;
  if (get_device_info(&dev) != NSB_OK) return NSB_ERR_CUDA;
  constexpr int threads = 256;
  const long long items = B * S * (D / ve);
  const int grid = (int)std::max<long long>(1, std::min<long long>((items + threads - 1) / threads,
                                                                   (long long)dev.sm_count * 16));
  auto a = static_cast<const T*>(shared);
  auto x = static_cast<const T*>(experts);
  auto w = static_cast<const T*>(weights);
  auto r = static_cast<const T*>(residual);
  auto o = static_cast<T*>(out);
  switch (ve) {
    case 8: frames_combine_fwd_kernel<T, (sizeof(T) == 2 ? 8 : 1)><<<grid, threads, 0, st>>>(a, x, w, r, o, B, S, D, E); break;
    case 4: frames_combine_fwd_kernel<T, 4><<<grid, threads, 0, st>>>(a, x, w, r, o, B, S, D, E); break;
    case 2: frames_combine_fwd_kernel<T, 2><<<grid, threads, 0, st>>>(a, x, w, r, o, B, S, D, E); break;
    default: frames_combine_fwd_kernel<T, 1><<<grid, threads, 0, st>>>(a, x, w, r, o, B, S, D, E); break;
  }
  NSB_CUDA_TRY(cudaGetLastError(), "launch frames_combine_fwd_kernel");
  return NSB_OK;
}

template <typename T>
int launch_bwd(const void* g_out, const void* shared, const void* experts, const void* weights,
               const void* residual, void* g_shared, void* g_experts, void* g_weights, void* g_residual,
               long long B, long long S, long long D, int E, cudaStream_t st) {
  const int ve = pick_ve<T>(D, {g_out, shared, experts, residual, g_shared, g_experts, g_residual}, 8);
  DeviceInfo dev;
  if (get_device_info(&dev) != NSB_OK) return NSB_ERR_CUDA;
  const long long dv = D / ve;
  const int threads = (int)std::min<long long>(kMaxWarps * 32, std::max<long long>(32, (dv + 31) / 32 * 32));
  const int grid = (int)std::max<long long>(1, std::min<long long>(B * S, (long long)dev.sm_count * 8));
  auto g = static_cast<const T*>(g_out);
  auto a = static_cast<const T*>(shared);
  auto x = static_cast<const T*>(experts);
  auto w = static_cast<const T*>(weights);
  auto r = static_cast<const T*>(residual);
  auto ga = static_cast<T*>(g_shared);
  auto gx = static_cast<T*>(g_experts);
  auto gw = static_cast<T*>(g_weights);
  auto gr = static_cast<T*>(g_residual);
  switch (ve) {
    case 4: frames_combine_bwd_kernel<T, (sizeof(T) == 2 ? 4 : 1)><<<grid, threads, 0, st>>>(g, a, x, w, r, ga, gx, gw, gr, B, S, D, E); break;
    case 2: frames_combine_bwd_kernel<T, 2><<<grid, threads, 0, st>>>(g, a, x, w, r, ga, gx, gw, gr, B, S, D, E); break;
    default: frames_combine_bwd_kernel<T, 1><<<grid, threads, 0, st>>>(g, a, x, w, r, ga, gx, gw, gr, B, S, D, E); break;
  }
  NSB_CUDA_TRY(cudaGetLastError(), "launch frames_combine_bwd_kernel");
  return NSB_OK;
}

bool dtype_ok(int d) { return d == NSB_F32 || d == NSB_BF16 || d == NSB_F16; }

}  // namespace
}  // namespace nsb

using namespace nsb;

extern "C" int nsb_frames_combine_fwd(const void* shared, const void* experts, const void* weights,
                                      const void* residual, void* out, int64_t B, int64_t S, int64_t D,
                                      int E, int dtype, void* stream) {
  if (B < 0 || S < 0 || D < 0 || E < 0 || E > kMaxExperts || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!shared || !residual || !out || (E > 0 && (!experts || !weights))) return NSB_ERR_INVALID_ARG;
  const size_t es = dtype_size(dtype);
  for (const void* p : {shared, experts, weights, residual, static_cast<const void*>(out)})
    if (p && !ptr_ok(p, es)) return NSB_ERR_INVALID_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NSB_F32: return launch_fwd<float>(shared, experts, weights, residual, out, B, S, D, E, st);
    case NSB_BF16: return launch_fwd<__nv_bfloat16>(shared, experts, weights, residual, out, B, S, D, E, st);
    default: return launch_fwd<__half>(shared, experts, weights, residual, out, B, S, D, E, st);
  }
}

extern "C" int nsb_frames_combine_bwd(const void* g_out, const void* shared, const void* experts,
                                      const void* weights, const void* residual, void* g_shared,
                                      void* g_experts, void* g_weights, void* g_residual, int64_t B,
                                      int64_t S, int64_t D, int E, int dtype, void* stream) {
  if (B < 0 || S < 0 || D < 0 || E < 0 || E > kMaxExperts || !dtype_ok(dtype)) return NSB_ERR_INVALID_ARG;
  if (B * S * D == 0) return NSB_OK;
  if (!g_out || (g_shared && !shared) || (g_residual && !residual) ||
      (E > 0 && (g_experts || g_weights) && (!experts || !weights)))
    return NSB_ERR_INVALID_ARG;
  const size_t es = dtype_size(dtype);
  for (const void* p : {g_out, shared, experts, weights, residual, static_cast<const void*>(g_shared),
                        static_cast<const void*>(g_experts), static_cast<const void*>(g_weights),
                        static_cast<const void*>(g_residual)})
    if (p && !ptr_ok(p, es)) return NSB_ERR_INVALID_ARG;
  if (!g_experts && !g_weights) E = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NSB_F32:
      return launch_bwd<float>(g_out, shared, experts, weights, residual, g_shared, g_experts, g_weights,
                               g_residual, B, S, D, E, st);
    case NSB_BF16:
      return launch_bwd<__nv_bfloat16>(g_out, shared, experts, weights, residual, g_shared, g_experts,
                                       g_weights, g_residual, B, S, D, E, st);
    default:
      return launch_bwd<__half>(g_out, shared, experts, weights, residual, g_shared, g_experts, g_weights,
                                g_residual, B, S, D, E, st);
  }
}
