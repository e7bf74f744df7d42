// Device functions of the FP16 bit-plane codec shared by the codec kernels and by the scan
// kernel that applies the binary residual to its own spikes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/neuronspark_b200.h"

namespace nsb {
namespace codec {

// fp32 -> half bit pattern as the reference does it: clamp to +-65504, round
// to nearest even. NaN maps to a quiet NaN with the input's sign.
__device__ __forceinline__ uint32_t half_bits_clamped(float f) {
  if (f != f) return ((__float_as_uint(f) >> 16) & 0x8000u) | 0x7e00u;
  f = fminf(fmaxf(f, -65504.0f), 65504.0f);
  return (uint32_t)__half_as_ushort(__float2half_rn(f));
}

__device__ __forceinline__ float round_through_bf16(float f) {
  return __bfloat162float(__float2bfloat16_rn(f));
}

// Decode 16 frame values (any reals, normally {0,1}) to a number with the
// reference's formula. EMU_BF16: round the mantissa sum, 1+m and the products
// to bf16 where the reference's bf16 arithmetic does.
template <bool EMU_BF16>
__device__ __forceinline__ float decode16(const float (&bit)[16]) {
  float sign = 1.0f - 2.0f * bit[0];
  float e = 16.0f * bit[1] + 8.0f * bit[2] + 4.0f * bit[3] + 2.0f * bit[4] + bit[5];
  float m = 0.0f;
  float w = 0.5f;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    m += bit[6 + i] * w;
    w *= 0.5f;
  }
  if (EMU_BF16) {
    sign = round_through_bf16(sign);
    e = round_through_bf16(e);
    m = round_through_bf16(m);
  }
  float val;
  if (e > 0.0f) {
    float opm = 1.0f + m;
    float p = sign * exp2f(e - 15.0f);
    if (EMU_BF16) {
      opm = round_through_bf16(opm);
      p = round_through_bf16(p);
    }
    val = p * opm;
  } else {
    val = (sign * 6.103515625e-05f) * m;
  }
  if (EMU_BF16) val = round_through_bf16(val);
  return val;
}

// Gradient of decode16 with respect to its 16 frame values, times g (fp32 formula; the frames
// are differentiated as reals: sign = 1 - 2*bit0, exponent and mantissa sums linear in their bits).
__device__ __forceinline__ void decode16_bwd(const float (&bit)[16], float g, float (&out)[16]) {
  const float sign = 1.0f - 2.0f * bit[0];
  const float e = 16.0f * bit[1] + 8.0f * bit[2] + 4.0f * bit[3] + 2.0f * bit[4] + bit[5];
  float m = 0.0f, w = 0.5f;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    m += bit[6 + i] * w;
    w *= 0.5f;
  }
  const bool normal = e > 0.0f;
  const float scale = normal ? exp2f(e - 15.0f) : 6.103515625e-05f;
  const float mag = normal ? scale * (1.0f + m) : scale * m;
  out[0] = -2.0f * mag * g;
  const float ge = normal ? g * sign * mag * 0.6931471805599453f : 0.0f;
  out[1] = ge * 16.0f;
  out[2] = ge * 8.0f;
  out[3] = ge * 4.0f;
  out[4] = ge * 2.0f;
  out[5] = ge;
  float gm = g * sign * scale * 0.5f;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    out[6 + i] = gm;
    gm *= 0.5f;
  }
}

// Half bit pattern of decode(a) + decode(b) for frames stored in DTYPE, with the roundings
// the reference's arithmetic in that dtype performs (atomic_ops/fp16_codec.py:115-164).
// bf16 frames have two reference behaviours (fp32 and fp16 frames have one: every intermediate
// is exact there). `compiled` = false: the ops evaluated one by one, each intermediate rounded
// to bf16 (eager PyTorch). `compiled` = true: the torch.compile'd residual (:168-170) as a GPU
// runs it: the decode stays in fp32 and only the sum, stored as a bf16 tensor between two fused
// kernels, is rounded. The flag is uniform over a launch.
template <int DTYPE>
__device__ __forceinline__ uint32_t residual_half_bits(const float (&a)[16], const float (&b)[16],
                                                       bool compiled) {
  constexpr bool EMU = DTYPE == NSB_BF16;
  float sum;
  if (EMU && !compiled)
    sum = decode16<true>(a) + decode16<true>(b);
  else
    sum = decode16<false>(a) + decode16<false>(b);
  if (EMU) sum = round_through_bf16(sum);
  if (DTYPE == NSB_F16) sum = __half2float(__float2half_rn(sum));
  return half_bits_clamped(sum);
}

// The 16 frames a half bit pattern stands for, as reals in {0,1} (frame 0 = sign = bit 15).
__device__ __forceinline__ void pattern_to_bits(uint32_t pat, float (&bit)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) bit[i] = ((pat >> (15 - i)) & 1u) ? 1.0f : 0.0f;
}

// decode16<false> of the frames a pattern stands for, straight from the bits. With frames in
// {0,1} every intermediate of the reference's formula is exact in fp32 (the mantissa sum has 10
// bits, 1+m has 11, the scale is a power of two), so the value is the fp32 number with the
// pattern's sign, exponent e + 112 and mantissa m << 13 - for every e from 1 to 31, an all-ones
// exponent included (the formula reads it as an ordinary normal number) - and sign * m * 2^-24
// for e = 0. A handful of integer instructions instead of sixteen selects and forty flops.
__device__ __forceinline__ float decode_pattern_exact(uint32_t pat) {
  const uint32_t sign = (pat & 0x8000u) << 16, e = (pat >> 10) & 31u, m = pat & 1023u;
  const float normal = __uint_as_float(sign | ((e + 112u) << 23) | (m << 13));
  const float sub = __uint_as_float(sign | __float_as_uint((float)m * 5.9604644775390625e-08f));
  return e ? normal : sub;
}

// encode(decode(a) + decode(b)) given the two decoded values: the sum's rounding for frames stored
// in DTYPE, then the half pattern.
template <int DTYPE>
__device__ __forceinline__ uint32_t half_bits_of_sum(float va, float vb) {
  float sum = va + vb;
  if (DTYPE == NSB_BF16) sum = round_through_bf16(sum);
  if (DTYPE == NSB_F16) sum = __half2float(__float2half_rn(sum));
  return half_bits_clamped(sum);
}

// residual_half_bits with the first operand given as a pattern (the scan's own spikes) and the
// second as 16 frames.
template <int DTYPE>
__device__ __forceinline__ uint32_t residual_pattern_frames(uint32_t pa, const float (&b)[16], bool compiled) {
  if (DTYPE == NSB_BF16 && !compiled) {
    float a[16];
    pattern_to_bits(pa, a);
    return residual_half_bits<DTYPE>(a, b, false);
  }
  return half_bits_of_sum<DTYPE>(decode_pattern_exact(pa), decode16<false>(b));
}

// residual_half_bits on two patterns, with the roundings of frames stored in `frame_dtype`
// (a run-time value here: packed patterns have no element type of their own).
__device__ __forceinline__ uint32_t residual_of_patterns(uint32_t pa, uint32_t pb, int frame_dtype, bool compiled) {
  if (frame_dtype == NSB_BF16 && !compiled) {
    float a[16], b[16];
    pattern_to_bits(pa, a);
    pattern_to_bits(pb, b);
    return residual_half_bits<NSB_BF16>(a, b, false);
  }
  const float va = decode_pattern_exact(pa), vb = decode_pattern_exact(pb);
  if (frame_dtype == NSB_BF16) return half_bits_of_sum<NSB_BF16>(va, vb);
  if (frame_dtype == NSB_F16) return half_bits_of_sum<NSB_F16>(va, vb);
  return half_bits_of_sum<NSB_F32>(va, vb);
}

}  // namespace codec
}  // namespace nsb
