/* Test infrastructure: BF16 value types with the conversions the reference kernels call
 * (round to nearest even, NaN kept quiet), for the host build described in hip_runtime.h. */
#pragma once

#include <cstdint>
#include <cstring>

namespace ref_bf16_detail {
inline float widen(uint16_t bits) {
  const uint32_t u = static_cast<uint32_t>(bits) << 16;
  float v;
  std::memcpy(&v, &u, 4);
  return v;
}
inline uint16_t narrow(float v) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
}  // namespace ref_bf16_detail

struct __hip_bfloat16 {
  uint16_t bits;
};
inline float __bfloat162float(__hip_bfloat16 v) { return ref_bf16_detail::widen(v.bits); }
inline __hip_bfloat16 __float2bfloat16(float v) { return __hip_bfloat16{ref_bf16_detail::narrow(v)}; }

/* the older class-style type used by the LM-head file */
struct hip_bfloat16 {
  uint16_t data;
  hip_bfloat16() = default;
  explicit hip_bfloat16(float v) : data(ref_bf16_detail::narrow(v)) {}
  operator float() const { return ref_bf16_detail::widen(data); }
};
