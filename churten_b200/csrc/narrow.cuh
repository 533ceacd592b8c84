// 8-byte accesses to fp16 / bf16 buffers that ride beside fp32 buffers: four 2-byte elements per
// access, widened exactly on load, rounded to nearest even on store.
#pragma once

#include "stream.cuh"

namespace cb200 {

template <bool STREAM>
__device__ __forceinline__ uint2 load8(const void* p) {
  if (STREAM) return __ldcs(reinterpret_cast<const uint2*>(p));
  return *reinterpret_cast<const uint2*>(p);
}
template <bool STREAM>
__device__ __forceinline__ void store8(void* p, const uint2& v) {
  if (STREAM) {
    __stcs(reinterpret_cast<uint2*>(p), v);
  } else {
    *reinterpret_cast<uint2*>(p) = v;
  }
}

// Four 2-byte elements in one 8-byte access.
template <class TM>
struct Quad;
template <>
struct Quad<__half> {
  __device__ static __forceinline__ void unpack(const uint2& v, float (&out)[4]) {
    const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
    out[0] = __low2float(a);
    out[1] = __high2float(a);
    out[2] = __low2float(b);
    out[3] = __high2float(b);
  }
  __device__ static __forceinline__ uint2 pack(const float (&in)[4]) {
    const __half2 a = __floats2half2_rn(in[0], in[1]), b = __floats2half2_rn(in[2], in[3]);
    return make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
  }
};
template <>
struct Quad<__nv_bfloat16> {
  __device__ static __forceinline__ void unpack(const uint2& v, float (&out)[4]) {
    out[0] = __uint_as_float(v.x << 16);  // a bf16 is the upper half of an fp32
    out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16);
    out[3] = __uint_as_float(v.y & 0xffff0000u);
  }
  __device__ static __forceinline__ uint2 pack(const float (&in)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(in[0], in[1]), b = __floats2bfloat162_rn(in[2], in[3]);
    return make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
  }
};

}  // namespace cb200
