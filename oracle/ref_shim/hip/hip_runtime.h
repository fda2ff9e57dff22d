/* Test infrastructure: a host-side stand-in for the few HIP device constructs the reference's
 * scalar MoE, pointwise and LM-head kernels use, so that those kernels -- taken unmodified from
 * the reference checkout at build time -- compile with g++ and run on the CPU.
 *
 * A kernel launch becomes a loop over blocks; the threads of a block run as cooperative
 * fibers on one OS thread (see ref_driver.cpp): __syncthreads() hands control to the next
 * fiber, so every fiber reaches barrier n before any continues past it, which is the barrier's
 * contract.  __shared__ variables become function-level statics (one block runs at a time).
 * Nothing here is part of the product; only tests, the smoke check and the CPU baseline of the
 * benchmark may load what is built from it. */
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>

struct ref_dim3 {
  unsigned x = 1, y = 1, z = 1;
};
extern ref_dim3 threadIdx, blockIdx, blockDim, gridDim;
void ref_syncthreads();

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static
#define __launch_bounds__(...)
#define __restrict__
#define __syncthreads() ref_syncthreads()

inline unsigned __float_as_uint(float v) { unsigned u; std::memcpy(&u, &v, 4); return u; }
inline float __uint_as_float(unsigned u) { float v; std::memcpy(&v, &u, 4); return v; }
inline float __int_as_float(int i) { float v; std::memcpy(&v, &i, 4); return v; }
/* The device rsqrtf is an approximation within one ulp; the reference corrects it to the rounded
 * value itself (pytorch_rounded_rsqrtf), so any seed within one ulp gives the same result. */
inline float rsqrtf(float v) { return 1.0f / std::sqrt(v); }

template <typename T>
inline T atomicAdd(T* address, T value) {
  const T old = *address;      /* fibers of a block run one at a time */
  *address = old + value;
  return old;
}
