// Shared helpers for the libmlkit_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mlkit_b200.h"

namespace mkb {

// ---- error reporting (per calling thread) ---------------------------------------------------
void set_error(const char* format, ...);
int cuda_fail(cudaError_t status, const char* what);

#define MKB_REQUIRE(cond, code, ...)  \
  do {                                \
    if (!(cond)) {                    \
      ::mkb::set_error(__VA_ARGS__);  \
      return (code);                  \
    }                                 \
  } while (0)

#define MKB_LAUNCH_CHECK(what)                                        \
  do {                                                                \
    cudaError_t status_ = cudaGetLastError();                         \
    if (status_ != cudaSuccess) return ::mkb::cuda_fail(status_, what); \
  } while (0)

// ---- device properties, cached per device ---------------------------------------------------
struct DeviceInfo {
  int sm_count;
  int max_smem_optin;
};
const DeviceInfo& device_info();

// ---- packing-word geometry -------------------------------------------------------------------
// One word is the fewest whole bytes holding a whole number of codes.
__host__ __device__ inline int gcd8(int bits) {
  return (bits % 8 == 0) ? 8 : (bits % 4 == 0) ? 4 : (bits % 2 == 0) ? 2 : 1;
}
__host__ __device__ inline int word_bytes(int bits) { return bits / gcd8(bits); }
__host__ __device__ inline int word_codes(int bits) { return 8 / gcd8(bits); }

// ---- typed loads / stores through a runtime dtype tag ------------------------------------------
__device__ __forceinline__ float load_as_float(const void* base, int64_t index, int dtype) {
  if (dtype == MKB_F16) return __half2float(reinterpret_cast<const __half*>(base)[index]);
  if (dtype == MKB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[index]);
  return reinterpret_cast<const float*>(base)[index];
}

__device__ __forceinline__ void store_from_float(void* base, int64_t index, int dtype, float value) {
  if (dtype == MKB_F16) reinterpret_cast<__half*>(base)[index] = __float2half_rn(value);
  else if (dtype == MKB_BF16) reinterpret_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(value);
  else reinterpret_cast<float*>(base)[index] = value;
}

// SwiGLU on two packed fp16 pairs, with the rounding points of separate fp16 operators: the
// activation silu(g) is rounded to fp16, then the product with u is rounded to fp16.
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t gate_bits, uint32_t up_bits) {
  const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&gate_bits));
  const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&up_bits));
  const float a = g.x / (1.f + __expf(-g.x)), b = g.y / (1.f + __expf(-g.y));
  const float2 act = __half22float2(__floats2half2_rn(a, b));
  const __half2 out = __floats2half2_rn(act.x * u.x, act.y * u.y);
  return *reinterpret_cast<const uint32_t*>(&out);
}

__host__ __device__ inline int dtype_bytes(int dtype) { return dtype == MKB_F32 ? 4 : 2; }

// The reference reconstruction: one binary32 multiply, then (with offsets) one separate binary32
// add; never a fused multiply-add.
__device__ __forceinline__ float reconstruct(float value, float scale) { return __fmul_rn(value, scale); }
__device__ __forceinline__ float reconstruct(float value, float scale, float zero) {
  return __fadd_rn(__fmul_rn(value, scale), zero);
}

}  // namespace mkb
