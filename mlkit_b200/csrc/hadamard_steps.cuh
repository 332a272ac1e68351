// Butterfly steps of the Walsh-Hadamard transform shared by the transform kernels and by the matvec that
// rotates its activations on load (sm_100a).  Pairing and order are those of a stage-by-stage transform:
// stage s pairs i with i ^ 2^s and forms (a + b, a - b), strides ascending, fp32, one rounding per
// operation, so every user rounds identically.
#pragma once

#include "mkb_common.cuh"

namespace mkb {

constexpr int kWarpRun = 16;                 // values per lane when a warp transforms 512 values
constexpr int kWarpSpan = 32 * kWarpRun;     // values per warp: nine stages without shared memory
constexpr int kWarpBits = 9;

template <int STAGES>
__device__ __forceinline__ void butterfly_pass(float* buf, int groups, int stride, int stride_bits, float scale) {
  for (int grp = threadIdx.x; grp < groups; grp += blockDim.x) {
    const int low = grp & (stride - 1);
    const int base = ((grp >> stride_bits) << (stride_bits + STAGES)) + low;
    float v[1 << STAGES];
    if (STAGES == 3 && stride == 1) {   // eight consecutive values: two 16-byte accesses, no bank conflicts
      const float4 lo = *reinterpret_cast<const float4*>(buf + base), hi = *reinterpret_cast<const float4*>(buf + base + 4);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
      v[4 % (1 << STAGES)] = hi.x; v[5 % (1 << STAGES)] = hi.y; v[6 % (1 << STAGES)] = hi.z; v[7 % (1 << STAGES)] = hi.w;
    } else {
#pragma unroll
      for (int j = 0; j < (1 << STAGES); ++j) v[j] = buf[base + j * stride];
    }
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const int span = 1 << s;
#pragma unroll
      for (int j = 0; j < (1 << STAGES); ++j) {
        if ((j & span) == 0) {
          const float a = v[j], b = v[j + span];
          v[j] = __fadd_rn(a, b);
          v[j + span] = __fsub_rn(a, b);
        }
      }
    }
    if (STAGES == 3 && stride == 1) {
      *reinterpret_cast<float4*>(buf + base) = make_float4(__fmul_rn(v[0], scale), __fmul_rn(v[1], scale),
                                                          __fmul_rn(v[2], scale), __fmul_rn(v[3], scale));
      *reinterpret_cast<float4*>(buf + base + 4) =
          make_float4(__fmul_rn(v[4 % (1 << STAGES)], scale), __fmul_rn(v[5 % (1 << STAGES)], scale),
                      __fmul_rn(v[6 % (1 << STAGES)], scale), __fmul_rn(v[7 % (1 << STAGES)], scale));
    } else {
#pragma unroll
      for (int j = 0; j < (1 << STAGES); ++j) buf[base + j * stride] = __fmul_rn(v[j], scale);
    }
  }
}

// the stages that are left after `done_bits` of them, on `count` values in shared memory (every thread
// of the CTA calls it)
__device__ __forceinline__ void remaining_passes(float* buf, int count, int log2p, int done_bits, float last_scale) {
  int remaining = log2p - done_bits, stride_bits = done_bits;
  while (remaining > 0) {
    const int stages = remaining >= 3 ? 3 : remaining;
    remaining -= stages;
    const float scale = remaining == 0 ? last_scale : 1.0f;
    const int groups = count >> stages;
    if (stages == 3) butterfly_pass<3>(buf, groups, 1 << stride_bits, stride_bits, scale);
    else if (stages == 2) butterfly_pass<2>(buf, groups, 1 << stride_bits, stride_bits, scale);
    else butterfly_pass<1>(buf, groups, 1 << stride_bits, stride_bits, scale);
    stride_bits += stages;
    __syncthreads();
  }
}

// The first `front` (4..9) stages on the 512 values a warp holds, sixteen consecutive ones per lane:
// strides 1..8 inside the lane, strides 16..256 between lanes.
__device__ __forceinline__ void warp_butterflies16(float (&v)[kWarpRun], int lane, int front) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int span = 1 << s;
#pragma unroll
    for (int j = 0; j < kWarpRun; ++j) {
      if ((j & span) == 0) {
        const float low = v[j], high = v[j + span];
        v[j] = __fadd_rn(low, high);
        v[j + span] = __fsub_rn(low, high);
      }
    }
  }
#pragma unroll
  for (int s = 4; s < kWarpBits; ++s) {
    if (s < front) {
      const int mask = 1 << (s - 4);
      // the lane with the bit clear keeps low + high, its partner low - high: one rounding of
      // (+-own + other), the same value as the add or the subtract
      const float sign = (lane & mask) ? -1.0f : 1.0f;
#pragma unroll
      for (int j = 0; j < kWarpRun; ++j) v[j] = __fmaf_rn(v[j], sign, __shfl_xor_sync(0xffffffffu, v[j], mask));
    }
  }
}

// The same stages for a warp that holds its 512 values as four groups of four consecutive ones, 128 apart:
// value v[4 * m + j] is element 128 * m + 4 * lane + j.  Strides 1 and 2 stay inside a group, strides 4..64
// are lane exchanges, strides 128 and 256 pair the groups; the order is still ascending.  Loads and stores of
// a group are 32 lanes x 4 consecutive values: fully coalesced in global memory, conflict-free in shared memory.
__device__ __forceinline__ void warp_butterflies4x4(float (&v)[kWarpRun], int lane, int front) {
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (s < front) {
      const int span = 1 << s;
#pragma unroll
      for (int j = 0; j < kWarpRun; ++j) {
        if ((j & span) == 0) {
          const float low = v[j], high = v[j + span];
          v[j] = __fadd_rn(low, high);
          v[j + span] = __fsub_rn(low, high);
        }
      }
    }
  }
#pragma unroll
  for (int s = 2; s < 7; ++s) {
    if (s < front) {
      const int mask = 1 << (s - 2);
      const float sign = (lane & mask) ? -1.0f : 1.0f;   // the partner with the bit set keeps low - high
#pragma unroll
      for (int j = 0; j < kWarpRun; ++j) v[j] = __fmaf_rn(v[j], sign, __shfl_xor_sync(0xffffffffu, v[j], mask));
    }
  }
#pragma unroll
  for (int s = 7; s < kWarpBits; ++s) {
    if (s < front) {
      const int span = 4 << (s - 7);   // groups m and m ^ 1 (stride 128), then m and m ^ 2 (stride 256)
#pragma unroll
      for (int j = 0; j < kWarpRun; ++j) {
        if ((j & span) == 0) {
          const float low = v[j], high = v[j + span];
          v[j] = __fadd_rn(low, high);
          v[j + span] = __fsub_rn(low, high);
        }
      }
    }
  }
}

}  // namespace mkb
