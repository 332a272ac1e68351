// Fused structured orthogonal transform of activation rows:  y = (B kron H_P)(x * signs).
//
// One CTA owns one row.  The row lives in shared memory as fp32 for the whole transform: sign
// flip on load, Walsh-Hadamard butterflies in ascending stride with three stages per pass (the
// same pairing and order as a stage-by-stage transform, so sums and differences round
// identically), the 1/sqrt(P) scale folded into the last pass as one multiply, the dense
// factor-by-factor mix across the blocks, and one rounding to the activation dtype on store.
// The reference needs ceil(log2(P)/3) global round trips plus casts, a sign multiply, two
// transposes and a small library matmul for the same result.
#include "mkb_common.cuh"

namespace mkb {
namespace {

struct HadamardArgs {
  const void* x;
  const int8_t* signs;
  const float* basis;
  void* y;
  int64_t M;
  int W, factor, pow2, log2p, dtype, inverse, vector_io;
  float scale;  // fp32(1) / fp32(sqrt(pow2)), or 1
};

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

__global__ void hadamard_kernel(HadamardArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  float* buf = smem_f;               // [W]
  float* basis_s = smem_f + ((a.W + 3) & ~3);   // [factor][factor padded to 4] when factor > 1; 16-byte aligned
  const int64_t row = blockIdx.x;
  const int64_t offset = row * a.W;

  if (a.vector_io) {
    // 16-bit activations, eight per 16-byte access
    const uint4* source = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.x) + offset);
    for (int i = threadIdx.x; i < a.W / 8; i += blockDim.x) {
      const uint4 raw = __ldg(source + i);
      const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
      float v[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 pair = a.dtype == MKB_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&words[q]))
                                               : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[q]));
        v[2 * q] = pair.x;
        v[2 * q + 1] = pair.y;
      }
      if (a.signs != nullptr && !a.inverse) {
        const uint2 flips = *reinterpret_cast<const uint2*>(a.signs + 8 * i);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const uint32_t word = q < 4 ? flips.x : flips.y;
          v[q] = __fmul_rn(v[q], float(int8_t((word >> (8 * (q & 3))) & 0xffu)));
        }
      }
      *reinterpret_cast<float4*>(buf + 8 * i) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(buf + 8 * i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
  } else {
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
      float v = load_as_float(a.x, offset + i, a.dtype);
      if (a.signs != nullptr && !a.inverse) v = __fmul_rn(v, float(a.signs[i]));
      buf[i] = v;
    }
  }
  // the factor mix, laid out [f][f' padded to 4]: mix[f][f'] multiplies h[f, :] into y[f', :]
  const int F4 = (a.factor + 3) & ~3;
  if (a.factor > 1)
    for (int i = threadIdx.x; i < a.factor * F4; i += blockDim.x) {
      const int f = i / F4, fo = i - f * F4;
      basis_s[i] = fo < a.factor ? (a.inverse ? a.basis[f * a.factor + fo] : a.basis[fo * a.factor + f]) : 0.f;
    }
  __syncthreads();

  int remaining = a.log2p, stride_bits = 0;
  while (remaining > 0) {
    const int stages = remaining >= 3 ? 3 : remaining;
    remaining -= stages;
    const float scale = remaining == 0 ? a.scale : 1.0f;
    const int groups = a.W >> stages;
    if (stages == 3) butterfly_pass<3>(buf, groups, 1 << stride_bits, stride_bits, scale);
    else if (stages == 2) butterfly_pass<2>(buf, groups, 1 << stride_bits, stride_bits, scale);
    else butterfly_pass<1>(buf, groups, 1 << stride_bits, stride_bits, scale);
    stride_bits += stages;
    __syncthreads();
  }

  if (a.factor == 1) {
    if (a.vector_io) {
      uint4* target = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.y) + offset);
      for (int i = threadIdx.x; i < a.W / 8; i += blockDim.x) {
        const float4 lo = *reinterpret_cast<const float4*>(buf + 8 * i), hi = *reinterpret_cast<const float4*>(buf + 8 * i + 4);
        float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        if (a.signs != nullptr && a.inverse) {
#pragma unroll
          for (int q = 0; q < 8; ++q) v[q] = __fmul_rn(v[q], float(a.signs[8 * i + q]));
        }
        uint32_t words[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (a.dtype == MKB_F16) {
            const __half2 pair = __floats2half2_rn(v[2 * q], v[2 * q + 1]);
            words[q] = *reinterpret_cast<const uint32_t*>(&pair);
          } else {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
            words[q] = *reinterpret_cast<const uint32_t*>(&pair);
          }
        }
        target[i] = make_uint4(words[0], words[1], words[2], words[3]);
      }
      return;
    }
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
      float v = buf[i];
      if (a.signs != nullptr && a.inverse) v = __fmul_rn(v, float(a.signs[i]));
      store_from_float(a.y, offset + i, a.dtype, v);
    }
    return;
  }
  // y[f', p] = sum_f mix[f][f'] h[f, p]: a thread forms four f' for one p, so one 16-byte broadcast
  // read of the mix and one read of h feed four multiply-adds; f runs in ascending order
  const int P = a.pow2, F = a.factor;
  for (int task = threadIdx.x; task < (F4 / 4) * P; task += blockDim.x) {
    const int quad = task / P, p = task - quad * P;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int f = 0; f < F; ++f) {
      const float4 m = *reinterpret_cast<const float4*>(basis_s + f * F4 + 4 * quad);
      const float h = buf[f * P + p];
      acc[0] = fmaf(m.x, h, acc[0]);
      acc[1] = fmaf(m.y, h, acc[1]);
      acc[2] = fmaf(m.z, h, acc[2]);
      acc[3] = fmaf(m.w, h, acc[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int fo = 4 * quad + j;
      if (fo < F) {
        const int i = fo * P + p;
        float value = acc[j];
        if (a.inverse && a.signs != nullptr) value = __fmul_rn(value, float(a.signs[i]));
        store_from_float(a.y, offset + i, a.dtype, value);
      }
    }
  }
}

}  // namespace
}  // namespace mkb

extern "C" int mkb_hadamard(const void* x, const int8_t* signs, const float* basis, void* y, int64_t M,
                            int W, int factor, int pow2, int dtype, int inverse, int normalize,
                            void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 0 && W >= 1, MKB_E_ARGUMENT, "hadamard: bad shape");
  MKB_REQUIRE(factor >= 1 && pow2 >= 1 && int64_t(factor) * pow2 == W, MKB_E_ARGUMENT,
              "hadamard: factor * pow2 != width");
  MKB_REQUIRE((pow2 & (pow2 - 1)) == 0, MKB_E_UNSUPPORTED, "hadamard: pow2=%d is not a power of two", pow2);
  MKB_REQUIRE(factor == 1 || basis != nullptr, MKB_E_ARGUMENT, "hadamard: factor > 1 needs a basis");
  MKB_REQUIRE(dtype >= MKB_F16 && dtype <= MKB_F32, MKB_E_ARGUMENT, "hadamard: unknown dtype");
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(x != nullptr && y != nullptr, MKB_E_ARGUMENT, "hadamard: null pointer");
  MKB_REQUIRE(M <= 0x7fffffffLL, MKB_E_UNSUPPORTED, "hadamard: too many rows");
  const size_t smem = (size_t((W + 3) & ~3) + (factor > 1 ? size_t(factor) * ((factor + 3) & ~3) : 0)) * sizeof(float);
  const DeviceInfo& info = device_info();
  MKB_REQUIRE(smem <= size_t(info.max_smem_optin), MKB_E_UNSUPPORTED,
              "hadamard: width %d needs %zu B shared memory", W, smem);
  static thread_local size_t opted[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && smem > 48 * 1024 && smem > opted[device]) {
    cudaError_t status = cudaFuncSetAttribute(hadamard_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              info.max_smem_optin);
    if (status != cudaSuccess) return cuda_fail(status, "hadamard: shared memory opt-in");
    opted[device] = size_t(info.max_smem_optin);
  }
  HadamardArgs a{};
  a.x = x; a.signs = signs; a.basis = basis; a.y = y; a.M = M;
  a.W = W; a.factor = factor; a.pow2 = pow2; a.dtype = dtype; a.inverse = inverse;
  a.vector_io = dtype != MKB_F32 && W % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(y) % 16 == 0 && (signs == nullptr || reinterpret_cast<uintptr_t>(signs) % 8 == 0);
  a.log2p = 0;
  while ((1 << a.log2p) < pow2) ++a.log2p;
  // the reference forms the scale in fp32: float(torch.tensor(1.0) / torch.tensor(math.sqrt(width)))
  a.scale = normalize ? 1.0f / float(sqrt(double(pow2))) : 1.0f;
  int threads = W >= 8192 ? 1024 : W >= 4096 ? 512 : W >= 1024 ? 256 : 128;
  hadamard_kernel<<<dim3((unsigned)M), threads, smem, static_cast<cudaStream_t>(stream)>>>(a);
  MKB_LAUNCH_CHECK("hadamard launch");
  return MKB_OK;
}
