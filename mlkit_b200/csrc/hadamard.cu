// Fused structured orthogonal transform of activation rows:  y = (B kron H_P)(x * signs).
//
// Three kernels, all with fp32 arithmetic and one rounding to the activation dtype on store.
//  * warp kernel (power-of-two widths that are multiples of 512): a warp owns 512 consecutive values,
//    sixteen per lane.  Strides 1..8 are butterflies between a lane's own registers, strides 16..256
//    are exchanges between lanes (shfl.xor), so nine stages need no shared memory and no barrier; a
//    width of 512 or less goes from global memory to global memory in one sweep.  Wider rows finish
//    the remaining stages in shared memory, three per pass.
//  * row kernel: any other power-of-two width, the whole row in shared memory, three stages per pass.
//  * factor kernel (width = F * P with a dense F x F basis): the transform is a Kronecker product, so
//    the F-point mix and the P-point butterflies commute.  A CTA owns four output blocks of one row:
//    it mixes the F input blocks into its four (reading the row straight from global memory), then
//    runs the butterflies on those 4 * P values.  A row is spread over ceil(F / 4) CTAs with no
//    exchange between them.
// The butterflies pair i with i ^ stride in ascending stride and form (a + b, a - b), the pairing and
// order of a stage-by-stage transform, so power-of-two widths round identically to one; the 1/sqrt(P)
// scale is one multiply after the last stage.
// The reference needs ceil(log2(P)/3) global round trips plus casts, a sign multiply, two transposes
// and a small library matmul for the same result.
#include "hadamard_steps.cuh"

namespace mkb {
namespace {

struct HadamardArgs {
  const void* x;
  const int8_t* signs;
  const float* basis;
  void* y;
  int64_t M;
  int W, factor, pow2, log2p, dtype, inverse;
  float scale;  // fp32(1) / fp32(sqrt(pow2)), or 1
};

__device__ __forceinline__ void depend_on_previous_grid() {
  // programmatic dependent launch: the kernel that follows in the stream (a packed matvec prefetching
  // its weights) may become resident now; this one waits for the producer of its input
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <int COUNT>
__device__ __forceinline__ void load_run(const void* x, int64_t index, int dtype, float* v) {
  // COUNT (8 or 16) consecutive activations starting at a 16-byte boundary
  if (dtype == MKB_F32) {
    const float4* source = reinterpret_cast<const float4*>(static_cast<const float*>(x) + index);
#pragma unroll
    for (int q = 0; q < COUNT / 4; ++q) {
      const float4 four = __ldg(source + q);
      v[4 * q] = four.x; v[4 * q + 1] = four.y; v[4 * q + 2] = four.z; v[4 * q + 3] = four.w;
    }
    return;
  }
  const uint4* source = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + index);
#pragma unroll
  for (int q = 0; q < COUNT / 8; ++q) {
    const uint4 raw = __ldg(source + q);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float2 pair = dtype == MKB_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&words[w]))
                                           : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[w]));
      v[8 * q + 2 * w] = pair.x;
      v[8 * q + 2 * w + 1] = pair.y;
    }
  }
}

template <int COUNT>
__device__ __forceinline__ void store_run(void* y, int64_t index, int dtype, const float* v) {
  if (dtype == MKB_F32) {
    float4* target = reinterpret_cast<float4*>(static_cast<float*>(y) + index);
#pragma unroll
    for (int q = 0; q < COUNT / 4; ++q) target[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    return;
  }
  uint4* target = reinterpret_cast<uint4*>(static_cast<uint16_t*>(y) + index);
#pragma unroll
  for (int q = 0; q < COUNT / 8; ++q) {
    uint32_t words[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      if (dtype == MKB_F16) {
        const __half2 pair = __floats2half2_rn(v[8 * q + 2 * w], v[8 * q + 2 * w + 1]);
        words[w] = *reinterpret_cast<const uint32_t*>(&pair);
      } else {
        const __nv_bfloat162 pair = __floats2bfloat162_rn(v[8 * q + 2 * w], v[8 * q + 2 * w + 1]);
        words[w] = *reinterpret_cast<const uint32_t*>(&pair);
      }
    }
    target[q] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

template <int COUNT>
__device__ __forceinline__ void flip_run(const int8_t* signs, int index, float* v) {
  // multiply by COUNT consecutive +-1 signs (the run starts on a COUNT-byte boundary)
  const uint2* source = reinterpret_cast<const uint2*>(signs + index);
#pragma unroll
  for (int q = 0; q < COUNT / 8; ++q) {
    const uint2 flips = source[q];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t word = j < 4 ? flips.x : flips.y;
      v[8 * q + j] = __fmul_rn(v[8 * q + j], float(int8_t((word >> (8 * (j & 3))) & 0xffu)));
    }
  }
}


// four consecutive activations starting at a multiple of four
__device__ __forceinline__ void load_four(const void* x, int64_t index, int dtype, float* v) {
  if (dtype == MKB_F32) {
    const float4 four = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(x) + index));
    v[0] = four.x; v[1] = four.y; v[2] = four.z; v[3] = four.w;
    return;
  }
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(x) + index));
  const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const float2 pair = dtype == MKB_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&words[w]))
                                         : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[w]));
    v[2 * w] = pair.x;
    v[2 * w + 1] = pair.y;
  }
}

__device__ __forceinline__ uint32_t pack_pair(float low, float high, int dtype) {
  if (dtype == MKB_F16) {
    const __half2 pair = __floats2half2_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
  }
  const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&pair);
}

__device__ __forceinline__ void store_four(void* y, int64_t index, int dtype, const float* v) {
  if (dtype == MKB_F32) {
    *reinterpret_cast<float4*>(static_cast<float*>(y) + index) = make_float4(v[0], v[1], v[2], v[3]);
    return;
  }
  *reinterpret_cast<uint2*>(static_cast<uint16_t*>(y) + index) = make_uint2(pack_pair(v[0], v[1], dtype), pack_pair(v[2], v[3], dtype));
}

__device__ __forceinline__ void flip_four(const int8_t* signs, int index, float* v) {
  // a sign of -1 is the byte 0xff: its top bit, moved to bit 31, flips the value's sign, which is what the
  // multiplication by +-1 does, bit for bit
  const uint32_t word = *reinterpret_cast<const uint32_t*>(signs + index);
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __uint_as_float(__float_as_uint(v[j]) ^ ((word << (24 - 8 * j)) & 0x80000000u));
}

// The last one to three stages, fused with the scale, the inverse sign flip and the store: a thread takes two
// neighbouring columns of a butterfly group (8-byte shared loads), so a warp stores 32 consecutive pairs.
template <int STAGES>
__device__ __forceinline__ void final_pass_store(const float* buf, const HadamardArgs& a, int64_t offset, int stride_bits) {
  const int stride = 1 << stride_bits, pairs = a.W >> (STAGES + 1);
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
    const int grp = 2 * pair, low = grp & (stride - 1);
    const int base = ((grp >> stride_bits) << (stride_bits + STAGES)) + low;
    float2 v[1 << STAGES];
#pragma unroll
    for (int j = 0; j < (1 << STAGES); ++j) v[j] = *reinterpret_cast<const float2*>(buf + base + j * stride);
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      const int span = 1 << s;
#pragma unroll
      for (int j = 0; j < (1 << STAGES); ++j) {
        if ((j & span) == 0) {
          const float2 p = v[j], q = v[j + span];
          v[j] = make_float2(__fadd_rn(p.x, q.x), __fadd_rn(p.y, q.y));
          v[j + span] = make_float2(__fsub_rn(p.x, q.x), __fsub_rn(p.y, q.y));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < (1 << STAGES); ++j) {
      const int at = base + j * stride;
      float x0 = __fmul_rn(v[j].x, a.scale), x1 = __fmul_rn(v[j].y, a.scale);
      if (a.signs != nullptr && a.inverse) {
        x0 = __fmul_rn(x0, float(a.signs[at]));
        x1 = __fmul_rn(x1, float(a.signs[at + 1]));
      }
      if (a.dtype == MKB_F32) *reinterpret_cast<float2*>(static_cast<float*>(a.y) + offset + at) = make_float2(x0, x1);
      else *reinterpret_cast<uint32_t*>(static_cast<uint16_t*>(a.y) + offset + at) = pack_pair(x0, x1, a.dtype);
    }
  }
}

__global__ void __launch_bounds__(1024) hadamard_warp_kernel(HadamardArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  depend_on_previous_grid();
  float* buf = smem_f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int64_t offset = int64_t(blockIdx.x) * a.W;
  const int front = a.log2p < kWarpBits ? a.log2p : kWarpBits;
  const bool direct = a.log2p <= kWarpBits;
  for (int chunk = warp; chunk < a.W / kWarpSpan; chunk += warps) {
    const int first = chunk * kWarpSpan + lane * 4;     // group m of the lane starts at first + 128 * m
    float v[kWarpRun];
#pragma unroll
    for (int m = 0; m < 4; ++m) load_four(a.x, offset + first + 128 * m, a.dtype, v + 4 * m);
    if (a.signs != nullptr && !a.inverse) {
#pragma unroll
      for (int m = 0; m < 4; ++m) flip_four(a.signs, first + 128 * m, v + 4 * m);
    }
    warp_butterflies4x4(v, lane, front);
    if (direct) {
#pragma unroll
      for (int j = 0; j < kWarpRun; ++j) v[j] = __fmul_rn(v[j], a.scale);
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        if (a.signs != nullptr && a.inverse) flip_four(a.signs, first + 128 * m, v + 4 * m);
        store_four(a.y, offset + first + 128 * m, a.dtype, v + 4 * m);
      }
    } else {
#pragma unroll
      for (int m = 0; m < 4; ++m)
        *reinterpret_cast<float4*>(buf + first + 128 * m) = make_float4(v[4 * m], v[4 * m + 1], v[4 * m + 2], v[4 * m + 3]);
    }
  }
  if (direct) return;
  __syncthreads();
  // all but the last pass in shared memory, three stages each; the last one to three stages go straight out
  int remaining = a.log2p - kWarpBits, stride_bits = kWarpBits;
  while (remaining > 3) {
    butterfly_pass<3>(buf, a.W >> 3, 1 << stride_bits, stride_bits, 1.0f);
    stride_bits += 3;
    remaining -= 3;
    __syncthreads();
  }
  if (remaining == 3) final_pass_store<3>(buf, a, offset, stride_bits);
  else if (remaining == 2) final_pass_store<2>(buf, a, offset, stride_bits);
  else final_pass_store<1>(buf, a, offset, stride_bits);
}

__global__ void hadamard_kernel(HadamardArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  depend_on_previous_grid();
  float* buf = smem_f;               // [W]
  const int64_t offset = int64_t(blockIdx.x) * a.W;
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    float v = load_as_float(a.x, offset + i, a.dtype);
    if (a.signs != nullptr && !a.inverse) v = __fmul_rn(v, float(a.signs[i]));
    buf[i] = v;
  }
  __syncthreads();
  remaining_passes(buf, a.W, a.log2p, 0, a.scale);
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    float v = buf[i];
    if (a.signs != nullptr && a.inverse) v = __fmul_rn(v, float(a.signs[i]));
    store_from_float(a.y, offset + i, a.dtype, v);
  }
}

__global__ void hadamard_factor_kernel(HadamardArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  depend_on_previous_grid();
  const int P = a.pow2, F = a.factor;
  float* buf = smem_f;                                         // [4][P]: this CTA's four output blocks
  float4* mix = reinterpret_cast<float4*>(smem_f + 4 * ((P + 3) & ~3));   // [F]: the four basis columns
  const int64_t offset = int64_t(blockIdx.x) * a.W;
  const int quad = blockIdx.y;
  // mix[f][j] multiplies input block f into output block 4 * quad + j
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float m[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int fo = 4 * quad + j;
      m[j] = fo < F ? (a.inverse ? a.basis[f * F + fo] : a.basis[fo * F + f]) : 0.f;
    }
    mix[f] = make_float4(m[0], m[1], m[2], m[3]);
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int f = 0; f < F; ++f) {      // f in ascending order
      float h = load_as_float(a.x, offset + f * P + p, a.dtype);
      if (a.signs != nullptr && !a.inverse) h = __fmul_rn(h, float(a.signs[f * P + p]));
      const float4 m = mix[f];
      acc[0] = fmaf(m.x, h, acc[0]);
      acc[1] = fmaf(m.y, h, acc[1]);
      acc[2] = fmaf(m.z, h, acc[2]);
      acc[3] = fmaf(m.w, h, acc[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) buf[j * P + p] = acc[j];
  }
  __syncthreads();
  remaining_passes(buf, 4 * P, a.log2p, 0, a.scale);
  for (int i = threadIdx.x; i < 4 * P; i += blockDim.x) {
    const int fo = 4 * quad + (i >> a.log2p), p = i & (P - 1);
    if (fo < F) {
      const int at = fo * P + p;
      float value = buf[i];
      if (a.inverse && a.signs != nullptr) value = __fmul_rn(value, float(a.signs[at]));
      store_from_float(a.y, offset + at, a.dtype, value);
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
  HadamardArgs a{};
  a.x = x; a.signs = signs; a.basis = basis; a.y = y; a.M = M;
  a.W = W; a.factor = factor; a.pow2 = pow2; a.dtype = dtype; a.inverse = inverse;
  a.log2p = 0;
  while ((1 << a.log2p) < pow2) ++a.log2p;
  // the reference forms the scale in fp32: float(torch.tensor(1.0) / torch.tensor(math.sqrt(width)))
  a.scale = normalize ? 1.0f / float(sqrt(double(pow2))) : 1.0f;
  const auto aligned = [](const void* p, uintptr_t to) { return reinterpret_cast<uintptr_t>(p) % to == 0; };
  const bool by_warp = factor == 1 && W % kWarpSpan == 0 && aligned(x, 16) && aligned(y, 16) &&
                       (signs == nullptr || aligned(signs, 4));
  void (*kernel)(HadamardArgs) = factor > 1 ? hadamard_factor_kernel : by_warp ? hadamard_warp_kernel : hadamard_kernel;
  size_t smem;
  dim3 grid((unsigned)M);
  int threads;
  if (factor > 1) {
    smem = (size_t(4) * ((pow2 + 3) & ~3) + size_t(4) * factor) * sizeof(float);
    grid.y = (factor + 3) / 4;
    threads = pow2 >= 1024 ? 1024 : pow2 >= 128 ? pow2 : 128;
  } else if (by_warp) {
    smem = a.log2p <= kWarpBits ? 0 : size_t(W) * sizeof(float);
    threads = W / kWarpRun >= 1024 ? 1024 : W / kWarpRun;
  } else {
    smem = size_t((W + 3) & ~3) * sizeof(float);
    threads = W >= 8192 ? 1024 : W >= 4096 ? 512 : W >= 1024 ? 256 : 128;
  }
  const DeviceInfo& info = device_info();
  MKB_REQUIRE(smem <= size_t(info.max_smem_optin), MKB_E_UNSUPPORTED,
              "hadamard: width %d needs %zu B shared memory", W, smem);
  const int which = factor > 1 ? 2 : by_warp ? 1 : 0;
  static thread_local bool opted[64][3];
  int device = 0;
  cudaGetDevice(&device);
  if (smem > 48 * 1024 && !(device >= 0 && device < 64 && opted[device][which])) {
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, info.max_smem_optin);
    if (status != cudaSuccess) return cuda_fail(status, "hadamard: shared memory opt-in");
    if (device >= 0 && device < 64) opted[device][which] = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = smem;
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t launched = cudaLaunchKernelEx(&config, kernel, a);
  if (launched != cudaSuccess) return cuda_fail(launched, "hadamard launch");
  return MKB_OK;
}
