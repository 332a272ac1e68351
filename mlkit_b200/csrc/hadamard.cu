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
  int W, factor, pow2, log2p, dtype, inverse;
  float scale;  // fp32(1) / fp32(sqrt(pow2)), or 1
};

template <int STAGES>
__device__ __forceinline__ void butterfly_pass(float* buf, int groups, int stride, int stride_bits, float scale) {
  for (int grp = threadIdx.x; grp < groups; grp += blockDim.x) {
    const int low = grp & (stride - 1);
    const int base = ((grp >> stride_bits) << (stride_bits + STAGES)) + low;
    float v[1 << STAGES];
#pragma unroll
    for (int j = 0; j < (1 << STAGES); ++j) v[j] = buf[base + j * stride];
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
#pragma unroll
    for (int j = 0; j < (1 << STAGES); ++j) buf[base + j * stride] = __fmul_rn(v[j], scale);
  }
}

__global__ void hadamard_kernel(HadamardArgs a) {
  extern __shared__ __align__(16) float smem_f[];
  float* buf = smem_f;               // [W]
  float* basis_s = smem_f + a.W;     // [factor * factor] when factor > 1
  const int64_t row = blockIdx.x;
  const int64_t offset = row * a.W;

  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    float v = load_as_float(a.x, offset + i, a.dtype);
    if (a.signs != nullptr && !a.inverse) v = __fmul_rn(v, float(a.signs[i]));
    buf[i] = v;
  }
  if (a.factor > 1)
    for (int i = threadIdx.x; i < a.factor * a.factor; i += blockDim.x) basis_s[i] = a.basis[i];
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
    for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
      float v = buf[i];
      if (a.signs != nullptr && a.inverse) v = __fmul_rn(v, float(a.signs[i]));
      store_from_float(a.y, offset + i, a.dtype, v);
    }
    return;
  }
  // y[f', p] = sum_f B[f', f] h[f, p]   (inverse: B[f, f'])
  const int P = a.pow2, F = a.factor;
  for (int i = threadIdx.x; i < a.W; i += blockDim.x) {
    const int fo = i / P, p = i - fo * P;
    float acc = 0.f;
    if (!a.inverse) {
      for (int f = 0; f < F; ++f) acc = fmaf(basis_s[fo * F + f], buf[f * P + p], acc);
    } else {
      for (int f = 0; f < F; ++f) acc = fmaf(basis_s[f * F + fo], buf[f * P + p], acc);
      if (a.signs != nullptr) acc = __fmul_rn(acc, float(a.signs[i]));
    }
    store_from_float(a.y, offset + i, a.dtype, acc);
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
  const size_t smem = (size_t(W) + (factor > 1 ? size_t(factor) * factor : 0)) * sizeof(float);
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
  a.log2p = 0;
  while ((1 << a.log2p) < pow2) ++a.log2p;
  // the reference forms the scale in fp32: float(torch.tensor(1.0) / torch.tensor(math.sqrt(width)))
  a.scale = normalize ? 1.0f / float(sqrt(double(pow2))) : 1.0f;
  int threads = W >= 4096 ? 512 : W >= 1024 ? 256 : 128;
  hadamard_kernel<<<dim3((unsigned)M), threads, smem, static_cast<cudaStream_t>(stream)>>>(a);
  MKB_LAUNCH_CHECK("hadamard launch");
  return MKB_OK;
}
