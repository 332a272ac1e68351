// Word-at-a-time packed matvec: the kernel that covers every layout the reference's fused kernel
// accepts (any width of 1..8 bits, any group that holds whole packing words, ragged K, fp16 / bf16 /
// fp32 activations and scales, offsets, bias).  It is the coverage kernel, not the fast one: the
// register-tiled kernel in gemv_tiled.cu takes the shapes that matter for throughput.
//
// One warp owns one output row.  Lanes stride over the packing words of the row; a lane assembles
// its word from bytes, expands the codes, forms w = lut[c] * scale (+ zero) in fp32 exactly like the
// reference kernel does, and multiplies by up to eight activation rows.  Lane partials meet in a
// shuffle tree; lane 0 adds the bias and stores in the activation dtype.
#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kWarps = 8;

struct ScalarArgs {
  const void* x;
  const uint8_t* packed;
  const void* scales;
  const float* lut;
  const void* zeros;
  const void* bias;
  void* y;
  int M, N, K, group, bits, lut_len, x_dtype, scale_dtype;
  int64_t packed_row_stride, scale_row_stride;
};

template <int MT>
__global__ void __launch_bounds__(kWarps * 32) gemv_scalar_kernel(ScalarArgs a) {
  __shared__ float lut_s[256];
  for (int i = threadIdx.x; i < 256; i += kWarps * 32) lut_s[i] = i < a.lut_len ? a.lut[i] : 0.f;
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (row >= a.N) return;

  const int wb = word_bytes(a.bits), wc = word_codes(a.bits);
  const int words = a.K / wc;
  const uint32_t mask = (1u << a.bits) - 1u;
  const uint8_t* row_bytes = a.packed + int64_t(row) * a.packed_row_stride;
  const bool has_zero = a.zeros != nullptr;

  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;

  for (int w = lane; w < words; w += 32) {
    uint64_t word = 0;
    const uint8_t* p = row_bytes + int64_t(w) * wb;
    for (int b = 0; b < wb; ++b) word |= uint64_t(__ldg(p + b)) << (8 * b);
    const int k0 = w * wc;
    const int64_t s_index = int64_t(row) * a.scale_row_stride + k0 / a.group;
    const float scale = load_as_float(a.scales, s_index, a.scale_dtype);
    const float zero = has_zero ? load_as_float(a.zeros, s_index, a.scale_dtype) : 0.f;
    for (int c = 0; c < wc; ++c) {
      const float value = lut_s[(word >> (c * a.bits)) & mask];
      const float weight = has_zero ? reconstruct(value, scale, zero) : reconstruct(value, scale);
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m < a.M) acc[m] = fmaf(weight, load_as_float(a.x, int64_t(m) * a.K + k0 + c, a.x_dtype), acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
    for (int offset = 16; offset; offset >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], offset);
  if (lane == 0) {
    const float b = a.bias ? load_as_float(a.bias, row, a.x_dtype) : 0.f;
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < a.M) store_from_float(a.y, int64_t(m) * a.N + row, a.x_dtype, acc[m] + b);
  }
}

}  // namespace

int gemv_scalar_supported(int K, int group, int bits) {
  if (bits < 1 || bits > 8) return 0;
  const int wc = word_codes(bits);
  return K % wc == 0 && group % wc == 0;
}

int launch_gemv_scalar(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                       const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                       int bits, int lut_len, int x_dtype, int scale_dtype, int64_t packed_row_stride,
                       int64_t scale_row_stride, cudaStream_t stream) {
  ScalarArgs a{x, packed, scales, lut, zeros, bias, y, M, N, K, group, bits, lut_len, x_dtype,
               scale_dtype, packed_row_stride, scale_row_stride};
  const dim3 grid((N + kWarps - 1) / kWarps);
  if (M == 1) gemv_scalar_kernel<1><<<grid, kWarps * 32, 0, stream>>>(a);
  else if (M == 2) gemv_scalar_kernel<2><<<grid, kWarps * 32, 0, stream>>>(a);
  else if (M <= 4) gemv_scalar_kernel<4><<<grid, kWarps * 32, 0, stream>>>(a);
  else gemv_scalar_kernel<8><<<grid, kWarps * 32, 0, stream>>>(a);
  MKB_LAUNCH_CHECK("gemv_scalar launch");
  return MKB_OK;
}

}  // namespace mkb
