// Bit-exact unpack + dequantisation of packed scalar codes.
//
// One thread owns eight consecutive codes.  Eight codes of `bits` bits occupy exactly `bits`
// bytes and start on a byte boundary whatever the width, so every thread reads a private,
// byte-aligned run and never needs its neighbour's bits.  The weight is formed as
// lut[code] * scale (+ zero) with separate IEEE multiply and add and rounded once on store.
#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kThreads = 256;

template <int BITS>
__device__ __forceinline__ uint64_t load_run(const uint8_t* __restrict__ p, int64_t valid_bytes,
                                             bool aligned) {
  // valid_bytes: bytes that exist from p onward (clamped by the caller to >= 1)
  uint64_t w = 0;
  if (valid_bytes >= BITS && aligned) {
    if constexpr (BITS == 8) {
      uint2 v = __ldg(reinterpret_cast<const uint2*>(p));
      return (uint64_t(v.y) << 32) | v.x;
    } else if constexpr (BITS == 4) {
      return __ldg(reinterpret_cast<const uint32_t*>(p));
    } else if constexpr (BITS == 2) {
      return __ldg(reinterpret_cast<const uint16_t*>(p));
    }
  }
#pragma unroll
  for (int b = 0; b < BITS; ++b)
    if (b < valid_bytes) w |= uint64_t(__ldg(p + b)) << (8 * b);
  return w;
}

template <typename OUT>
__device__ __forceinline__ OUT narrow(float v);
template <>
__device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float narrow<float>(float v) { return v; }

template <typename OUT>
struct alignas(sizeof(OUT) * 8) Pack8 { OUT v[8]; };

struct DequantArgs {
  const uint8_t* packed;
  const void* scales;
  const float* lut;
  const void* zeros;
  void* w_out;
  uint8_t* codes_out;
  const int64_t* rows;  // row gather list, or null for the flat stream
  int64_t count;        // gathered rows
  int64_t N, K;
  int64_t scale_row_stride;
  int64_t total_bytes;  // bytes in the stream
  int group, bits, lut_len, scale_dtype;
  int uniform;          // eight codes of a thread share row and group
  int aligned;          // packed base allows the vector loads
};

// FLAT: thread t owns flat codes [8t, 8t+8) of the whole [N,K] stream.
// !FLAT: thread owns chunk c of gathered row i: codes [8c, 8c+8) of row rows[i].
template <int BITS, typename OUT, bool FLAT>
__global__ void __launch_bounds__(kThreads) dequant_kernel(DequantArgs a) {
  __shared__ float lut_s[256];
  for (int i = threadIdx.x; i < 256; i += kThreads) lut_s[i] = i < a.lut_len ? a.lut[i] : 0.f;
  __syncthreads();

  const int64_t tid = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  int64_t row, col, out_base, byte_offset, valid_bytes;
  int live;  // codes of this thread that exist
  if constexpr (FLAT) {
    const int64_t total = a.N * a.K;
    const int64_t first = tid * 8;
    if (first >= total) return;
    live = int(total - first < 8 ? total - first : 8);
    row = first / a.K;
    col = first - row * a.K;
    out_base = first;
    byte_offset = tid * BITS;
    valid_bytes = a.total_bytes - byte_offset;
  } else {
    const int64_t chunks = (a.K + 7) / 8;
    const int64_t i = tid / chunks;
    if (i >= a.count) return;
    const int64_t chunk = tid - i * chunks;
    row = a.rows[i];
    col = chunk * 8;
    live = int(a.K - col < 8 ? a.K - col : 8);
    out_base = i * a.K + col;
    const int64_t row_bytes = a.K * BITS / 8;
    byte_offset = row * row_bytes + chunk * BITS;
    valid_bytes = row_bytes - chunk * BITS;
    if (row < 0 || row >= a.N) return;
  }
  const uint64_t run = load_run<BITS>(a.packed + byte_offset, valid_bytes, a.aligned != 0);
  constexpr uint32_t mask = (1u << BITS) - 1u;

  uint8_t codes[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) codes[e] = uint8_t((run >> (e * BITS)) & mask);

  if (a.codes_out != nullptr) {
    if (live == 8 && (out_base & 7) == 0) {
      uint2 v;
      v.x = codes[0] | (codes[1] << 8) | (codes[2] << 16) | (uint32_t(codes[3]) << 24);
      v.y = codes[4] | (codes[5] << 8) | (codes[6] << 16) | (uint32_t(codes[7]) << 24);
      *reinterpret_cast<uint2*>(a.codes_out + out_base) = v;
    } else {
      for (int e = 0; e < live; ++e) a.codes_out[out_base + e] = codes[e];
    }
  }
  if (a.w_out == nullptr) return;

  OUT* out = reinterpret_cast<OUT*>(a.w_out);
  const bool has_zero = a.zeros != nullptr;
  if (a.uniform && live == 8) {
    const int64_t s_index = row * a.scale_row_stride + col / a.group;
    const float scale = load_as_float(a.scales, s_index, a.scale_dtype);
    const float zero = has_zero ? load_as_float(a.zeros, s_index, a.scale_dtype) : 0.f;
    Pack8<OUT> result;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float value = lut_s[codes[e]];
      result.v[e] = narrow<OUT>(has_zero ? reconstruct(value, scale, zero) : reconstruct(value, scale));
    }
    if ((reinterpret_cast<uintptr_t>(out + out_base) & (sizeof(Pack8<OUT>) - 1)) == 0) {
      *reinterpret_cast<Pack8<OUT>*>(out + out_base) = result;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) out[out_base + e] = result.v[e];
    }
    return;
  }
  for (int e = 0; e < live; ++e) {
    int64_t r = row, c = col + e;
    if constexpr (FLAT) {
      while (c >= a.K) { c -= a.K; ++r; }
    }
    const int64_t s_index = r * a.scale_row_stride + c / a.group;
    const float scale = load_as_float(a.scales, s_index, a.scale_dtype);
    const float value = lut_s[codes[e]];
    const float w = has_zero ? reconstruct(value, scale, load_as_float(a.zeros, s_index, a.scale_dtype))
                             : reconstruct(value, scale);
    out[out_base + e] = narrow<OUT>(w);
  }
}

template <int BITS, bool FLAT>
int launch_typed(const DequantArgs& a, int out_dtype, int64_t threads, cudaStream_t stream) {
  const int64_t blocks = (threads + kThreads - 1) / kThreads;
  MKB_REQUIRE(blocks <= 0x7fffffffLL, MKB_E_UNSUPPORTED, "dequant: %lld blocks exceed the grid limit",
              (long long)blocks);
  if (blocks == 0) return MKB_OK;
  const dim3 grid((unsigned)blocks);
  switch (out_dtype) {
    case MKB_F16: dequant_kernel<BITS, __half, FLAT><<<grid, kThreads, 0, stream>>>(a); break;
    case MKB_BF16: dequant_kernel<BITS, __nv_bfloat16, FLAT><<<grid, kThreads, 0, stream>>>(a); break;
    default: dequant_kernel<BITS, float, FLAT><<<grid, kThreads, 0, stream>>>(a); break;
  }
  MKB_LAUNCH_CHECK("dequant launch");
  return MKB_OK;
}

template <bool FLAT>
int launch_bits(const DequantArgs& a, int out_dtype, int64_t threads, cudaStream_t stream) {
  switch (a.bits) {
    case 1: return launch_typed<1, FLAT>(a, out_dtype, threads, stream);
    case 2: return launch_typed<2, FLAT>(a, out_dtype, threads, stream);
    case 3: return launch_typed<3, FLAT>(a, out_dtype, threads, stream);
    case 4: return launch_typed<4, FLAT>(a, out_dtype, threads, stream);
    case 5: return launch_typed<5, FLAT>(a, out_dtype, threads, stream);
    case 6: return launch_typed<6, FLAT>(a, out_dtype, threads, stream);
    case 7: return launch_typed<7, FLAT>(a, out_dtype, threads, stream);
    default: return launch_typed<8, FLAT>(a, out_dtype, threads, stream);
  }
}

int check_common(const uint8_t* packed, const void* scales, const float* lut, int64_t N, int64_t K,
                 int group, int bits, int lut_len, int scale_dtype, int out_dtype, bool need_params) {
  MKB_REQUIRE(N >= 0 && K >= 0, MKB_E_ARGUMENT, "dequant: negative shape");
  MKB_REQUIRE(bits >= 1 && bits <= 8, MKB_E_UNSUPPORTED, "dequant: bits=%d outside 1..8", bits);
  MKB_REQUIRE(out_dtype >= MKB_F16 && out_dtype <= MKB_F32, MKB_E_ARGUMENT, "dequant: unknown out dtype");
  if (N * K == 0) return MKB_OK;
  MKB_REQUIRE(packed != nullptr, MKB_E_ARGUMENT, "dequant: packed is null");
  if (need_params) {
    MKB_REQUIRE(scales != nullptr && lut != nullptr, MKB_E_ARGUMENT, "dequant: scales or lut is null");
    MKB_REQUIRE(group >= 1, MKB_E_ARGUMENT, "dequant: group must be positive");
    MKB_REQUIRE(lut_len >= 1 && lut_len <= (1 << bits), MKB_E_ARGUMENT,
                "dequant: lut_len=%d does not fit %d-bit codes", lut_len, bits);
    MKB_REQUIRE(scale_dtype >= MKB_F16 && scale_dtype <= MKB_F32, MKB_E_ARGUMENT,
                "dequant: unknown scale dtype");
  }
  return MKB_OK;
}

}  // namespace
}  // namespace mkb

extern "C" int mkb_dequant(const uint8_t* packed, const void* scales, const float* lut,
                           const void* zeros, void* w_out, uint8_t* codes_out, int64_t N, int64_t K,
                           int group, int bits, int lut_len, int scale_dtype, int out_dtype,
                           int64_t scale_row_stride, void* stream) {
  using namespace mkb;
  int status = check_common(packed, scales, lut, N, K, group, bits, lut_len, scale_dtype, out_dtype,
                            w_out != nullptr);
  if (status != MKB_OK || N * K == 0) return status;
  MKB_REQUIRE(w_out != nullptr || codes_out != nullptr, MKB_E_ARGUMENT, "dequant: no output requested");
  DequantArgs a{};
  a.packed = packed; a.scales = scales; a.lut = lut; a.zeros = zeros;
  a.w_out = w_out; a.codes_out = codes_out; a.rows = nullptr; a.count = 0;
  a.N = N; a.K = K; a.scale_row_stride = scale_row_stride;
  a.total_bytes = (N * K * bits + 7) / 8;
  a.group = group < 1 ? 1 : group; a.bits = bits; a.lut_len = w_out ? lut_len : 0; a.scale_dtype = scale_dtype;
  a.uniform = (K % 8 == 0) && (a.group % 8 == 0);
  a.aligned = (reinterpret_cast<uintptr_t>(packed) % 8) == 0;
  const int64_t threads = (N * K + 7) / 8;
  return launch_bits<true>(a, out_dtype, threads, static_cast<cudaStream_t>(stream));
}

extern "C" int mkb_dequant_rows(const uint8_t* packed, const void* scales, const float* lut,
                                const void* zeros, const int64_t* rows, void* out, int64_t count,
                                int64_t N, int64_t K, int group, int bits, int lut_len,
                                int scale_dtype, int out_dtype, int64_t scale_row_stride, void* stream) {
  using namespace mkb;
  int status = check_common(packed, scales, lut, N, K, group, bits, lut_len, scale_dtype, out_dtype, true);
  if (status != MKB_OK) return status;
  MKB_REQUIRE(count >= 0, MKB_E_ARGUMENT, "dequant_rows: negative row count");
  if (count == 0 || K == 0) return MKB_OK;
  MKB_REQUIRE(rows != nullptr && out != nullptr, MKB_E_ARGUMENT, "dequant_rows: rows or out is null");
  MKB_REQUIRE((K * bits) % 8 == 0, MKB_E_UNSUPPORTED,
              "dequant_rows: rows of %lld %d-bit codes do not hold whole bytes", (long long)K, bits);
  DequantArgs a{};
  a.packed = packed; a.scales = scales; a.lut = lut; a.zeros = zeros;
  a.w_out = out; a.codes_out = nullptr; a.rows = rows; a.count = count;
  a.N = N; a.K = K; a.scale_row_stride = scale_row_stride;
  a.total_bytes = N * (K * bits / 8);
  a.group = group; a.bits = bits; a.lut_len = lut_len; a.scale_dtype = scale_dtype;
  a.uniform = (group % 8 == 0);
  const int64_t row_bytes = K * bits / 8;
  a.aligned = (reinterpret_cast<uintptr_t>(packed) % 8) == 0 && (row_bytes % 8) == 0;
  const int64_t threads = count * ((K + 7) / 8);
  return launch_bits<false>(a, out_dtype, threads, static_cast<cudaStream_t>(stream));
}
