// Round-to-nearest encoding of a weight matrix onto a scalar grid with one fp16 scale per row group,
// and packing of the codes into the little-endian bit stream, in one launch (sm_100a).
//
// The arithmetic is the tensor route of the reference, operation for operation, so codes and scales
// are bit-equal to it: per group, scale = max(|w|) clamped from below at 1e-12, times the fp32
// reciprocal of the largest level magnitude, rounded to fp16 (clamped to [2^-24, 65504]); code =
// round-half-even(w / scale) clamped to the grid for integer grids, the nearest level (a tie takes
// the lower one) for codebooks; the division is IEEE binary32.
// One warp encodes one group: a pass for the range, a pass for the codes (through shared memory),
// then each lane assembles whole bytes of the stream.
#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kEncodeWarps = 8;
constexpr int kMaxGroup = 1024;

struct EncodeArgs {
  const void* weight;
  const float* levels;
  uint8_t* packed;
  __half* scales;
  uint8_t* codes;
  int64_t rows;
  int width, group, groups, bits, level_count, integer, weight_dtype;
  float low, high, reciprocal;
};

__device__ __forceinline__ int nearest_level(float x, const float* levels, int count) {
  // first level >= x (binary search), then the closer of it and the one below; a tie goes below
  int lo = 0, hi = count;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (levels[mid] < x) lo = mid + 1;
    else hi = mid;
  }
  const int above = min(lo, count - 1), below = max(above - 1, 0);
  return fabsf(__fsub_rn(x, levels[below])) <= fabsf(__fsub_rn(x, levels[above])) ? below : above;
}

__global__ void __launch_bounds__(kEncodeWarps * 32) rtn_encode_kernel(const EncodeArgs a) {
  __shared__ uint8_t code_s[kEncodeWarps][kMaxGroup];
  __shared__ float level_s[256];
  for (int i = threadIdx.x; i < a.level_count; i += blockDim.x) level_s[i] = a.levels[i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = a.rows * a.groups;
  for (int64_t item = int64_t(blockIdx.x) * kEncodeWarps + warp; item < total; item += int64_t(gridDim.x) * kEncodeWarps) {
    const int64_t row = item / a.groups;
    const int gi = int(item - row * a.groups);
    const int first = gi * a.group, count = min(a.group, a.width - first);
    const int64_t base = row * a.width + first;
    float biggest = 0.f;
    for (int i = lane; i < count; i += 32) biggest = fmaxf(biggest, fabsf(load_as_float(a.weight, base + i, a.weight_dtype)));
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) biggest = fmaxf(biggest, __shfl_xor_sync(0xffffffffu, biggest, offset));
    float scale = __fmul_rn(fmaxf(biggest, 1e-12f), a.reciprocal);
    const __half stored = __float2half_rn(fminf(fmaxf(scale, 5.9604644775390625e-08f), 65504.f));
    scale = __half2float(stored);
    if (lane == 0) a.scales[row * a.groups + gi] = stored;
    for (int i = lane; i < count; i += 32) {
      const float normalized = __fdiv_rn(load_as_float(a.weight, base + i, a.weight_dtype), scale);
      int code;
      if (a.integer) code = int(fminf(fmaxf(rintf(normalized), a.low), a.high) - a.low);
      else code = nearest_level(normalized, level_s, a.level_count);
      code_s[warp][i] = uint8_t(code);
      if (a.codes != nullptr) a.codes[base + i] = uint8_t(code);
    }
    __syncwarp();
    // the group starts on a byte of the stream (group * bits and width * bits are multiples of 8)
    const int64_t first_byte = (row * int64_t(a.width) + first) * a.bits / 8;
    const int bytes = count * a.bits / 8;
    for (int j = lane; j < bytes; j += 32) {
      uint32_t value = 0;
      const int bit0 = j * 8;
      for (int i = bit0 / a.bits; i * a.bits < bit0 + 8 && i < count; ++i) {
        const int shift = i * a.bits - bit0;  // position of the code's lowest bit relative to the byte
        const uint32_t code = code_s[warp][i];
        value |= shift >= 0 ? code << shift : code >> -shift;
      }
      a.packed[first_byte + j] = uint8_t(value);
    }
    __syncwarp();
  }
}

}  // namespace
}  // namespace mkb

extern "C" int mkb_rtn_encode(const void* weight, const float* levels, uint8_t* packed, void* scales, uint8_t* codes,
                              int64_t N, int K, int group, int bits, int level_count, int integer_grid,
                              float grid_low, float grid_high, float reciprocal, int weight_dtype, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(N >= 0 && K >= 1 && group >= 1 && bits >= 1 && bits <= 8, MKB_E_ARGUMENT, "rtn_encode: bad shape");
  MKB_REQUIRE(level_count >= 1 && level_count <= (1 << bits), MKB_E_ARGUMENT,
              "rtn_encode: %d levels do not fit %d-bit codes", level_count, bits);
  MKB_REQUIRE(weight_dtype >= MKB_F16 && weight_dtype <= MKB_F32, MKB_E_ARGUMENT, "rtn_encode: unknown dtype");
  MKB_REQUIRE(grid_high >= grid_low && reciprocal > 0.f, MKB_E_ARGUMENT, "rtn_encode: bad grid range");
  if (N == 0) return MKB_OK;
  MKB_REQUIRE(weight && levels && packed && scales, MKB_E_ARGUMENT, "rtn_encode: null pointer");
  if (group > K) group = K;
  MKB_REQUIRE(group <= kMaxGroup, MKB_E_UNSUPPORTED, "rtn_encode: groups of more than %d codes", kMaxGroup);
  MKB_REQUIRE((int64_t(group) * bits) % 8 == 0 && (int64_t(K) * bits) % 8 == 0, MKB_E_UNSUPPORTED,
              "rtn_encode: a group or a row of %d-bit codes does not end on a byte", bits);
  EncodeArgs a{};
  a.weight = weight; a.levels = levels; a.packed = packed; a.scales = static_cast<__half*>(scales); a.codes = codes;
  a.rows = N; a.width = K; a.group = group; a.groups = (K + group - 1) / group; a.bits = bits;
  a.level_count = level_count; a.integer = integer_grid; a.weight_dtype = weight_dtype;
  a.low = grid_low; a.high = grid_high; a.reciprocal = reciprocal;
  const int64_t items = N * a.groups;
  const int64_t wanted = (items + kEncodeWarps - 1) / kEncodeWarps;
  const int blocks = int(wanted < 148 * 16 ? wanted : 148 * 16);
  rtn_encode_kernel<<<blocks, kEncodeWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  MKB_LAUNCH_CHECK("rtn_encode launch");
  return MKB_OK;
}
