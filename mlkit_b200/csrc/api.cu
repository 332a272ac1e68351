// C ABI entry points that are not tied to one kernel file: error text, device cache, matvec dispatch.
#include <cstdarg>
#include <cstdio>

#include "mkb_common.cuh"

namespace mkb {

static thread_local char g_error[512] = "";

void set_error(const char* format, ...) {
  va_list arguments;
  va_start(arguments, format);
  vsnprintf(g_error, sizeof(g_error), format, arguments);
  va_end(arguments);
}

int cuda_fail(cudaError_t status, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(status));
  return MKB_E_CUDA;
}

const DeviceInfo& device_info() {
  static DeviceInfo cache[64];
  static bool known[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64) device = 0;
  if (!known[device]) {
    DeviceInfo info{148, 232448};
    cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&info.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    cache[device] = info;
    known[device] = true;
  }
  return cache[device];
}

int gemv_scalar_supported(int K, int group, int bits);
int launch_gemv_scalar(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                       const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                       int bits, int lut_len, int x_dtype, int scale_dtype, int64_t packed_row_stride,
                       int64_t scale_row_stride, cudaStream_t stream);
int gemv_tiled_supported(int M, int K, int group, int bits, int x_dtype, int scale_dtype,
                         const void* x, const uint8_t* packed, int64_t packed_row_stride);
int launch_gemv_tiled(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                      const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                      int bits, int lut_len, int64_t packed_row_stride, int64_t scale_row_stride,
                      int integer_grid, float grid_minimum, int gated, cudaStream_t stream);

int gemv_umma_supported(int M, int K, int group, int bits, int x_dtype, int scale_dtype, const void* x,
                        const uint8_t* packed, int64_t packed_row_stride, const void* zeros, int integer_grid);
int64_t gemv_umma_workspace_bytes(int M, int N, int K);
bool prefer_tmem();
int launch_gemv_umma(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                     void* workspace, int M, int N, int K, int group, int64_t packed_row_stride,
                     int64_t scale_row_stride, float grid_minimum, cudaStream_t stream);

int gemv_bulk_supported(int M, int N, int K, int group, int bits, int x_dtype, int scale_dtype, const void* x,
                        const uint8_t* packed, int64_t packed_row_stride, const void* zeros, int integer_grid,
                        float grid_minimum);
int64_t gemv_bulk_workspace_bytes(int M, int N, int K);
int launch_gemv_bulk(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                     void* workspace, int64_t workspace_bytes, int M, int N, int K, int group,
                     int64_t packed_row_stride, int64_t scale_row_stride, float grid_minimum, cudaStream_t stream);
bool prefer_bulk(int M, int N, int K);

int gemv_stream_supported(int M, int N, int K, int group, int bits, int lut_len, int x_dtype, int scale_dtype,
                          const void* x, const uint8_t* packed, const void* scales, int64_t packed_row_stride,
                          int64_t scale_row_stride, const void* zeros, int integer_grid, float grid_minimum);
int launch_gemv_stream(const void* x, const uint8_t* packed, const void* scales, const float* lut, const void* bias,
                       void* y, int M, int N, int K, int group, int bits, int lut_len, int64_t packed_row_stride,
                       int64_t scale_row_stride, int integer_grid, float grid_minimum, int gated, cudaStream_t stream);
int gemv_stream_rotation_supported(int M, int N, int K, int group, int bits, int lut_len, int integer_grid,
                                   float grid_minimum, const void* signs);
int launch_gemv_stream_rotated(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                               const void* bias, void* y, int M, int N, int K, int group, int bits, int lut_len,
                               int64_t packed_row_stride, int64_t scale_row_stride, int integer_grid,
                               float grid_minimum, int gated, const int8_t* signs, int rotate, int normalize,
                               cudaStream_t stream);

}  // namespace mkb



extern "C" int mkb_version(void) { return 102; }

namespace mkb {
// Which kernel MKB_GEMV_AUTO takes when both cover the arguments (set from measurements).
bool prefer_tmem() { return false; }
// Measured on B200 (CUDA-graph replays over weights that are cold in L2): the TMA-fed kernel's time
// hardly grows with the row count (its activations sit in registers), the tiled kernel's does; the
// tiled kernel starts faster, which decides small layers.
bool prefer_bulk(int M, int N, int K) {
  const int64_t codes = int64_t(N) * K;
  if (codes < (int64_t(20) << 20)) return false;
  if (M >= 3) return true;
  return K > 16384 || (K <= 4096 && N >= 24576);
}
}  // namespace mkb

extern "C" const char* mkb_last_error(void) { return mkb::g_error; }

extern "C" int64_t mkb_gemv_workspace_bytes(int M, int N, int K, int bits) {
  if (bits != 4 || M < 1 || M > 8 || N < 1 || K < 256) return 0;
  const int64_t tmem = K % 512 == 0 ? mkb::gemv_umma_workspace_bytes(M, N, K) : 0;
  const int64_t bulk = K % 256 == 0 ? mkb::gemv_bulk_workspace_bytes(M, N, K) : 0;
  return tmem > bulk ? tmem : bulk;
}

extern "C" int mkb_gemv_workspace_status(const void* workspace, int64_t workspace_bytes, int* status) {
  using namespace mkb;
  MKB_REQUIRE(workspace != nullptr && status != nullptr && workspace_bytes >= 65536, MKB_E_ARGUMENT,
              "gemv_workspace_status: no workspace head");
  // the status word follows the arrival counters in the 64 KB head of the workspace
  const uint8_t* word = static_cast<const uint8_t*>(workspace) + (65536 / 4 - 1) * 4;
  int value = 0;
  const cudaError_t copied = cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost);
  if (copied != cudaSuccess) return cuda_fail(copied, "gemv_workspace_status");
  *status = value;
  return MKB_OK;
}

extern "C" int mkb_gemv_ws(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                           const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                           int bits, int lut_len, int x_dtype, int scale_dtype,
                           int64_t packed_row_stride, int64_t scale_row_stride, int integer_grid,
                           float grid_minimum, int kernel, void* workspace, int64_t workspace_bytes,
                           void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 1 && M <= 8, MKB_E_UNSUPPORTED, "gemv: M=%d outside 1..8", M);
  MKB_REQUIRE(N >= 0 && K >= 0, MKB_E_ARGUMENT, "gemv: negative shape");
  MKB_REQUIRE(bits >= 1 && bits <= 8, MKB_E_UNSUPPORTED, "gemv: bits=%d outside 1..8", bits);
  MKB_REQUIRE(group >= 1, MKB_E_ARGUMENT, "gemv: group must be positive");
  MKB_REQUIRE(x_dtype >= MKB_F16 && x_dtype <= MKB_F32 && scale_dtype >= MKB_F16 && scale_dtype <= MKB_F32,
              MKB_E_ARGUMENT, "gemv: unknown dtype");
  MKB_REQUIRE(lut_len >= 1 && lut_len <= (1 << bits), MKB_E_ARGUMENT,
              "gemv: lut_len=%d does not fit %d-bit codes", lut_len, bits);
  const int gated = (kernel & MKB_GEMV_GATED) != 0;
  kernel &= ~MKB_GEMV_GATED;
  MKB_REQUIRE(kernel >= MKB_GEMV_AUTO && kernel <= MKB_GEMV_STREAM, MKB_E_ARGUMENT, "gemv: unknown kernel choice");
  if (N == 0) return MKB_OK;
  MKB_REQUIRE(x && packed && scales && lut && y, MKB_E_ARGUMENT, "gemv: null pointer");
  MKB_REQUIRE(gemv_scalar_supported(K, group, bits), MKB_E_UNSUPPORTED,
              "gemv: K=%d or group=%d splits a packing word of %d-bit codes", K, group, bits);
  MKB_REQUIRE(K > 0, MKB_E_UNSUPPORTED, "gemv: empty reduction");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool stream_ok = gemv_stream_supported(M, N, K, group, bits, lut_len, x_dtype, scale_dtype, x, packed, scales,
                                               packed_row_stride, scale_row_stride, zeros, integer_grid, grid_minimum);
  if (kernel == MKB_GEMV_STREAM)
    MKB_REQUIRE(stream_ok, MKB_E_UNSUPPORTED, "gemv: the streaming kernel does not cover these arguments");
  if (kernel == MKB_GEMV_STREAM || (kernel == MKB_GEMV_AUTO && stream_ok))
    return launch_gemv_stream(x, packed, scales, lut, bias, y, M, N, K, group, bits, lut_len, packed_row_stride,
                              scale_row_stride, integer_grid, grid_minimum, gated, s);
  const bool tiled_ok = gemv_tiled_supported(M, K, group, bits, x_dtype, scale_dtype, x, packed, packed_row_stride);
  const bool tmem_ok = workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) % 16) == 0 && lut_len == 16 &&
                       gemv_umma_supported(M, K, group, bits, x_dtype, scale_dtype, x, packed, packed_row_stride, zeros,
                                           integer_grid) &&
                       workspace_bytes >= gemv_umma_workspace_bytes(M, N, K);
  if (kernel == MKB_GEMV_TMEM)
    MKB_REQUIRE(tmem_ok, MKB_E_UNSUPPORTED,
                "gemv: the tensor-memory kernel does not cover these arguments or the workspace is too small");
  MKB_REQUIRE(!(gated && kernel == MKB_GEMV_TMEM), MKB_E_UNSUPPORTED, "gemv: the tensor-memory kernel takes no gated input");
  if (kernel == MKB_GEMV_TMEM || (!gated && kernel == MKB_GEMV_AUTO && tmem_ok && mkb::prefer_tmem()))
    return launch_gemv_umma(x, packed, scales, bias, y, workspace, M, N, K, group, packed_row_stride,
                            scale_row_stride, grid_minimum, s);
  const bool workspace_aligned = workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) % 16) == 0;
  const bool bulk_ok = lut_len == 16 && workspace_aligned &&
                       gemv_bulk_supported(M, N, K, group, bits, x_dtype, scale_dtype, x, packed, packed_row_stride,
                                           zeros, integer_grid, grid_minimum) &&
                       (gemv_bulk_workspace_bytes(M, N, K) == 0 ||
                        (workspace != nullptr && workspace_bytes >= gemv_bulk_workspace_bytes(M, N, K)));
  if (kernel == MKB_GEMV_BULK)
    MKB_REQUIRE(bulk_ok, MKB_E_UNSUPPORTED,
                "gemv: the TMA-fed kernel does not cover these arguments or the workspace is too small");
  MKB_REQUIRE(!(gated && kernel == MKB_GEMV_BULK), MKB_E_UNSUPPORTED, "gemv: the TMA-fed kernel takes no gated input");
  if (kernel == MKB_GEMV_BULK || (!gated && kernel == MKB_GEMV_AUTO && bulk_ok && mkb::prefer_bulk(M, N, K)))
    return launch_gemv_bulk(x, packed, scales, bias, y, workspace, workspace_bytes, M, N, K, group,
                            packed_row_stride, scale_row_stride, grid_minimum, s);
  if (kernel == MKB_GEMV_TILED)
    MKB_REQUIRE(tiled_ok, MKB_E_UNSUPPORTED, "gemv: the tiled kernel does not cover these arguments");
  if (kernel == MKB_GEMV_TILED || (kernel == MKB_GEMV_AUTO && tiled_ok)) {
    const int launched = launch_gemv_tiled(x, packed, scales, lut, zeros, bias, y, M, N, K, group, bits, lut_len,
                                           packed_row_stride, scale_row_stride, integer_grid, grid_minimum, gated, s);
    // the tiled kernel sizes its shared memory from M, K, bits and the decode mode and refuses, before
    // it launches anything, a combination that does not fit one SM (a 256-entry table with K = 28672
    // at more than four rows, say): under AUTO such a call takes the scalar kernel
    if (launched != MKB_E_UNSUPPORTED || kernel == MKB_GEMV_TILED || gated) return launched;
  }
  MKB_REQUIRE(!gated, MKB_E_UNSUPPORTED, "gemv: the gated input needs the tiled kernel");
  return launch_gemv_scalar(x, packed, scales, lut, zeros, bias, y, M, N, K, group, bits, lut_len, x_dtype,
                            scale_dtype, packed_row_stride, scale_row_stride, s);
}

extern "C" int mkb_gemv_ex(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                           const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                           int bits, int lut_len, int x_dtype, int scale_dtype,
                           int64_t packed_row_stride, int64_t scale_row_stride, int integer_grid,
                           float grid_minimum, int kernel, void* stream) {
  return mkb_gemv_ws(x, packed, scales, lut, zeros, bias, y, M, N, K, group, bits, lut_len, x_dtype, scale_dtype,
                     packed_row_stride, scale_row_stride, integer_grid, grid_minimum, kernel, nullptr, 0, stream);
}

extern "C" int mkb_gemv(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                        const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                        int bits, int lut_len, int x_dtype, int scale_dtype, int64_t packed_row_stride,
                        int64_t scale_row_stride, int integer_grid, float grid_minimum, void* stream) {
  return mkb_gemv_ex(x, packed, scales, lut, zeros, bias, y, M, N, K, group, bits, lut_len, x_dtype,
                     scale_dtype, packed_row_stride, scale_row_stride, integer_grid, grid_minimum,
                     MKB_GEMV_AUTO, stream);
}

extern "C" int mkb_gemv_hadamard(const void* x, const int8_t* signs, const uint8_t* packed, const void* scales,
                                 const float* lut, const void* bias, void* y, int M, int N, int K, int group, int bits,
                                 int lut_len, int x_dtype, int scale_dtype, int64_t packed_row_stride,
                                 int64_t scale_row_stride, int integer_grid, float grid_minimum, int normalize,
                                 void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 1 && N >= 1 && K >= 1 && group >= 1, MKB_E_ARGUMENT, "gemv_hadamard: bad shape");
  MKB_REQUIRE(x && packed && scales && lut && y, MKB_E_ARGUMENT, "gemv_hadamard: null pointer");
  MKB_REQUIRE(gemv_stream_supported(M, N, K, group, bits, lut_len, x_dtype, scale_dtype, x, packed, scales, packed_row_stride,
                                    scale_row_stride, nullptr, integer_grid, grid_minimum) &&
                  gemv_stream_rotation_supported(M, N, K, group, bits, lut_len, integer_grid, grid_minimum, signs),
              MKB_E_UNSUPPORTED,
              "gemv_hadamard: needs a layer the streaming matvec covers, K a power of two of at least 512, "
              "M * K * 4 <= 65536 and 16-byte aligned signs");
  return launch_gemv_stream_rotated(x, packed, scales, lut, bias, y, M, N, K, group, bits, lut_len, packed_row_stride,
                                    scale_row_stride, integer_grid, grid_minimum, 0, signs, 1, normalize,
                                    static_cast<cudaStream_t>(stream));
}
