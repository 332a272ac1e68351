// One-shot all-reduce over peer memory for the row-parallel linears of the tensor-parallel decode
// step (sm_100a, NVLink/NVSwitch), fused with the residual add and RMS norm that consume it: ONE
// kernel per reduction, no library collective.
//
// Every rank owns one exchange buffer that all ranks of the node have mapped:
//   [ header: sent: 8 x uint32 | status | poll limit | pad to 2 KB ]
//   [ slots: 2 parities x world x rows x H/2 packets of 8 bytes ]
// A packet is one 32-bit word of data (two fp16 values) and one 32-bit flag; data and flag travel in the
// same store, so a receiver that sees the flag has the data: no fence, no second message.  (The stores are
// 16 bytes = two packets; each 8-byte half validates itself, so it does not matter whether a 16-byte
// store stays whole on its way.)
// CTA m of the kernel handles row m of the partial [M, H]:
//   * push: it writes row m, as packets flagged v, into slot[parity][rank] of every rank's buffer (its own
//     included) with plain stores over NVLink.  v counts the reductions this row has taken part in (kept
//     in the rank's own buffer); all ranks run the same sequence of reductions, so v is the same number
//     everywhere, and parity = v & 1 keeps a fast rank's next reduction out of the slots a slow rank is
//     still reading; a slot sees v, v + 2, v + 4, ..., so a stale packet never carries the awaited flag;
//   * wait + add: every thread polls (bounded) the packets it needs of source 0, adds them, then source 1,
//     ...: the sum is formed in rank order in fp32 (every rank gets the same bits).  Every CTA pushes before
//     it waits and packets persist, so no rank can wait for a rank that waits for it;
//   * norm: the sum is rounded to fp16 as the library all-reduce would, added to the residual, normalised.
// A wait that gives up sets the status word and lets the kernel finish; later waits are skipped.
#include "mkb_common.cuh"

#include <mutex>
#include <unordered_map>

namespace mkb {
namespace {

constexpr int kHeaderBytes = 2048;
constexpr int kMaxWorld = 16;
constexpr int kMaxRows = 8;
constexpr int kGatherThreads = 1024;
constexpr uint32_t kDefaultPolls = 60000000;  // of the order of half a minute: ranks are separate processes

constexpr int kMaxSplit = 8;      // CTAs that share one row

struct Header {
  uint32_t sent[kMaxRows][kMaxSplit];      // reductions CTA (m, s) has taken part in (touched by that CTA only)
  uint2 squares[2][kMaxRows][kMaxSplit];   // [parity][row][split]: a partial sum of squares and its flag
  uint32_t status;                // non-zero when a wait expired
  uint32_t poll_limit;            // polls of one packet before a wait gives up
};
static_assert(sizeof(Header) <= kHeaderBytes, "header does not fit");

// packets of (parity, source): [rows][H / 4] units of 16 bytes (two packets: four fp16 values)
__device__ __forceinline__ uint4* slot_of(void* buffer, int parity, int source, int world, int64_t slot_units) {
  return reinterpret_cast<uint4*>(static_cast<uint8_t*>(buffer) + kHeaderBytes) + (int64_t(parity) * world + source) * slot_units;
}

__device__ __forceinline__ uint4 load_volatile16(const uint4* address) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(address));
  return v;
}
__device__ __forceinline__ uint2 load_volatile8(const uint2* address) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(address));
  return v;
}

// CTA (m, s) owns slice s of row m: push, wait, then residual[m, slice] += sum over ranks of slot[r][m, slice];
// the slices' sums of squares meet through the rank's own header; normed = rmsnorm(residual) * weight.
// `reduced` (optional) receives the fp16 sum, for callers that need the all-reduced tensor itself.
// One CTA pushes world * slice * 4 bytes over NVLink; a single SM sustains only a few tens of GB/s of remote
// stores, so wide worlds split the row over several CTAs (measured at 8 ranks: 256 KB from one SM cost ~10 us).
constexpr int kGatherPieces = 2;   // slices up to 1024 * 2 * 8 = 16384 elements stay in registers

__global__ void __launch_bounds__(kGatherThreads) peer_reduce_add_rmsnorm_kernel(
    const __half* __restrict__ partial, void* const* peers, void* own, __half* __restrict__ residual,
    const __half* __restrict__ weight, __half* __restrict__ normed, __half* __restrict__ reduced, int H, int world,
    int rank, int64_t slot_units, float eps) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float part_s[kGatherThreads / 32];
  __shared__ float total_s;
  Header* mine = static_cast<Header*>(own);
  const int m = blockIdx.x, split = gridDim.y, part = blockIdx.y;
  const int slice = H / split, first = part * slice;       // this CTA's elements of the row
  // the norm weights are constants of the model: fetched before the wait, they cost no latency after the sum
  uint4 scale_of[kGatherPieces];
#pragma unroll
  for (int piece = 0; piece < kGatherPieces; ++piece) {
    const int i = (piece * kGatherThreads + threadIdx.x) * 8;
    scale_of[piece] = i < slice ? __ldg(reinterpret_cast<const uint4*>(weight + first + i)) : make_uint4(0u, 0u, 0u, 0u);
  }
  // (nothing of the header is read before the wait: the reduction launched just before this one may be the one
  // that writes this CTA's counter, and with the status and the poll limit read early the two-GPU decode test
  // failed)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t first_limit = mine->status != 0 ? 0u : mine->poll_limit;
  const uint32_t v = mine->sent[m][part] + 1;   // only CTA (m, part) of a reduction touches sent[m][part]
  const int parity = int(v & 1u);
  const int64_t row_units = int64_t(m) * (H / 4) + first / 4;   // 16-byte units of the slice inside a slot
  {
    // push the slice, as flagged packets, into this rank's slot on every rank
    const uint4* source = reinterpret_cast<const uint4*>(partial + int64_t(m) * H + first);
    uint4 piece[kGatherPieces];
#pragma unroll
    for (int k = 0; k < kGatherPieces; ++k) {
      const int i = k * kGatherThreads + threadIdx.x;
      piece[k] = i * 8 < slice ? source[i] : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int p = 0; p < world; ++p) {
      uint4* target = slot_of(peers[p], parity, rank, world, slot_units) + row_units;
#pragma unroll
      for (int k = 0; k < kGatherPieces; ++k) {
        const int i = k * kGatherThreads + threadIdx.x;
        if (i * 8 < slice) {
          target[2 * i] = make_uint4(piece[k].x, v, piece[k].y, v);
          target[2 * i + 1] = make_uint4(piece[k].z, v, piece[k].w, v);
        }
      }
    }
  }
  // a wait that expired once is not repeated: every later reduction of a broken exchange would otherwise
  // add its own timeout
  uint32_t limit = first_limit;
  bool expired = false;

  const int64_t base = int64_t(blockIdx.x) * H + first;
  uint4 kept[kGatherPieces];
  float sq = 0.f;
#pragma unroll
  for (int piece = 0; piece < kGatherPieces; ++piece) {
    const int unit = piece * kGatherThreads + threadIdx.x;
    const int i = unit * 8;
    kept[piece] = make_uint4(0u, 0u, 0u, 0u);
    if (i < slice) {
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        // the slot is written from outside this GPU: volatile loads, until both units carry the flag
        const uint4* from = slot_of(own, parity, r, world, slot_units) + row_units + 2 * unit;
        uint4 low = load_volatile16(from), high = load_volatile16(from + 1);
        uint32_t polls = 0;
        while ((low.y != v || low.w != v || high.y != v || high.w != v) && polls < limit) {
          low = load_volatile16(from);
          high = load_volatile16(from + 1);
          ++polls;
        }
        if (low.y != v || low.w != v || high.y != v || high.w != v) {
          expired = true;
          limit = 0;
          continue;     // on expiry the kernel still runs through, without what did not arrive
        }
        const uint32_t words[4] = {low.x, low.z, high.x, high.z};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&words[q]));
          sum[2 * q] += f.x;
          sum[2 * q + 1] += f.y;
        }
      }
      uint4 delta;
      __half2* dh = reinterpret_cast<__half2*>(&delta);
#pragma unroll
      for (int q = 0; q < 4; ++q) dh[q] = __floats2half2_rn(sum[2 * q], sum[2 * q + 1]);
      if (reduced != nullptr) *reinterpret_cast<uint4*>(reduced + base + i) = delta;
      uint4 value = *reinterpret_cast<const uint4*>(residual + base + i);
      __half2* vh = reinterpret_cast<__half2*>(&value);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __half22float2(vh[q]), y = __half22float2(dh[q]);
        vh[q] = __floats2half2_rn(x.x + y.x, x.y + y.y);
      }
      *reinterpret_cast<uint4*>(residual + base + i) = value;
      kept[piece] = value;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __half22float2(vh[q]);
        sq += x.x * x.x + x.y * x.y;
      }
    }
  }
  if (threadIdx.x == 0) mine->sent[m][part] = v;
#pragma unroll
  for (int offset = 16; offset; offset >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, offset);
  if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < int(blockDim.x) / 32; ++w) total += part_s[w];
    if (split > 1) {
      // the slices' sums meet in this rank's own header, as packets like the data; every CTA of the row adds
      // them in slice order, so all of them normalise with the same bits
      asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(&mine->squares[parity][m][part]),
                   "r"(__float_as_uint(total)), "r"(v) : "memory");
      total = 0.f;
      for (int other = 0; other < split; ++other) {
        const uint2* from = &mine->squares[parity][m][other];
        uint2 got = load_volatile8(from);
        uint32_t polls = 0;
        while (got.y != v && polls < limit) {
          got = load_volatile8(from);
          ++polls;
        }
        if (got.y != v) {
          expired = true;
          limit = 0;
          continue;
        }
        total += __uint_as_float(got.x);
      }
    }
    total_s = total;
  }
  if (expired) atomicExch(&mine->status, 1u);
  __syncthreads();
  const float inv = rsqrtf(total_s / float(H) + eps);
#pragma unroll
  for (int piece = 0; piece < kGatherPieces; ++piece) {
    const int i = (piece * kGatherThreads + threadIdx.x) * 8;
    if (i < slice) {
      const __half2* vh = reinterpret_cast<const __half2*>(&kept[piece]);
      const __half2* wh = reinterpret_cast<const __half2*>(&scale_of[piece]);
      uint4 result;
      __half2* rh = reinterpret_cast<__half2*>(&result);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = __half22float2(vh[q]), ww = __half22float2(wh[q]);
        const float2 u = __half22float2(__floats2half2_rn(x.x * inv, x.y * inv));
        rh[q] = __floats2half2_rn(u.x * ww.x, u.y * ww.y);
      }
      *reinterpret_cast<uint4*>(normed + base + i) = result;
    }
  }
}

// CTAs per row a caller fixed for a buffer (tests force the split path on small worlds); 0: automatic
std::mutex g_split_lock;
std::unordered_map<const void*, uint32_t> g_split;
uint32_t split_of(const void* own) {
  std::lock_guard<std::mutex> guard(g_split_lock);
  const auto found = g_split.find(own);
  return found == g_split.end() ? 0u : found->second;
}

template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, void* stream, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = 0;
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

}  // namespace
}  // namespace mkb

extern "C" int64_t mkb_peer_buffer_bytes(int rows, int H, int world) {
  if (rows < 1 || rows > mkb::kMaxRows || H < 8 || world < 1 || world > mkb::kMaxWorld) return 0;
  return mkb::kHeaderBytes + int64_t(2) * world * rows * H * 4;   // packets: 4 bytes of flags per 4 bytes of data
}

extern "C" int mkb_peer_set_poll_limit(void* own, int64_t polls) {
  using namespace mkb;
  MKB_REQUIRE(own != nullptr && polls >= 1 && polls <= int64_t(0xffffffffu), MKB_E_ARGUMENT, "peer_set_poll_limit: bad arguments");
  const uint32_t value = uint32_t(polls);
  const cudaError_t copied = cudaMemcpy(&static_cast<Header*>(own)->poll_limit, &value, sizeof(value), cudaMemcpyHostToDevice);
  if (copied != cudaSuccess) return cuda_fail(copied, "peer_set_poll_limit");
  return MKB_OK;
}

extern "C" int mkb_peer_set_split(void* own, int split) {
  using namespace mkb;
  MKB_REQUIRE(own != nullptr && split >= 0 && split <= kMaxSplit && (split & (split - 1)) == 0, MKB_E_ARGUMENT,
              "peer_set_split: 0 (automatic) or a power of two up to %d", kMaxSplit);
  std::lock_guard<std::mutex> guard(g_split_lock);
  g_split[own] = uint32_t(split);
  return MKB_OK;
}

extern "C" int mkb_peer_alloc(int64_t bytes, void** buffer) {
  using namespace mkb;
  MKB_REQUIRE(bytes > 0 && buffer != nullptr, MKB_E_ARGUMENT, "peer_alloc: bad arguments");
  cudaError_t status = cudaMalloc(buffer, size_t(bytes));
  if (status != cudaSuccess) return cuda_fail(status, "peer_alloc");
  status = cudaMemset(*buffer, 0, size_t(bytes));
  if (status != cudaSuccess) return cuda_fail(status, "peer_alloc: clearing");
  return mkb_peer_set_poll_limit(*buffer, int64_t(kDefaultPolls));
}

extern "C" int mkb_peer_free(void* buffer) {
  using namespace mkb;
  {
    std::lock_guard<std::mutex> guard(g_split_lock);
    g_split.erase(buffer);
  }
  const cudaError_t status = cudaFree(buffer);
  if (status != cudaSuccess) return cuda_fail(status, "peer_free");
  return MKB_OK;
}

extern "C" int mkb_peer_export(void* buffer, void* handle64) {
  using namespace mkb;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  MKB_REQUIRE(buffer != nullptr && handle64 != nullptr, MKB_E_ARGUMENT, "peer_export: null pointer");
  const cudaError_t status = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), buffer);
  if (status != cudaSuccess) return cuda_fail(status, "peer_export");
  return MKB_OK;
}

extern "C" int mkb_peer_open(const void* handle64, void** buffer) {
  using namespace mkb;
  MKB_REQUIRE(handle64 != nullptr && buffer != nullptr, MKB_E_ARGUMENT, "peer_open: null pointer");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle64, sizeof(handle));
  const cudaError_t status = cudaIpcOpenMemHandle(buffer, handle, cudaIpcMemLazyEnablePeerAccess);
  if (status != cudaSuccess) return cuda_fail(status, "peer_open");
  return MKB_OK;
}

extern "C" int mkb_peer_close(void* buffer) {
  using namespace mkb;
  const cudaError_t status = cudaIpcCloseMemHandle(buffer);
  if (status != cudaSuccess) return cuda_fail(status, "peer_close");
  return MKB_OK;
}

extern "C" int mkb_peer_reduce_add_rmsnorm(const void* partial, void* const* peers, void* own, void* residual,
                                           const void* weight, void* normed, void* reduced, int M, int H, int rows,
                                           int world, int rank, float eps, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(partial && peers && own && residual && weight && normed, MKB_E_ARGUMENT,
              "peer_reduce_add_rmsnorm: null pointer");
  MKB_REQUIRE(M >= 1 && M <= rows && rows <= kMaxRows && H % 8 == 0 && H >= 8 &&
                  H <= kGatherThreads * kGatherPieces * 8 && world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world,
              MKB_E_UNSUPPORTED, "peer_reduce_add_rmsnorm: unsupported shape");
  MKB_REQUIRE(((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(residual) |
                reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(normed) |
                reinterpret_cast<uintptr_t>(reduced)) & 15) == 0,
              MKB_E_ARGUMENT, "peer_reduce_add_rmsnorm: pointers must be 16-byte aligned");
  // CTAs per row: wide worlds push more bytes than one SM moves quickly (the header may fix the number)
  const uint32_t wanted = split_of(own);
  // measured (70B-shaped decode, H = 8192, tokens/s with 1 / 2 / 4 / 8 CTAs per row): 2 ranks, one row: 152 / 155 /
  // 155 / -, eight rows: 1117 / 1119 / 1101 / -; 4 ranks, one row: 186 / 190 / 194 / 190, eight rows best with
  // one; 8 ranks: four CTAs per row ahead of one at one row (205 against 179) and at eight rows.  So: about four
  // pushing CTAs per launch, thirty-two when eight ranks make every row a 256 KB push.
  int split = int(wanted);
  if (split == 0) {
    const int budget = world >= 8 ? 32 : world >= 2 ? 4 : 1;   // a single rank pushes nothing over NVLink
    split = 1;
    while (split < 4 && 2 * split * M <= budget) split *= 2;
  }
  while (split > 1 && (H % (split * 8) != 0 || H / split < 256)) split >>= 1;
  const int slice = H / split;
  int threads = (slice / 8 + 31) / 32 * 32;
  if (threads > kGatherThreads) threads = kGatherThreads;
  const cudaError_t launched = launch_dependent(
      peer_reduce_add_rmsnorm_kernel, dim3(M, split), dim3(threads), stream, static_cast<const __half*>(partial), peers,
      own, static_cast<__half*>(residual), static_cast<const __half*>(weight), static_cast<__half*>(normed),
      static_cast<__half*>(reduced), H, world, rank, int64_t(rows) * (H / 4), eps);
  if (launched != cudaSuccess) return cuda_fail(launched, "peer_reduce_add_rmsnorm launch");
  return MKB_OK;
}

extern "C" int mkb_peer_status(const void* own, int* status) {
  using namespace mkb;
  MKB_REQUIRE(own && status, MKB_E_ARGUMENT, "peer_status: null pointer");
  uint32_t value = 0;
  const cudaError_t copied = cudaMemcpy(&value, &static_cast<const Header*>(own)->status, sizeof(value), cudaMemcpyDeviceToHost);
  if (copied != cudaSuccess) return cuda_fail(copied, "peer_status");
  *status = int(value);
  return MKB_OK;
}
