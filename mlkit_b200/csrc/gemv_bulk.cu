// Packed INT4 matvec fed by the tensor memory accelerator (TMA), M <= 8, fp16 (sm_100a).
//
// A decode matvec moves a few hundred KB of packed weights per SM and does almost no arithmetic per
// byte, so what decides its speed is (1) how soon and how many bytes are in flight and (2) how few
// instructions stand between an arrived byte and the tensor core.  Here
//   * one persistent CTA per SM owns a contiguous run of units; a unit is 16 weight rows x W chunks
//     of 256 codes (128 bytes per row and chunk), W = number of consumer warps (8..16);
//   * one producer thread moves whole units global -> shared with cp.async.bulk.tensor (a 3-D tensor
//     map {128 bytes, rows, chunks}, 128-byte swizzle) into a ring that holds ~200 KB -- for the
//     decoder shapes that is nearly everything the SM will ever read, so all of it is in flight from
//     the first microsecond; completion is tracked by mbarriers, nobody computes an address per tile;
//   * consumer warp w owns chunk w of every unit of a K slab.  Its activations never change inside
//     a slab, so its tensor-core B fragments (and min * sum(x) per scale group) live in registers for
//     the whole kernel: a unit costs a warp four conflict-free 16-byte shared loads, the nibble
//     decode (one AND per pair of codes: the masked bits are the fp16 subnormal c * 2^-24 or
//     c * 2^-20, each lift class with its own accumulator, so nothing is rounded), 16 m16n8k16
//     tensor-core steps and two scale multiplies;
//   * the W partial sums of a unit meet in shared memory; two reducer warps add them in warp order,
//     add the bias and store fp16.  When K is split over S slabs the reducers park the unit's sum in
//     a workspace and the last slab to arrive (atomic counter per row tile, left at zero) adds the S
//     partials in slab order -- the result does not depend on timing.
// Every wait is bounded: on expiry the CTA records a status word, stops issuing and drains.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kMaxConsumers = 16;
constexpr int kReducerWarps = 2;
constexpr int kMaxThreadsB = (kMaxConsumers + 1 + kReducerWarps) * 32;
constexpr int kChunkBytes = 2048;         // 16 rows x 128 bytes: what one consumer warp takes from a unit
constexpr int kMaxStages = 24;
constexpr uint32_t kSpinLimitB = 4000000;
constexpr int64_t kHeadBytes = 65536;     // workspace head: one counter per row tile, then a status word
constexpr int64_t kMaxRowTiles = kHeadBytes / 4 - 1;

struct BulkArgs {
  const __half* x;
  const __half* scales;
  const __half* bias;
  __half* y;
  float* partials;   // [row tile][slab][16 * M]
  int* counters;     // [row tile], zero between launches
  int* status;       // set non-zero when a bounded wait expired
  int M, N, K, group_shift;
  int64_t scale_row_stride;
  int consumers, slabs, row_tiles, units, stages, chunks;  // chunks of 256 codes per row
  int rows_outer;    // 0: a stage is [chunk][row][128 B]; 1: [row][chunk][128 B] (tensor map with natural dimension order)
  float grid_min;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase of the given parity; false when it gave up or another role did.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  const uint32_t address = smem_u32(bar);
  for (uint32_t spins = 0; spins < kSpinLimitB; ++spins) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(address), "r"(parity) : "memory");
    if (done) return true;
    if ((spins & 255) == 255 && *failed) return false;
  }
  *failed = 1;
  return false;
}

// One unit: box {128 bytes, 16 rows, W chunks} at (0, first row, first chunk); rows and chunks past
// the tensor are filled with zeros and still count toward the barrier's byte total.
__device__ __forceinline__ void unit_load(uint32_t dst, const CUtensorMap* map, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
  return v;
}

__device__ __forceinline__ void mma_step(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Position p = 8*w + 2*j + h of a lane's 32 activations (unit w, register j, half h) faces this code
// of the lane's 32-code chunk: a mask pair of a 4-bit word is (c, c + 4); registers 0,1 of a unit
// hold the pairs of the low nibbles of each byte (codes 0,2), registers 2,3 those of the high
// nibbles (codes 1,3).
__host__ __device__ constexpr int facing_code(int p) {
  const int w = p >> 3, j = (p >> 1) & 3, h = p & 1;
  return 8 * w + ((j & 1) * 2 + (j >> 1)) + 4 * h;
}

// The 32 activations x[0..31] of one lane and scale group, reordered into four B-fragment units.
__device__ __forceinline__ void fragment_units(const uint32_t (&xr)[16], uint4 (&unit)[4]) {
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e0 = facing_code(8 * w + 2 * j), e1 = facing_code(8 * w + 2 * j + 1);
      const uint32_t lo = (e0 & 1) ? (xr[e0 >> 1] >> 16) : (xr[e0 >> 1] & 0xffffu);
      const uint32_t hi = (e1 & 1) ? (xr[e1 >> 1] & 0xffff0000u) : (xr[e1 >> 1] << 16);
      out[j] = lo | hi;
    }
    unit[w] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// 32 codes of rows g and g+8 against the lane's activations of that scale group: 8 tensor-core
// steps; low-nibble codes (c * 2^-24) accumulate in lo, high-nibble codes (c * 2^-20) in hi.
__device__ __forceinline__ void group_steps(const uint4& c0, const uint4& c1, const uint4 (&b)[4], float (&lo)[4],
                                            float (&hi)[4]) {
  const uint32_t q0[4] = {c0.x, c0.y, c0.z, c0.w}, q1[4] = {c1.x, c1.y, c1.z, c1.w};
  const uint32_t bb[4][4] = {{b[0].x, b[0].y, b[0].z, b[0].w}, {b[1].x, b[1].y, b[1].z, b[1].w},
                             {b[2].x, b[2].y, b[2].z, b[2].w}, {b[3].x, b[3].y, b[3].z, b[3].w}};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t r0 = q0[w], r1 = q1[w], s0 = r0 >> 8, s1 = r1 >> 8;
    mma_step(lo, r0 & 0x000f000fu, r1 & 0x000f000fu, s0 & 0x000f000fu, s1 & 0x000f000fu, bb[w][0], bb[w][1]);
    mma_step(hi, r0 & 0x00f000f0u, r1 & 0x00f000f0u, s0 & 0x00f000f0u, s1 & 0x00f000f0u, bb[w][2], bb[w][3]);
  }
}

// ---- the kernel ----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kMaxThreadsB, 1)
gemv_bulk_kernel(const __grid_constant__ CUtensorMap weights, const BulkArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // the swizzle pattern repeats every 1024 bytes: stages start on that boundary
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int W = a.consumers;
  const int stage_bytes = W * kChunkBytes;
  const int outputs = 16 * a.M;                 // results of one unit: [m][row]
  float* red = reinterpret_cast<float*>(smem + size_t(a.stages) * stage_bytes);   // [2][W][outputs]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * W * outputs);             // [stages]
  uint64_t* empty = full + a.stages;                                                // [stages]
  uint64_t* red_full = empty + a.stages;                                            // [2]
  uint64_t* red_empty = red_full + 2;                                               // [2]
  volatile int* failed = reinterpret_cast<volatile int*>(red_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int u0 = int(int64_t(blockIdx.x) * a.units / gridDim.x);
  const int u1 = int(int64_t(blockIdx.x + 1) * a.units / gridDim.x);
  const int n_units = u1 - u0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      bar_init(full + s, 1);
      bar_init(empty + s, W);
    }
    for (int b = 0; b < 2; ++b) {
      bar_init(red_full + b, W);
      bar_init(red_empty + b, 1);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == W) {
    // ---- producer: weights are constants, so it does not wait for the previous kernel ----
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < n_units; ++i) {
        const int stage = i % a.stages, round = i / a.stages;
        if (round > 0 && !bar_wait(empty + stage, (round - 1) & 1, failed)) break;
        const int u = u0 + i, slab = u / a.row_tiles, rt = u - slab * a.row_tiles;
        bar_expect(full + stage, uint32_t(stage_bytes));
        const uint32_t dst = smem_u32(smem + size_t(stage) * stage_bytes);
        if (a.rows_outer) unit_load(dst, &weights, slab * W, rt * 16, full + stage);
        else unit_load(dst, &weights, rt * 16, slab * W, full + stage);
        issued = i + 1;
      }
      if (*failed) {
        // copies still in flight must land before the CTA may go: wait (bounded) for the last ones
        if (a.status != nullptr) atomicExch(a.status, 1);
        const int first = issued > a.stages ? issued - a.stages : 0;
        for (int i = first; i < issued; ++i) {
          const uint32_t address = smem_u32(full + i % a.stages), parity = uint32_t(i / a.stages) & 1u;
          for (uint32_t spins = 0; spins < kSpinLimitB; ++spins) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                         : "=r"(done) : "r"(address), "r"(parity) : "memory");
            if (done) break;
          }
        }
      }
    }
  } else if (warp < W) {
    // ---- consumers ----
    const int g = lane >> 2, t = lane & 3;
    // fragment row g reads memory row rho(g) of the tile: the two rows of a quarter warp then differ
    // in bit 2, which the swizzle turns into disjoint bank sets
    const int rho = (g >> 1) + 4 * (g & 1);
    // the 128-byte swizzle XORs the 16-byte index of a line with bits 7..9 of its address (stages are
    // 1024-byte aligned, so the offset inside the stage decides)
    const uint32_t row_pitch = a.rows_outer ? uint32_t(W) * 128u : 128u, chunk_pitch = a.rows_outer ? 128u : 2048u;
    const uint32_t line0 = warp * chunk_pitch + rho * row_pitch, line1 = line0 + 8 * row_pitch;
    const uint32_t x0 = (line0 >> 7) & 7u, x1 = (line1 >> 7) & 7u;
    const uint32_t base = smem_u32(smem);
    const uint32_t a00 = base + line0 + ((uint32_t(t) ^ x0) << 4), a01 = base + line0 + ((uint32_t(t + 4) ^ x0) << 4);
    const uint32_t a10 = base + line1 + ((uint32_t(t) ^ x1) << 4), a11 = base + line1 + ((uint32_t(t + 4) ^ x1) << 4);

    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint4 b0[4], b1[4];            // B fragments of the chunk's two scale groups
    float bias0[2], bias1[2];      // min * sum(x) * 2^-24 of the two groups for activation rows 2t, 2t+1
    int slab_now = -1;
    auto load_activations = [&](int slab) {
      const int chunk = slab * W + warp;
      float sums[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t xr[16];
        const bool live = g < a.M && chunk < a.chunks;
        const uint4* src = reinterpret_cast<const uint4*>(a.x + int64_t(live ? g : 0) * a.K +
                                                          int64_t(live ? chunk : 0) * 256 + j * 128 + t * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 v = live ? __ldg(src + q) : make_uint4(0u, 0u, 0u, 0u);
          xr[4 * q] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
        }
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&xr[q]));
          sum += pair.x;
          sum += pair.y;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sums[j] = sum * a.grid_min * 5.9604644775390625e-08f;  // 2^-24
        if (j == 0) fragment_units(xr, b0); else fragment_units(xr, b1);
      }
      // the sum of activation row m sits on lanes with g == m; accumulator columns are rows 2t, 2t+1
      bias0[0] = __shfl_sync(0xffffffffu, sums[0], (2 * t) * 4);
      bias0[1] = __shfl_sync(0xffffffffu, sums[0], (2 * t + 1) * 4);
      bias1[0] = __shfl_sync(0xffffffffu, sums[1], (2 * t) * 4);
      bias1[1] = __shfl_sync(0xffffffffu, sums[1], (2 * t + 1) * 4);
    };
    // the four scales of a unit: rows rho, rho + 8 of the tile, the chunk's two groups
    auto load_scales = [&](int u, __half (&s)[4]) {
      const int slab = u / a.row_tiles, rt = u - slab * a.row_tiles;
      const int chunk = min(slab * W + warp, a.chunks - 1);
      const int64_t r0 = min(rt * 16 + rho, a.N - 1), r1 = min(rt * 16 + rho + 8, a.N - 1);
      const int c0 = (chunk * 256) >> a.group_shift, c1 = (chunk * 256 + 128) >> a.group_shift;
      s[0] = __ldg(a.scales + r0 * a.scale_row_stride + c0);
      s[1] = __ldg(a.scales + r0 * a.scale_row_stride + c1);
      s[2] = __ldg(a.scales + r1 * a.scale_row_stride + c0);
      s[3] = __ldg(a.scales + r1 * a.scale_row_stride + c1);
    };
    __half scale_next[4];
    if (n_units > 0) load_scales(u0, scale_next);
    for (int i = 0; i < n_units; ++i) {
      const int u = u0 + i, slab = u / a.row_tiles;
      if (slab != slab_now) {
        load_activations(slab);
        slab_now = slab;
      }
      const float s00 = __half2float(scale_next[0]), s01 = __half2float(scale_next[1]);
      const float s10 = __half2float(scale_next[2]), s11 = __half2float(scale_next[3]);
      if (i + 1 < n_units) load_scales(u + 1, scale_next);

      const int stage = i % a.stages;
      if (!bar_wait(full + stage, uint32_t(i / a.stages) & 1u, failed)) break;
      const uint32_t stage_offset = uint32_t(stage) * uint32_t(stage_bytes);
      const uint4 c00 = lds128(a00 + stage_offset), c10 = lds128(a10 + stage_offset);   // group 0: rows g, g+8
      const uint4 c01 = lds128(a01 + stage_offset), c11 = lds128(a11 + stage_offset);   // group 1
      __syncwarp();
      if (lane == 0) bar_arrive(empty + stage);

      float lo[4] = {bias0[0], bias0[1], bias0[0], bias0[1]}, hi[4] = {0.f, 0.f, 0.f, 0.f};
      group_steps(c00, c10, b0, lo, hi);
      float y[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) y[q] = (q < 2 ? s00 : s10) * fmaf(hi[q], 0.0625f, lo[q]);
      float lo1[4] = {bias1[0], bias1[1], bias1[0], bias1[1]}, hi1[4] = {0.f, 0.f, 0.f, 0.f};
      group_steps(c01, c11, b1, lo1, hi1);
#pragma unroll
      for (int q = 0; q < 4; ++q) y[q] = fmaf(q < 2 ? s01 : s11, fmaf(hi1[q], 0.0625f, lo1[q]), y[q]);

      // partial sums of this warp: [m][memory row of the tile]
      const int buffer = i & 1, use = i >> 1;
      if (use > 0 && !bar_wait(red_empty + buffer, uint32_t(use - 1) & 1u, failed)) break;
      float* mine = red + (buffer * W + warp) * outputs;
      if (2 * t < a.M) {
        mine[(2 * t) * 16 + rho] = y[0];
        mine[(2 * t) * 16 + rho + 8] = y[2];
      }
      if (2 * t + 1 < a.M) {
        mine[(2 * t + 1) * 16 + rho] = y[1];
        mine[(2 * t + 1) * 16 + rho + 8] = y[3];
      }
      __syncwarp();
      if (lane == 0) bar_arrive(red_full + buffer);
    }
  } else {
    // ---- reducers: warp r takes the units of parity r ----
    const int r = warp - W - 1;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = r; i < n_units; i += kReducerWarps) {
      const int u = u0 + i, slab = u / a.row_tiles, rt = u - slab * a.row_tiles;
      const int use = i >> 1;
      if (!bar_wait(red_full + r, uint32_t(use) & 1u, failed)) break;
      float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int j = lane + 32 * q;
        if (j < outputs) {
          const float* partial = red + r * W * outputs + j;
          for (int w = 0; w < W; ++w) sum[q] += partial[w * outputs];
        }
      }
      __syncwarp();
      if (lane == 0) bar_arrive(red_empty + r);

      bool finish = true;
      if (a.slabs > 1) {
        float* slot = a.partials + (int64_t(rt) * a.slabs + slab) * outputs;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (lane + 32 * q < outputs) slot[lane + 32 * q] = sum[q];
        __threadfence();
        __syncwarp();
        int arrived = 0;
        if (lane == 0) arrived = atomicAdd(a.counters + rt, 1);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        finish = arrived == a.slabs - 1;
        if (finish) {
          __threadfence();
          const float* first = a.partials + int64_t(rt) * a.slabs * outputs;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            sum[q] = 0.f;
            if (lane + 32 * q < outputs)
              for (int s = 0; s < a.slabs; ++s) sum[q] += __ldcg(first + s * outputs + lane + 32 * q);
          }
          if (lane == 0) a.counters[rt] = 0;
        }
      }
      if (finish) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = lane + 32 * q, m = j >> 4, row = rt * 16 + (j & 15);
          if (j < outputs && row < a.N) {
            float value = sum[q] * 16777216.f;  // codes were c * 2^-24
            if (a.bias != nullptr) value += __half2float(a.bias[row]);
            a.y[int64_t(m) * a.N + row] = __float2half_rn(value);
          }
        }
      }
    }
    if (*failed && lane == 0 && a.status != nullptr) atomicExch(a.status, 1);
  }
}

// ---- host side -----------------------------------------------------------------------------------
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
  static EncodeTiled function = []() -> EncodeTiled {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiled>(entry);
  }();
  return function;
}

struct MapEntry {
  CUtensorMap map;
  int rows_outer;
};

// Tensor maps are pure functions of (pointer, shape, stride, box): built once per weight and kept.
int weight_map(const uint8_t* packed, int N, int chunks, int64_t row_stride, int consumers, MapEntry& out) {
  static std::mutex lock;
  static std::map<std::tuple<const void*, int, int, int64_t, int>, MapEntry> cache;
  static int preferred_order_works = -1;  // unknown, 0, 1
  const auto key = std::make_tuple(static_cast<const void*>(packed), N, chunks, row_stride, consumers);
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) { out = found->second; return MKB_OK; }
  EncodeTiled encode = encoder();
  MKB_REQUIRE(encode != nullptr, MKB_E_CUDA, "gemv_bulk: the driver does not offer cuTensorMapEncodeTiled");
  MapEntry entry{};
  const cuuint32_t unit_strides[3] = {1, 1, 1};
  CUresult result = CUDA_ERROR_INVALID_VALUE;
  if (preferred_order_works != 0) {
    // dimensions {byte in line, row, chunk}: a stage is [chunk][row][128 B] and the swizzle follows the row
    const cuuint64_t dims[3] = {128, cuuint64_t(N), cuuint64_t(chunks)};
    const cuuint64_t strides[2] = {cuuint64_t(row_stride), 128};
    const cuuint32_t box[3] = {128, 16, cuuint32_t(consumers)};
    result = encode(&entry.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(packed), dims, strides, box,
                    unit_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    entry.rows_outer = 0;
    preferred_order_works = result == CUDA_SUCCESS ? 1 : 0;
  }
  if (result != CUDA_SUCCESS) {
    // natural order {byte in line, chunk, row}: a stage is [row][chunk][128 B]
    const cuuint64_t dims[3] = {128, cuuint64_t(chunks), cuuint64_t(N)};
    const cuuint64_t strides[2] = {128, cuuint64_t(row_stride)};
    const cuuint32_t box[3] = {128, cuuint32_t(consumers), 16};
    result = encode(&entry.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(packed), dims, strides, box,
                    unit_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    entry.rows_outer = 1;
  }
  MKB_REQUIRE(result == CUDA_SUCCESS, MKB_E_CUDA, "gemv_bulk: cuTensorMapEncodeTiled failed with %d", int(result));
  if (cache.size() > 65536) cache.clear();
  cache[key] = entry;
  out = entry;
  return MKB_OK;
}

// K split: W consumer warps take one 256-code chunk each, S slabs of W chunks cover a row.
void split_for(int N, int K, int sm_count, int& consumers, int& slabs) {
  const int chunks = K / 256, row_tiles = (N + 15) / 16;
  slabs = (chunks + kMaxConsumers - 1) / kMaxConsumers;
  consumers = (chunks + slabs - 1) / slabs;
  // small layers: more, thinner units until every SM has a few
  while (consumers >= 8 && consumers % 2 == 0 && int64_t(slabs) * row_tiles < 2 * sm_count) {
    slabs *= 2;
    consumers /= 2;
  }
}

}  // namespace

int gemv_bulk_supported(int M, int N, int K, int group, int bits, int x_dtype, int scale_dtype, const void* x,
                        const uint8_t* packed, int64_t packed_row_stride, const void* zeros, int integer_grid,
                        float grid_minimum) {
  if (bits != 4 || x_dtype != MKB_F16 || scale_dtype != MKB_F16 || zeros != nullptr || !integer_grid) return 0;
  if (M < 1 || M > 8 || N < 1 || K < 256 || K % 256 != 0) return 0;
  if (group < 128 || (group & (group - 1)) != 0) return 0;
  if (grid_minimum != float(int(grid_minimum)) || grid_minimum < -512.f || grid_minimum > 512.f) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(packed) % 16 || packed_row_stride % 16) return 0;
  if ((N + 15) / 16 > kMaxRowTiles) return 0;
  return 1;
}

// Bytes of workspace the K split of this shape needs (0: none).
int64_t gemv_bulk_workspace_bytes(int M, int N, int K) {
  if (K < 256 || K % 256 != 0 || N < 1) return 0;
  int consumers = 0, slabs = 0;
  split_for(N, K, device_info().sm_count, consumers, slabs);
  if (slabs <= 1) return 0;
  return kHeadBytes + int64_t((N + 15) / 16) * slabs * 16 * M * 4;
}

int launch_gemv_bulk(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                     void* workspace, int64_t workspace_bytes, int M, int N, int K, int group,
                     int64_t packed_row_stride, int64_t scale_row_stride, float grid_minimum, cudaStream_t stream) {
  BulkArgs a{};
  a.x = static_cast<const __half*>(x); a.scales = static_cast<const __half*>(scales);
  a.bias = static_cast<const __half*>(bias); a.y = static_cast<__half*>(y);
  a.M = M; a.N = N; a.K = K; a.scale_row_stride = scale_row_stride; a.grid_min = grid_minimum;
  a.group_shift = 0;
  while ((1 << a.group_shift) < group) ++a.group_shift;
  const DeviceInfo& info = device_info();
  a.chunks = K / 256;
  a.row_tiles = (N + 15) / 16;
  split_for(N, K, info.sm_count, a.consumers, a.slabs);
  a.units = a.row_tiles * a.slabs;
  if (a.slabs > 1) {
    MKB_REQUIRE(workspace != nullptr && workspace_bytes >= gemv_bulk_workspace_bytes(M, N, K), MKB_E_UNSUPPORTED,
                "gemv_bulk: K=%d is split over %d slabs and needs a workspace of %lld B", K, a.slabs,
                (long long)gemv_bulk_workspace_bytes(M, N, K));
    a.counters = static_cast<int*>(workspace);
    a.status = a.counters + kMaxRowTiles;
    a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kHeadBytes);
  } else if (workspace != nullptr && workspace_bytes >= kHeadBytes) {
    a.status = static_cast<int*>(workspace) + kMaxRowTiles;
  }

  const int stage_bytes = a.consumers * kChunkBytes;
  const size_t fixed = 1024 + size_t(2) * a.consumers * 16 * M * 4 + size_t(2 * kMaxStages + 4) * 8 + 16;
  int stages = int((size_t(info.max_smem_optin) - fixed) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  MKB_REQUIRE(stages >= 2, MKB_E_UNSUPPORTED, "gemv_bulk: shared memory holds fewer than two stages");
  int grid = info.sm_count < a.units ? info.sm_count : a.units;
  const int most = (a.units + grid - 1) / grid;
  if (stages > most) stages = most;  // no CTA ever has more units than this
  a.stages = stages;
  const size_t smem = 1024 + size_t(stages) * stage_bytes + size_t(2) * a.consumers * 16 * M * 4 +
                      size_t(2 * stages + 4) * 8 + 16;

  MapEntry entry;
  int status = weight_map(packed, N, a.chunks, packed_row_stride, a.consumers, entry);
  if (status != MKB_OK) return status;
  a.rows_outer = entry.rows_outer;

  static bool configured[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    cudaError_t set = cudaFuncSetAttribute(gemv_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           info.max_smem_optin);
    if (set != cudaSuccess) return cuda_fail(set, "gemv_bulk: shared memory opt-in");
    configured[device] = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3((a.consumers + 1 + kReducerWarps) * 32, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t launched = cudaLaunchKernelEx(&config, gemv_bulk_kernel, entry.map, a);
  if (launched != cudaSuccess) return cuda_fail(launched, "gemv_bulk launch");
  return MKB_OK;
}

}  // namespace mkb
