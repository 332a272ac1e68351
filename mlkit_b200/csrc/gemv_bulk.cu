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
constexpr int kMaxReducers = 2;
constexpr int kMaxThreadsB = (kMaxConsumers + 1 + kMaxReducers) * 32;
constexpr int kRedBuffers = 4;            // ring of partial-sum buffers between consumers and reducers
constexpr int kBatch = 4;                 // units a reducer publishes together when K is split
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
  int reducers;
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

// One look at the barrier, no waiting.
__device__ __forceinline__ bool bar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
               : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
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

// The first step of an accumulator chain: C = 0 comes from the zero register, no initialisation.
__device__ __forceinline__ void mma_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
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

// 2 x 32 codes of rows g and g+8 (the chunk's two scale groups) against the lane's activations: 16
// tensor-core steps.  Low-nibble codes (c * 2^-24) and high-nibble codes (c * 2^-20) of each group
// have accumulators of their own, so four independent chains are in flight.
__device__ __forceinline__ void group_steps(const uint4& c00, const uint4& c10, const uint4& c01, const uint4& c11,
                                            const uint4 (&b0)[4], const uint4 (&b1)[4], float (&lo0)[4], float (&hi0)[4],
                                            float (&lo1)[4], float (&hi1)[4]) {
  const uint32_t q00[4] = {c00.x, c00.y, c00.z, c00.w}, q10[4] = {c10.x, c10.y, c10.z, c10.w};
  const uint32_t q01[4] = {c01.x, c01.y, c01.z, c01.w}, q11[4] = {c11.x, c11.y, c11.z, c11.w};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t r0 = q00[w], r1 = q10[w], s0 = r0 >> 8, s1 = r1 >> 8;
    const uint32_t u0 = q01[w], u1 = q11[w], v0 = u0 >> 8, v1 = u1 >> 8;
    if (w == 0) {
      mma_first(lo0, r0 & 0x000f000fu, r1 & 0x000f000fu, s0 & 0x000f000fu, s1 & 0x000f000fu, b0[w].x, b0[w].y);
      mma_first(lo1, u0 & 0x000f000fu, u1 & 0x000f000fu, v0 & 0x000f000fu, v1 & 0x000f000fu, b1[w].x, b1[w].y);
      mma_first(hi0, r0 & 0x00f000f0u, r1 & 0x00f000f0u, s0 & 0x00f000f0u, s1 & 0x00f000f0u, b0[w].z, b0[w].w);
      mma_first(hi1, u0 & 0x00f000f0u, u1 & 0x00f000f0u, v0 & 0x00f000f0u, v1 & 0x00f000f0u, b1[w].z, b1[w].w);
    } else {
      mma_step(lo0, r0 & 0x000f000fu, r1 & 0x000f000fu, s0 & 0x000f000fu, s1 & 0x000f000fu, b0[w].x, b0[w].y);
      mma_step(lo1, u0 & 0x000f000fu, u1 & 0x000f000fu, v0 & 0x000f000fu, v1 & 0x000f000fu, b1[w].x, b1[w].y);
      mma_step(hi0, r0 & 0x00f000f0u, r1 & 0x00f000f0u, s0 & 0x00f000f0u, s1 & 0x00f000f0u, b0[w].z, b0[w].w);
      mma_step(hi1, u0 & 0x00f000f0u, u1 & 0x00f000f0u, v0 & 0x00f000f0u, v1 & 0x00f000f0u, b1[w].z, b1[w].w);
    }
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
  float* red = reinterpret_cast<float*>(smem + size_t(a.stages) * stage_bytes);   // [kRedBuffers][W][outputs]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + kRedBuffers * W * outputs);   // [stages]
  uint64_t* empty = full + a.stages;                                                // [stages]
  uint64_t* red_full = empty + a.stages;                                            // [kRedBuffers]
  uint64_t* red_empty = red_full + kRedBuffers;                                     // [kRedBuffers]
  volatile int* failed = reinterpret_cast<volatile int*>(red_empty + kRedBuffers);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int u0 = int(int64_t(blockIdx.x) * a.units / gridDim.x);
  const int u1 = int(int64_t(blockIdx.x + 1) * a.units / gridDim.x);
  const int n_units = u1 - u0;
  const int slab_first = u0 / a.row_tiles, rt_first = u0 - slab_first * a.row_tiles;

  // The producer thread sets the barriers up and has the first ring of units on its way before
  // anyone else runs: weights are constants, so it does not wait for the previous kernel either.
  int issue_slab = slab_first, issue_rt = rt_first, issue_stage = 0;
  auto issue_unit = [&]() {
    const int stage = issue_stage, slab = issue_slab, rt = issue_rt;
    if (++issue_stage == a.stages) issue_stage = 0;
    if (++issue_rt == a.row_tiles) { issue_rt = 0; ++issue_slab; }
    bar_expect(full + stage, uint32_t(stage_bytes));
    const uint32_t dst = smem_u32(smem + size_t(stage) * stage_bytes);
    if (a.rows_outer) unit_load(dst, &weights, slab * W, rt * 16, full + stage);
    else unit_load(dst, &weights, rt * 16, slab * W, full + stage);
  };
  const int first_wave = n_units < a.stages ? n_units : a.stages;
  if (warp == W && lane == 0) {
    for (int s = 0; s < a.stages; ++s) {
      bar_init(full + s, 1);
      bar_init(empty + s, W);
    }
    for (int b = 0; b < kRedBuffers; ++b) {
      bar_init(red_full + b, W);
      bar_init(red_empty + b, 1);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int i = 0; i < first_wave; ++i) issue_unit();
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == W) {
    // ---- producer: refill a stage as soon as all consumer warps have read it ----
    if (lane == 0) {
      int issued = first_wave;
      uint32_t empty_phase = 0;
      for (int i = first_wave; i < n_units; ++i) {
        if (!bar_wait(empty + issue_stage, empty_phase, failed)) break;
        if (issue_stage == a.stages - 1) empty_phase ^= 1u;
        issue_unit();
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

    uint4 b0[4], b1[4];            // B fragments of the chunk's two scale groups
    float bias0[2], bias1[2];      // min * sum(x) * 2^-24 of the two groups for activation rows 2t, 2t+1
    auto load_activations = [&](int slab) {
      const int chunk = slab * W + warp;
      const bool live = g < a.M && chunk < a.chunks;
      const uint4* src = reinterpret_cast<const uint4*>(a.x + int64_t(live ? g : 0) * a.K +
                                                        int64_t(live ? chunk : 0) * 256 + t * 32);
      uint4 v[8];   // all eight requests leave before the first is used
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = live ? __ldg(src + (q >> 2) * 16 + (q & 3)) : make_uint4(0u, 0u, 0u, 0u);
      float sums[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t xr[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          xr[4 * q] = v[4 * j + q].x; xr[4 * q + 1] = v[4 * j + q].y; xr[4 * q + 2] = v[4 * j + q].z; xr[4 * q + 3] = v[4 * j + q].w;
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
    // the four scales of a unit (rows rho, rho + 8 of the tile x the chunk's two groups) as two
    // packed pairs; they are constants, so the first ones are requested before the dependency wait,
    // and the loop keeps two units of them in flight
    const bool paired = a.group_shift == 7 && (a.scale_row_stride & 1) == 0 && (reinterpret_cast<uintptr_t>(a.scales) & 3) == 0;
    auto load_scales = [&](int slab, int rt, uint32_t (&s)[2]) {
      const int chunk = min(slab * W + warp, a.chunks - 1);
      const int64_t r0 = min(rt * 16 + rho, a.N - 1), r1 = min(rt * 16 + rho + 8, a.N - 1);
      const __half* p0 = a.scales + r0 * a.scale_row_stride;
      const __half* p1 = a.scales + r1 * a.scale_row_stride;
      if (paired) {
        s[0] = __ldg(reinterpret_cast<const uint32_t*>(p0 + chunk * 2));
        s[1] = __ldg(reinterpret_cast<const uint32_t*>(p1 + chunk * 2));
      } else {
        const int c0 = (chunk * 256) >> a.group_shift, c1 = (chunk * 256 + 128) >> a.group_shift;
        const unsigned short* q0 = reinterpret_cast<const unsigned short*>(p0);
        const unsigned short* q1 = reinterpret_cast<const unsigned short*>(p1);
        s[0] = uint32_t(__ldg(q0 + c0)) | (uint32_t(__ldg(q0 + c1)) << 16);
        s[1] = uint32_t(__ldg(q1 + c0)) | (uint32_t(__ldg(q1 + c1)) << 16);
      }
    };
    auto advance = [&](int& slab, int& rt) {
      if (++rt == a.row_tiles) { rt = 0; ++slab; }
    };
    int slab = slab_first, rt = rt_first;             // this unit
    int slab_ahead = slab, rt_ahead = rt;             // the unit whose scales are requested next
    int slab_now = -1;
    uint32_t scale_now[2] = {0u, 0u}, scale_next[2] = {0u, 0u};
    if (n_units > 0) { load_scales(slab_ahead, rt_ahead, scale_now); advance(slab_ahead, rt_ahead); }
    if (n_units > 1) { load_scales(slab_ahead, rt_ahead, scale_next); advance(slab_ahead, rt_ahead); }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    int stage = 0;
    uint32_t phase = 0, stage_offset = 0;
    for (int i = 0; i < n_units; ++i) {
      if (slab != slab_now) {
        load_activations(slab);
        slab_now = slab;
      }
      uint32_t scale_after[2] = {0u, 0u};
      if (i + 2 < n_units) { load_scales(slab_ahead, rt_ahead, scale_after); advance(slab_ahead, rt_ahead); }

      if (!bar_wait(full + stage, phase, failed)) break;
      if (warp == 0 && lane == 0) {
      }
      const uint4 d00 = lds128(a00 + stage_offset), d10 = lds128(a10 + stage_offset);   // group 0: rows g, g+8
      const uint4 d01 = lds128(a01 + stage_offset), d11 = lds128(a11 + stage_offset);   // group 1
      __syncwarp();
      if (lane == 0) bar_arrive(empty + stage);
      if (++stage == a.stages) { stage = 0; phase ^= 1u; stage_offset = 0; } else { stage_offset += uint32_t(stage_bytes); }
      advance(slab, rt);

      // 16 tensor-core steps in four independent accumulator chains (two groups x two lift classes)
      float lo0[4], hi0[4], lo1[4], hi1[4];
      group_steps(d00, d10, d01, d11, b0, b1, lo0, hi0, lo1, hi1);
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&scale_now[0]));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&scale_now[1]));
      float y[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float first = (q < 2 ? f0.x : f1.x) * (fmaf(hi0[q], 0.0625f, lo0[q]) + bias0[q & 1]);
        y[q] = fmaf(q < 2 ? f0.y : f1.y, fmaf(hi1[q], 0.0625f, lo1[q]) + bias1[q & 1], first);
      }
      scale_now[0] = scale_next[0]; scale_now[1] = scale_next[1];
      scale_next[0] = scale_after[0]; scale_next[1] = scale_after[1];

      // partial sums of this warp: [m][memory row of the tile]
      const int buffer = i & (kRedBuffers - 1), use = i / kRedBuffers;
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
    // ---- reducers: warp r of R takes the units i = r, r + R, ... in batches, so that the slow part
    // of a K split (fence, counter, reading the other slabs' sums) is paid once per batch ----
    const int r = warp - W - 1, R = a.reducers;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int next_slab = slab_first, next_rt = rt_first + r;
    while (next_rt >= a.row_tiles) { next_rt -= a.row_tiles; ++next_slab; }
    auto store_rows = [&](const float (&sum)[4], int rt) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int j = lane + 32 * q, m = j >> 4, row = rt * 16 + (j & 15);
        if (j < outputs && row < a.N) {
          float value = sum[q] * 16777216.f;  // codes were c * 2^-24
          if (a.bias != nullptr) value += __half2float(a.bias[row]);
          a.y[int64_t(m) * a.N + row] = __float2half_rn(value);
        }
      }
    };
    bool alive = true;
    for (int i0 = r; i0 < n_units && alive; i0 += R * kBatch) {
      int my_rt = -1;   // lane b keeps the row tile of the batch's unit b
      for (int b = 0; b < kBatch; ++b) {
        const int i = i0 + b * R;
        if (i >= n_units) break;
        const int slab = next_slab, rt = next_rt;
        next_rt += R;
        while (next_rt >= a.row_tiles) { next_rt -= a.row_tiles; ++next_slab; }
        const int buffer = i & (kRedBuffers - 1), use = i / kRedBuffers;
        if (!bar_wait(red_full + buffer, uint32_t(use) & 1u, failed)) { alive = false; break; }
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int j = lane + 32 * q;
          if (j < outputs) {
            const float* partial = red + buffer * W * outputs + j;
            float part[kMaxConsumers];
#pragma unroll
            for (int w = 0; w < kMaxConsumers; ++w) part[w] = w < W ? partial[w * outputs] : 0.f;
#pragma unroll
            for (int w = 0; w < kMaxConsumers; ++w) sum[q] += part[w];
          }
        }
        __syncwarp();
        if (lane == 0) bar_arrive(red_empty + buffer);
        if (a.slabs == 1) {
          store_rows(sum, rt);
        } else {
          float* slot = a.partials + (int64_t(rt) * a.slabs + slab) * outputs;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (lane + 32 * q < outputs) slot[lane + 32 * q] = sum[q];
          if (lane == b) my_rt = rt;
        }
      }
      if (a.slabs > 1) {
        // publish the batch: the sums above must be visible before the counters move
        __threadfence();
        __syncwarp();
        const int arrived = my_rt >= 0 ? atomicAdd(a.counters + my_rt, 1) : -1;
        unsigned finishing = __ballot_sync(0xffffffffu, arrived == a.slabs - 1);
        if (finishing) __threadfence();
        while (finishing) {
          const int b = __ffs(finishing) - 1;
          finishing &= finishing - 1;
          const int rt = __shfl_sync(0xffffffffu, my_rt, b);
          const float* first = a.partials + int64_t(rt) * a.slabs * outputs;
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
          for (int s = 0; s < a.slabs; ++s)
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (lane + 32 * q < outputs) sum[q] += __ldcg(first + s * outputs + lane + 32 * q);
          store_rows(sum, rt);
          if (lane == b) a.counters[rt] = 0;
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

// K split: W consumer warps take one 256-code chunk each, S slabs of W chunks cover a row.  Thin
// CTAs (W <= 8) run two to an SM with one reducer warp, wide ones alone with two.
struct Split {
  int consumers, slabs, ctas_per_sm, reducers;
};

Split split_for(int N, int K, int sm_count) {
  const int chunks = K / 256, row_tiles = (N + 15) / 16;
  Split split{};
  split.slabs = (chunks + kMaxConsumers - 1) / kMaxConsumers;
  split.consumers = (chunks + split.slabs - 1) / split.slabs;
  // small layers: more, thinner units until every SM has a few
  while (split.consumers >= 8 && split.consumers % 2 == 0 && int64_t(split.slabs) * row_tiles < 2 * sm_count) {
    split.slabs *= 2;
    split.consumers /= 2;
  }
  split.ctas_per_sm = split.consumers <= 8 ? 2 : 1;
  split.reducers = split.consumers <= 8 ? 1 : 2;
  return split;
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
  const Split split = split_for(N, K, device_info().sm_count);
  if (split.slabs <= 1) return 0;
  return kHeadBytes + int64_t((N + 15) / 16) * split.slabs * 16 * M * 4;
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
  const Split split = split_for(N, K, info.sm_count);
  a.consumers = split.consumers; a.slabs = split.slabs; a.reducers = split.reducers;
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

  // shared memory: the ring takes what the partial-sum buffers and barriers leave of the CTA's share
  const int stage_bytes = a.consumers * kChunkBytes;
  const size_t share = split.ctas_per_sm == 1 ? size_t(info.max_smem_optin)
                                              : (size_t(info.max_smem_optin) + 1024) / 2 - 1024;
  const size_t red_bytes = size_t(kRedBuffers) * a.consumers * 16 * M * 4;
  const size_t fixed = 1024 + red_bytes + size_t(2 * kMaxStages + 2 * kRedBuffers) * 8 + 16;
  MKB_REQUIRE(share > fixed + 2 * size_t(stage_bytes), MKB_E_UNSUPPORTED, "gemv_bulk: shared memory holds fewer than two stages");
  int stages = int((share - fixed) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  int grid = info.sm_count * split.ctas_per_sm;
  if (grid > a.units) grid = a.units;
  const int most = (a.units + grid - 1) / grid;
  if (stages > most) stages = most;  // no CTA ever has more units than this
  a.stages = stages;
  const size_t smem = 1024 + size_t(stages) * stage_bytes + red_bytes + size_t(2 * stages + 2 * kRedBuffers) * 8 + 16;

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
    if (set == cudaSuccess)
      set = cudaFuncSetAttribute(gemv_bulk_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared);
    if (set != cudaSuccess) return cuda_fail(set, "gemv_bulk: shared memory opt-in");
    configured[device] = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3((a.consumers + 1 + a.reducers) * 32, 1, 1);
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
