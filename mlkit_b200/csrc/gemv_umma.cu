// Packed INT4 matvec on the 5th-generation tensor cores (tcgen05, sm_100a), M <= 8, fp16.
//
// Why tensor memory: at 4 bits per weight one SM must turn ~46 weights per clock into products to
// keep up with HBM.  With register-fragment tensor-core instructions every lane pays for operand
// shuffling, fragment loads and per-tile bookkeeping; here a thread owns one weight ROW, decodes its
// codes with one AND per pair, and hands them to the tensor core through tensor memory (TMEM) as the
// A operand of tcgen05.mma.  Activations are the B operand, read by the tensor core from shared
// memory; accumulators live in TMEM.  A thread touches nothing but its own row.
//
// Work: a unit is 128 output rows x 512 codes (4 scale groups, 32 KB of codes).  A CTA keeps one K
// slab (so its activation tiles are staged once, 16 KB) and walks units blockIdx.x,
// blockIdx.x + gridDim.x, ...  Roles inside the CTA (224 threads):
//   * warps 0-3, "row" threads: thread r owns row r of the current unit.  Per group of 128 codes the
//     128 x 64 B code tile arrives by cp.async (coalesced) in a shared-memory ring; the thread reads
//     its 64 bytes, masks codes into fp16 subnormals c * 2^-24 (low nibbles) and c * 2^-20 (high
//     nibbles) and stores them to its TMEM lane (tcgen05.st), 64 columns of the A buffer of that
//     group's parity; one group later it loads its row of the accumulators (tcgen05.ld) and adds
//     scale[r, group] * (D0 + D1 / 16 + min * sum(x)) to its fp32 outputs;
//   * warps 4 and 6, "issuers": one lane of each waits for an A buffer and issues four of the group's
//     eight tcgen05.mma (M128 N16 K16) -- warp 4 the low-nibble steps, which accumulate in D0, warp 6 the
//     high-nibble steps, which accumulate in D1, so no operand is rescaled and nothing is rounded -- and
//     commits them to an mbarrier.  A and D are double buffered, so issuing overlaps the decode of the
//     next group;
//   * warp 5, "publisher": K is split over slabs, so a unit ends with a partial [M x 128] in the
//     workspace.  This warp publishes the unit (fence, atomic counter per row block) and, when its
//     unit was the last of the row block, adds the partials in slab order, adds the bias and
//     stores fp16.  The counter is left at zero, so the workspace needs zeroing only once.
// All hand-offs are mbarriers; every wait is bounded: on expiry the CTA records a status word,
// stops issuing and drains.
#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kRowThreads = 128;
constexpr int kThreadsU = 224;            // 4 row warps, issuer warp, publisher warp, second issuer warp
constexpr int kSlabGroups = 4;            // scale groups (of 128 codes) per unit
constexpr int kDepthU = 8;                // ring stages, one group each
constexpr int kPitch = 80;                // bytes per row in a stage: 64 of codes + 16 of padding
constexpr int kStageBytes = 128 * kPitch;
constexpr int kTileBytes = 512;           // one B tile: [2 k-chunks][16 rows][8 halves]
constexpr int kTmemColumns = 256;         // A[2]: 0..127; D[2][2]: 128..191
constexpr uint32_t kSpinLimit = 2000000;

struct UmmaArgs {
  const __half* x;
  const uint8_t* packed;
  const __half* scales;
  const __half* bias;
  __half* y;
  float* partials;   // [row_blocks][slabs][M][128]
  int* counters;     // [row_blocks], zero between launches
  int* status;       // set non-zero when a bounded wait expired
  int M, N, K, group_shift;
  int64_t packed_row_stride, scale_row_stride;
  int row_blocks, slabs, units;
  float grid_min;
};


struct Barriers {          // shared-memory mbarriers
  uint64_t a_full[2];      // row threads -> issuer: A buffer written (128 arrivals)
  uint64_t d_full[2];      // issuers -> row threads: steps of the group complete (two tcgen05.commit)
  uint64_t d_empty[2];     // row threads -> issuer: accumulators read (128 arrivals)
  uint64_t unit_done[2];   // row threads -> publisher: partials of a unit stored (128 arrivals)
  uint64_t slot_free[2];   // publisher -> row threads: partial slot bookkeeping consumed (1 arrival)
};

__device__ __forceinline__ uint32_t smem_address(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void copy16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__device__ __forceinline__ void barrier_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(count));
}
__device__ __forceinline__ void barrier_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when it gave up (or another role did).
__device__ __forceinline__ bool barrier_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  uint32_t done = 0;
  for (uint32_t spins = 0; spins < kSpinLimit; ++spins) {
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(smem_address(bar)), "r"(parity) : "memory");
    if (done) return true;
    if ((spins & 1023) == 1023 && *failed) return false;
  }
  *failed = 1;
  return false;
}

// which code of a 32-code chunk faces K index kk (0..15) of the tensor-core step of class cls:
// register i = kk / 2 holds the mask pair of word i / 2; class 0 pairs are (0,4) and (2,6),
// class 1 pairs are (1,5) and (3,7)
__device__ __forceinline__ int chunk_code(int cls, int kk) {
  const int i = kk >> 1, h = kk & 1, w = i >> 1, second = i & 1;
  return 8 * w + cls + 2 * second + 4 * h;
}

__global__ void __launch_bounds__(kThreadsU) gemv_umma_kernel(const UmmaArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* tiles_s = smem;                                                  // [groups][4 chunks][2 classes][512 B]
  float* corr_s = reinterpret_cast<float*>(smem + kSlabGroups * 8 * kTileBytes);  // [groups][8]
  float* part_s = corr_s + kSlabGroups * 8;                                 // [groups][8][4 chunks]
  uint8_t* ring_s = reinterpret_cast<uint8_t*>(part_s + kSlabGroups * 32);  // [depth][128][pitch]
  __shared__ __align__(8) Barriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool row_thread = tid < kRowThreads;
  const int slab = int(blockIdx.x) % a.slabs;
  const int n_units = a.units > int(blockIdx.x) ? (a.units - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  const int total = n_units * kSlabGroups;  // groups (= ring stages) this CTA consumes
  volatile int* failed = &failed_s;

  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_address(&tmem_base_s)),
                 "r"(kTmemColumns));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  if (tid == 0) {
    failed_s = 0;
    for (int b = 0; b < 2; ++b) {
      barrier_init(&bars.a_full[b], kRowThreads);
      barrier_init(&bars.d_full[b], 2);  // one commit per issuer
      barrier_init(&bars.d_empty[b], kRowThreads);
      barrier_init(&bars.unit_done[b], kRowThreads);
      barrier_init(&bars.slot_free[b], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // ---- code stream (row threads): stage t = (unit t / 4, group t % 4); vector j * 128 + tid is 16 bytes of
  // row (j * 32 + tid / 4) at chunk tid % 4, so a warp instruction reads 8 rows x 64 B ----
  const uint32_t ring_base = smem_address(ring_s);
  const uint32_t ring_lane = ring_base + (tid >> 2) * kPitch + (tid & 3) * 16;
  const int64_t lane_column = int64_t(slab) * kSlabGroups * 64 + (tid & 3) * 16;
  int ld_stage = 0, ld_group = 0, ld_slot = 0, ld_unit = int(blockIdx.x);
  const uint8_t* ld_pointer[4] = {nullptr, nullptr, nullptr, nullptr};
  auto ld_rows = [&]() {
    const int row_block = ld_unit / a.slabs;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t global_row = min(row_block * 128 + j * 32 + (tid >> 2), a.N - 1);
      ld_pointer[j] = a.packed + global_row * a.packed_row_stride + lane_column;
    }
  };
  auto issue = [&]() {
    if (ld_stage < total) {
      const uint32_t slot = ring_lane + ld_slot * kStageBytes;
#pragma unroll
      for (int j = 0; j < 4; ++j) copy16(slot + j * 32 * kPitch, ld_pointer[j] + ld_group * 64);
      ++ld_stage;
      if (++ld_group == kSlabGroups) {
        ld_group = 0;
        ld_unit += int(gridDim.x);
        ld_rows();
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    ld_slot = ld_slot + 1 == kDepthU ? 0 : ld_slot + 1;
  };
  if (row_thread) {
    ld_rows();
#pragma unroll
    for (int d = 0; d < kDepthU - 1; ++d) issue();
  }

  // ---- activation tiles of this slab (B operand), and min * sum(x) * 2^-24 per group and row ----
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int i = tid; i < kSlabGroups * 8 * kTileBytes / 16; i += kThreadsU)
    reinterpret_cast<uint4*>(tiles_s)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  if (tid < a.M * kSlabGroups * 4) {
    const int chunk = tid & 3, group = (tid >> 2) % kSlabGroups, m = (tid >> 2) / kSlabGroups;
    const __half* source = a.x + int64_t(m) * a.K + (int64_t(slab) * kSlabGroups + group) * 128 + chunk * 32;
    __half values[32];
#pragma unroll
    for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(values + 8 * q) = __ldg(reinterpret_cast<const uint4*>(source) + q);
    float sum = 0.f;
#pragma unroll
    for (int q = 0; q < 32; ++q) sum += __half2float(values[q]);
    part_s[(group * 8 + m) * 4 + chunk] = sum;
#pragma unroll
    for (int cls = 0; cls < 2; ++cls) {
      uint8_t* tile = tiles_s + ((group * 4 + chunk) * 2 + cls) * kTileBytes;
#pragma unroll
      for (int kc = 0; kc < 2; ++kc) {
        __half out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = values[chunk_code(cls, kc * 8 + i)];
        *reinterpret_cast<uint4*>(tile + (kc * 16 + m) * 16) = *reinterpret_cast<uint4*>(out);
      }
    }
  }
  __syncthreads();
  if (tid < kSlabGroups * 8) {
    const float* p = part_s + tid * 4;
    const bool live = (tid & 7) < a.M;
    corr_s[tid] = live ? ((p[0] + p[1]) + (p[2] + p[3])) * a.grid_min * 5.9604644775390625e-08f : 0.f;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (row_thread) {
    // ================================ row threads ================================
    const uint32_t lane_base = uint32_t(warp * 32) << 16;
    float y_acc[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) y_acc[m] = 0.f;
    int group = 0, slot_index = 0, unit = int(blockIdx.x), local_unit = 0;
    int row_block = unit / a.slabs;
    const __half* scale_row = a.scales + int64_t(min(row_block * 128 + tid, a.N - 1)) * a.scale_row_stride;
    __half unit_scales[kSlabGroups];  // the four group scales of this row for the current unit, loaded at its start
    auto load_scales = [&]() {
#pragma unroll
      for (int gi = 0; gi < kSlabGroups; ++gi)
        unit_scales[gi] = __ldg(scale_row + (((slab * kSlabGroups + gi) * 128) >> a.group_shift));
    };
    load_scales();
    float previous_scale = 0.f;
    int previous_group = 0, previous_row_block = row_block;
    bool alive = true;

    // reads the accumulators of group t (buffer t & 1) and folds them into y_acc; ends the unit after its last group
    auto retire = [&](int t) {
      const int b = t & 1;
      if (!barrier_wait(&bars.d_full[b], uint32_t(t >> 1) & 1u, failed)) { alive = false; return; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t d0[8], d1[8];
      const uint32_t address = tmem_base + lane_base + 128 + b * 32;
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(d0[0]), "=r"(d0[1]), "=r"(d0[2]), "=r"(d0[3]), "=r"(d0[4]), "=r"(d0[5]), "=r"(d0[6]), "=r"(d0[7])
                   : "r"(address) : "memory");
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(d1[0]), "=r"(d1[1]), "=r"(d1[2]), "=r"(d1[3]), "=r"(d1[4]), "=r"(d1[5]), "=r"(d1[6]), "=r"(d1[7])
                   : "r"(address + 16) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      barrier_arrive(&bars.d_empty[b]);
      const float4 c_lo = *reinterpret_cast<const float4*>(corr_s + previous_group * 8);
      const float4 c_hi = *reinterpret_cast<const float4*>(corr_s + previous_group * 8 + 4);
      const float corr[8] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w, c_hi.x, c_hi.y, c_hi.z, c_hi.w};
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const float tile_sum = fmaf(__uint_as_float(d1[m]), 0.0625f, __uint_as_float(d0[m])) + corr[m];
        y_acc[m] = fmaf(previous_scale, tile_sum, y_acc[m]);
      }
      if (previous_group == kSlabGroups - 1) {
        // the partial slot of this parity is reused every second unit: wait until the publisher is done with it
        if (local_unit >= 2 && !barrier_wait(&bars.slot_free[local_unit & 1], uint32_t((local_unit >> 1) - 1) & 1u, failed)) {
          alive = false;
          return;
        }
        float* slot = a.partials + (int64_t(previous_row_block) * a.slabs + slab) * a.M * 128;
        for (int m = 0; m < a.M; ++m) slot[m * 128 + tid] = y_acc[m] * 16777216.f;  // 2^24: codes were c * 2^-24
#pragma unroll
        for (int m = 0; m < 8; ++m) y_acc[m] = 0.f;
        barrier_arrive(&bars.unit_done[local_unit & 1]);
        ++local_unit;
      }
    };

    for (int t = 0; t < total && alive; ++t) {
      asm volatile("cp.async.wait_group %0;" ::"n"(kDepthU - 2) : "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");  // every row thread's share of stage t has landed
      issue();                                         // refills the stage read one iteration ago
      const uint8_t* mine = ring_s + slot_index * kStageBytes + tid * kPitch;
      slot_index = slot_index + 1 == kDepthU ? 0 : slot_index + 1;
      uint4 chunk[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) chunk[c] = *reinterpret_cast<const uint4*>(mine + 16 * c);
      const uint32_t a_address = tmem_base + lane_base + (t & 1) * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t words[4] = {chunk[c].x, chunk[c].y, chunk[c].z, chunk[c].w};
        uint32_t r[16];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t q = words[w], q8 = q >> 8;
          r[2 * w] = q & 0x000f000fu;          // class 0: codes (0,4) then (2,6), c * 2^-24
          r[2 * w + 1] = q8 & 0x000f000fu;
          r[8 + 2 * w] = q & 0x00f000f0u;      // class 1: codes (1,5) then (3,7), c * 2^-20
          r[8 + 2 * w + 1] = q8 & 0x00f000f0u;
        }
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     :: "r"(a_address + 16 * c), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      barrier_arrive(&bars.a_full[t & 1]);
      if (t > 0) retire(t - 1);
      previous_scale = __half2float(group == 0 ? unit_scales[0] : group == 1 ? unit_scales[1]
                                    : group == 2 ? unit_scales[2] : unit_scales[3]);
      previous_group = group;
      previous_row_block = row_block;
      if (++group == kSlabGroups) {
        group = 0;
        unit += int(gridDim.x);
        row_block = unit / a.slabs;
        scale_row = a.scales + int64_t(min(row_block * 128 + tid, a.N - 1)) * a.scale_row_stride;
        if (t + 1 < total) load_scales();
      }
    }
    if (alive && total > 0) retire(total - 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == 4 || warp == 6) {
    // ================================ issuers: warp 4 takes the low-nibble steps, warp 6 the high-nibble steps =====
    if (lane == 0) {
      const int cls = warp == 4 ? 0 : 1;
      const uint32_t idesc = (1u << 4) | (2u << 17) | (8u << 24);  // fp32 accumulate, fp16 A/B, K-major, N = 16, M = 128
      // shared-memory descriptor: version 1, no swizzle, leading (next 8 K) 256 B, stride (next 8 rows) 128 B
      const uint64_t desc_base = (uint64_t(256 >> 4) << 16) | (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46) |
                                 uint64_t((smem_address(tiles_s) & 0x3FFFF) >> 4);
      int group = 0;
      for (int g = 0; g < total; ++g) {
        const int b = g & 1;
        if (!barrier_wait(&bars.a_full[b], uint32_t(g >> 1) & 1u, failed)) break;
        if (g >= 2 && !barrier_wait(&bars.d_empty[b], uint32_t((g >> 1) - 1) & 1u, failed)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t desc_group = desc_base + uint64_t(group * 8 * (kTileBytes >> 4));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint64_t desc = desc_group + uint64_t((c * 2 + cls) * (kTileBytes >> 4));
          const uint32_t d = tmem_base + 128 + b * 32 + cls * 16;
          const uint32_t a_columns = tmem_base + b * 64 + 16 * c + 8 * cls;
          if (c == 0)
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%4, %4, %4, %4}, p;\n\t}\n"
                         :: "r"(d), "r"(a_columns), "l"(desc), "r"(idesc), "r"(0u) : "memory");
          else
            asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
                         "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%4, %4, %4, %4}, p;\n\t}\n"
                         :: "r"(d), "r"(a_columns), "l"(desc), "r"(idesc), "r"(0u) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_address(&bars.d_full[b]))
                     : "memory");
        group = group + 1 == kSlabGroups ? 0 : group + 1;
      }
    }
  } else if (warp == 5) {
    // ================================ publisher ================================
    for (int i = 0; i < n_units; ++i) {
      int ok = 1;
      if (lane == 0) ok = barrier_wait(&bars.unit_done[i & 1], uint32_t(i >> 1) & 1u, failed) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int row_block = (int(blockIdx.x) + i * int(gridDim.x)) / a.slabs;
      int last = 0;
      if (lane == 0) {
        __threadfence();  // cumulative: publishes the partials whose stores the barrier ordered before this point
        last = atomicAdd(a.counters + row_block, 1) == a.slabs - 1;
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence();
        const float* first = a.partials + int64_t(row_block) * a.slabs * a.M * 128 + lane * 4;
        const int row = row_block * 128 + lane * 4;
        for (int m = 0; m < a.M; ++m) {
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s = 0; s < a.slabs; ++s) {
            const float4 part = __ldcg(reinterpret_cast<const float4*>(first + (int64_t(s) * a.M + m) * 128));
            sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
          }
          const float values[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (row + e < a.N) {
              float v = values[e];
              if (a.bias != nullptr) v += __half2float(a.bias[row + e]);
              a.y[int64_t(m) * a.N + row + e] = __float2half_rn(v);
            }
          }
        }
        if (lane == 0) a.counters[row_block] = 0;
      }
      __syncwarp();
      if (lane == 0) barrier_arrive(&bars.slot_free[i & 1]);
    }
  }

  if (tid == 0 && failed_s) atomicExch(a.status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && failed_s) atomicExch(a.status, 1);
  if (warp == 4)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns));
}

constexpr size_t kSmemU = size_t(kSlabGroups) * 8 * kTileBytes + kSlabGroups * 8 * 4 + kSlabGroups * 32 * 4 +
                          size_t(kDepthU) * kStageBytes;

}  // namespace

int gemv_umma_supported(int M, int K, int group, int bits, int x_dtype, int scale_dtype, const void* x,
                        const uint8_t* packed, int64_t packed_row_stride, const void* zeros, int integer_grid) {
  if (bits != 4 || !integer_grid || zeros != nullptr) return 0;
  if (x_dtype != MKB_F16 || scale_dtype != MKB_F16 || M < 1 || M > 8) return 0;
  if (K < 128 * kSlabGroups || K % (128 * kSlabGroups) != 0 || group % 128 != 0 || (group & (group - 1)) != 0) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(packed) % 16 || packed_row_stride % 16) return 0;
  return 1;
}

// Workspace layout: a fixed head of kCounterBytes (one counter per row block, then a status word),
// then the partials.  The head has the same place for every problem size, and every launch leaves
// its counters at zero, so one zero-filled buffer serves calls of different shapes in turn.
constexpr int64_t kCounterBytes = 65536;
constexpr int64_t kMaxRowBlocks = kCounterBytes / 4 - 1;

int64_t gemv_umma_workspace_bytes(int M, int N, int K) {
  const int64_t row_blocks = (N + 127) / 128, slabs = K / (128 * kSlabGroups);
  if (row_blocks > kMaxRowBlocks) return 0;
  return kCounterBytes + row_blocks * slabs * M * 128 * 4;
}

int launch_gemv_umma(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                     void* workspace, int M, int N, int K, int group, int64_t packed_row_stride,
                     int64_t scale_row_stride, float grid_minimum, cudaStream_t stream) {
  UmmaArgs a{};
  a.x = static_cast<const __half*>(x); a.packed = packed; a.scales = static_cast<const __half*>(scales);
  a.bias = static_cast<const __half*>(bias); a.y = static_cast<__half*>(y);
  a.M = M; a.N = N; a.K = K; a.packed_row_stride = packed_row_stride; a.scale_row_stride = scale_row_stride;
  a.group_shift = 0;
  while ((1 << a.group_shift) < group) ++a.group_shift;
  a.grid_min = grid_minimum;
  a.row_blocks = (N + 127) / 128;
  a.slabs = K / (128 * kSlabGroups);
  a.units = a.row_blocks * a.slabs;
  MKB_REQUIRE(a.row_blocks <= kMaxRowBlocks, MKB_E_UNSUPPORTED, "gemv_umma: %d row blocks exceed the counter area", a.row_blocks);
  a.counters = static_cast<int*>(workspace);
  a.status = a.counters + kMaxRowBlocks;
  a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kCounterBytes);

  const DeviceInfo& info = device_info();
  static bool configured[64];
  int device = 0;
  cudaGetDevice(&device);
  static int ctas_per_sm[64];
  if (device >= 0 && device < 64 && !configured[device]) {
    // opt in to the device maximum and the largest shared-memory carve-out, so that several CTAs fit one SM
    cudaError_t status = cudaFuncSetAttribute(gemv_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              info.max_smem_optin - 1024);  // the kernel also has static shared
    if (status != cudaSuccess) return cuda_fail(status, "gemv_umma: shared memory opt-in");
    status = cudaFuncSetAttribute(gemv_umma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared);
    if (status != cudaSuccess) return cuda_fail(status, "gemv_umma: shared memory carve-out");
    int blocks = 0;
    status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, gemv_umma_kernel, kThreadsU, kSmemU);
    if (status != cudaSuccess) return cuda_fail(status, "gemv_umma: occupancy query");
    MKB_REQUIRE(blocks >= 1, MKB_E_UNSUPPORTED, "gemv_umma: kernel does not fit one SM");
    // tensor memory has 512 columns per SM: at most four CTAs of this kernel share one; the kernel
    // is correct for any grid, so the grid is sized for that bound even where the query is more cautious
    (void)blocks;
    ctas_per_sm[device] = 512 / kTmemColumns;
    configured[device] = true;
  }
  int grid = info.sm_count * ctas_per_sm[device] / a.slabs * a.slabs;  // a multiple of the slab count
  if (grid < a.slabs) grid = a.slabs;
  if (grid > a.units) grid = a.units;

  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3(kThreadsU, 1, 1);
  config.dynamicSmemBytes = kSmemU;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t launched = cudaLaunchKernelEx(&config, gemv_umma_kernel, a);
  if (launched != cudaSuccess) return cuda_fail(launched, "gemv_umma launch");
  return MKB_OK;
}

}  // namespace mkb

// ---- the matvec for callers that cannot allocate ---------------------------------------------------
// Some hosts of this library have no way to hand over a workspace: a serving runtime that gave all
// of HBM to its KV cache at start-up, a plugin that is forbidden to call the CUDA allocator, code
// that runs while a stream is being captured (where cudaMalloc is an error).  For them the split-K
// scratch of the tensor-memory kernel lives in the library image itself.
namespace mkb {
namespace {

constexpr int64_t kStaticScratchBytes = int64_t(8) << 20;  // 8 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel may use comes from cudaGetSymbolAddress, asked once per device while that
// device is current.
int static_scratch_address(void** address) {
  static void* cached[64];
  int device = 0;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess) return cuda_fail(status, "gemv_static: cudaGetDevice");
  MKB_REQUIRE(device >= 0 && device < 64, MKB_E_UNSUPPORTED, "gemv_static: device ordinal %d out of range", device);
  if (cached[device] == nullptr) {
    void* pointer = nullptr;
    status = cudaGetSymbolAddress(&pointer, g_static_scratch);
    if (status != cudaSuccess) return cuda_fail(status, "gemv_static: cudaGetSymbolAddress");
    MKB_REQUIRE(pointer != nullptr, MKB_E_CUDA, "gemv_static: the scratch symbol has no device address");
    cached[device] = pointer;
  }
  *address = cached[device];
  return MKB_OK;
}

}  // namespace
}  // namespace mkb

extern "C" int64_t mkb_gemv_static_scratch_bytes(void) { return mkb::kStaticScratchBytes; }

extern "C" int mkb_gemv_static(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                               int M, int N, int K, int group, int64_t packed_row_stride, int64_t scale_row_stride,
                               float grid_minimum, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 1 && M <= 8 && N >= 1 && K >= 1 && group >= 1, MKB_E_ARGUMENT, "gemv_static: bad shape");
  MKB_REQUIRE(x && packed && scales && y, MKB_E_ARGUMENT, "gemv_static: null pointer");
  MKB_REQUIRE(grid_minimum == float(int(grid_minimum)) && grid_minimum >= -512.f && grid_minimum <= 512.f, MKB_E_ARGUMENT,
              "gemv_static: grid_minimum must be a small integer");
  MKB_REQUIRE(gemv_umma_supported(M, K, group, 4, MKB_F16, MKB_F16, x, packed, packed_row_stride, nullptr, 1),
              MKB_E_UNSUPPORTED,
              "gemv_static: needs K a multiple of 512, a power-of-two group of at least 128 and 16-byte aligned x and packed");
  const int64_t need = gemv_umma_workspace_bytes(M, N, K);
  MKB_REQUIRE(need > 0 && need <= kStaticScratchBytes, MKB_E_UNSUPPORTED,
              "gemv_static: M=%d N=%d K=%d needs %lld B of scratch, the built-in scratch holds %lld B", M, N, K,
              (long long)need, (long long)kStaticScratchBytes);
  void* scratch = nullptr;
  const int status = static_scratch_address(&scratch);
  if (status != MKB_OK) return status;
  // the array keeps what the previous call left: the row-block counters of this launch must start at
  // zero.  The status word is sticky (a wait that expired stays visible until mkb_gemv_static_status
  // reads and clears it), as the status of a caller's workspace is.
  const int64_t row_blocks = (N + 127) / 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const cudaError_t cleared = cudaMemsetAsync(scratch, 0, size_t(row_blocks) * 4, s);
  if (cleared != cudaSuccess) return cuda_fail(cleared, "gemv_static: clearing the counters");
  return launch_gemv_umma(x, packed, scales, bias, y, scratch, M, N, K, group, packed_row_stride, scale_row_stride,
                          grid_minimum, s);
}

extern "C" int mkb_gemv_static_status(int* status) {
  using namespace mkb;
  MKB_REQUIRE(status != nullptr, MKB_E_ARGUMENT, "gemv_static_status: null pointer");
  void* scratch = nullptr;
  const int looked_up = static_scratch_address(&scratch);
  if (looked_up != MKB_OK) return looked_up;
  // the status word follows the row-block counters; read it, then clear it for the calls to come
  uint8_t* word = static_cast<uint8_t*>(scratch) + kMaxRowBlocks * 4;
  int value = 0;
  cudaError_t done = cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost);
  if (done == cudaSuccess && value != 0) done = cudaMemset(word, 0, sizeof(value));
  if (done != cudaSuccess) return cuda_fail(done, "gemv_static_status");
  *status = value;
  return MKB_OK;
}
