// Fused dequantise + GEMM for packed INT4 weights on the 5th-generation tensor cores (tcgen05, sm_100a):
// y[M, N] = x[M, K] . W^T with 9 <= M <= 128 activation rows, fp16, groups of 128 codes.
//
// The reference leaves this range to its dense route: reconstruct the whole fp16 weight in global
// memory (N * K * 2 bytes written, then read again by a library GEMM).  Here the packed codes are read
// once (N * K / 2 bytes) and the reconstructed weights never leave the SM: a thread decodes the codes
// of one weight row, multiplies by the group scale -- (c - 8) * scale rounded once to fp16, the bits
// the reference's reconstruction holds -- and stores them to tensor memory (TMEM) as the A operand of
// tcgen05.mma.  Activations are the B operand in shared memory, accumulators live in TMEM in fp32.
//
// Work: a unit is 128 weight rows x one K slab; one CTA computes one unit.  Roles (512 threads):
//   * warps 0-7, "decoders": warp w owns rows 32 * (w % 4) .. + 31 and the 128-code blocks of parity w / 4,
//     so the two warp groups alternate and one decodes while the other's block is multiplied.  The 32 x
//     64 B code tile of a block arrives by cp.async in the warp's own shared-memory ring (five stages; the
//     rings are what keeps enough bytes in flight towards HBM, and only the warp itself reads its ring, so
//     the loop has no CTA-wide barrier); a thread reads the 64 bytes of its row, turns each byte into two
//     fp16 weights (PRMT + LOP3 + HFMA2 + HMUL2) in natural K order and stores the 64 columns of one of four
//     A buffers (tcgen05.st).  At the end of the unit the same threads read the accumulators (tcgen05.ld) and store y,
//     or a partial when K is split over slabs;
//   * warps 8-11, "loaders": warp w copies the [Mpad x 128] activation tiles of the blocks t = w (mod 4) into a
//     ring of four or eight stages in the canonical K-major core-matrix layout (cp.async, 16 B = 8 K of one row);
//   * warps 12-15, "issuers": one lane of issuer i waits for A and B of the blocks t = i (mod issuers), issues
//     their eight tcgen05.mma each (M128, N = Mpad, K16) into its own accumulator columns and commits them to
//     the mbarriers that free the A buffer and the B stage.  Issuing a step costs the thread about a hundred
//     cycles whatever N is, so two (Mpad > 64) or four issuers share the blocks.
// With K split over slabs the last CTA of a row block (atomic counter) adds the partials in slab order.
// All hand-offs are mbarriers; every wait is bounded: on expiry the CTA records a status word, stops
// issuing and drains.
#include "mkb_common.cuh"

namespace mkb {
namespace {

constexpr int kDecoders = 256;
constexpr int kLoaders = 128;
constexpr int kMaxIssuers = 4;
constexpr int kThreadsG = kDecoders + kLoaders + 32 * kMaxIssuers;   // warps 12..15 issue
constexpr int kWarpStage = 32 * 64;       // bytes of codes per block of 128 K and decoder warp: 32 rows x 64 B
constexpr int kCodeStages = 5;            // ring stages per decoder warp: 8 warps x 5 x 2 KB = 80 KB in flight per SM
constexpr int kCodeBytes = 8 * kCodeStages * kWarpStage;
constexpr int kABuffers = 4;              // A operand buffers in tensor memory, 64 columns each
constexpr int kMaxBStages = 8;            // activation tiles in shared memory: eight if they fit, else four
constexpr int kMaxUnitBlocks = 32;        // blocks of 128 K per unit: its scales sit in shared memory
constexpr int kScalePitch = kMaxUnitBlocks + 2;   // halves per row of the scale table (17 words: no bank conflicts)
constexpr int kTmemColumnsG = 512;        // A[4]: 0..255; D_i: 256 + i * Mpad, one per issuer
constexpr int kDColumn = kABuffers * 64;
constexpr int kMaxRowsG = 128;
constexpr uint32_t kSpinLimitG = 200000;   // tries of up to 20 us each: a few seconds

struct GemmArgs {
  const __half* x;
  const uint8_t* packed;
  const __half* scales;
  const __half* bias;
  __half* y;
  float* partials;   // [row_blocks][slabs][Mpad][128]
  int* counters;     // [row_blocks], zero between launches
  int* status;       // set non-zero when a bounded wait expired
  int M, Mpad, N, K;
  int64_t packed_row_stride, scale_row_stride;
  int row_blocks, slabs, slab_blocks, k_blocks, b_stage_bytes, b_stages, issuers;
};

struct GemmBarriers {
  uint64_t a_full[kABuffers];    // decoders -> issuer (128 arrivals: the four warps that own the block)
  uint64_t a_empty[kABuffers];   // issuer -> decoders (tcgen05.commit)
  uint64_t b_full[kMaxBStages];  // loaders -> issuer (32 arrivals: the warp that copied the tile)
  uint64_t b_empty[kMaxBStages]; // issuer -> loaders (tcgen05.commit)
  uint64_t d_full;               // issuer -> decoders: every step of the unit is complete
};

__device__ __forceinline__ uint32_t shared_address(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void async_copy16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false when it gave up (or another role did).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  uint32_t done = 0;
  for (uint32_t spins = 0; spins < kSpinLimitG; ++spins) {
    // the hint lets the hardware park the thread (up to that many nanoseconds, or until the phase completes)
    // instead of spinning through the issue slots the decoders need
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(shared_address(bar)), "r"(parity), "r"(20000u) : "memory");
    if (done) return true;
    if ((spins & 1023) == 1023 && *failed) return false;
  }
  *failed = 1;
  return false;
}
__device__ __forceinline__ void commit_to(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(shared_address(bar)) : "memory");
}

// codes 2j and 2j+1 of a packed word (byte j) as the fp16 pair ((c0 - 8) * s, (c1 - 8) * s): the byte is
// copied into both halves, one mask keeps c0 in the low half and 16 * c1 in the high half on top of
// the fp16 exponent of 1024, one fused multiply-add (exact) maps (1024 + c0, 1024 + 16 c1) to
// (c0 - 8, c1 - 8), one multiply applies the scale with the single rounding of the reconstruction.
template <int BYTE>
__device__ __forceinline__ uint32_t weight_pair(uint32_t word, __half2 scale) {
  constexpr uint32_t selector = BYTE == 0 ? 0x1010u : BYTE == 1 ? 0x2121u : BYTE == 2 ? 0x3232u : 0x0303u;
  const uint32_t both = __byte_perm(word, word, selector);
  uint32_t biased;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(biased) : "r"(both), "r"(0x00f0000fu), "r"(0x64006400u));   // (both & mask) | exponent
  const __half2 one_sixteenth = __halves2half2(__ushort_as_half(0x3c00), __ushort_as_half(0x2c00));  // (1, 1/16)
  const __half2 offset = __halves2half2(__ushort_as_half(0xe408), __ushort_as_half(0xd480));         // (-1032, -72)
  const __half2 centred = __hfma2(*reinterpret_cast<const __half2*>(&biased), one_sixteenth, offset);
  const __half2 weight = __hmul2(centred, scale);
  return *reinterpret_cast<const uint32_t*>(&weight);
}

__device__ __forceinline__ void store_columns16(uint32_t address, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               :: "r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                  "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

__global__ void __launch_bounds__(kThreadsG, 1) gemm_umma_kernel(const GemmArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* code_s = smem;                                               // [8 warps][stages][32 rows][64 B], 16-byte chunks swizzled
  uint8_t* b_s = code_s + kCodeBytes;             // [b_stages][16 chunks][Mpad + 1][16 B]
  __half* scale_s = reinterpret_cast<__half*>(b_s + size_t(a.b_stages) * a.b_stage_bytes);   // [128][kScalePitch]
  __shared__ __align__(8) GemmBarriers bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int failed_s, last_s;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_block = int(blockIdx.x) / a.slabs, slab = int(blockIdx.x) - row_block * a.slabs;
  const int first_block = slab * a.slab_blocks;
  const int blocks = min(a.slab_blocks, a.k_blocks - first_block);     // blocks of 128 K in this unit
  volatile int* failed = &failed_s;

  if (warp == 12) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(shared_address(&tmem_base_s)),
                 "r"(kTmemColumnsG));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  if (tid == 0) {
    failed_s = 0;
    last_s = 0;
    for (int b = 0; b < kABuffers; ++b) {
      mbar_init(&bars.a_full[b], kDecoders / 2);
      mbar_init(&bars.a_empty[b], 1);
    }
    for (int b = 0; b < kMaxBStages; ++b) {
      mbar_init(&bars.b_full[b], 32);
      mbar_init(&bars.b_empty[b], 1);
    }
    mbar_init(&bars.d_full, a.issuers);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }

  // ---- decoders: one code ring per warp.  Warp w decodes rows 32 * (w % 4) .. + 31 of the blocks of
  // parity w / 4, so a stage is 32 rows x 64 B; copy i of a stage is chunk i % 4 of row i / 4, and chunk c
  // of row r sits at chunk position c ^ ((r >> 1) & 3): a quarter warp reading one chunk of eight rows
  // meets every bank once.  Nothing but the warp itself reads its ring: no CTA-wide barrier per block.
  const int parity = (warp >> 2) & 1;
  const int own_blocks = tid < kDecoders ? (blocks + 1 - parity) >> 1 : 0;
  int issued = 0, issue_slot = 0;
  const uint8_t* code_source[4] = {nullptr, nullptr, nullptr, nullptr};
  uint32_t code_target[4] = {0u, 0u, 0u, 0u};
  auto issue_codes = [&]() {
    if (issued < own_blocks) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        async_copy16(code_target[j] + issue_slot * kWarpStage, code_source[j] + int64_t(2 * issued + parity) * 64);
      ++issued;
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    issue_slot = issue_slot + 1 == kCodeStages ? 0 : issue_slot + 1;
  };
  if (tid < kDecoders) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j, r = i >> 2, c = i & 3;
      const int64_t global_row = min(row_block * 128 + (warp & 3) * 32 + r, a.N - 1);
      code_source[j] = a.packed + global_row * a.packed_row_stride + int64_t(first_block) * 64 + c * 16;
      code_target[j] = shared_address(code_s) + warp * (kCodeStages * kWarpStage) + r * 64 + ((c ^ ((r >> 1) & 3)) << 4);
    }
#pragma unroll
    for (int d = 0; d < kCodeStages - 1; ++d) issue_codes();
  }
  // the scales of the unit: row r, block t at scale_s[r * pitch + t] (weights: no dependency on the previous grid)
  {
    // all of a thread's loads are issued before the first is stored: one memory latency, not one per scale
    constexpr int kLoads = 128 * kMaxUnitBlocks / kThreadsG;
    __half held[kLoads];
#pragma unroll
    for (int j = 0; j < kLoads; ++j) {
      const int i = tid + j * kThreadsG, r = i / blocks, t = i - r * blocks;
      const int64_t global_row = min(row_block * 128 + r, a.N - 1);
      held[j] = i < 128 * blocks ? __ldg(a.scales + global_row * a.scale_row_stride + first_block + t) : __half();
    }
#pragma unroll
    for (int j = 0; j < kLoads; ++j) {
      const int i = tid + j * kThreadsG, r = i / blocks, t = i - r * blocks;
      if (i < 128 * blocks) scale_s[r * kScalePitch + t] = held[j];
    }
  }
  // rows M..Mpad of the activation tiles are never copied: they read as zero
  for (int i = tid; i < a.b_stages * a.b_stage_bytes / 16; i += kThreadsG)
    reinterpret_cast<uint4*>(b_s)[i] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (tid < kDecoders) {
    // ================================ decoders ================================
    const int r = tid & 127, half_block = tid >> 7;
    const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
    const int swizzle = (lane >> 1) & 3;
    const uint8_t* my_codes = code_s + warp * (kCodeStages * kWarpStage) + lane * 64;
    const __half* my_scales = scale_s + r * kScalePitch;
    int slot = 0;
    bool alive = true;
    for (int j = 0; j < own_blocks && alive; ++j) {
      const int t = 2 * j + parity;                   // the block this warp decodes now
      asm volatile("cp.async.wait_group %0;" ::"n"(kCodeStages - 2) : "memory");
      __syncwarp();                                    // every lane's share of the stage has landed
      issue_codes();                                   // refills the stage read one iteration ago
      const uint8_t* stage = my_codes + slot * kWarpStage;
      slot = slot + 1 == kCodeStages ? 0 : slot + 1;
      uint4 chunk[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) chunk[c] = *reinterpret_cast<const uint4*>(stage + ((c ^ swizzle) << 4));
      const __half2 scale = __half2half2(my_scales[t]);
      // this A buffer was last read by the steps of block t - 4
      if (t >= kABuffers && !mbar_wait(&bars.a_empty[t & 3], uint32_t((t >> 2) - 1) & 1u, failed)) { alive = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_address = tmem_base + lane_base + (t & 3) * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t words[4] = {chunk[c].x, chunk[c].y, chunk[c].z, chunk[c].w};
        uint32_t weights[16];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          weights[4 * w] = weight_pair<0>(words[w], scale);
          weights[4 * w + 1] = weight_pair<1>(words[w], scale);
          weights[4 * w + 2] = weight_pair<2>(words[w], scale);
          weights[4 * w + 3] = weight_pair<3>(words[w], scale);
        }
        store_columns16(a_address + 16 * c, weights);
      }
      // publish at once: the steps of this block then run under the decode of the next two
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&bars.a_full[t & 3]);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- the unit's accumulators: thread (r, h) takes columns [h * Mpad / 2, (h + 1) * Mpad / 2) of row r ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (alive && blocks > 0 && mbar_wait(&bars.d_full, 0u, failed)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int n = row_block * 128 + r;
      const int half_columns = a.Mpad >> 1;
      const int live = min(a.issuers, blocks);      // accumulators that took part in this unit
      const float bias = (a.slabs == 1 && a.bias != nullptr && n < a.N) ? __half2float(a.bias[n]) : 0.f;
      float* slot_out = a.partials + (int64_t(row_block) * a.slabs + slab) * a.Mpad * 128;
      for (int c = 0; c < half_columns; c += 8) {
        const int m0 = half_block * half_columns + c;
        float d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = 0.f;
        for (int i = 0; i < live; ++i) {
          uint32_t part[8];
          asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                       : "=r"(part[0]), "=r"(part[1]), "=r"(part[2]), "=r"(part[3]), "=r"(part[4]), "=r"(part[5]), "=r"(part[6]), "=r"(part[7])
                       : "r"(tmem_base + lane_base + kDColumn + i * a.Mpad + m0) : "memory");
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] += __uint_as_float(part[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = m0 + j;
          if (a.slabs == 1) {
            if (m < a.M && n < a.N) a.y[int64_t(m) * a.N + n] = __float2half_rn(d[j] + bias);
          } else if (m < a.M) {
            slot_out[m * 128 + r] = d[j];
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (a.slabs > 1) {
      // publish the partial; the last unit of the row block adds all of them in slab order
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (tid == 0) {
        __threadfence();
        last_s = atomicAdd(a.counters + row_block, 1) == a.slabs - 1;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (last_s) {
        __threadfence();
        const float* first = a.partials + int64_t(row_block) * a.slabs * a.Mpad * 128;
        for (int i = tid; i < a.M * 128; i += kDecoders) {
          const int m = i >> 7, rr = i & 127, n = row_block * 128 + rr;
          float sum = 0.f;
          for (int s = 0; s < a.slabs; ++s) sum += __ldcg(first + (int64_t(s) * a.Mpad + m) * 128 + rr);
          if (n < a.N) {
            if (a.bias != nullptr) sum += __half2float(a.bias[n]);
            a.y[int64_t(m) * a.N + n] = __float2half_rn(sum);
          }
        }
        if (tid == 0) a.counters[row_block] = 0;
      }
    }
  } else if (warp < 12) {
    // ================================ loaders ================================
    // item i of a block is chunk i % 16 (8 K) of activation row i / 16: sixteen threads read 256 contiguous
    // bytes; chunk c of row m lands at (c * (Mpad + 1) + m) * 16, the odd pitch spreads the chunks over banks
    // loader warp w copies the tiles of the blocks t = w (mod 4): a block's round trip (wait for its
    // stage, issue, land, publish) is about a thousand cycles whatever its size, so four of them run side
    // by side.  Lane l copies chunk l % 16 (8 K) of rows l / 16, l / 16 + 2, ...: sixteen lanes read 256
    // contiguous bytes; chunk c of row m lands at (c * (Mpad + 1) + m) * 16, the odd pitch spreads the
    // chunks over the banks.
    const int me = warp - 8;
    const uint32_t b_base = shared_address(b_s);
    const __half* my_source = a.x + int64_t(lane >> 4) * a.K + int64_t(first_block) * 128 + (lane & 15) * 8;
    const uint32_t my_target = b_base + ((lane & 15) * (a.Mpad + 1) + (lane >> 4)) * 16;
    const int64_t row_step = int64_t(2) * a.K;
    const int own = blocks > me ? (blocks - me + 3) >> 2 : 0;
    const int lag = a.b_stages >= 8 ? 1 : 0;       // own tiles still in flight when one is published
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool alive = true;
    for (int j = 0; j < own + lag && alive; ++j) {
      if (j < own) {
        const int t = me + 4 * j, stage = t % a.b_stages, round = t / a.b_stages;
        if (round > 0 && !mbar_wait(&bars.b_empty[stage], uint32_t(round - 1) & 1u, failed)) { alive = false; break; }
        const __half* source = my_source + int64_t(t) * 128;
        uint32_t target = my_target + stage * a.b_stage_bytes;
#pragma unroll 4
        for (int m = lane >> 4; m < a.M; m += 2) {
          async_copy16(target, source);
          source += row_step;
          target += 32;
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      if (j >= lag) {
        if (lag) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&bars.b_full[(me + 4 * (j - lag)) % a.b_stages]);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (lane == 0 && warp - 12 < a.issuers) {
    // ================================ issuers ================================
    // issuer i takes the blocks t = i (mod issuers) and accumulates them in its own columns D_i: the cost
    // of a step is in issuing it, so the issuers work side by side; the decoders add the D_i at the end
    const int me = warp - 12;
    const uint32_t idesc = (1u << 4) | (uint32_t(a.Mpad >> 3) << 17) | (8u << 24);  // fp32 accumulate, fp16 A/B, K-major, N = Mpad, M = 128
    const uint32_t chunk_pitch = uint32_t(a.Mpad + 1) * 16;     // bytes from one 8-K chunk to the next
    // shared-memory descriptor: version 1, no swizzle, leading (next 8 K) chunk_pitch, stride (next 8 rows) 128 B
    const uint64_t desc_fixed = (uint64_t(chunk_pitch >> 4) << 16) | (uint64_t(128 >> 4) << 32) | (uint64_t(1) << 46);
    const uint32_t d_columns = tmem_base + kDColumn + me * a.Mpad;
    int stage = me % a.b_stages, round = me / a.b_stages;     // the tile ring: stage t % b_stages on its (t / b_stages)-th use
    bool sent = false;
    for (int t = me; t < blocks; t += a.issuers) {
      const int b = t & 3;
      if (!mbar_wait(&bars.a_full[b], uint32_t(t >> 2) & 1u, failed)) break;
      if (!mbar_wait(&bars.b_full[stage], uint32_t(round) & 1u, failed)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tile = shared_address(b_s) + stage * a.b_stage_bytes;
      uint64_t desc = desc_fixed | uint64_t((tile & 0x3FFFFu) >> 4);
      const uint64_t desc_step = uint64_t((2 * chunk_pitch) >> 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a_columns = tmem_base + b * 64 + 8 * j;
        const uint32_t accumulate = (t > me || j > 0) ? 1u : 0u;
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
                     :: "r"(d_columns), "r"(a_columns), "l"(desc), "r"(idesc), "r"(accumulate) : "memory");
        desc += desc_step;
      }
      commit_to(&bars.a_empty[b]);
      commit_to(&bars.b_empty[stage]);
      if (t + a.issuers >= blocks) {
        commit_to(&bars.d_full);
        sent = true;
      }
      stage += a.issuers;
      while (stage >= a.b_stages) { stage -= a.b_stages; ++round; }
    }
    if (!sent && me >= blocks) mbar_arrive(&bars.d_full);   // a unit with fewer blocks than issuers
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && failed_s) atomicExch(a.status, 1);
  if (warp == 12)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumnsG));
}

}  // namespace

// Workspace layout: a fixed head (one counter per row block, then a status word), then the partials.
// Every launch leaves its counters at zero, so one zero-filled buffer serves calls of different shapes.
constexpr int64_t kGemmHeadBytes = 65536;
constexpr int64_t kGemmMaxRowBlocks = kGemmHeadBytes / 4 - 1;

struct GemmPlan {
  int Mpad, row_blocks, k_blocks, slabs, slab_blocks, b_stage_bytes, b_stages;
  size_t smem;
};

static GemmPlan plan_gemm(int M, int N, int K, int sm_count, int max_smem) {
  GemmPlan p{};
  p.Mpad = (M + 15) & ~15;
  p.row_blocks = (N + 127) / 128;
  p.k_blocks = K / 128;
  // enough units for every SM, units of at most kMaxUnitBlocks blocks and at least four
  int slabs = sm_count / p.row_blocks;
  const int least = (p.k_blocks + kMaxUnitBlocks - 1) / kMaxUnitBlocks, most = p.k_blocks >= 4 ? p.k_blocks / 4 : 1;
  if (slabs > most) slabs = most;
  if (slabs < least) slabs = least;
  if (slabs < 1) slabs = 1;
  p.slab_blocks = (p.k_blocks + slabs - 1) / slabs;
  p.slabs = (p.k_blocks + p.slab_blocks - 1) / p.slab_blocks;   // no empty slab
  p.b_stage_bytes = 16 * (p.Mpad + 1) * 16;
  const int fixed = kCodeBytes + 128 * kScalePitch * 2 + 2048;   // 2 KB: static shared memory and slack
  // four loader warps fill the ring, warp w the blocks t = w (mod 4): with four or eight stages a stage has
  // one producer, which keeps every waiter within one phase of its mbarrier
  const int fit = (max_smem - fixed) / p.b_stage_bytes;
  p.b_stages = fit >= 8 ? 8 : fit >= 4 ? 4 : 0;
  p.smem = size_t(kCodeBytes) + size_t(p.b_stages) * p.b_stage_bytes + size_t(128) * kScalePitch * 2;
  return p;
}

int gemm_umma_supported(int M, int N, int K, int group, int bits, int lut_len, int x_dtype, int scale_dtype, const void* x,
                        const uint8_t* packed, int64_t packed_row_stride, const void* zeros, int integer_grid,
                        float grid_minimum) {
  if (bits != 4 || !integer_grid || zeros != nullptr || grid_minimum != -8.f || lut_len != 16) return 0;
  if (x_dtype != MKB_F16 || scale_dtype != MKB_F16 || M < 1 || M > kMaxRowsG || N < 1) return 0;
  if (K < 128 || K % 128 != 0 || group != 128) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(packed) % 16 || packed_row_stride % 16) return 0;
  if ((N + 127) / 128 > kGemmMaxRowBlocks) return 0;
  return 1;
}

int64_t gemm_umma_workspace_bytes(int M, int N, int K) {
  const GemmPlan p = plan_gemm(M, N, K, device_info().sm_count, device_info().max_smem_optin);
  return kGemmHeadBytes + (p.slabs > 1 ? int64_t(p.row_blocks) * p.slabs * p.Mpad * 128 * 4 : 0);
}

int launch_gemm_umma(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y, void* workspace,
                     int M, int N, int K, int64_t packed_row_stride, int64_t scale_row_stride, cudaStream_t stream) {
  const DeviceInfo& info = device_info();
  const GemmPlan p = plan_gemm(M, N, K, info.sm_count, info.max_smem_optin);
  GemmArgs a{};
  a.x = static_cast<const __half*>(x); a.packed = packed; a.scales = static_cast<const __half*>(scales);
  a.bias = static_cast<const __half*>(bias); a.y = static_cast<__half*>(y);
  a.M = M; a.Mpad = p.Mpad; a.N = N; a.K = K;
  a.packed_row_stride = packed_row_stride; a.scale_row_stride = scale_row_stride;
  a.row_blocks = p.row_blocks; a.slabs = p.slabs; a.slab_blocks = p.slab_blocks; a.k_blocks = p.k_blocks;
  a.b_stage_bytes = p.b_stage_bytes; a.b_stages = p.b_stages;
  a.issuers = p.Mpad <= 64 ? 4 : 2;     // issuers * Mpad accumulator columns beside the 256 of the A buffers
  MKB_REQUIRE(p.b_stages >= 4, MKB_E_UNSUPPORTED, "gemm: the activation tiles do not fit shared memory");
  a.counters = static_cast<int*>(workspace);
  a.status = a.counters + kGemmMaxRowBlocks;
  a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kGemmHeadBytes);
  MKB_REQUIRE(p.smem + 1024 <= size_t(info.max_smem_optin), MKB_E_UNSUPPORTED, "gemm: %zu B of shared memory do not fit", p.smem);
  static bool configured[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < 64 && !configured[device]) {
    const cudaError_t status = cudaFuncSetAttribute(gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                    info.max_smem_optin - 1024);   // the kernel also has static shared
    if (status != cudaSuccess) return cuda_fail(status, "gemm: shared memory opt-in");
    configured[device] = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(unsigned(p.row_blocks * p.slabs), 1, 1);
  config.blockDim = dim3(kThreadsG, 1, 1);
  config.dynamicSmemBytes = p.smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  const cudaError_t launched = cudaLaunchKernelEx(&config, gemm_umma_kernel, a);
  if (launched != cudaSuccess) return cuda_fail(launched, "gemm launch");
  return MKB_OK;
}

}  // namespace mkb

extern "C" int64_t mkb_gemm_workspace_bytes(int M, int N, int K) {
  if (M < 1 || M > mkb::kMaxRowsG || N < 1 || K < 128 || K % 128 != 0) return 0;
  return mkb::gemm_umma_workspace_bytes(M, N, K);
}

extern "C" int mkb_gemm(const void* x, const uint8_t* packed, const void* scales, const float* lut, const void* zeros,
                        const void* bias, void* y, int M, int N, int K, int group, int bits, int lut_len, int x_dtype,
                        int scale_dtype, int64_t packed_row_stride, int64_t scale_row_stride, int integer_grid,
                        float grid_minimum, void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace mkb;
  (void)lut;
  MKB_REQUIRE(M >= 1 && N >= 1 && K >= 1 && group >= 1, MKB_E_ARGUMENT, "gemm: bad shape");
  MKB_REQUIRE(x && packed && scales && y && workspace, MKB_E_ARGUMENT, "gemm: null pointer");
  MKB_REQUIRE(gemm_umma_supported(M, N, K, group, bits, lut_len, x_dtype, scale_dtype, x, packed, packed_row_stride, zeros,
                                  integer_grid, grid_minimum),
              MKB_E_UNSUPPORTED,
              "gemm: needs 1..%d fp16 rows, symmetric INT4 on the integer grid -8..7 with fp16 scales per 128 codes, "
              "K a multiple of 128 and 16-byte aligned x and packed", kMaxRowsG);
  MKB_REQUIRE(workspace_bytes >= gemm_umma_workspace_bytes(M, N, K), MKB_E_ARGUMENT,
              "gemm: workspace of %lld B, %lld needed", (long long)workspace_bytes, (long long)gemm_umma_workspace_bytes(M, N, K));
  return launch_gemm_umma(x, packed, scales, bias, y, workspace, M, N, K, packed_row_stride, scale_row_stride,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int mkb_gemm_status(const void* workspace, int* status) {
  using namespace mkb;
  MKB_REQUIRE(workspace != nullptr && status != nullptr, MKB_E_ARGUMENT, "gemm_status: null pointer");
  const cudaError_t done = cudaMemcpy(status, static_cast<const int*>(workspace) + kGemmMaxRowBlocks, sizeof(int),
                                      cudaMemcpyDeviceToHost);
  if (done != cudaSuccess) return cuda_fail(done, "gemm_status");
  return MKB_OK;
}
