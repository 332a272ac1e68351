// Register-tiled packed matvec for fp16 activations, M <= 8 (sm_100a).
//
// Work decomposition
//   * a row tile is 16 output rows; a k-tile is 128 consecutive codes (16*bits bytes per row);
//   * a persistent CTA of 8 warps owns row tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the
//     warps split the CTA's k-tiles into contiguous runs, so per row a warp streams one
//     contiguous byte range;
//   * with `splits` > 1 the CTAs of a thread-block cluster (1 x splits) split K between them and
//     meet once, at the end, through distributed shared memory (fixed summation order).
//
// Data path per warp and k-tile
//   * lane (g = lane / 4, t = lane % 4) owns 32 codes (4*bits bytes) of row g and of row g + 8.
//     They travel global -> shared with per-thread asynchronous copies (cp.async, L1 bypass) into a
//     private ring of DEPTH k-tiles per warp; the ring runs ahead across row-tile boundaries.
//     Completion is tracked by copy groups, not by register scoreboards, so DEPTH tiles really are
//     in flight;
//   * codes become fp16 tensor-core operands in registers.  Integer grids with group % 128 == 0
//     ("raw"): the masked bits of a code are used directly as an fp16 subnormal, c * 2^-24, or a
//     power of two more for codes that sit higher in their 16-bit lane; codes of equal lift share
//     tensor-core steps and an accumulator, and the accumulators are recombined with exact
//     power-of-two weights, so a pair of codes costs one AND and nothing is rounded; the grid
//     minimum enters as min * sum(x) per k-tile, precomputed, and the group scale multiplies the
//     fp32 k-tile sum.  Integer grids with small groups or offsets ("fold"): magic-number decode, scale
//     and offset folded into the fp16 weight.  Other codebooks ("table"): a bank-conflict-free
//     shared-memory table, fp32 multiply by the scale and one rounding, which reproduces the
//     reference's fp16 weight exactly;
//   * eight m16n8k16 tensor-core products per k-tile accumulate in fp32: the 16 weight rows are the
//     A operand, the (up to 8) activation rows the B operand.  Activations are staged once per CTA
//     in shared memory, permuted so that the B fragments of one lane are four 16-byte reads.
// Warp partials meet in shared memory once per row tile; 128 threads add them in warp order, add
// the bias and store fp16.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>

#include "mkb_common.cuh"

namespace cg = cooperative_groups;

namespace mkb {
namespace {

constexpr int kWarpsT = 8;
constexpr int kThreadsT = kWarpsT * 32;
constexpr int kMaxRowTilesPerCta = 64;  // bound on the cluster-split accumulator

enum { MODE_RAW = 0, MODE_FOLD = 1, MODE_TABLE = 2 };
enum { PERM_IDENTITY = 0, PERM_NIBBLE = 1, PERM_CRUMB = 2 };

struct TiledArgs {
  const __half* x;
  const uint8_t* packed;
  const __half* scales;
  const float* lut;
  const __half* zeros;
  const __half* bias;
  __half* y;
  int M, N, K, group, lut_len;
  int64_t packed_row_stride, scale_row_stride;
  int row_tiles, first_tile, k_tiles, k_tiles_cta, splits, mpad, group_shift;  // row tiles [first_tile, first_tile + row_tiles)
  float grid_min;
  int gated;  // x is [M, 2K] = gate | up: the staged activation is silu(gate) * up
};

// ---- asynchronous global -> shared copies (per thread; no register scoreboard involved) ----------
template <int BYTES>
__device__ __forceinline__ void copy_async(uint32_t smem_address, const void* global) {
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_address), "l"(global) : "memory");
  else if constexpr (BYTES == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_address), "l"(global) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_address), "l"(global) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// 32 codes of one row: BITS 32-bit words, moved in vectors of VEC bytes.
template <int BITS>
struct Chunk { uint32_t q[BITS]; };
template <int BITS>
struct ChunkGeometry {
  static constexpr int BYTES = 4 * BITS;
  static constexpr int VEC = BITS % 4 == 0 ? 16 : BITS % 2 == 0 ? 8 : 4;
  static constexpr int VECS = BYTES / VEC;
  static constexpr int SLOT_BYTES = 2 * VECS * 32 * VEC;  // two rows, one warp
};

// One ring slot of a warp is [row 0/1][vector][lane]: copies and reads of a warp touch 32
// consecutive vectors.  `lane_address` already includes lane * VEC.
template <int BITS>
__device__ __forceinline__ void chunk_copy_async(uint32_t lane_address, int row, const uint8_t* p) {
  using G = ChunkGeometry<BITS>;
#pragma unroll
  for (int v = 0; v < G::VECS; ++v)
    copy_async<G::VEC>(lane_address + (row * G::VECS + v) * 32 * G::VEC, p + v * G::VEC);
}

template <int BITS>
__device__ __forceinline__ void chunk_read(Chunk<BITS>& c, uint32_t lane_address, int row) {
  using G = ChunkGeometry<BITS>;
#pragma unroll
  for (int v = 0; v < G::VECS; ++v) {
    const uint32_t address = lane_address + (row * G::VECS + v) * 32 * G::VEC;
    if constexpr (G::VEC == 16) {
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(c.q[4 * v]), "=r"(c.q[4 * v + 1]), "=r"(c.q[4 * v + 2]), "=r"(c.q[4 * v + 3]) : "r"(address));
    } else if constexpr (G::VEC == 8) {
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(c.q[2 * v]), "=r"(c.q[2 * v + 1]) : "r"(address));
    } else {
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c.q[v]) : "r"(address));
    }
  }
}

// ---- the staged activation order -------------------------------------------------------------------
// A lane's 32 activations of a k-tile are kept as four 16-byte units; position p = 8*w + 2*j + h is
// unit w, register j, half h.  Register j of unit w is the B fragment {b0b1 | b2b3} of tensor-core
// step 2w (j = 0, 1) and step 2w+1 (j = 2, 3).  source_code(p) names the code of the lane's chunk
// whose weight the decode puts opposite that position.
template <int PERM>
__host__ __device__ constexpr int source_code(int p) {
  const int w = p >> 3, j = (p >> 1) & 3, h = p & 1;
  if (PERM == PERM_NIBBLE) {
    // 4-bit words of 8 codes: a mask pair is (c, c+4); registers 0,1 hold the pairs of the low
    // nibbles of each byte (codes 0,2), registers 2,3 those of the high nibbles (codes 1,3)
    return 8 * w + ((j & 1) * 2 + (j >> 1)) + 4 * h;
  }
  if (PERM == PERM_CRUMB) {
    // 2-bit words of 16 codes: a mask pair is (c, c+8); tensor-core step cl of a word takes the
    // pairs cl and cl+4, which sit at the same bit offset 2*cl of their bytes
    const int cl = 2 * (w & 1) + (j >> 1), r = j & 1;
    return 16 * (w >> 1) + cl + 4 * r + 8 * h;
  }
  return p;
}

template <int BITS, int MODE>
__host__ __device__ constexpr int perm_of() {
  return MODE == MODE_TABLE ? PERM_IDENTITY : BITS == 4 ? PERM_NIBBLE : BITS == 2 ? PERM_CRUMB : PERM_IDENTITY;
}

// Raw decode: tensor-core step s of a k-tile holds codes lifted by 2^(LIFT * (s % ACCS)) over
// c * 2^-24; steps of equal lift share accumulator s % ACCS.
template <int BITS>
struct RawClasses {
  static constexpr int ACCS = BITS == 2 ? 4 : 2;
  static constexpr int LIFT = BITS == 4 ? 4 : BITS == 2 ? 2 : 0;
};

// ---- code -> fp16 operand registers: h[4w + j] faces register j of activation unit w ---------------
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

template <int BITS>
__device__ __forceinline__ void decode_raw(const Chunk<BITS>& c, uint32_t (&h)[16]) {
  if constexpr (BITS == 4) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t q = c.q[w], q8 = q >> 8;
      h[4 * w + 0] = q & 0x000f000fu;   // codes 0,4      * 2^-24
      h[4 * w + 1] = q8 & 0x000f000fu;  // codes 2,6
      h[4 * w + 2] = q & 0x00f000f0u;   // codes 1,5      * 2^-20
      h[4 * w + 3] = q8 & 0x00f000f0u;  // codes 3,7
    }
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // word j: codes 4j..4j+3 -> tensor-core step j
      const int base = 4 * (j >> 1) + 2 * (j & 1);
      h[base + 0] = __byte_perm(c.q[j], 0u, 0x4140);  // {code0, 0, code1, 0}
      h[base + 1] = __byte_perm(c.q[j], 0u, 0x4342);
    }
  } else {  // BITS == 2
#pragma unroll
    for (int wd = 0; wd < 2; ++wd) {
      const uint32_t q = c.q[wd], q8 = q >> 8;
#pragma unroll
      for (int cl = 0; cl < 4; ++cl) {  // step cl of the word: pairs cl (codes cl, cl+8) and cl+4
        const int base = 4 * (2 * wd + (cl >> 1)) + 2 * (cl & 1);
        h[base + 0] = q & (0x00030003u << (2 * cl));
        h[base + 1] = q8 & (0x00030003u << (2 * cl));
      }
    }
  }
}

struct FoldConsts {
  __half2 sub1;        // 1024 - min
  __half2 mul4, add4;  // 1/4,  min - 256
  __half2 mul16, add16;
  __half2 mul64, add64;
};

__device__ __forceinline__ FoldConsts make_fold(float grid_min) {
  FoldConsts k;
  k.sub1 = __float2half2_rn(1024.f - grid_min);
  k.mul4 = __float2half2_rn(0.25f);      k.add4 = __float2half2_rn(grid_min - 256.f);
  k.mul16 = __float2half2_rn(0.0625f);   k.add16 = __float2half2_rn(grid_min - 64.f);
  k.mul64 = __float2half2_rn(0.015625f); k.add64 = __float2half2_rn(grid_min - 16.f);
  return k;
}

// lut[c] = min + c as exact fp16 values (magic number 1024 | c, then one subtract or one fma).
template <int BITS>
__device__ __forceinline__ void decode_fold(const Chunk<BITS>& c, const FoldConsts& k, uint32_t (&h)[16]) {
  constexpr uint32_t magic = 0x64006400u;  // half2(1024, 1024)
  if constexpr (BITS == 4) {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t q = c.q[w], q8 = q >> 8;
      h[4 * w + 0] = h2_bits(__hsub2(bits_h2((q & 0x000f000fu) | magic), k.sub1));
      h[4 * w + 1] = h2_bits(__hsub2(bits_h2((q8 & 0x000f000fu) | magic), k.sub1));
      h[4 * w + 2] = h2_bits(__hfma2(bits_h2((q & 0x00f000f0u) | magic), k.mul16, k.add16));
      h[4 * w + 3] = h2_bits(__hfma2(bits_h2((q8 & 0x00f000f0u) | magic), k.mul16, k.add16));
    }
  } else if constexpr (BITS == 8) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int base = 4 * (j >> 1) + 2 * (j & 1);
      h[base + 0] = h2_bits(__hsub2(bits_h2(__byte_perm(c.q[j], magic, 0x5150)), k.sub1));
      h[base + 1] = h2_bits(__hsub2(bits_h2(__byte_perm(c.q[j], magic, 0x5352)), k.sub1));
    }
  } else {  // BITS == 2
#pragma unroll
    for (int wd = 0; wd < 2; ++wd) {
      const uint32_t q = c.q[wd], q8 = q >> 8;
#pragma unroll
      for (int cl = 0; cl < 4; ++cl) {
        const int base = 4 * (2 * wd + (cl >> 1)) + 2 * (cl & 1);
        const uint32_t lo = (q & (0x00030003u << (2 * cl))) | magic, hi = (q8 & (0x00030003u << (2 * cl))) | magic;
        if (cl == 0) {
          h[base + 0] = h2_bits(__hsub2(bits_h2(lo), k.sub1));
          h[base + 1] = h2_bits(__hsub2(bits_h2(hi), k.sub1));
        } else {
          const __half2 mul = cl == 1 ? k.mul4 : cl == 2 ? k.mul16 : k.mul64;
          const __half2 add = cl == 1 ? k.add4 : cl == 2 ? k.add16 : k.add64;
          h[base + 0] = h2_bits(__hfma2(bits_h2(lo), mul, add));
          h[base + 1] = h2_bits(__hfma2(bits_h2(hi), mul, add));
        }
      }
    }
  }
}

// Any width through the shared table.  table_lane[c * 32] holds lut[c]; the weight is formed in
// fp32 (multiply, optional add) and rounded once, pairwise, to fp16.
template <int BITS, bool HAS_ZERO>
__device__ __forceinline__ void decode_table(const Chunk<BITS>& c, const float* table_lane, float scale,
                                             float zero, uint32_t (&h)[16]) {
  constexpr uint32_t mask = (1u << BITS) - 1u;
  float w[2];
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    const int bit = e * BITS, word = bit >> 5, shift = bit & 31;
    uint32_t code;
    if (shift + BITS <= 32) code = (c.q[word] >> shift) & mask;
    else code = __funnelshift_r(c.q[word], c.q[(word + 1) % BITS], shift) & mask;
    const float value = table_lane[code * 32];
    w[e & 1] = HAS_ZERO ? reconstruct(value, scale, zero) : reconstruct(value, scale);
    if (e & 1) h[e >> 1] = h2_bits(__floats2half2_rn(w[0], w[1]));
  }
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- the kernel ----------------------------------------------------------------------------------
template <int BITS, int MODE, bool HAS_ZERO, int DEPTH>
__global__ void __launch_bounds__(kThreadsT, MODE == MODE_TABLE ? 2 : 3) gemv_tiled_kernel(const TiledArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  using G = ChunkGeometry<BITS>;
  constexpr int PERM = perm_of<BITS, MODE>();
  constexpr int TILE_BYTES = 16 * BITS;  // 128 codes of one row
  constexpr bool RAW = MODE == MODE_RAW;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // K range of this CTA (cluster rank) and of this warp
  const int rank = a.splits > 1 ? int(blockIdx.y) : 0;
  const int kt0 = rank * a.k_tiles_cta;
  const int kt1 = min(a.k_tiles, kt0 + a.k_tiles_cta);
  const int nk_cta = max(0, kt1 - kt0);
  const int per_warp = (nk_cta + kWarpsT - 1) / kWarpsT;
  const int wk0 = min(kt1, kt0 + warp * per_warp);
  const int nk_w = max(0, min(kt1, wk0 + per_warp) - wk0);
  const int stride_rt = int(gridDim.x);
  const int n_rt = a.row_tiles > int(blockIdx.x) ? (a.row_tiles - 1 - int(blockIdx.x)) / stride_rt + 1 : 0;

  // shared memory carve-up
  uint4* x_s = reinterpret_cast<uint4*>(smem);                      // [k-tile][unit w][m][t] 16-byte units
  const int x_units = a.k_tiles_cta * 4 * a.mpad * 4;
  float* sum_s = reinterpret_cast<float*>(smem + size_t(x_units) * 16);           // [k-tile][8]: min*sum(x)*2^-24
  uint8_t* ring_s = reinterpret_cast<uint8_t*>(sum_s + a.k_tiles_cta * 8);        // [warps][DEPTH] slots
  float* red_s = reinterpret_cast<float*>(ring_s + kWarpsT * DEPTH * G::SLOT_BYTES);  // [2][warps][128]
  float* table_s = red_s + 2 * kWarpsT * 128;                                     // [2^BITS][32] (table decode)
  float* acc_s = table_s + (MODE == MODE_TABLE ? (32 << BITS) : 0);               // [n_rt][128] (cluster split)

  // ---- 1. first weight copies: they depend on nothing the previous kernel wrote ----
  const uint32_t ring_begin = uint32_t(__cvta_generic_to_shared(ring_s)) + warp * DEPTH * G::SLOT_BYTES + lane * G::VEC;
  const uint32_t ring_end = ring_begin + DEPTH * G::SLOT_BYTES;
  const int64_t lane_column = int64_t(wk0) * TILE_BYTES + t * G::BYTES;
  uint32_t ld_address = ring_begin;
  int ld_left = n_rt * nk_w, ld_k_left = nk_w, ld_rt = a.first_tile + int(blockIdx.x);
  const uint8_t *ld_p0, *ld_p1;
  auto ld_rows = [&]() {
    const int64_t r0 = min(ld_rt * 16 + g, a.N - 1), r1 = min(ld_rt * 16 + g + 8, a.N - 1);
    ld_p0 = a.packed + r0 * a.packed_row_stride + lane_column;
    ld_p1 = a.packed + r1 * a.packed_row_stride + lane_column;
  };
  ld_rows();
  auto issue = [&]() {
    if (ld_left > 0) {
      chunk_copy_async<BITS>(ld_address, 0, ld_p0);
      chunk_copy_async<BITS>(ld_address, 1, ld_p1);
      ld_p0 += TILE_BYTES;
      ld_p1 += TILE_BYTES;
      --ld_left;
      if (--ld_k_left == 0) {
        ld_k_left = nk_w;
        ld_rt += stride_rt;
        ld_rows();
      }
    }
    copy_commit();  // one group per ring slot, empty past the end, so the pending count stays exact
    ld_address += G::SLOT_BYTES;
    if (ld_address == ring_end) ld_address = ring_begin;
  };
#pragma unroll
  for (int d = 0; d < DEPTH - 1; ++d) issue();

  // ---- 2. stage activations (permuted) with their k-tile sums, and the decode table ----
  asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    const int chunks = a.M * nk_cta * 4;  // (m, local k-tile, quarter)
    const int rounded = (chunks + 31) & ~31;
    for (int c = threadIdx.x; c < rounded; c += kThreadsT) {
      const bool live = c < chunks;
      const int tt = c & 3, kl = live ? (c >> 2) % nk_cta : 0, m = live ? (c >> 2) / nk_cta : 0;
      const int64_t x_row = a.gated ? 2 * int64_t(a.K) : int64_t(a.K);
      const uint4* src = reinterpret_cast<const uint4*>(a.x + int64_t(m) * x_row + int64_t(kt0 + kl) * 128 + tt * 32);
      uint32_t xr[16];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 v = live ? __ldg(src + q) : make_uint4(0u, 0u, 0u, 0u);
        if (a.gated && live) {
          const uint4 up = __ldg(src + a.K / 8 + q);
          v = make_uint4(swiglu_pair(v.x, up.x), swiglu_pair(v.y, up.y), swiglu_pair(v.z, up.z), swiglu_pair(v.w, up.w));
        }
        xr[4 * q] = v.x; xr[4 * q + 1] = v.y; xr[4 * q + 2] = v.z; xr[4 * q + 3] = v.w;
      }
      if constexpr (RAW) {
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float2 pair = __half22float2(bits_h2(xr[q]));
          sum += pair.x;
          sum += pair.y;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (live && tt == 0) sum_s[kl * 8 + m] = sum * a.grid_min * 5.9604644775390625e-08f;  // 2^-24
      }
      if (live) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          uint32_t out[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int e0 = source_code<PERM>(8 * w + 2 * j), e1 = source_code<PERM>(8 * w + 2 * j + 1);
            const uint32_t lo = (e0 & 1) ? (xr[e0 >> 1] >> 16) : (xr[e0 >> 1] & 0xffffu);
            const uint32_t hi = (e1 & 1) ? (xr[e1 >> 1] & 0xffff0000u) : (xr[e1 >> 1] << 16);
            out[j] = lo | hi;
          }
          x_s[((kl * 4 + w) * a.mpad + m) * 4 + tt] = make_uint4(out[0], out[1], out[2], out[3]);
        }
      }
    }
    if constexpr (MODE == MODE_TABLE) {
      for (int q = threadIdx.x; q < (32 << BITS); q += kThreadsT) {
        const int code = q >> 5;
        table_s[q] = code < a.lut_len ? a.lut[code] : 0.f;
      }
    }
    if constexpr (RAW) {  // rows m >= M of the sums are read by idle accumulator lanes: keep them finite
      for (int q = threadIdx.x; q < nk_cta * 8; q += kThreadsT)
        if ((q & 7) >= a.M) sum_s[q] = 0.f;
    }
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const FoldConsts fold = make_fold(a.grid_min);
  const bool lane_has_x = g < a.M;
  // this lane's B fragments: unit w of local k-tile kl sits at x_lane + (kl * 4 + w) * x_step
  const uint4* x_lane = x_s + g * 4 + t;
  const int x_step = a.mpad * 4;
  const float* sum_lane = sum_s + 2 * t;  // activation rows 2t, 2t+1 of this lane's accumulators

  // ---- 3. main loop: row tiles of this CTA, k-tiles of this warp ----
  uint32_t cs_address = ring_begin;
  uint4 b[4];  // lanes without an activation row keep zeros here for the whole kernel
#pragma unroll
  for (int w = 0; w < 4; ++w) b[w] = make_uint4(0u, 0u, 0u, 0u);
  float y_even[4] = {0.f, 0.f, 0.f, 0.f}, y_odd[4] = {0.f, 0.f, 0.f, 0.f};
  for (int rt_local = 0; rt_local < n_rt; ++rt_local) {
    const int rt = a.first_tile + int(blockIdx.x) + rt_local * stride_rt;
    const int64_t r0 = min(rt * 16 + g, a.N - 1), r1 = min(rt * 16 + g + 8, a.N - 1);
    const __half* scale_row0 = a.scales + r0 * a.scale_row_stride;
    const __half* scale_row1 = a.scales + r1 * a.scale_row_stride;
    const __half* zero_row0 = HAS_ZERO ? a.zeros + r0 * a.scale_row_stride : nullptr;
    const __half* zero_row1 = HAS_ZERO ? a.zeros + r1 * a.scale_row_stride : nullptr;
    for (int kk = 0; kk < nk_w; ++kk) {
      const int kt = wk0 + kk;
      const int scale_column = (RAW ? kt * 128 : kt * 128 + t * 32) >> a.group_shift;
      const __half s0h = __ldg(scale_row0 + scale_column), s1h = __ldg(scale_row1 + scale_column);
      issue();                 // keeps DEPTH - 1 k-tiles in flight behind the one consumed now
      copy_wait<DEPTH - 1>();  // the oldest group, this k-tile, has landed
      Chunk<BITS> c0, c1;
      chunk_read<BITS>(c0, cs_address, 0);
      chunk_read<BITS>(c1, cs_address, 1);
      cs_address += G::SLOT_BYTES;
      if (cs_address == ring_end) cs_address = ring_begin;

      uint32_t h0[16], h1[16];
      if constexpr (MODE == MODE_RAW) {
        decode_raw<BITS>(c0, h0);
        decode_raw<BITS>(c1, h1);
      } else if constexpr (MODE == MODE_FOLD) {
        decode_fold<BITS>(c0, fold, h0);
        decode_fold<BITS>(c1, fold, h1);
        const __half2 s0 = __half2half2(s0h), s1 = __half2half2(s1h);
        if constexpr (HAS_ZERO) {
          const __half2 z0 = __half2half2(__ldg(zero_row0 + scale_column));
          const __half2 z1 = __half2half2(__ldg(zero_row1 + scale_column));
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            h0[q] = h2_bits(__hfma2(bits_h2(h0[q]), s0, z0));
            h1[q] = h2_bits(__hfma2(bits_h2(h1[q]), s1, z1));
          }
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            h0[q] = h2_bits(__hmul2(bits_h2(h0[q]), s0));
            h1[q] = h2_bits(__hmul2(bits_h2(h1[q]), s1));
          }
        }
      } else {
        const float z0 = HAS_ZERO ? __half2float(__ldg(zero_row0 + scale_column)) : 0.f;
        const float z1 = HAS_ZERO ? __half2float(__ldg(zero_row1 + scale_column)) : 0.f;
        decode_table<BITS, HAS_ZERO>(c0, table_s + lane, __half2float(s0h), z0, h0);
        decode_table<BITS, HAS_ZERO>(c1, table_s + lane, __half2float(s1h), z1, h1);
      }

      const int kl = kt - kt0;
      const uint4* x_tile = x_lane + kl * 4 * x_step;
      if constexpr (RAW) {
        // accumulator 0 starts at min * sum(x) * 2^-24; the group scale multiplies the k-tile sum
        using C = RawClasses<BITS>;
        const float2 bias2 = *reinterpret_cast<const float2*>(sum_lane + kl * 8);
        float acc[C::ACCS][4];
#pragma unroll
        for (int i = 0; i < C::ACCS; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[i][q] = i == 0 ? ((q & 1) ? bias2.y : bias2.x) : 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if (lane_has_x) b[w] = x_tile[w * x_step];
          mma16816(acc[(2 * w) % C::ACCS], h0[4 * w], h1[4 * w], h0[4 * w + 1], h1[4 * w + 1], b[w].x, b[w].y);
          mma16816(acc[(2 * w + 1) % C::ACCS], h0[4 * w + 2], h1[4 * w + 2], h0[4 * w + 3], h1[4 * w + 3], b[w].z, b[w].w);
        }
        const float s0 = __half2float(s0h), s1 = __half2float(s1h);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float tile_sum = acc[C::ACCS - 1][q];
#pragma unroll
          for (int i = C::ACCS - 2; i >= 0; --i)  // Horner in 2^-LIFT: exact scalings
            tile_sum = fmaf(tile_sum, 1.f / float(1 << C::LIFT), acc[i][q]);
          y_even[q] = fmaf(q < 2 ? s0 : s1, tile_sum, y_even[q]);
        }
      } else {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if (lane_has_x) b[w] = x_tile[w * x_step];
          mma16816(y_even, h0[4 * w], h1[4 * w], h0[4 * w + 1], h1[4 * w + 1], b[w].x, b[w].y);
          mma16816(y_odd, h0[4 * w + 2], h1[4 * w + 2], h0[4 * w + 3], h1[4 * w + 3], b[w].z, b[w].w);
        }
      }
    }
    // ---- warp partials -> shared memory, summed in warp order by 128 threads ----
    const float lift = RAW ? 16777216.f : 1.f;  // 2^24: raw codes were c * 2^-24
    float* mine = red_s + ((rt_local & 1) * kWarpsT + warp) * 128;
    mine[(2 * t) * 16 + g] = (y_even[0] + y_odd[0]) * lift;
    mine[(2 * t + 1) * 16 + g] = (y_even[1] + y_odd[1]) * lift;
    mine[(2 * t) * 16 + g + 8] = (y_even[2] + y_odd[2]) * lift;
    mine[(2 * t + 1) * 16 + g + 8] = (y_even[3] + y_odd[3]) * lift;
#pragma unroll
    for (int q = 0; q < 4; ++q) y_even[q] = y_odd[q] = 0.f;
    __syncthreads();
    if (threadIdx.x < 128) {
      const float* partial = red_s + (rt_local & 1) * kWarpsT * 128 + threadIdx.x;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarpsT; ++w) sum += partial[w * 128];
      if (a.splits > 1) {
        acc_s[rt_local * 128 + threadIdx.x] = sum;
      } else {
        const int m = threadIdx.x >> 4;
        const int row = rt * 16 + (threadIdx.x & 15);
        if (m < a.M && row < a.N) {
          if (a.bias != nullptr) sum += __half2float(a.bias[row]);
          a.y[int64_t(m) * a.N + row] = __float2half_rn(sum);
        }
      }
    }
  }

  // ---- 4. K split over the cluster: one exchange through distributed shared memory ----
  if (a.splits > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (threadIdx.x < 128) {
      for (int rt_local = rank; rt_local < n_rt; rt_local += a.splits) {
        float sum = 0.f;
        for (int peer = 0; peer < a.splits; ++peer)
          sum += cluster.map_shared_rank(acc_s, peer)[rt_local * 128 + threadIdx.x];
        const int m = threadIdx.x >> 4;
        const int row = (a.first_tile + int(blockIdx.x) + rt_local * stride_rt) * 16 + (threadIdx.x & 15);
        if (m < a.M && row < a.N) {
          if (a.bias != nullptr) sum += __half2float(a.bias[row]);
          a.y[int64_t(m) * a.N + row] = __float2half_rn(sum);
        }
      }
    }
    cluster.sync();
  }
}

// ---- host side -----------------------------------------------------------------------------------
template <typename Kernel>
int occupancy_for(Kernel kernel, size_t smem, int& ctas_per_sm) {
  static std::mutex lock;
  static std::map<std::tuple<const void*, size_t, int>, int> cache;
  int device = 0;
  cudaGetDevice(&device);
  const auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), smem, device);
  std::lock_guard<std::mutex> guard(lock);
  auto found = cache.find(key);
  if (found != cache.end()) { ctas_per_sm = found->second; return MKB_OK; }
  // opt in to the device maximum once: a later, smaller request must not lower the limit again
  cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            device_info().max_smem_optin);
  if (status != cudaSuccess) return cuda_fail(status, "gemv_tiled: shared memory opt-in");
  int blocks = 0;
  status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kThreadsT, smem);
  if (status != cudaSuccess) return cuda_fail(status, "gemv_tiled: occupancy query");
  MKB_REQUIRE(blocks >= 1, MKB_E_UNSUPPORTED, "gemv_tiled: kernel does not fit one SM with %zu B shared", smem);
  ctas_per_sm = blocks;
  cache[key] = blocks;
  return MKB_OK;
}

template <int BITS, int MODE, bool HAS_ZERO>
int launch_variant(TiledArgs a, cudaStream_t stream) {
  // ring depth: about 48 KB of weights in flight per CTA
  constexpr int DEPTH = BITS >= 7 ? 3 : BITS >= 5 ? 4 : BITS == 4 ? 6 : 8;
  auto kernel = gemv_tiled_kernel<BITS, MODE, HAS_ZERO, DEPTH>;
  const DeviceInfo& info = device_info();

  // K split: keep the staged activations of one CTA under ~64 KB and give small-N layers
  // enough CTAs; the split is a cluster dimension, so it stays in {1, 2, 4}.
  a.mpad = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : 8;
  a.row_tiles = (a.N + 15) / 16;
  a.k_tiles = a.K / 128;
  int splits = 1;
  while (splits < 4 && size_t(a.k_tiles + splits - 1) / splits * 256 * a.mpad > 65536) splits *= 2;
  while (splits < 4 && a.row_tiles * splits < info.sm_count && a.k_tiles / (splits * 2) >= kWarpsT) splits *= 2;
  a.splits = splits;
  a.k_tiles_cta = (a.k_tiles + splits - 1) / splits;

  const size_t x_bytes = size_t(a.k_tiles_cta) * (256 * a.mpad + 32);
  const size_t fixed = 2 * kWarpsT * 128 * 4 + (MODE == MODE_TABLE ? (size_t(32) << BITS) * 4 : 0) +
                       size_t(kWarpsT) * DEPTH * ChunkGeometry<BITS>::SLOT_BYTES;
  const size_t smem = x_bytes + fixed + (splits > 1 ? size_t(kMaxRowTilesPerCta) * 512 : 0);
  MKB_REQUIRE(smem <= size_t(info.max_smem_optin), MKB_E_UNSUPPORTED,
              "gemv_tiled: %zu B shared memory exceed the device limit", smem);
  int ctas_per_sm = 1;
  int status = occupancy_for(kernel, smem, ctas_per_sm);
  if (status != MKB_OK) return status;
  int columns = info.sm_count * ctas_per_sm / splits;
  if (columns < 1) columns = 1;
  // with a K split every CTA keeps one accumulator per row tile it owns: bound the tiles per launch
  const int total_tiles = a.row_tiles;
  const int tiles_per_launch = splits > 1 ? columns * kMaxRowTilesPerCta : total_tiles;
  for (int first = 0; first < total_tiles; first += tiles_per_launch) {
    a.first_tile = first;
    a.row_tiles = total_tiles - first < tiles_per_launch ? total_tiles - first : tiles_per_launch;
    const int grid_columns = columns > a.row_tiles ? a.row_tiles : columns;

    cudaLaunchConfig_t config{};
    config.gridDim = dim3(grid_columns, splits, 1);
    config.blockDim = dim3(kThreadsT, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    // Programmatic dependent launch: the kernel may become resident while its predecessor in the
    // stream drains.  It prefetches weights at once (constants) and executes griddepcontrol.wait
    // before it reads activations or writes anything.
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    if (splits > 1) {
      attribute[1].id = cudaLaunchAttributeClusterDimension;
      attribute[1].val.clusterDim.x = 1;
      attribute[1].val.clusterDim.y = splits;
      attribute[1].val.clusterDim.z = 1;
      config.numAttrs = 2;
    }
    cudaError_t launched = cudaLaunchKernelEx(&config, kernel, a);
    if (launched != cudaSuccess) return cuda_fail(launched, "gemv_tiled launch");
  }
  return MKB_OK;
}

template <int BITS>
int launch_integer(const TiledArgs& a, bool raw, bool has_zero, cudaStream_t stream) {
  if (raw) return launch_variant<BITS, MODE_RAW, false>(a, stream);
  if (has_zero) return launch_variant<BITS, MODE_FOLD, true>(a, stream);
  return launch_variant<BITS, MODE_FOLD, false>(a, stream);
}

template <int BITS>
int launch_table(const TiledArgs& a, bool has_zero, cudaStream_t stream) {
  if (has_zero) return launch_variant<BITS, MODE_TABLE, true>(a, stream);
  return launch_variant<BITS, MODE_TABLE, false>(a, stream);
}

}  // namespace

int gemv_tiled_supported(int M, int K, int group, int bits, int x_dtype, int scale_dtype,
                         const void* x, const uint8_t* packed, int64_t packed_row_stride) {
  if (x_dtype != MKB_F16 || scale_dtype != MKB_F16) return 0;
  if (M < 1 || M > 8 || bits < 1 || bits > 8) return 0;
  if (K % 128 != 0 || K < 128 || group % 32 != 0 || (group & (group - 1)) != 0) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(packed) % 16) return 0;
  if (packed_row_stride % 16) return 0;
  return 1;
}

// integer_grid != 0 promises lut[c] == grid_minimum + c exactly (an integer minimum): the codes are
// then expanded arithmetically instead of through the table.
int launch_gemv_tiled(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                      const void* zeros, const void* bias, void* y, int M, int N, int K, int group,
                      int bits, int lut_len, int64_t packed_row_stride, int64_t scale_row_stride,
                      int integer_grid, float grid_minimum, int gated, cudaStream_t stream) {
  TiledArgs a{};
  a.gated = gated;
  a.x = static_cast<const __half*>(x); a.packed = packed; a.scales = static_cast<const __half*>(scales);
  a.lut = lut; a.zeros = static_cast<const __half*>(zeros); a.bias = static_cast<const __half*>(bias);
  a.y = static_cast<__half*>(y);
  a.M = M; a.N = N; a.K = K; a.group = group; a.lut_len = lut_len;
  a.packed_row_stride = packed_row_stride; a.scale_row_stride = scale_row_stride;
  const bool has_zero = zeros != nullptr;
  const bool integer = integer_grid != 0 && (bits == 2 || bits == 4 || bits == 8) &&
                       grid_minimum == float(int(grid_minimum)) && grid_minimum >= -512.f && grid_minimum <= 512.f;
  a.grid_min = integer ? grid_minimum : 0.f;
  a.group_shift = 0;
  while ((1 << a.group_shift) < group) ++a.group_shift;
  const bool raw = integer && !has_zero && group % 128 == 0;
  if (integer) {
    switch (bits) {
      case 2: return launch_integer<2>(a, raw, has_zero, stream);
      case 4: return launch_integer<4>(a, raw, has_zero, stream);
      default: return launch_integer<8>(a, raw, has_zero, stream);
    }
  }
  switch (bits) {
    case 1: return launch_table<1>(a, has_zero, stream);
    case 2: return launch_table<2>(a, has_zero, stream);
    case 3: return launch_table<3>(a, has_zero, stream);
    case 4: return launch_table<4>(a, has_zero, stream);
    case 5: return launch_table<5>(a, has_zero, stream);
    case 6: return launch_table<6>(a, has_zero, stream);
    case 7: return launch_table<7>(a, has_zero, stream);
    default: return launch_table<8>(a, has_zero, stream);
  }
}

}  // namespace mkb
