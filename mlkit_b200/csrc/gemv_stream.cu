// Streaming packed matvec for integer grids with one scale per 128 codes (sm_100a), M <= 8, fp16.
//
// The kernel is written around two budgets.  At the HBM rate an SM has about 45 cycles per KB of
// packed weights, i.e. roughly 90 integer-pipe operations and 180 issue slots per 16-row x 128-code
// tile; and a launch streams for only a few microseconds, so whatever happens before the first
// tensor-core step or after the last one is paid in full.  Hence:
//
//   * one CTA of up to 16 warps per SM owns row tiles blockIdx.x, blockIdx.x + gridDim.x, ... ("visits").
//     A warp owns the SAME KT k-tiles of every row tile it visits, so its activation fragments, their
//     per-tile sums and all shared-memory offsets are loop invariants held in registers: nothing is
//     staged per CTA and no activation byte is read from shared memory in the loop;
//   * weights travel global -> shared by per-thread cp.async (L1 bypass) into a private ring of DV
//     visits per warp (up to ~190 KB per SM in flight, far more than bandwidth x latency needs), so
//     the ring fills before `griddepcontrol.wait` returns and while activations are fetched.  One copy
//     instruction of a warp covers whole 128-byte lines; the shared layout is chosen so that both
//     the copies and the 16-byte fragment reads are free of bank conflicts;
//   * codes become fp16 tensor-core operands with one AND per PAIR of codes: the masked bits of a
//     code are the fp16 subnormal c * 2^-24 (or c * 2^-20 for odd codes, which keep their own
//     accumulator, so nothing is rounded; the two are recombined with an exact power of two).  The
//     grid minimum enters as min * sum(x) per k-tile, preloaded as the accumulator's start value; the
//     group scale multiplies the fp32 k-tile sum;
//   * a visit's partial sums (one per warp) meet in shared memory; every R visits the CTA adds them in
//     warp order and stores fp16.  When K is split over the CTAs of a thread-block cluster (large K or
//     small N) the per-CTA sums meet once more, at the end, through distributed shared memory in a
//     fixed order.  Results do not depend on timing.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>
#include <utility>

#include "hadamard_steps.cuh"

namespace cg = cooperative_groups;

namespace mkb {
namespace {

constexpr int kMaxWarps = 16;
constexpr int kMaxClusterVisits = 128;  // bound on the per-CTA sums kept for the cluster exchange

struct StreamArgs {
  const __half* x;
  const uint8_t* packed;
  const __half* scales;
  const __half* bias;
  const float* lut;   // table codecs: the levels
  int lut_len;
  __half* y;
  int M, N, K;
  int64_t packed_row_stride, scale_row_stride;
  int row_tiles;    // ceil(N / 16)
  int k_warps;      // K / (128 * KT): warp-sized shares of K over all slabs
  int KW, RG;       // warps along K and row tiles per visit of one CTA (the CTA has KW * RG warps)
  int slabs;        // CTAs of a cluster along K (gridDim.y)
  int visits;       // visits of every CTA
  int batch;        // visits whose partial sums shared memory holds between two reductions (a multiple of R)
  int gated;        // x is [M, 2K] = gate | up of a SwiGLU MLP: the activation is silu(gate) * up, formed on load
  // rotation on load (K a power of two): the CTA transforms x * signs with the Walsh-Hadamard butterflies in
  // shared memory and its warps take their activations from there, rounded to fp16 as the transform's own
  // launch would store them
  const int8_t* rot_signs;
  int rot_log2;     // 0: no rotation
  uint32_t rot_offset;   // of the [M][K] fp32 buffer in shared memory
  float rot_scale;
  int early;        // visits copied before the dependency wait; the rest of the ring follows the activation loads
  int kw_inverse, rg_inverse;  // ceil(65536 / KW), ceil(65536 / RG): small quotients by multiply and shift
  float grid_min;
};

__device__ __forceinline__ void copy16(uint32_t smem_address, const void* global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_address), "l"(global) : "memory");
}
__device__ __forceinline__ void copy4(uint32_t smem_address, const void* global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_address), "l"(global) : "memory");
}
// base + index * step, as one multiply-add on the fp32/integer-multiply pipe
template <typename T>
__device__ __forceinline__ const T* offset_pointer(const T* base, uint32_t index, uint32_t step_bytes) {
  uint64_t out;
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(out) : "r"(index), "r"(step_bytes), "l"(reinterpret_cast<uint64_t>(base)));
  return reinterpret_cast<const T*>(out);
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// d = a * b + c on the tensor cores, 16 weight rows x 16 codes times 16 codes x 8 activation rows.
__device__ __forceinline__ void mma_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
__device__ __forceinline__ void mma_next(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// How codes become tensor-core operands.
//   RAW   integer grids (lut[c] = min + c) of 2 to 8 bits with one scale per 128 codes: masked bits
//         used as fp16 subnormals (see the head of this file); the scale multiplies the k-tile sum.
//   TABLE any table of at most 16 levels with 3- or 4-bit codes and one scale per 64 or 128 codes: a
//         pair of neighbouring codes indexes a shared-memory table of fp16 pairs (one copy per lane,
//         so the gather has no bank conflicts), the pair is multiplied by the fp16 scale of its row
//         group (one scale per k-tile: the scale multiplies the tile's sum instead), and the products
//         accumulate directly.  The table holds fp16(lut[c]): the matvec is
//         within the 2e-3 bound of reconstruct-then-matmul, not bit-equal to it (the dequantisation
//         kernel is the bit-exact route).
enum { MODE_RAW = 0, MODE_TABLE = 1 };

// Geometry of one visit of one warp: 16 rows x KT k-tiles of 128 codes.  GPT = scale groups per k-tile.
template <int BITS, int MODE, int GPT, int KT>
struct Visit {
  static constexpr int TILE_ROW_BYTES = 16 * BITS;               // 128 codes of one row
  static constexpr int TILE_BYTES = 16 * TILE_ROW_BYTES;         // 16 rows
  static constexpr int SEGMENT = KT * TILE_ROW_BYTES;            // contiguous bytes of one row per visit
  static constexpr int VECTORS_PER_ROW = SEGMENT / 16;           // 16-byte vectors per row segment
  static constexpr int VECTORS_PER_TILE_ROW = TILE_ROW_BYTES / 16;
  static constexpr int VECTORS = 16 * VECTORS_PER_ROW;           // per visit and warp
  static constexpr int COPIES = (VECTORS + 31) / 32;             // copy instructions per lane and visit
  // the scales of a visit follow its codes: 16 rows x SCALE_ROW_BYTES (at least one 4-byte copy)
  static constexpr int SCALE_ROW_BYTES = KT * GPT * 2 < 4 ? 4 : KT * GPT * 2;
  static constexpr int SCALE_OFFSET = KT * TILE_BYTES;
  static constexpr int SLOT_BYTES = KT * TILE_BYTES + 16 * SCALE_ROW_BYTES;
  [[maybe_unused]] static constexpr int CLASSES = MODE == MODE_RAW ? (BITS == 4 ? 2 : BITS == 2 ? 4 : BITS == 3 ? 8 : BITS == 8 ? 1 : 11 - BITS) : 1;
  [[maybe_unused]] static constexpr int TABLE_ENTRIES = MODE == MODE_TABLE ? (1 << (2 * BITS)) : 0;   // pairs of codes
  static_assert(SEGMENT % 16 == 0 && SLOT_BYTES % 16 == 0, "visit geometry");
  static_assert(MODE == MODE_TABLE ? (BITS == 3 || BITS == 4) : (BITS >= 2 && BITS <= 8), "codec");
};

__device__ __forceinline__ uint4 load_shared16(uint32_t address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
  return v;
}
__device__ __forceinline__ uint32_t load_shared4(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}
__device__ __forceinline__ uint2 load_shared8(uint32_t address) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(address));
  return v;
}
__device__ __forceinline__ uint32_t load_shared2(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}
__device__ __forceinline__ void copy8(uint32_t smem_address, const void* global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_address), "l"(global) : "memory");
}
__device__ __forceinline__ void store_shared16(uint32_t address, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(address), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Position of 16-byte vector `vector` of row `row` inside k-tile `tile` of a slot.  The layouts keep
// the copies (a warp writes whole 128-byte lines) and the fragment reads (a lane reads its 32 codes
// of rows g and g + 8) free of bank conflicts: 4-bit rows of odd k-tiles swap with their neighbour,
// 8-bit rows keep their vectors swapped in pairs on odd rows.
template <int BITS>
__host__ __device__ constexpr uint32_t tile_offset(int tile, int row, int vector) {
  if (BITS == 4) return uint32_t(tile) * 1024u + uint32_t(row ^ (tile & 1)) * 64u + uint32_t(vector) * 16u;
  if (BITS == 8) return uint32_t(tile) * 2048u + uint32_t(row) * 128u + uint32_t(vector ^ (row & 1)) * 16u;
  return uint32_t(tile) * (256u * BITS) + uint32_t(row) * (16u * BITS) + uint32_t(vector) * 16u;
}

// Integer grids of 5, 6 or 7 bits.  A lane's 32 codes of a row are 4 B bytes whose halves (16 codes, 2 B
// bytes) repeat each other's bit positions, so a register that pairs bytes (i, i + 1) of the first half
// with the same bytes of the second holds code c and code c + 16 at one offset of its two 16-bit lanes.
// Code c starts at bit (B c) % 8 of byte (B c) / 8; where that leaves it reaching past the ten mantissa
// bits of an fp16 the register is moved down four bits first.  What remains is the lift 2^offset of the
// subnormal the mask cuts out: codes of equal offset share an accumulator.
template <int B>
struct Spread {
  __host__ __device__ static constexpr int window(int c) { return (B * c) / 8; }
  __host__ __device__ static constexpr int shift(int c) { return (B * c) % 8 + B <= 10 ? 0 : 4; }
  __host__ __device__ static constexpr int offset(int c) { return (B * c) % 8 - shift(c); }
  static constexpr int LIFTS = 11 - B;   // offsets 0 .. 10 - B
  // the codes in the order the tensor-core steps take them: by offset, two per step
  __host__ __device__ static constexpr int code_of(int step, int which) {
    int n = 0;
    for (int o = 0; o < LIFTS; ++o)
      for (int c = 0; c < 16; ++c)
        if (offset(c) == o) {
          if (n == 2 * step + which) return c;
          ++n;
        }
    return -1;
  }
  __host__ __device__ static constexpr bool opens_class(int step) { return step == 0 || offset(code_of(step, 0)) != offset(code_of(step - 1, 0)); }
  __host__ __device__ static constexpr bool used(int o) {
    for (int c = 0; c < 16; ++c)
      if (offset(c) == o) return true;
    return false;
  }
  __host__ __device__ static constexpr bool paired() {
    for (int step = 0; step < 8; ++step)
      if (offset(code_of(step, 0)) != offset(code_of(step, 1))) return false;
    return true;
  }
};

// the register and the byte positions in it that hold bytes (I, I + 1) of a lane's 4 B bytes
template <int B, int I>
__device__ __forceinline__ uint32_t piece_register(const uint32_t (&w)[B]) {
  if constexpr (I % 4 == 3 && I / 4 + 1 < B) return __funnelshift_r(w[I / 4], w[I / 4 + 1], 16);
  else return w[I / 4];
}
template <int B>
__host__ __device__ constexpr uint32_t piece_bytes(int I) {   // two selector digits: where byte I and byte I + 1 sit
  if (I % 4 == 3 && I / 4 + 1 < B) return 0x21u;
  if (I % 4 == 3) return 0x33u;           // the last byte of all: its neighbour does not exist and is not needed
  return uint32_t(I % 4) | uint32_t(I % 4 + 1) << 4;
}
template <int B, int I>
__device__ __forceinline__ uint32_t paired_window(const uint32_t (&w)[B]) {
  constexpr uint32_t selector = piece_bytes<B>(I) | (piece_bytes<B>(I + 2 * B) + 0x44u) << 8;
  return __byte_perm(piece_register<B, I>(w), piece_register<B, I + 2 * B>(w), selector);
}

template <int... I, typename F>
__device__ __forceinline__ void static_for_each(std::integer_sequence<int, I...>, F&& f) {
  (f(std::integral_constant<int, I>{}), ...);
}
template <int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_each(std::make_integer_sequence<int, N>{}, f);
}

// ROTATE: the instance that transforms its activations on load; the plain instance carries none of that code
// (with the rotation a run-time branch of one kernel the plain matvec measured 4-7 % slower)
template <int BITS, int MODE, int GPT, int KT, int R, bool ROTATE>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) gemv_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  using V = Visit<BITS, MODE, GPT, KT>;
  constexpr bool RAW = MODE == MODE_RAW;
  // dependents may become resident at once: they only copy constants until their own wait returns
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rg = (warp * a.kw_inverse) >> 16, kw = warp - rg * a.KW;   // warp / KW, warp % KW
  const int slab = int(blockIdx.y);
  const int k_warp = slab * a.KW + kw;           // this warp's share of K
  const int tile0 = k_warp * KT;                 // first k-tile
  const int visit_stride = int(gridDim.x) * a.RG;
  const int first_row_tile = int(blockIdx.x) * a.RG + rg;
  // visits in which this warp has a row tile: all of the CTA's, or all but the last; a warp past the
  // end of K has none.  The last row tile of a layer may be partial: the visits before `whole_visits`
  // have all 16 rows.
  int my_visits = a.visits - (first_row_tile + (a.visits - 1) * visit_stride >= a.row_tiles ? 1 : 0);
  if (k_warp >= a.k_warps) my_visits = 0;
  const int whole_visits = (a.N & 15) ? my_visits - 1 : my_visits;

  // shared memory: rings [warp][R][slot], partial sums [warp][batch][128], cluster sums [visit][RG][128],
  // then the pair table [entry][lane] of the table codecs
  const uint32_t smem_base = uint32_t(__cvta_generic_to_shared(smem));
  const uint32_t ring_base = smem_base + warp * R * V::SLOT_BYTES;
  float* red_s = reinterpret_cast<float*>(smem + size_t(warps) * R * V::SLOT_BYTES);
  const uint32_t red_base = smem_base + warps * R * V::SLOT_BYTES;
  float* acc_s = red_s + size_t(warps) * a.batch * 128;
  const uint32_t table_base = red_base + (warps * a.batch + (a.slabs > 1 ? a.visits * a.RG : 0)) * 512;

  // ---- copy side: vector v = i * 32 + lane of the visit's 16 x SEGMENT bytes -> (row, column) ----
  // one 64-bit source per copy of a lane; a visit adds visit * step with one multiply-add (no carries
  // to propagate on the integer pipe, which the code expansion needs for itself)
  const uint8_t* copy_base[V::COPIES];
  uint32_t copy_to[V::COPIES];
  uint32_t copy_rows = 0;   // row of copy i in bits [4i, 4i + 4)
#pragma unroll
  for (int i = 0; i < V::COPIES; ++i) {
    const int vector = i * 32 + lane, row = vector / V::VECTORS_PER_ROW, column = vector % V::VECTORS_PER_ROW;
    copy_base[i] = a.packed + int64_t(first_row_tile * 16 + row) * a.packed_row_stride +
                   int64_t(tile0) * V::TILE_ROW_BYTES + column * 16;
    copy_to[i] = ring_base + tile_offset<BITS>(column / V::VECTORS_PER_TILE_ROW, row, column % V::VECTORS_PER_TILE_ROW);
    copy_rows |= uint32_t(row) << (4 * i);
  }
  const uint32_t copy_visit_step = uint32_t(visit_stride) * 16u * uint32_t(a.packed_row_stride);
  // the scales of a visit ride in its slot: lane r < 16 copies the SCALE_ROW_BYTES that hold row r's
  // scales of the visit (for a single scale the aligned pair around it), so they arrive with the weights
  constexpr int SCALES = KT * GPT;   // scales per row and visit
  const int64_t scale_index = int64_t(first_row_tile * 16 + (lane & 15)) * a.scale_row_stride + int64_t(tile0) * GPT;
  const __half* scale_base = a.scales + (SCALES == 1 ? scale_index & ~int64_t(1) : scale_index);
  const uint32_t scale_visit_step = uint32_t(visit_stride) * 32u * uint32_t(a.scale_row_stride);  // bytes
  const uint32_t scale_to = ring_base + V::SCALE_OFFSET + (lane & 15) * V::SCALE_ROW_BYTES;
  const bool copies_scales = lane < 16;
  // `exists`: the warp owns this visit.  `whole` == false: rows past N are left out (their slots keep
  // stale bytes; the sums of such rows are never stored).
  auto issue = [&](int visit, int slot, bool exists, bool whole) {
    if (exists) {
      const int first_row = whole ? 0 : (first_row_tile + visit * visit_stride) * 16;
#pragma unroll
      for (int i = 0; i < V::COPIES; ++i)
        if ((V::VECTORS % 32 == 0 || i * 32 + lane < V::VECTORS) &&
            (whole || first_row + int((copy_rows >> (4 * i)) & 15u) < a.N))
          copy16(copy_to[i] + slot * V::SLOT_BYTES, offset_pointer(copy_base[i], uint32_t(visit), copy_visit_step));
      if (copies_scales && (whole || first_row + (lane & 15) < a.N)) {
        const __half* from = offset_pointer(scale_base, uint32_t(visit), scale_visit_step);
        if constexpr (V::SCALE_ROW_BYTES == 4) copy4(scale_to + slot * V::SLOT_BYTES, from);
        else if constexpr (V::SCALE_ROW_BYTES == 8) copy8(scale_to + slot * V::SLOT_BYTES, from);
        else copy16(scale_to + slot * V::SLOT_BYTES, from);
      }
    }
    copy_commit();  // one group per visit, empty past the end, so the pending count stays exact
  };
#pragma unroll
  for (int d = 0; d < R - 1; ++d)
    if (d < a.early) issue(d, d, d < my_visits, d < whole_visits);

  // ---- the pair table of the table codecs: entry (lo | hi << BITS) = fp16 (lut[lo], lut[hi]) ----
  if constexpr (!RAW) {
    __half2* table = reinterpret_cast<__half2*>(smem + (table_base - smem_base));
    for (int index = threadIdx.x; index < V::TABLE_ENTRIES * 32; index += blockDim.x) {
      const int entry = index >> 5, lo = entry & ((1 << BITS) - 1), hi = entry >> BITS;
      table[index] = __floats2half2_rn(lo < a.lut_len ? a.lut[lo] : 0.f, hi < a.lut_len ? a.lut[hi] : 0.f);
    }
    __syncthreads();
  }

  // ---- activations: the B fragments of this warp's k-tiles, permuted in registers ----
  asm volatile("griddepcontrol.wait;" ::: "memory");
  [[maybe_unused]] float* rotated = reinterpret_cast<float*>(smem + a.rot_offset);   // [M][K] when the rotation is on
  if constexpr (ROTATE) {
    // nine stages per 512 values in a warp's registers, the rest in shared memory, three stages per pass
    const int front = a.rot_log2 < kWarpBits ? a.rot_log2 : kWarpBits;
    const int chunks_per_row = a.K / kWarpSpan;
    // a warp takes chunks warp, warp + warps, ...: two at a time, so both chunks' loads are in flight together
    const int chunks = a.M * chunks_per_row;
    for (int chunk0 = warp; chunk0 < chunks; chunk0 += 2 * warps) {
      uint4 raw[2][2];
      int row[2], first[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int chunk = chunk0 + c * warps;
        row[c] = chunk / chunks_per_row;
        first[c] = (chunk - row[c] * chunks_per_row) * kWarpSpan + lane * kWarpRun;
        if (chunk < chunks) {
          const uint4* source = reinterpret_cast<const uint4*>(a.x + int64_t(row[c]) * a.K + first[c]);
          raw[c][0] = __ldg(source);
          raw[c][1] = __ldg(source + 1);
        }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (chunk0 + c * warps >= chunks) break;
        float values[kWarpRun];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t words[4] = {raw[c][q].x, raw[c][q].y, raw[c][q].z, raw[c][q].w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&words[w]));
            values[8 * q + 2 * w] = pair.x;
            values[8 * q + 2 * w + 1] = pair.y;
          }
        }
        if (a.rot_signs != nullptr) {
          const uint4 flips = *reinterpret_cast<const uint4*>(a.rot_signs + first[c]);
          const uint32_t words[4] = {flips.x, flips.y, flips.z, flips.w};
#pragma unroll
          for (int j = 0; j < kWarpRun; ++j)   // the sign byte's top bit flips the value's sign: the product with +-1
            values[j] = __uint_as_float(__float_as_uint(values[j]) ^ ((words[j >> 2] << (24 - 8 * (j & 3))) & 0x80000000u));
        }
        warp_butterflies16(values, lane, front);
        if (a.rot_log2 <= kWarpBits) {
#pragma unroll
          for (int j = 0; j < kWarpRun; ++j) values[j] = __fmul_rn(values[j], a.rot_scale);
        }
        float4* target = reinterpret_cast<float4*>(rotated + row[c] * a.K + first[c]);
#pragma unroll
        for (int q = 0; q < 4; ++q) target[q] = make_float4(values[4 * q], values[4 * q + 1], values[4 * q + 2], values[4 * q + 3]);
      }
    }
    __syncthreads();
    remaining_passes(rotated, a.M * a.K, a.rot_log2, kWarpBits, a.rot_scale);
  }
  uint32_t b[KT][16];     // tensor-core step s of a k-tile multiplies by b[2s], b[2s + 1]
  float start[KT][4];     // RAW: accumulator start, min * sum(x) * 2^-24 for activation rows 2t, 2t+1 (twice)
  {
    const __half* x_lane = a.x + int64_t(g) * (a.gated ? 2 * a.K : a.K) + int64_t(tile0) * 128 + t * 32;
    const bool has_x = my_visits > 0 && g < a.M;
    uint4 v[KT][4];
#pragma unroll
    for (int kk = 0; kk < KT; ++kk)
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        v[kk][w] = make_uint4(0u, 0u, 0u, 0u);
        if (ROTATE && has_x) {
          const float* from = rotated + g * a.K + tile0 * 128 + t * 32 + kk * 128 + w * 8;
          const float4 lo = *reinterpret_cast<const float4*>(from), hi = *reinterpret_cast<const float4*>(from + 4);
          const __half2 h0 = __floats2half2_rn(lo.x, lo.y), h1 = __floats2half2_rn(lo.z, lo.w);
          const __half2 h2 = __floats2half2_rn(hi.x, hi.y), h3 = __floats2half2_rn(hi.z, hi.w);
          v[kk][w] = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                                *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
        } else if (has_x) {
          v[kk][w] = __ldg(reinterpret_cast<const uint4*>(x_lane + kk * 128 + w * 8));
        }
      }
    if (a.gated && has_x) {  // the up half sits K elements further in the same row; lanes without a row keep their
                             // zeros (and stay off the slow path a division of zero would take)
#pragma unroll
      for (int kk = 0; kk < KT; ++kk)
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          uint4 up = make_uint4(0u, 0u, 0u, 0u);
          if (has_x) up = __ldg(reinterpret_cast<const uint4*>(x_lane + a.K + kk * 128 + w * 8));
          v[kk][w] = make_uint4(swiglu_pair(v[kk][w].x, up.x), swiglu_pair(v[kk][w].y, up.y),
                                swiglu_pair(v[kk][w].z, up.z), swiglu_pair(v[kk][w].w, up.w));
        }
    }
    // the rest of the ring is requested behind the activations, so these are not queued behind it
#pragma unroll
    for (int d = 0; d < R - 1; ++d)
      if (d >= a.early) issue(d, d, d < my_visits, d < whole_visits);
    const float unit = a.grid_min * 5.9604644775390625e-08f;   // min * 2^-24: the unit of the accumulators
#pragma unroll
    for (int kk = 0; kk < KT; ++kk) {
      const uint32_t r[16] = {v[kk][0].x, v[kk][0].y, v[kk][0].z, v[kk][0].w, v[kk][1].x, v[kk][1].y, v[kk][1].z, v[kk][1].w,
                              v[kk][2].x, v[kk][2].y, v[kk][2].z, v[kk][2].w, v[kk][3].x, v[kk][3].y, v[kk][3].z, v[kk][3].w};
      if constexpr (RAW && BITS == 4) {
        // a mask keeps codes (c, c + 4) of a word of 8: pairs (x0,x4) (x2,x6) for the even codes, (x1,x5) (x3,x7) for the odd
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          b[kk][4 * w + 0] = __byte_perm(r[4 * w], r[4 * w + 2], 0x5410);
          b[kk][4 * w + 1] = __byte_perm(r[4 * w + 1], r[4 * w + 3], 0x5410);
          b[kk][4 * w + 2] = __byte_perm(r[4 * w], r[4 * w + 2], 0x7632);
          b[kk][4 * w + 3] = __byte_perm(r[4 * w + 1], r[4 * w + 3], 0x7632);
        }
      } else if constexpr (RAW && BITS == 2) {
        // a mask keeps codes (i, i + 8) of a word of 16; step 4 * word + i also takes (i + 4, i + 12)
#pragma unroll
        for (int word = 0; word < 2; ++word)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t selector = (i & 1) ? 0x7632 : 0x5410;
            b[kk][2 * (4 * word + i) + 0] = __byte_perm(r[8 * word + i / 2], r[8 * word + i / 2 + 4], selector);
            b[kk][2 * (4 * word + i) + 1] = __byte_perm(r[8 * word + i / 2 + 2], r[8 * word + i / 2 + 6], selector);
          }
      } else if constexpr (RAW && BITS == 3) {
        // step c takes codes (c, c + 16) and (c + 8, c + 24) of the lane's 32: the halves of a lane's 96 bits
        // repeat each other's bit positions, so one mask keeps a code of each
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t selector = (c & 1) ? 0x7632 : 0x5410;
          b[kk][2 * c + 0] = __byte_perm(r[c / 2], r[c / 2 + 8], selector);
          b[kk][2 * c + 1] = __byte_perm(r[c / 2 + 4], r[c / 2 + 12], selector);
        }
      } else if constexpr (RAW && BITS >= 5 && BITS <= 7) {
        // step s takes codes (c, c + 16) and (c', c' + 16), c and c' the two codes of the step's offset class
        static_for<8>([&](auto step) {
          constexpr int c0 = Spread<BITS>::code_of(decltype(step)::value, 0), c1 = Spread<BITS>::code_of(decltype(step)::value, 1);
          b[kk][2 * decltype(step)::value + 0] = __byte_perm(r[c0 / 2], r[c0 / 2 + 8], (c0 & 1) ? 0x7632 : 0x5410);
          b[kk][2 * decltype(step)::value + 1] = __byte_perm(r[c1 / 2], r[c1 / 2 + 8], (c1 & 1) ? 0x7632 : 0x5410);
        });
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) b[kk][j] = r[j];   // neighbouring codes pair up: the natural order
      }
      if constexpr (RAW) {
        // sum of the k-tile's activations per activation row, on the tensor cores: a weight tile of ones
        // gives every weight row the same sums, laid out as the accumulators want them
        constexpr uint32_t ones = 0x3c003c00u;
        float sums[4];
        mma_first(sums, ones, ones, ones, ones, b[kk][0], b[kk][1], 0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int step = 1; step < 8; ++step) mma_next(sums, ones, ones, ones, ones, b[kk][2 * step], b[kk][2 * step + 1]);
#pragma unroll
        for (int q = 0; q < 4; ++q) start[kk][q] = sums[q] * unit;
      }
    }
  }

  // ---- fragment side: lane (g, t) reads its 32 codes of rows g and g + 8 of every k-tile ----
  const uint32_t table_lane = table_base + lane * 4;
  // scales of rows g and g + 8 in the slot; a single scale per row and visit sits in the half of an
  // aligned pair that the parity of its index says (the same in every visit, the visit step being even)
  const uint32_t scale_begin = ring_base + V::SCALE_OFFSET + g * V::SCALE_ROW_BYTES;
  const int64_t index_low = int64_t(first_row_tile * 16 + g) * a.scale_row_stride + int64_t(tile0) * GPT;
  const int64_t index_high = index_low + 8 * a.scale_row_stride;
  const uint32_t odd_scale_0 = SCALES == 1 && (index_low & 1) ? 2u : 0u, odd_scale_1 = SCALES == 1 && (index_high & 1) ? 2u : 0u;
  const uint32_t red_to = red_base + ((warp * a.batch) * 128 + lane * 4) * 4;

  // One k-tile of one visit: `slot_at` is the shared address of the visit's slot.
  auto tile_product = [&](uint32_t slot_at, int kk, float (&y)[4]) {
    const uint32_t scales_at = slot_at + (scale_begin - ring_base);
    if constexpr (RAW) {
      const float f0 = __half2float(__ushort_as_half((unsigned short)load_shared2(scales_at + kk * 2 + odd_scale_0)));
      const float f1 = __half2float(__ushort_as_half((unsigned short)load_shared2(scales_at + 8 * V::SCALE_ROW_BYTES + kk * 2 + odd_scale_1)));
      float acc[V::CLASSES][4];
      if constexpr (BITS == 4) {
        const uint4 lo = load_shared16(slot_at + tile_offset<4>(kk, g, t)), hi = load_shared16(slot_at + tile_offset<4>(kk, g + 8, t));
        const uint32_t q[4] = {lo.x, lo.y, lo.z, lo.w}, p[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t q8 = q[w] >> 8, p8 = p[w] >> 8;  // codes 2, 3, 6, 7 of a word move down one byte
          if (w == 0) {
            mma_first(acc[0], q[w] & 0x000f000fu, p[w] & 0x000f000fu, q8 & 0x000f000fu, p8 & 0x000f000fu,
                      b[kk][0], b[kk][1], start[kk][0], start[kk][1], start[kk][2], start[kk][3]);
            mma_first(acc[1], q[w] & 0x00f000f0u, p[w] & 0x00f000f0u, q8 & 0x00f000f0u, p8 & 0x00f000f0u,
                      b[kk][2], b[kk][3], 0.f, 0.f, 0.f, 0.f);
          } else {
            mma_next(acc[0], q[w] & 0x000f000fu, p[w] & 0x000f000fu, q8 & 0x000f000fu, p8 & 0x000f000fu,
                     b[kk][4 * w], b[kk][4 * w + 1]);
            mma_next(acc[1], q[w] & 0x00f000f0u, p[w] & 0x00f000f0u, q8 & 0x00f000f0u, p8 & 0x00f000f0u,
                     b[kk][4 * w + 2], b[kk][4 * w + 3]);
          }
        }
      } else if constexpr (BITS == 8) {
        // a byte is the fp16 subnormal c * 2^-24 once it sits in the low byte of a 16-bit lane
        const uint4 lo0 = load_shared16(slot_at + tile_offset<8>(kk, g, 2 * t)), lo1 = load_shared16(slot_at + tile_offset<8>(kk, g, 2 * t + 1));
        const uint4 hi0 = load_shared16(slot_at + tile_offset<8>(kk, g + 8, 2 * t)), hi1 = load_shared16(slot_at + tile_offset<8>(kk, g + 8, 2 * t + 1));
        const uint32_t q[8] = {lo0.x, lo0.y, lo0.z, lo0.w, lo1.x, lo1.y, lo1.z, lo1.w};
        const uint32_t p[8] = {hi0.x, hi0.y, hi0.z, hi0.w, hi1.x, hi1.y, hi1.z, hi1.w};
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          const uint32_t a0 = __byte_perm(q[step], 0u, 0x4140), a1 = __byte_perm(p[step], 0u, 0x4140);
          const uint32_t a2 = __byte_perm(q[step], 0u, 0x4342), a3 = __byte_perm(p[step], 0u, 0x4342);
          if (step == 0) mma_first(acc[0], a0, a1, a2, a3, b[kk][0], b[kk][1], start[kk][0], start[kk][1], start[kk][2], start[kk][3]);
          else mma_next(acc[0], a0, a1, a2, a3, b[kk][2 * step], b[kk][2 * step + 1]);
        }
      } else if constexpr (BITS == 3) {
        // A lane's 32 codes of a row are 12 bytes B0..B11; code c sits at bit 3 c and code c + 16 exactly 48
        // bits later.  Four registers pair a 16-bit window of the first half with the same window of the
        // second; in each, and in its copy moved down one byte, whole codes sit at bit offsets 0..7 of both
        // halves: offset o is the lift 2^o, with an accumulator of its own (eight classes, one step each).
        const uint32_t at0 = slot_at + tile_offset<3>(kk, g, 0) + t * 12, at1 = slot_at + tile_offset<3>(kk, g + 8, 0) + t * 12;
        uint32_t q[4], p[4];
        auto windows = [](uint32_t at, uint32_t (&r)[4]) {
          const uint32_t w0 = load_shared4(at), w1 = load_shared4(at + 4), w2 = load_shared4(at + 8);
          const uint32_t u = __funnelshift_r(w0, w1, 16), v = __funnelshift_r(w1, w2, 16);   // B2..B5, B6..B9
          r[0] = __byte_perm(w0, v, 0x5410);   // B0 B1 | B6 B7:   codes 0 1 2 at offsets 0 3 6, codes 3 4 at 9 12
          r[1] = __byte_perm(w0, v, 0x6521);   // B1 B2 | B7 B8:   code 5 at 7, codes 6 7 at 10 13
          r[2] = __byte_perm(u, w2, 0x6521);   // B3 B4 | B9 B10:  codes 8 9 10 at 0 3 6, codes 11 12 at 9 12
          r[3] = __byte_perm(u, w2, 0x7632);   // B4 B5 | B10 B11: code 13 at 7, codes 14 15 at 10 13
        };
        windows(at0, q);
        windows(at1, p);
        // class (bit offset) of step c, and where its two pairs of codes come from
        auto step = [&](auto code, auto offset, uint32_t x0, uint32_t x1, uint32_t y0, uint32_t y1) {
          constexpr int c = decltype(code)::value, o = decltype(offset)::value;
          constexpr uint32_t mask = 0x00070007u << o;
          if constexpr (o == 0)
            mma_first(acc[o], x0 & mask, x1 & mask, y0 & mask, y1 & mask, b[kk][2 * c], b[kk][2 * c + 1],
                      start[kk][0], start[kk][1], start[kk][2], start[kk][3]);
          else
            mma_first(acc[o], x0 & mask, x1 & mask, y0 & mask, y1 & mask, b[kk][2 * c], b[kk][2 * c + 1], 0.f, 0.f, 0.f, 0.f);
        };
        using std::integral_constant;
        const uint32_t q0 = q[0] >> 8, p0 = p[0] >> 8, q1 = q[1] >> 8, p1 = p[1] >> 8;
        const uint32_t q2 = q[2] >> 8, p2 = p[2] >> 8, q3 = q[3] >> 8, p3 = p[3] >> 8;
        step(integral_constant<int, 0>{}, integral_constant<int, 0>{}, q[0], p[0], q[2], p[2]);
        step(integral_constant<int, 1>{}, integral_constant<int, 3>{}, q[0], p[0], q[2], p[2]);
        step(integral_constant<int, 2>{}, integral_constant<int, 6>{}, q[0], p[0], q[2], p[2]);
        step(integral_constant<int, 3>{}, integral_constant<int, 1>{}, q0, p0, q2, p2);
        step(integral_constant<int, 4>{}, integral_constant<int, 4>{}, q0, p0, q2, p2);
        step(integral_constant<int, 5>{}, integral_constant<int, 7>{}, q[1], p[1], q[3], p[3]);
        step(integral_constant<int, 6>{}, integral_constant<int, 2>{}, q1, p1, q3, p3);
        step(integral_constant<int, 7>{}, integral_constant<int, 5>{}, q1, p1, q3, p3);
      } else if constexpr (BITS >= 5 && BITS <= 7) {
        static_assert(Spread<BITS>::paired(), "every offset class holds an even number of codes");
        uint32_t q[BITS], p[BITS];
        const uint32_t at0 = slot_at + tile_offset<BITS>(kk, g, 0) + t * (4 * BITS);
        const uint32_t at1 = slot_at + tile_offset<BITS>(kk, g + 8, 0) + t * (4 * BITS);
#pragma unroll
        for (int i = 0; i < BITS; ++i) {
          q[i] = load_shared4(at0 + 4 * i);
          p[i] = load_shared4(at1 + 4 * i);
        }
        static_for<8>([&](auto step) {
          using S = Spread<BITS>;
          constexpr int s = decltype(step)::value, c0 = S::code_of(s, 0), c1 = S::code_of(s, 1), o = S::offset(c0);
          constexpr uint32_t mask = (((1u << BITS) - 1u) * 0x00010001u) << o;
          const uint32_t a0 = (paired_window<BITS, S::window(c0)>(q) >> S::shift(c0)) & mask;
          const uint32_t a1 = (paired_window<BITS, S::window(c0)>(p) >> S::shift(c0)) & mask;
          const uint32_t a2 = (paired_window<BITS, S::window(c1)>(q) >> S::shift(c1)) & mask;
          const uint32_t a3 = (paired_window<BITS, S::window(c1)>(p) >> S::shift(c1)) & mask;
          if constexpr (s == 0)
            mma_first(acc[o], a0, a1, a2, a3, b[kk][0], b[kk][1], start[kk][0], start[kk][1], start[kk][2], start[kk][3]);
          else if constexpr (S::opens_class(s))
            mma_first(acc[o], a0, a1, a2, a3, b[kk][2 * s], b[kk][2 * s + 1], 0.f, 0.f, 0.f, 0.f);
          else
            mma_next(acc[o], a0, a1, a2, a3, b[kk][2 * s], b[kk][2 * s + 1]);
        });
      } else {  // BITS == 2: codes of equal position in their byte share a lift of 4^i and an accumulator
        const uint2 lo = load_shared8(slot_at + tile_offset<2>(kk, g, 0) + t * 8), hi = load_shared8(slot_at + tile_offset<2>(kk, g + 8, 0) + t * 8);
        const uint32_t q[2] = {lo.x, lo.y}, p[2] = {hi.x, hi.y};
#pragma unroll
        for (int word = 0; word < 2; ++word) {
          const uint32_t q8 = q[word] >> 8, p8 = p[word] >> 8;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t mask = 0x00030003u << (2 * i);
            const int step = 4 * word + i;
            if (word == 0 && i == 0)
              mma_first(acc[0], q[word] & mask, p[word] & mask, q8 & mask, p8 & mask, b[kk][0], b[kk][1],
                        start[kk][0], start[kk][1], start[kk][2], start[kk][3]);
            else if (word == 0)
              mma_first(acc[i], q[word] & mask, p[word] & mask, q8 & mask, p8 & mask, b[kk][2 * step], b[kk][2 * step + 1],
                        0.f, 0.f, 0.f, 0.f);
            else
              mma_next(acc[i], q[word] & mask, p[word] & mask, q8 & mask, p8 & mask, b[kk][2 * step], b[kk][2 * step + 1]);
          }
        }
      }
      // classes of higher lift were c * 2^-24 times a power of two: recombine exactly (Horner), then one
      // scale per row and k-tile
      if constexpr (BITS >= 5 && BITS <= 7) {   // the offsets in use need not be consecutive
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float total = acc[0][q];
          static_for<V::CLASSES - 1>([&](auto index) {
            constexpr int o = decltype(index)::value + 1;
            if constexpr (Spread<BITS>::used(o)) total = fmaf(acc[o][q], 1.f / float(1 << o), total);
          });
          y[q] = fmaf(q < 2 ? f0 : f1, total, y[q]);
        }
      } else {
        constexpr float down = BITS == 4 ? 0.0625f : BITS == 3 ? 0.5f : 0.25f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float total = acc[V::CLASSES - 1][q];
#pragma unroll
          for (int c = V::CLASSES - 2; c >= 0; --c) total = fmaf(total, down, acc[c][q]);
          y[q] = fmaf(q < 2 ? f0 : f1, total, y[q]);
        }
      }
    } else {
      // table codecs: a pair of codes -> fp16 pair from the lane's copy of the table, times the scale of
      // the lane's row group; the products accumulate directly
      const uint32_t group_of_lane = (t * GPT) >> 2;   // scale group of codes 32t .. 32t+31 inside the k-tile
      const uint32_t s0 = load_shared2(scales_at + (kk * GPT + group_of_lane) * 2 + odd_scale_0);
      const uint32_t s1 = load_shared2(scales_at + 8 * V::SCALE_ROW_BYTES + (kk * GPT + group_of_lane) * 2 + odd_scale_1);
      const uint32_t scale_0 = s0 | (s0 << 16), scale_1 = s1 | (s1 << 16);
      const __half2 f0 = *reinterpret_cast<const __half2*>(&scale_0), f1 = *reinterpret_cast<const __half2*>(&scale_1);
      // with one scale per k-tile (GPT == 1) the scale multiplies the tile's sum, as in the RAW codecs: the
      // table values go to the tensor core as they are; with two groups per k-tile a step mixes groups,
      // so every pair is scaled before it
      constexpr bool SCALE_SUM = GPT == 1;
      auto weight_pair = [&](uint32_t entry, __half2 scale) -> uint32_t {
        const uint32_t bits = load_shared4(table_lane + entry * 128u);
        if constexpr (SCALE_SUM) return bits;
        const __half2 scaled = __hmul2(*reinterpret_cast<const __half2*>(&bits), scale);
        return *reinterpret_cast<const uint32_t*>(&scaled);
      };
      float tile_sum[4] = {0.f, 0.f, 0.f, 0.f};
      float (&into)[4] = SCALE_SUM ? tile_sum : y;
      if constexpr (BITS == 4) {
        const uint4 lo = load_shared16(slot_at + tile_offset<4>(kk, g, t)), hi = load_shared16(slot_at + tile_offset<4>(kk, g + 8, t));
        const uint32_t q[4] = {lo.x, lo.y, lo.z, lo.w}, p[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int step = 0; step < 8; ++step) {   // bytes 2 * step and 2 * step + 1 of the lane's 16
          const int w = step >> 1, low = (step & 1) ? 0x4442 : 0x4440, high = (step & 1) ? 0x4443 : 0x4441;
          mma_next(into, weight_pair(__byte_perm(q[w], 0u, low), f0), weight_pair(__byte_perm(p[w], 0u, low), f1),
                   weight_pair(__byte_perm(q[w], 0u, high), f0), weight_pair(__byte_perm(p[w], 0u, high), f1),
                   b[kk][2 * step], b[kk][2 * step + 1]);
        }
      } else {  // BITS == 3: 32 codes are 96 bits; pair j is the 6-bit field at bit 6 j
        const uint32_t at0 = slot_at + tile_offset<3>(kk, g, 0) + t * 12, at1 = slot_at + tile_offset<3>(kk, g + 8, 0) + t * 12;
        const uint32_t q[3] = {load_shared4(at0), load_shared4(at0 + 4), load_shared4(at0 + 8)};
        const uint32_t p[3] = {load_shared4(at1), load_shared4(at1 + 4), load_shared4(at1 + 8)};
        auto field = [](const uint32_t (&w)[3], int j) -> uint32_t {
          const int bit = 6 * j, word = bit >> 5, shift = bit & 31;
          const uint32_t value = shift + 6 <= 32 ? w[word] >> shift : __funnelshift_r(w[word], w[word + 1], shift);
          return value & 63u;
        };
#pragma unroll
        for (int step = 0; step < 8; ++step)
          mma_next(into, weight_pair(field(q, 2 * step), f0), weight_pair(field(p, 2 * step), f1),
                   weight_pair(field(q, 2 * step + 1), f0), weight_pair(field(p, 2 * step + 1), f1),
                   b[kk][2 * step], b[kk][2 * step + 1]);
      }
      if constexpr (SCALE_SUM) {
        const float scale_low = __half2float(__low2half(f0)), scale_high = __half2float(__low2half(f1));
#pragma unroll
        for (int q = 0; q < 4; ++q) y[q] = fmaf(q < 2 ? scale_low : scale_high, tile_sum[q], y[q]);
      }
    }
  };

  // One round: R visits, unrolled over the ring, so every shared-memory offset is an immediate.  With
  // CHECKED == false the caller promises that this warp owns every visit of the round and every visit
  // the round issues copies for, and the body has no branches.
  auto round = [&](int visit0, uint32_t red_at, auto checked) {
    constexpr bool CHECKED = decltype(checked)::value;
#pragma unroll
    for (int d = 0; d < R; ++d) {
      const int visit = visit0 + d;
      __syncwarp();  // every lane has read the slot that the next copies overwrite
      issue(visit + R - 1, (d + R - 1) % R, !CHECKED || visit + R - 1 < my_visits, !CHECKED || visit + R - 1 < whole_visits);
      copy_wait<R - 1>();
      __syncwarp();  // the lanes' copies of this visit are visible to the whole warp
      float y[4] = {0.f, 0.f, 0.f, 0.f};
      if (!CHECKED || visit < my_visits) {
#pragma unroll
        for (int kk = 0; kk < KT; ++kk) tile_product(ring_base + d * V::SLOT_BYTES, kk, y);
      }
      store_shared16(red_at + d * 512, y[0], y[1], y[2], y[3]);
    }
  };

  int batch_first = 0;   // first visit of the batch whose sums shared memory holds
  for (int visit0 = 0; visit0 < a.visits; visit0 += R) {
    const uint32_t red_at = red_to + (visit0 - batch_first) * 512;
    if (visit0 + 2 * R - 2 < whole_visits) round(visit0, red_at, std::false_type{});
    else round(visit0, red_at, std::true_type{});
    if (visit0 + R - batch_first < a.batch && visit0 + R < a.visits) continue;

    // ---- end of a batch: add the warps' partial sums in warp order, four outputs per thread ----
    __syncthreads();
    const int in_batch = min(a.batch, a.visits - batch_first);
    const int quads = in_batch * a.RG * 32;
    for (int o = threadIdx.x; o < quads; o += blockDim.x) {
      const int source_lane = o & 31, group_index = o >> 5;
      const int d = (group_index * a.rg_inverse) >> 16, rgi = group_index - d * a.RG;   // / RG, % RG
      const float4* partial = reinterpret_cast<const float4*>(red_s) + (size_t(rgi) * a.KW * a.batch + d) * 32 + source_lane;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int w = 0; w < a.KW; ++w) {
        const float4 v = partial[w * a.batch * 32];
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
      const int v = batch_first + d;
      if (a.slabs > 1) {
        reinterpret_cast<float4*>(acc_s)[(size_t(v) * a.RG + rgi) * 32 + source_lane] = sum;
      } else {
        // the lane that produced this quad held weight rows g, g + 8 and activation rows 2t, 2t + 1
        const int rt = int(blockIdx.x) * a.RG + rgi + v * visit_stride;
        const int row = rt * 16 + (source_lane >> 2), m = (source_lane & 3) * 2;
        if (rt < a.row_tiles) {
          const float out[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int mq = m + (q & 1), rq = row + (q & 2) * 4;
            if (mq < a.M && rq < a.N) {
              float value = RAW ? out[q] * 16777216.f : out[q];  // RAW sums are in units of 2^-24
              if (a.bias != nullptr) value += __half2float(a.bias[rq]);
              a.y[int64_t(mq) * a.N + rq] = __float2half_rn(value);
            }
          }
        }
      }
    }
    batch_first = visit0 + R;
    if (batch_first < a.visits) __syncthreads();   // the next batch overwrites the sums
  }
  copy_wait<0>();

  // ---- K split over the cluster: one exchange through distributed shared memory, slab order ----
  if (a.slabs > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int outputs = a.visits * a.RG * 128;
    for (int o = slab * int(blockDim.x) + threadIdx.x; o < outputs; o += a.slabs * int(blockDim.x)) {
      float sum = 0.f;
      for (int peer = 0; peer < a.slabs; ++peer) sum += cluster.map_shared_rank(acc_s, peer)[o];
      const int e = o & 127, group_index = o >> 7;
      const int v = group_index / a.RG, rgi = group_index - v * a.RG;
      const int rt = int(blockIdx.x) * a.RG + rgi + v * visit_stride;
      const int row = rt * 16 + (e >> 4) + ((e & 2) ? 8 : 0), m = ((e >> 2) & 3) * 2 + (e & 1);
      if (rt < a.row_tiles && row < a.N && m < a.M) {
        if (RAW) sum *= 16777216.f;
        if (a.bias != nullptr) sum += __half2float(a.bias[row]);
        a.y[int64_t(m) * a.N + row] = __float2half_rn(sum);
      }
    }
    cluster.sync();  // no CTA leaves while a peer may still read its sums
  }
}

// ---- host side -----------------------------------------------------------------------------------
template <typename Kernel>
int opt_in_shared(Kernel kernel) {
  static std::mutex lock;
  static std::map<std::pair<const void*, int>, bool> done;
  int device = 0;
  cudaGetDevice(&device);
  const auto key = std::make_pair(reinterpret_cast<const void*>(kernel), device);
  std::lock_guard<std::mutex> guard(lock);
  if (done.count(key)) return MKB_OK;
  cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            device_info().max_smem_optin);
  if (status != cudaSuccess) return cuda_fail(status, "gemv_stream: shared memory opt-in");
  status = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  if (status != cudaSuccess) return cuda_fail(status, "gemv_stream: cluster size opt-in");
  done[key] = true;
  return MKB_OK;
}

constexpr size_t kMaxRotationBytes = 64 * 1024;   // of fp32 activations a CTA rotates in shared memory

struct StreamPlan {
  int bits, mode, gpt;   // the codec: code width, MODE_*, scale groups per k-tile
  int KT, KW, RG, slabs, columns, visits, depth, batch, per_sm;
  size_t smem;
};

// Chooses the decomposition: slabs of K (CTAs of a cluster), warps along K and row tiles per visit of a
// CTA, CTAs per SM (small CTAs share an SM), ring depth (= visits per round).
// `cluster_cap` > 0 bounds the number of clusters in flight.  bits, mode, gpt are inputs.
bool plan_stream(int M, int N, int K, int sm_count, int max_smem, int cluster_cap, StreamPlan& p, size_t extra = 0) {
  (void)M;
  const int k_tiles = K / 128;
  const int KT = k_tiles % 2 == 0 ? 2 : 1;
  const int k_warps = k_tiles / KT;
  const int row_tiles = (N + 15) / 16;
  const int scale_row_bytes = KT * p.gpt * 2 < 4 ? 4 : KT * p.gpt * 2;
  const size_t slot = size_t(KT) * 256 * p.bits + 16 * scale_row_bytes;
  const size_t table = p.mode == MODE_TABLE ? (size_t(128) << (2 * p.bits)) : 0;
  // fewest slabs that give every warp of a 16-warp CTA one share of K.  The choice depends on K alone,
  // so a layer and the same rows inside a wider (concatenated) layer are summed in the same order.
  const int slabs = (k_warps + kMaxWarps - 1) / kMaxWarps;
  if (slabs > 8) return false;
  const int KW = (k_warps + slabs - 1) / slabs;
  int RG = kMaxWarps / KW;
  while (RG > 1 && (row_tiles + RG - 1) / RG * slabs < sm_count) --RG;  // keep every SM busy first
  const int warps = KW * RG;
  const int per_sm = table ? 1 : kMaxWarps / warps;
  int clusters = sm_count * per_sm / slabs;
  if (cluster_cap > 0 && clusters > cluster_cap) clusters = cluster_cap;  // what the GPU can co-schedule
  if (clusters < 1) return false;
  const int items = (row_tiles + RG - 1) / RG;
  const int columns = items < clusters ? items : clusters;
  const int visits = (items + columns - 1) / columns;
  if (slabs > 1 && visits > kMaxClusterVisits) return false;
  int depth = visits < 2 ? 2 : visits > 3 ? 3 : visits;
  const size_t budget = (size_t(max_smem) + 1024) / per_sm - 1024;  // every resident CTA reserves 1 KB
  const size_t sums = (slabs > 1 ? size_t(visits) * RG * 512 : 0) + table + extra;   // extra: the rotation buffer, last
  while (depth > 2 && size_t(depth) * warps * (slot + 512) + sums > budget) --depth;
  if (size_t(depth) * warps * (slot + 512) + sums > budget) return false;
  // partial sums of as many visits as fit (whole rounds), ideally all: one reduction at the end
  const int rounds = (visits + depth - 1) / depth;
  int batch_rounds = int((budget - sums - size_t(depth) * warps * slot) / (size_t(depth) * warps * 512));
  if (batch_rounds > rounds) batch_rounds = rounds;
  const int batch = batch_rounds * depth;
  p.KT = KT; p.KW = KW; p.RG = RG; p.slabs = slabs; p.columns = columns; p.visits = visits;
  p.depth = depth; p.batch = batch; p.per_sm = per_sm;
  p.smem = size_t(depth) * warps * slot + size_t(batch) * warps * 512 + sums;
  return true;
}

template <int BITS, int MODE, int GPT, int KT, int R>
int launch_stream(const StreamArgs& a, const StreamPlan& p, cudaStream_t stream, int* cluster_cap) {
  auto kernel = a.rot_log2 ? gemv_stream_kernel<BITS, MODE, GPT, KT, R, true> : gemv_stream_kernel<BITS, MODE, GPT, KT, R, false>;
  int status = opt_in_shared(kernel);
  if (status != MKB_OK) return status;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(p.columns, p.slabs, 1);
  config.blockDim = dim3(p.KW * p.RG * 32, 1, 1);
  config.dynamicSmemBytes = p.smem;
  config.stream = stream;
  // Programmatic dependent launch: CTAs may start while the previous kernel of the stream drains; they
  // copy weights (constants) at once and execute griddepcontrol.wait before they read activations.
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (p.slabs > 1) {
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = 1;
    attribute[1].val.clusterDim.y = p.slabs;
    attribute[1].val.clusterDim.z = 1;
    config.numAttrs = 2;
  }
  if (cluster_cap != nullptr) {
    // how many clusters of this shape the GPU holds at once (cached): a grid beyond it runs in waves
    static std::mutex lock;
    static std::map<std::tuple<const void*, int, size_t, int, int>, int> known;
    int device = 0;
    cudaGetDevice(&device);
    const auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), int(config.blockDim.x), p.smem, p.slabs, device);
    std::lock_guard<std::mutex> guard(lock);
    auto found = known.find(key);
    if (found == known.end()) {
      int clusters = 0;
      config.gridDim = dim3(1024, p.slabs, 1);
      const cudaError_t asked = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
      if (asked != cudaSuccess) return cuda_fail(asked, "gemv_stream: cluster occupancy query");
      found = known.emplace(key, clusters).first;
    }
    *cluster_cap = found->second;
    return MKB_OK;
  }
  const cudaError_t launched = cudaLaunchKernelEx(&config, kernel, a);
  if (launched != cudaSuccess) return cuda_fail(launched, "gemv_stream launch");
  return MKB_OK;
}

template <int BITS, int MODE, int GPT>
int dispatch_shape(const StreamArgs& a, const StreamPlan& p, cudaStream_t stream, int* cluster_cap) {
  if (p.KT == 2) {
    if (p.depth == 2) return launch_stream<BITS, MODE, GPT, 2, 2>(a, p, stream, cluster_cap);
    return launch_stream<BITS, MODE, GPT, 2, 3>(a, p, stream, cluster_cap);
  }
  if (p.depth == 2) return launch_stream<BITS, MODE, GPT, 1, 2>(a, p, stream, cluster_cap);
  return launch_stream<BITS, MODE, GPT, 1, 3>(a, p, stream, cluster_cap);
}

int dispatch_stream(const StreamArgs& a, const StreamPlan& p, cudaStream_t stream, int* cluster_cap) {
  if (p.mode == MODE_RAW) {
    if (p.bits == 4) return dispatch_shape<4, MODE_RAW, 1>(a, p, stream, cluster_cap);
    if (p.bits == 2) return dispatch_shape<2, MODE_RAW, 1>(a, p, stream, cluster_cap);
    if (p.bits == 3) return dispatch_shape<3, MODE_RAW, 1>(a, p, stream, cluster_cap);
    if (p.bits == 5) return dispatch_shape<5, MODE_RAW, 1>(a, p, stream, cluster_cap);
    if (p.bits == 6) return dispatch_shape<6, MODE_RAW, 1>(a, p, stream, cluster_cap);
    if (p.bits == 7) return dispatch_shape<7, MODE_RAW, 1>(a, p, stream, cluster_cap);
    return dispatch_shape<8, MODE_RAW, 1>(a, p, stream, cluster_cap);
  }
  if (p.bits == 4) return p.gpt == 1 ? dispatch_shape<4, MODE_TABLE, 1>(a, p, stream, cluster_cap)
                                     : dispatch_shape<4, MODE_TABLE, 2>(a, p, stream, cluster_cap);
  return p.gpt == 1 ? dispatch_shape<3, MODE_TABLE, 1>(a, p, stream, cluster_cap)
                    : dispatch_shape<3, MODE_TABLE, 2>(a, p, stream, cluster_cap);
}

// The codec a call maps to: false when the streaming kernel does not cover it.
bool codec_of(int group, int bits, int lut_len, const void* zeros, int integer_grid, float grid_minimum, StreamPlan& p) {
  if (zeros != nullptr || lut_len < 1 || lut_len > (1 << bits)) return false;
  const bool ramp = integer_grid && lut_len == (1 << bits) && grid_minimum == float(int(grid_minimum)) &&
                    grid_minimum >= -512.f && grid_minimum <= 512.f;
  if (ramp && group == 128 && bits >= 2 && bits <= 8) {
    p.bits = bits; p.mode = MODE_RAW; p.gpt = 1;
    return true;
  }
  if ((bits == 3 || bits == 4) && (group == 64 || group == 128)) {
    p.bits = bits; p.mode = MODE_TABLE; p.gpt = 128 / group;
    return true;
  }
  return false;
}

}  // namespace

int gemv_stream_supported(int M, int N, int K, int group, int bits, int lut_len, int x_dtype, int scale_dtype,
                          const void* x, const uint8_t* packed, const void* scales, int64_t packed_row_stride,
                          int64_t scale_row_stride, const void* zeros, int integer_grid, float grid_minimum) {
  if (x_dtype != MKB_F16 || scale_dtype != MKB_F16) return 0;
  if (M < 1 || M > 8 || N < 1 || K < 128 || K % 128 != 0) return 0;
  StreamPlan plan{};
  if (!codec_of(group, bits, lut_len, zeros, integer_grid, grid_minimum, plan)) return 0;
  if (reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(packed) % 16 || packed_row_stride % 16) return 0;
  // the scales of a row and visit are copied as one aligned piece of 4, 8 or 16 bytes
  const int scales_per_visit = ((K / 128) % 2 == 0 ? 2 : 1) * plan.gpt;
  if (scales_per_visit == 1) {
    if (reinterpret_cast<uintptr_t>(scales) % 4 || (int64_t(N) * scale_row_stride) % 2) return 0;  // aligned pairs
  } else if (reinterpret_cast<uintptr_t>(scales) % (scales_per_visit * 2) || scale_row_stride % scales_per_visit) {
    return 0;
  }
  if (int64_t(N) * packed_row_stride >= (int64_t(1) << 32) || int64_t(N) * scale_row_stride >= (int64_t(1) << 30)) return 0;
  const DeviceInfo& info = device_info();
  return plan_stream(M, N, K, info.sm_count, info.max_smem_optin, 0, plan) ? 1 : 0;
}

// Rotation on load: K = 2^log2 >= 512 and M * K fp32 values of shared memory beside the rings.
int gemv_stream_rotation_supported(int M, int N, int K, int group, int bits, int lut_len, int integer_grid,
                                   float grid_minimum, const void* signs) {
  if (K < kWarpSpan || (K & (K - 1)) != 0 || size_t(M) * K * 4 > kMaxRotationBytes) return 0;
  if (reinterpret_cast<uintptr_t>(signs) % 16) return 0;
  StreamPlan plan{};
  if (!codec_of(group, bits, lut_len, nullptr, integer_grid, grid_minimum, plan)) return 0;
  const DeviceInfo& info = device_info();
  return plan_stream(M, N, K, info.sm_count, info.max_smem_optin, 0, plan, size_t(M) * K * 4) ? 1 : 0;
}

int launch_gemv_stream_rotated(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                               const void* bias, void* y, int M, int N, int K, int group, int bits, int lut_len,
                               int64_t packed_row_stride, int64_t scale_row_stride, int integer_grid,
                               float grid_minimum, int gated, const int8_t* signs, int rotate, int normalize,
                               cudaStream_t stream) {
  const DeviceInfo& info = device_info();
  StreamPlan p{};
  const size_t extra = rotate ? size_t(M) * K * 4 : 0;
  MKB_REQUIRE(codec_of(group, bits, lut_len, nullptr, integer_grid, grid_minimum, p) &&
                  plan_stream(M, N, K, info.sm_count, info.max_smem_optin, 0, p, extra),
              MKB_E_UNSUPPORTED, "gemv_stream: no decomposition for N=%d K=%d bits=%d group=%d", N, K, bits, group);
  StreamArgs a{};
  if (p.slabs > 1) {  // a grid of clusters must be resident as a whole, or it runs in waves
    int cap = 0;
    const int status = dispatch_stream(a, p, stream, &cap);
    if (status != MKB_OK) return status;
    MKB_REQUIRE(cap >= 1, MKB_E_UNSUPPORTED, "gemv_stream: no cluster of %d CTAs fits the GPU", p.slabs);
    if (p.columns > cap)
      MKB_REQUIRE(plan_stream(M, N, K, info.sm_count, info.max_smem_optin, cap, p, extra),
                  MKB_E_UNSUPPORTED, "gemv_stream: no decomposition for N=%d K=%d in %d clusters", N, K, cap);
  }
  a.x = static_cast<const __half*>(x); a.packed = packed; a.scales = static_cast<const __half*>(scales);
  a.bias = static_cast<const __half*>(bias); a.y = static_cast<__half*>(y); a.lut = lut; a.lut_len = lut_len;
  a.M = M; a.N = N; a.K = K; a.packed_row_stride = packed_row_stride; a.scale_row_stride = scale_row_stride;
  a.row_tiles = (N + 15) / 16; a.k_warps = K / (128 * p.KT); a.KW = p.KW; a.RG = p.RG; a.slabs = p.slabs;
  a.visits = p.visits; a.grid_min = p.mode == MODE_RAW ? grid_minimum : 0.f; a.batch = p.batch; a.early = 1; a.gated = gated;
  a.kw_inverse = (65536 + p.KW - 1) / p.KW; a.rg_inverse = (65536 + p.RG - 1) / p.RG;
  if (rotate) {
    a.rot_signs = signs;
    while ((1 << a.rot_log2) < K) ++a.rot_log2;
    a.rot_offset = uint32_t(p.smem - extra);
    // the reference forms the scale in fp32: float(torch.tensor(1.0) / torch.tensor(math.sqrt(width)))
    a.rot_scale = normalize ? 1.0f / float(sqrt(double(K))) : 1.0f;
  }
  return dispatch_stream(a, p, stream, nullptr);
}

int launch_gemv_stream(const void* x, const uint8_t* packed, const void* scales, const float* lut, const void* bias,
                       void* y, int M, int N, int K, int group, int bits, int lut_len, int64_t packed_row_stride,
                       int64_t scale_row_stride, int integer_grid, float grid_minimum, int gated, cudaStream_t stream) {
  return launch_gemv_stream_rotated(x, packed, scales, lut, bias, y, M, N, K, group, bits, lut_len, packed_row_stride,
                                    scale_row_stride, integer_grid, grid_minimum, gated, nullptr, 0, 0, stream);
}

}  // namespace mkb
