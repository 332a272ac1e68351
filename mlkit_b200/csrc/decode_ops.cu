// The small operators between the packed matvecs of a Llama-style decode step, one launch each:
// residual add + RMS norm, rotary embedding + KV-cache append, single-token attention over the cache
// (grouped-query), SiLU(gate) * up.  fp16 storage, fp32 arithmetic.  They exist so that a decode step
// is a short chain of launches that a CUDA graph replays; none of them is bandwidth critical.
#include "mkb_common.cuh"

namespace mkb {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// residual[m,:] += delta[m,:] (when delta != null); normed[m,:] = residual[m,:] * rsqrt(mean(sq) + eps) * weight.
// One CTA of 1024 threads per row; a thread keeps its (up to two) 8-element pieces in registers
// between the two passes, so the row is read once.
constexpr int kNormThreads = 1024;
constexpr int kNormPieces = 2;   // rows up to 1024 * 2 * 8 = 16384 elements stay in registers

__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(__half* __restrict__ residual,
                                                                   const __half* __restrict__ delta,
                                                                   const __half* __restrict__ weight,
                                                                   __half* __restrict__ normed, int H, float eps) {
  // programmatic dependent launch: let the next kernel in the stream become resident now (a matvec
  // starts streaming its weights), then wait for everything this kernel reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the norm weights are constants of the model: fetched before the wait, they cost no latency after the sum
  uint4 scale_of[kNormPieces];
#pragma unroll
  for (int piece = 0; piece < kNormPieces; ++piece) {
    const int i = (piece * kNormThreads + threadIdx.x) * 8;
    scale_of[piece] = i < H ? __ldg(reinterpret_cast<const uint4*>(weight + i)) : make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ float part_s[kNormThreads / 32];
  const int64_t base = int64_t(blockIdx.x) * H;
  uint4 kept[kNormPieces];
  float sq = 0.f;
#pragma unroll
  for (int piece = 0; piece < kNormPieces; ++piece) {
    const int i = (piece * kNormThreads + threadIdx.x) * 8;
    kept[piece] = make_uint4(0u, 0u, 0u, 0u);
    if (i < H) {
      uint4 v = *reinterpret_cast<const uint4*>(residual + base + i);
      if (delta != nullptr) {
        const uint4 d = *reinterpret_cast<const uint4*>(delta + base + i);
        // the sum is stored back in fp16: the running residual of the model is an fp16 tensor
        __half2* vh = reinterpret_cast<__half2*>(&v);
        const __half2* dh = reinterpret_cast<const __half2*>(&d);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 a = __half22float2(vh[q]), b = __half22float2(dh[q]);
          vh[q] = __floats2half2_rn(a.x + b.x, a.y + b.y);
        }
        *reinterpret_cast<uint4*>(residual + base + i) = v;
      }
      kept[piece] = v;
      const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __half22float2(vh[q]);
        sq += a.x * a.x + a.y * a.y;
      }
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5] = sq;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kNormThreads / 32; ++w) total += part_s[w];
  const float inv = rsqrtf(total / float(H) + eps);
#pragma unroll
  for (int piece = 0; piece < kNormPieces; ++piece) {
    const int i = (piece * kNormThreads + threadIdx.x) * 8;
    if (i < H) {
      const __half2* vh = reinterpret_cast<const __half2*>(&kept[piece]);
      const __half2* wh = reinterpret_cast<const __half2*>(&scale_of[piece]);
      uint4 result;
      __half2* rh = reinterpret_cast<__half2*>(&result);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __half22float2(vh[q]), ww = __half22float2(wh[q]);
        // same rounding points as the usual fp16 module: the normalised value is rounded, then scaled
        const float2 u = __half22float2(__floats2half2_rn(a.x * inv, a.y * inv));
        rh[q] = __floats2half2_rn(u.x * ww.x, u.y * ww.y);
      }
      *reinterpret_cast<uint4*>(normed + base + i) = result;
    }
  }
}

// Any even row length (rows staged in shared memory): residual[m,:] += delta[m,:] (when delta != null); normed[m,:] = residual[m,:] * rsqrt(mean(sq) + eps) * weight
__global__ void __launch_bounds__(256) add_rmsnorm_generic_kernel(__half* __restrict__ residual, const __half* __restrict__ delta,
                                                          const __half* __restrict__ weight, __half* __restrict__ normed,
                                                          int H, float eps) {
  // programmatic dependent launch: let the next kernel in the stream become resident now (a matvec
  // starts streaming its weights), then wait for everything this kernel reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  extern __shared__ float row_s[];  // [H]
  __shared__ float part_s[8];
  const int64_t base = int64_t(blockIdx.x) * H;
  float sq = 0.f;
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    float2 v = __half22float2(*reinterpret_cast<const __half2*>(residual + base + i));
    if (delta != nullptr) {
      const float2 d = __half22float2(*reinterpret_cast<const __half2*>(delta + base + i));
      // the sum is stored back in fp16: the running residual of the model is an fp16 tensor
      const __half2 summed = __floats2half2_rn(v.x + d.x, v.y + d.y);
      *reinterpret_cast<__half2*>(residual + base + i) = summed;
      v = __half22float2(summed);
    }
    row_s[i] = v.x;
    row_s[i + 1] = v.y;
    sq += v.x * v.x + v.y * v.y;
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5] = sq;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < (blockDim.x >> 5); ++w) total += part_s[w];
  const float inv = rsqrtf(total / float(H) + eps);
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    const float2 w = __half22float2(*reinterpret_cast<const __half2*>(weight + i));
    // same rounding points as the usual fp16 module: the normalised value is rounded, then scaled
    const __half2 unit = __floats2half2_rn(row_s[i] * inv, row_s[i + 1] * inv);
    const float2 u = __half22float2(unit);
    *reinterpret_cast<__half2*>(normed + base + i) = __floats2half2_rn(u.x * w.x, u.y * w.y);
  }
}

// qkv[m] = [q heads | k heads | v heads], head_dim D (even).  Rotates q and k in place (pairs (i, i + D/2),
// angle position * theta^(-2i/D)) and writes k, v into the caches at `positions[m]`.
// A cache position outside [0, capacity) must never become an address: the kernels clamp it, skip the
// append, and raise this word, which mkb_decode_status reads (and clears).
__device__ unsigned int g_decode_status = 0;

__device__ __forceinline__ int checked_position(int position, int capacity, bool& valid) {
  valid = position >= 0 && position < capacity;
  if (!valid) {
    if (threadIdx.x == 0) atomicOr(&g_decode_status, 1u);
    position = position < 0 ? 0 : capacity - 1;
  }
  return position;
}

__global__ void rope_append_kernel(__half* __restrict__ qkv, const int* __restrict__ positions,
                                   __half* __restrict__ k_cache, __half* __restrict__ v_cache, int q_heads,
                                   int kv_heads, int D, int capacity, float theta) {
  // programmatic dependent launch: let the next kernel in the stream become resident now (a matvec
  // starts streaming its weights), then wait for everything this kernel reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.x, head = blockIdx.y;  // head over q_heads + kv_heads (+ kv_heads for v)
  bool in_cache;
  const int position = checked_position(positions[m], capacity, in_cache);
  const int row = (q_heads + 2 * kv_heads) * D;
  __half* vec = qkv + int64_t(m) * row + int64_t(head) * D;
  const int half_dim = D / 2;
  if (head < q_heads + kv_heads) {
    for (int i = threadIdx.x; i < half_dim; i += blockDim.x) {
      const float freq = powf(theta, -2.f * float(i) / float(D));
      float s, c;
      sincosf(float(position) * freq, &s, &c);
      const float a = __half2float(vec[i]), b = __half2float(vec[i + half_dim]);
      vec[i] = __float2half_rn(a * c - b * s);
      vec[i + half_dim] = __float2half_rn(b * c + a * s);
    }
  }
  if (head >= q_heads && in_cache) {
    __syncthreads();
    const bool is_v = head >= q_heads + kv_heads;
    const int kv = head - q_heads - (is_v ? kv_heads : 0);
    __half* cache = (is_v ? v_cache : k_cache) + ((int64_t(m) * kv_heads + kv) * capacity + position) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) cache[i] = vec[i];
  }
}

// One CTA of 512 threads per (sequence m, query head), head_dim 128.
//   1. scores: a thread owns whole cached positions (16 independent 16-byte key reads, q in shared
//      memory, read as broadcasts);
//   2. block-wide max and sum of exp;
//   3. values: warp w takes positions w, w + 16, ...; a lane owns four dimensions (one 8-byte read
//      per position, a warp reads a whole 256-byte row), eight positions in flight; the 16 warps
//      meet in shared memory.
constexpr int kAttentionThreads = 512;
constexpr int kAttentionWarps = kAttentionThreads / 32;

__global__ void __launch_bounds__(kAttentionThreads) attention_decode_kernel(
    const __half* __restrict__ qkv, const int* __restrict__ positions, const __half* __restrict__ k_cache,
    const __half* __restrict__ v_cache, __half* __restrict__ out, int q_heads, int kv_heads, int capacity, float scale) {
  // programmatic dependent launch: let the next kernel in the stream become resident now (a matvec
  // starts streaming its weights), then wait for everything this kernel reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int D = 128;
  extern __shared__ float score_s[];  // [capacity]
  __shared__ float q_s[D];
  __shared__ float part_s[kAttentionWarps];
  __shared__ float acc_s[kAttentionWarps][D];
  const int m = blockIdx.x, head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool in_cache;
  const int length = checked_position(positions[m], capacity, in_cache) + 1;  // the new token was appended already
  const int kv = head / (q_heads / kv_heads);
  const int row = (q_heads + 2 * kv_heads) * D;
  if (threadIdx.x < D) q_s[threadIdx.x] = __half2float(qkv[int64_t(m) * row + int64_t(head) * D + threadIdx.x]) * scale;
  __syncthreads();
  const __half* keys = k_cache + (int64_t(m) * kv_heads + kv) * capacity * D;
  const __half* values = v_cache + (int64_t(m) * kv_heads + kv) * capacity * D;

  float local_max = -INFINITY;
  for (int p = threadIdx.x; p < length; p += kAttentionThreads) {
    const uint4* key = reinterpret_cast<const uint4*>(keys + int64_t(p) * D);
    uint4 raw[D / 8];
#pragma unroll
    for (int v = 0; v < D / 8; ++v) raw[v] = __ldg(key + v);
    float dot0 = 0.f, dot1 = 0.f;
#pragma unroll
    for (int v = 0; v < D / 8; ++v) {
      const uint32_t words[4] = {raw[v].x, raw[v].y, raw[v].z, raw[v].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
        dot0 = fmaf(q_s[v * 8 + 2 * i], k2.x, dot0);
        dot1 = fmaf(q_s[v * 8 + 2 * i + 1], k2.y, dot1);
      }
    }
    const float dot = dot0 + dot1;
    score_s[p] = dot;
    local_max = fmaxf(local_max, dot);
  }
  local_max = warp_max(local_max);
  if (lane == 0) part_s[warp] = local_max;
  __syncthreads();
  float top = part_s[0];
#pragma unroll
  for (int w = 1; w < kAttentionWarps; ++w) top = fmaxf(top, part_s[w]);
  __syncthreads();
  float local_sum = 0.f;
  for (int p = threadIdx.x; p < length; p += kAttentionThreads) {
    const float weight = __expf(score_s[p] - top);
    score_s[p] = weight;
    local_sum += weight;
  }
  local_sum = warp_sum(local_sum);
  if (lane == 0) part_s[warp] = local_sum;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kAttentionWarps; ++w) total += part_s[w];

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const __half* column = values + 4 * lane;
  int p = warp;
  for (; p + 7 * kAttentionWarps < length; p += 8 * kAttentionWarps) {
    uint2 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint2*>(column + int64_t(p + u * kAttentionWarps) * D);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float weight = score_s[p + u * kAttentionWarps];
      const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&v[u].x));
      const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&v[u].y));
      acc[0] = fmaf(weight, lo.x, acc[0]); acc[1] = fmaf(weight, lo.y, acc[1]);
      acc[2] = fmaf(weight, hi.x, acc[2]); acc[3] = fmaf(weight, hi.y, acc[3]);
    }
  }
  for (; p < length; p += kAttentionWarps) {
    const uint2 v = *reinterpret_cast<const uint2*>(column + int64_t(p) * D);
    const float weight = score_s[p];
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
    acc[0] = fmaf(weight, lo.x, acc[0]); acc[1] = fmaf(weight, lo.y, acc[1]);
    acc[2] = fmaf(weight, hi.x, acc[2]); acc[3] = fmaf(weight, hi.y, acc[3]);
  }
  *reinterpret_cast<float4*>(&acc_s[warp][4 * lane]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  __syncthreads();
  if (threadIdx.x < D) {
    float value = 0.f;
#pragma unroll
    for (int w = 0; w < kAttentionWarps; ++w) value += acc_s[w][threadIdx.x];
    out[(int64_t(m) * q_heads + head) * D + threadIdx.x] = __float2half_rn(value / total);
  }
}

// ---- attention with grouped query heads on the tensor cores ----------------------------------------
constexpr int kGroupWarps = 12;
constexpr int kGroupThreads = kGroupWarps * 32;
constexpr int kPitch = 272;                 // bytes per staged row: 256 of data + 16 of padding (ldmatrix conflict-free)
constexpr int kTileBytes = 16 * kPitch;     // one 16-position tile of K or of V

__device__ __forceinline__ uint32_t shared_address(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One CTA per (sequence m, key-value head): the G query heads that share the head are the rows of the
// tensor-core tiles, so every cached key and value is read once.  A warp owns 16-position tiles
// (warp, warp + 16, ...): S = Q K^T (16 steps), running softmax per row, O += P V (16 steps); the
// warps' (max, sum, O) meet in shared memory in warp order.
__global__ void __launch_bounds__(kGroupThreads) attention_group_kernel(const __half* __restrict__ qkv, const int* __restrict__ positions,
                                                                 const __half* __restrict__ k_cache,
                                                                 const __half* __restrict__ v_cache, __half* __restrict__ out,
                                                                 int q_heads, int kv_heads, int capacity, float scale,
                                                                 float theta, int fuse_rope) {
  // programmatic dependent launch: let the next kernel in the stream become resident now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int D = 128;
  extern __shared__ __align__(16) uint8_t smem[];
  const int m = blockIdx.x, kv = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = q_heads / kv_heads;               // <= 8: rows g of the tiles; rows g + 8 are padding
  // the positions are an input of the step, not a product of the kernel before this one: they are read,
  // and the rotation table is formed (powf and a large-argument sincosf: about a microsecond), before
  // the wait for the kernel that produces the queries, keys and values
  bool in_cache;
  const int length = checked_position(positions[m], capacity, in_cache) + 1;
  __shared__ float cos_s[D / 2], sin_s[D / 2];
  if (fuse_rope && threadIdx.x < D / 2) {
    const float freq = powf(theta, -2.f * float(threadIdx.x) / float(D));
    sincosf(float(length - 1) * freq, &sin_s[threadIdx.x], &cos_s[threadIdx.x]);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int row = (q_heads + 2 * kv_heads) * D;
  const __half* keys = k_cache + (int64_t(m) * kv_heads + kv) * capacity * D;
  const __half* values = v_cache + (int64_t(m) * kv_heads + kv) * capacity * D;
  uint8_t* k_tile = smem + warp * 2 * kTileBytes;
  uint8_t* v_tile = k_tile + kTileBytes;
  if (fuse_rope) {
    // rotary embedding fused in: this CTA rotates the new key of its head and appends key and value
    // to the caches itself (nobody else reads that slot), and rotates its query heads in registers;
    // nothing is appended for a position outside the cache
    const int position = length - 1;
    if (in_cache && threadIdx.x < D / 2) {
      const float cosine = cos_s[threadIdx.x], sine = sin_s[threadIdx.x];   // written by this same thread
      const __half* k = qkv + int64_t(m) * row + int64_t(q_heads + kv) * D;
      const float a = __half2float(k[threadIdx.x]), b = __half2float(k[threadIdx.x + D / 2]);
      __half* slot = const_cast<__half*>(keys) + int64_t(position) * D;
      slot[threadIdx.x] = __float2half_rn(a * cosine - b * sine);
      slot[threadIdx.x + D / 2] = __float2half_rn(b * cosine + a * sine);
    } else if (in_cache && threadIdx.x < D / 2 + D) {
      const int i = threadIdx.x - D / 2;
      const_cast<__half*>(values)[int64_t(position) * D + i] = qkv[int64_t(m) * row + int64_t(q_heads + kv_heads + kv) * D + i];
    }
    // the appended row is read back by this CTA only: the barrier orders the stores for its own threads
    __syncthreads();
  }

  // Q fragments of this group: a[ks] = rows (g, g+8) x dims 16ks + (2t, 2t+1, 2t+8, 2t+9)
  uint32_t qa[8][4];
  {
    const __half* q = qkv + int64_t(m) * row + int64_t(kv * G + g) * D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(q + 16 * ks + 2 * t) : 0u;
      qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(q + 16 * ks + 8 + 2 * t) : 0u;
      qa[ks][1] = 0u;
      qa[ks][3] = 0u;
    }
  }
  if (fuse_rope) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int part = 0; part < 4; part += 2) {   // registers 0 and 2 of the fragment: dims 16ks + 2t and 16ks + 8 + 2t
        const int d = 16 * ks + (part ? 8 : 0) + 2 * t;
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks][part]));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&qa[ks + 4][part]));
        const float c0 = cos_s[d], s0 = sin_s[d], c1 = cos_s[d + 1], s1 = sin_s[d + 1];
        qa[ks][part] = pack_half2(lo.x * c0 - hi.x * s0, lo.y * c1 - hi.y * s1);
        qa[ks + 4][part] = pack_half2(hi.x * c0 + lo.x * s0, hi.y * c1 + lo.y * s1);
      }
  }
  float o[16][2];   // row g x dims 8jn + (2t, 2t+1)
#pragma unroll
  for (int jn = 0; jn < 16; ++jn) o[jn][0] = o[jn][1] = 0.f;
  float row_max = -INFINITY, row_sum = 0.f;   // of row g, over this lane's columns (sum) / the quad (max)

  const int tiles = (length + 15) / 16;
  for (int tile = warp; tile < tiles; tile += kGroupWarps) {
    const int p0 = tile * 16;
    // stage K and V rows p0 .. p0+15: 16 rows x 256 B each = 2 x 256 vectors of 16 B, 8 per lane each
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int vector = i * 32 + lane, r = vector >> 4, c = vector & 15;
      const int p = min(p0 + r, length - 1);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(shared_address(k_tile + r * kPitch + c * 16)),
                   "l"(keys + int64_t(p) * D + c * 8) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(shared_address(v_tile + r * kPitch + c * 16)),
                   "l"(values + int64_t(p) * D + c * 8) : "memory");
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncwarp();
    // S[16 heads][16 positions]: two n-tiles of 8 positions
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      // matrices: (pos 0-7, k 16ks..+7), (pos 0-7, k +8..+15), (pos 8-15, k ..+7), (pos 8-15, k +8..)
      uint32_t b[4];
      const int mat = lane >> 3, r = (lane & 7) + (mat >> 1) * 8, c = 16 * ks + (mat & 1) * 8;
      ldmatrix_x4(b, shared_address(k_tile + r * kPitch + c * 2));
      mma16816(s[0], qa[ks], b[0], b[1]);
      mma16816(s[1], qa[ks], b[2], b[3]);
    }
    // running softmax of row g (rows g + 8 are padding)
    float tile_max = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int p = p0 + nt * 8 + 2 * t + e;
        s[nt][e] = p < length ? s[nt][e] * scale : -INFINITY;
        tile_max = fmaxf(tile_max, s[nt][e]);
      }
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
    tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
    const float new_max = fmaxf(row_max, tile_max);
    const float correction = __expf(row_max - new_max);   // 0 on the first tile (row_max = -inf)
    row_max = new_max;
    float p_[2][2];
    float partial = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p_[nt][e] = __expf(s[nt][e] - new_max);
        partial += p_[nt][e];
      }
    row_sum = row_sum * correction + partial;
#pragma unroll
    for (int jn = 0; jn < 16; ++jn) { o[jn][0] *= correction; o[jn][1] *= correction; }
    // P as the A operand of the second product: k = positions
    uint32_t pa[4] = {pack_half2(p_[0][0], p_[0][1]), 0u, pack_half2(p_[1][0], p_[1][1]), 0u};
#pragma unroll
    for (int pair = 0; pair < 8; ++pair) {
      // matrices (transposed on load): (pos 0-7, dims 16pair..+7), (pos 8-15, same dims), (pos 0-7, dims +8..), (pos 8-15, dims +8..)
      uint32_t b[4];
      const int mat = lane >> 3, r = (lane & 7) + (mat & 1) * 8, c = 16 * pair + (mat >> 1) * 8;
      ldmatrix_x4_trans(b, shared_address(v_tile + r * kPitch + c * 2));
      float d0[4] = {o[2 * pair][0], o[2 * pair][1], 0.f, 0.f}, d1[4] = {o[2 * pair + 1][0], o[2 * pair + 1][1], 0.f, 0.f};
      mma16816(d0, pa, b[0], b[1]);
      mma16816(d1, pa, b[2], b[3]);
      o[2 * pair][0] = d0[0]; o[2 * pair][1] = d0[1];
      o[2 * pair + 1][0] = d1[0]; o[2 * pair + 1][1] = d1[1];
    }
  }
  row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 1);
  row_sum += __shfl_xor_sync(0xffffffffu, row_sum, 2);

  // meet: [warp][8 heads] max and sum, [warp][8 heads][128] outputs (the staging area is free now)
  __syncthreads();
  float* max_s = reinterpret_cast<float*>(smem);            // [kGroupWarps][8]
  float* sum_s = max_s + kGroupWarps * 8;                         // [kGroupWarps][8]
  float* out_s = sum_s + kGroupWarps * 8;                         // [kGroupWarps][8][D]
  if (t == 0) { max_s[warp * 8 + g] = row_max; sum_s[warp * 8 + g] = row_sum; }
#pragma unroll
  for (int jn = 0; jn < 16; ++jn)
    *reinterpret_cast<float2*>(out_s + (warp * 8 + g) * D + 8 * jn + 2 * t) = make_float2(o[jn][0], o[jn][1]);
  __syncthreads();
  for (int index = threadIdx.x; index < G * D; index += kGroupThreads) {
    const int head = index / D, dim = index - head * D;
    float top = -INFINITY;
    for (int w = 0; w < kGroupWarps; ++w) top = fmaxf(top, max_s[w * 8 + head]);
    float total = 0.f, value = 0.f;
    for (int w = 0; w < kGroupWarps; ++w) {
      const float weight = __expf(max_s[w * 8 + head] - top);   // 0 for warps that saw no position
      total += sum_s[w * 8 + head] * weight;
      value += out_s[(w * 8 + head) * D + dim] * weight;
    }
    out[(int64_t(m) * q_heads + kv * G + head) * D + dim] = __float2half_rn(value / total);
  }
}

// out[m, i] = silu(gate_up[m, i]) * gate_up[m, I + i]
__global__ void silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ out, int64_t rows, int I) {
  // programmatic dependent launch: let the next kernel in the stream become resident now (a matvec
  // starts streaming its weights), then wait for everything this kernel reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int64_t index = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 2;
  if (index >= rows * I) return;
  const int64_t m = index / I, i = index - m * I;
  const float2 g = __half22float2(*reinterpret_cast<const __half2*>(gate_up + m * 2 * I + i));
  const float2 u = __half22float2(*reinterpret_cast<const __half2*>(gate_up + m * 2 * I + I + i));
  const float a = g.x / (1.f + __expf(-g.x)), b = g.y / (1.f + __expf(-g.y));
  // the activation is rounded to fp16 before the product, as separate fp16 module ops would do
  const float2 act = __half22float2(__floats2half2_rn(a, b));
  *reinterpret_cast<__half2*>(out + m * I + i) = __floats2half2_rn(act.x * u.x, act.y * u.y);
}

// Launch with the programmatic-stream-serialization attribute: the kernel may become resident while
// its predecessor drains; it executes griddepcontrol.wait before it touches memory.
template <typename... Params, typename... Args>
cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, void* stream, Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
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

extern "C" int mkb_add_rmsnorm(void* residual, const void* delta, const void* weight, void* normed, int M, int H,
                               float eps, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 0 && H > 0 && H % 2 == 0, MKB_E_ARGUMENT, "add_rmsnorm: bad shape");
  MKB_REQUIRE(H * 4 <= 160 * 1024, MKB_E_UNSUPPORTED, "add_rmsnorm: hidden size %d too large", H);
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(residual && weight && normed, MKB_E_ARGUMENT, "add_rmsnorm: null pointer");
  const bool aligned = ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) |
                         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(normed)) & 15) == 0;
  cudaError_t launched;
  if (aligned && H % 8 == 0 && H <= kNormThreads * kNormPieces * 8) {
    launched = launch_dependent(add_rmsnorm_kernel, dim3(M), dim3(kNormThreads), 0, stream,
                                static_cast<__half*>(residual), static_cast<const __half*>(delta),
                                static_cast<const __half*>(weight), static_cast<__half*>(normed), H, eps);
  } else {
    const size_t smem = size_t(H) * 4;
    static bool opted = false;
    if (smem > 48 * 1024 && !opted) {
      cudaFuncSetAttribute(add_rmsnorm_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      opted = true;
    }
    launched = launch_dependent(add_rmsnorm_generic_kernel, dim3(M), dim3(256), smem, stream,
                                static_cast<__half*>(residual), static_cast<const __half*>(delta),
                                static_cast<const __half*>(weight), static_cast<__half*>(normed), H, eps);
  }
  if (launched != cudaSuccess) return cuda_fail(launched, "add_rmsnorm launch");
  return MKB_OK;
}

extern "C" int mkb_rope_append(void* qkv, const int* positions, void* k_cache, void* v_cache, int M, int q_heads,
                               int kv_heads, int head_dim, int capacity, float theta, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 0 && q_heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && capacity > 0,
              MKB_E_ARGUMENT, "rope_append: bad shape");
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(qkv && positions && k_cache && v_cache, MKB_E_ARGUMENT, "rope_append: null pointer");
  const cudaError_t launched = launch_dependent(
      rope_append_kernel, dim3(M, q_heads + 2 * kv_heads), dim3(64), 0, stream, static_cast<__half*>(qkv), positions,
      static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), q_heads, kv_heads, head_dim, capacity, theta);
  if (launched != cudaSuccess) return cuda_fail(launched, "rope_append launch");
  return MKB_OK;
}

extern "C" int mkb_attention_decode(const void* qkv, const int* positions, const void* k_cache, const void* v_cache,
                                    void* out, int M, int q_heads, int kv_heads, int head_dim, int capacity,
                                    float scale, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(head_dim == 128, MKB_E_UNSUPPORTED, "attention_decode: head_dim %d (128 supported)", head_dim);
  MKB_REQUIRE(M >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && capacity > 0, MKB_E_ARGUMENT,
              "attention_decode: bad shape");
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(qkv && positions && k_cache && v_cache && out, MKB_E_ARGUMENT, "attention_decode: null pointer");
  MKB_REQUIRE(capacity <= 40960, MKB_E_UNSUPPORTED, "attention_decode: capacity %d exceeds 40960 positions", capacity);
  if (q_heads / kv_heads <= 8) {
    // grouped heads: one CTA per (sequence, key-value head), every cached row read once
    const size_t group_smem = size_t(kGroupWarps) * 2 * kTileBytes;   // the meeting area (64.5 KB) fits inside
    static bool group_opted = false;
    if (!group_opted) {
      cudaFuncSetAttribute(attention_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(group_smem));
      group_opted = true;
    }
    const cudaError_t launched = launch_dependent(
        attention_group_kernel, dim3(M, kv_heads), dim3(kGroupThreads), group_smem, stream,
        static_cast<const __half*>(qkv), positions, static_cast<const __half*>(k_cache),
        static_cast<const __half*>(v_cache), static_cast<__half*>(out), q_heads, kv_heads, capacity, scale, 0.f, 0);
    if (launched != cudaSuccess) return cuda_fail(launched, "attention_decode launch");
    return MKB_OK;
  }
  const size_t smem = size_t(capacity) * 4;
  static bool opted = false;
  if (smem > 40 * 1024 && !opted) {
    cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024);
    opted = true;
  }
  const cudaError_t launched = launch_dependent(
      attention_decode_kernel, dim3(M, q_heads), dim3(kAttentionThreads), smem, stream, static_cast<const __half*>(qkv), positions,
      static_cast<const __half*>(k_cache), static_cast<const __half*>(v_cache), static_cast<__half*>(out), q_heads,
      kv_heads, capacity, scale);
  if (launched != cudaSuccess) return cuda_fail(launched, "attention_decode launch");
  return MKB_OK;
}

extern "C" int mkb_rope_attention_decode(const void* qkv, const int* positions, void* k_cache, void* v_cache, void* out,
                                         int M, int q_heads, int kv_heads, int head_dim, int capacity, float theta,
                                         float scale, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(head_dim == 128, MKB_E_UNSUPPORTED, "rope_attention_decode: head_dim %d (128 supported)", head_dim);
  MKB_REQUIRE(M >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && capacity > 0, MKB_E_ARGUMENT,
              "rope_attention_decode: bad shape");
  MKB_REQUIRE(q_heads / kv_heads <= 8, MKB_E_UNSUPPORTED,
              "rope_attention_decode: %d query heads per key-value head (at most 8)", q_heads / kv_heads);
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(qkv && positions && k_cache && v_cache && out, MKB_E_ARGUMENT, "rope_attention_decode: null pointer");
  const size_t group_smem = size_t(kGroupWarps) * 2 * kTileBytes;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(attention_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(group_smem));
    opted = true;
  }
  const cudaError_t launched = launch_dependent(
      attention_group_kernel, dim3(M, kv_heads), dim3(kGroupThreads), group_smem, stream,
      static_cast<const __half*>(qkv), positions, static_cast<const __half*>(k_cache),
      static_cast<const __half*>(v_cache), static_cast<__half*>(out), q_heads, kv_heads, capacity, scale, theta, 1);
  if (launched != cudaSuccess) return cuda_fail(launched, "rope_attention_decode launch");
  return MKB_OK;
}

namespace mkb {
namespace {
// best[m] = (max over i of logits[m, i], smallest such i + offset), one CTA of 1024 threads per row.
// The pair is packed so that an integer maximum orders it: the fp16 value mapped to a sortable key in
// the high word, the complement of the index in the low word (a tie keeps the smallest index).
__global__ void __launch_bounds__(1024) argmax_kernel(const __half* __restrict__ logits, int64_t width, int64_t row_stride,
                                                      int64_t offset, unsigned long long* __restrict__ best) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __shared__ unsigned long long part_s[32];
  const __half* row = logits + int64_t(blockIdx.x) * row_stride;
  unsigned long long top = 0;
  for (int64_t i = threadIdx.x; i < width; i += blockDim.x) {
    const unsigned short bits = __half_as_ushort(row[i]);
    // monotone map of fp16 to unsigned: flip all bits of negatives, the sign bit of the others (NaN ranks lowest)
    unsigned int key = (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
    if ((bits & 0x7fffu) > 0x7c00u) key = 0;
    const unsigned long long candidate = (static_cast<unsigned long long>(key) << 32) | (0xffffffffu - static_cast<unsigned int>(i + offset));
    top = candidate > top ? candidate : top;
  }
#pragma unroll
  for (int step = 16; step; step >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, top, step);
    top = other > top ? other : top;
  }
  if ((threadIdx.x & 31) == 0) part_s[threadIdx.x >> 5] = top;
  __syncthreads();
  if (threadIdx.x < 32) {
    top = part_s[threadIdx.x];
#pragma unroll
    for (int step = 16; step; step >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, top, step);
      top = other > top ? other : top;
    }
    if (threadIdx.x == 0) best[blockIdx.x] = top;
  }
}
}  // namespace
}  // namespace mkb

extern "C" int mkb_argmax(const void* logits, void* best, int M, int64_t width, int64_t row_stride, int64_t offset,
                          void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 0 && width >= 1 && row_stride >= width && offset >= 0 && offset + width <= 0xffffffffLL, MKB_E_ARGUMENT,
              "argmax: bad shape");
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(logits && best, MKB_E_ARGUMENT, "argmax: null pointer");
  const cudaError_t launched = launch_dependent(argmax_kernel, dim3(M), dim3(1024), 0, stream,
                                                static_cast<const __half*>(logits), width, row_stride, offset,
                                                static_cast<unsigned long long*>(best));
  if (launched != cudaSuccess) return cuda_fail(launched, "argmax launch");
  return MKB_OK;
}

extern "C" int mkb_decode_status(int* status) {
  using namespace mkb;
  MKB_REQUIRE(status != nullptr, MKB_E_ARGUMENT, "decode_status: null pointer");
  unsigned int value = 0, zero = 0;
  cudaError_t done = cudaMemcpyFromSymbol(&value, g_decode_status, sizeof(value));
  if (done == cudaSuccess && value != 0) done = cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(zero));
  if (done != cudaSuccess) return cuda_fail(done, "decode_status");
  *status = int(value);
  return MKB_OK;
}

extern "C" int mkb_silu_mul(const void* gate_up, void* out, int M, int I, void* stream) {
  using namespace mkb;
  MKB_REQUIRE(M >= 0 && I > 0 && I % 2 == 0, MKB_E_ARGUMENT, "silu_mul: bad shape");
  if (M == 0) return MKB_OK;
  MKB_REQUIRE(gate_up && out, MKB_E_ARGUMENT, "silu_mul: null pointer");
  const int64_t pairs = int64_t(M) * I / 2;
  const cudaError_t launched = launch_dependent(silu_mul_kernel, dim3(unsigned((pairs + 255) / 256)), dim3(256), 0,
                                                stream, static_cast<const __half*>(gate_up), static_cast<__half*>(out),
                                                int64_t(M), I);
  if (launched != cudaSuccess) return cuda_fail(launched, "silu_mul launch");
  return MKB_OK;
}
