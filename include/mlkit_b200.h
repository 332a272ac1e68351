/*
 * C ABI of libmlkit_b200: sm_100a kernels for mlkit's packed-inference path.
 *
 * Every pointer is a DEVICE pointer owned by the caller unless a comment says
 * otherwise.  Nothing here allocates device memory.  Every entry point queues
 * its work on `stream` (a cudaStream_t passed as void*) and returns without
 * synchronising.  Return value: 0 on success, a negative MKB_E_* code on a
 * rejected call (nothing was launched); mkb_last_error() then describes the
 * reason for the calling thread.
 *
 * Citations name files of the reference project (mlkit) whose interface or
 * arithmetic an entry point stands in for.
 */
#ifndef MLKIT_B200_H
#define MLKIT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of activations, scales/offsets and dense outputs */
enum { MKB_F16 = 0, MKB_BF16 = 1, MKB_F32 = 2 };

/* error codes */
enum {
  MKB_OK = 0,
  MKB_E_ARGUMENT = -1,    /* null pointer, non-positive size, unknown dtype */
  MKB_E_UNSUPPORTED = -2, /* shape / layout outside what the kernels cover */
  MKB_E_ALIGNMENT = -3,   /* pointer or stride alignment the fast path needs */
  MKB_E_CUDA = -4         /* the CUDA runtime refused the launch */
};

/* kernel choice for mkb_gemv_ex */
enum {
  MKB_GEMV_AUTO = 0,   /* fastest kernel that covers the arguments */
  MKB_GEMV_SCALAR = 1, /* word-at-a-time fp32 kernel: every layout the reference's fused kernel accepts */
  MKB_GEMV_TILED = 2,  /* 16-row x 128-code register-tiled kernel (fp16 activations) */
  MKB_GEMV_TMEM = 3,   /* tcgen05 kernel: weights through tensor memory (INT4 integer grid, fp16, needs a workspace) */
  MKB_GEMV_GATED = 0x100, /* flag, OR-ed into a choice (mkb_gemv_ex, mkb_gemv_ws): x is [M, 2K] = gate | up of a
                             SwiGLU MLP and the kernel forms silu(gate) * up while it loads the activations
                             (rounded to fp16 after the activation and after the product, as separate fp16
                             operators would); tiled and streaming kernels (AUTO takes one of them).  In the
                             streaming kernel every warp forms the activation of its own share of K once, so
                             the cost is M * K activations per CTA; it replaces a launch.  The reference leaves
                             this product to the model code between two PackedLinear calls */
  MKB_GEMV_BULK = 4,   /* TMA-fed kernel: whole 16-row units by cp.async.bulk.tensor into a shared-memory ring
                          (INT4 integer grid, fp16, K % 256 == 0; needs the workspace when K is split) */
  MKB_GEMV_STREAM = 5  /* streaming kernel: activations in registers, weights through per-warp cp.async rings
                          (integer grid, fp16, group 128, K % 128 == 0); what AUTO takes when it applies */
};

int mkb_version(void);
const char* mkb_last_error(void);

/*
 * Packed matvec for one to eight activation rows:
 *   y[m,n] = sum_k x[m,k] * (lut[code[n,k]] * scales[n,k/group] (+ zeros[n,k/group])) (+ bias[n])
 * accumulated in fp32 and stored in the activation dtype.
 *
 * Replaces the reference's Triton launch `packed_matrix_vector`
 * (src/mlkit/kernels/packed_linear.py:107-173) as issued by
 * `PackedLinear._launch_directly` (src/mlkit/inference/packed_linear.py:181-245)
 * and `matrix_vector` (src/mlkit/kernels/packed_linear.py:181-226).
 *
 * packed: the little-endian code stream of src/mlkit/quantization/operations/bit_packing.py:13-29;
 *         row n starts at packed + n*packed_row_stride and holds K*bits/8 bytes.
 * scales/zeros/bias: element type scale_dtype / scale_dtype / x_dtype; zeros and bias may be null.
 * lut: fp32 code values, lut_len <= 2^bits entries.
 * integer_grid / grid_minimum: the caller's promise that lut[c] == grid_minimum + c exactly for
 *         every code, with an integer grid_minimum (the counterpart of the reference's
 *         uniform_grid / grid_minimum / grid_step launch constants,
 *         src/mlkit/inference/packed_linear.py:90-97); pass 0 when unsure, the table is used then.
 * Constraints (src/mlkit/kernels/packed_linear.py:63-79): 1 <= bits <= 8, K and group are
 * multiples of the codes in one packing word, 1 <= M <= 8.
 */
int mkb_gemv(const void* x, const uint8_t* packed, const void* scales, const float* lut,
             const void* zeros, const void* bias, void* y,
             int M, int N, int K, int group, int bits, int lut_len,
             int x_dtype, int scale_dtype,
             int64_t packed_row_stride, int64_t scale_row_stride,
             int integer_grid, float grid_minimum, void* stream);

/* Same, with an explicit kernel choice (MKB_GEMV_*); returns MKB_E_UNSUPPORTED when the chosen
 * kernel does not cover the arguments. */
int mkb_gemv_ex(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                const void* zeros, const void* bias, void* y,
                int M, int N, int K, int group, int bits, int lut_len,
                int x_dtype, int scale_dtype,
                int64_t packed_row_stride, int64_t scale_row_stride,
                int integer_grid, float grid_minimum, int kernel, void* stream);

/*
 * The matvec with a caller-provided workspace, which lets MKB_GEMV_AUTO choose the kernels that
 * split K over CTAs and meet through the workspace (MKB_GEMV_BULK, MKB_GEMV_TMEM).  Same contract as
 * mkb_gemv_ex.
 * workspace: device memory of at least mkb_gemv_workspace_bytes(M, N, K, bits) bytes, 16-byte aligned,
 *         ZERO-FILLED ONCE before its first use; the kernel leaves it ready for the next call.  Calls
 *         that may overlap on the GPU (different streams) need workspaces of their own.  A null or
 *         short workspace simply rules those kernels out for the shapes that need it.
 * mkb_gemv_workspace_bytes returns 0 when no workspace is of use for the shape.
 * No counterpart in the reference: its Triton kernel gives every program whole rows
 * (src/mlkit/kernels/packed_linear.py:131-167).
 */
int64_t mkb_gemv_workspace_bytes(int M, int N, int K, int bits);
/* Reads the workspace's status word (synchronises with the device): 0, or non-zero when a bounded
 * wait inside a kernel that used this workspace expired (the results of that call are not valid). */
int mkb_gemv_workspace_status(const void* workspace, int64_t workspace_bytes, int* status);
int mkb_gemv_ws(const void* x, const uint8_t* packed, const void* scales, const float* lut,
                const void* zeros, const void* bias, void* y,
                int M, int N, int K, int group, int bits, int lut_len,
                int x_dtype, int scale_dtype,
                int64_t packed_row_stride, int64_t scale_row_stride,
                int integer_grid, float grid_minimum, int kernel,
                void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The INT4 matvec for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  Same arithmetic and kernel as mkb_gemv_ws with MKB_GEMV_TMEM (fp16 activations and
 * scales, integer grid lut[c] = grid_minimum + c with 16 levels, no offsets, K a multiple of 512,
 * power-of-two group >= 128), but the split-K scratch is a fixed array inside the library image
 * instead of a caller workspace: mkb_gemv_static_scratch_bytes() bytes (8 MiB), held by every GPU
 * that loads the library until the process exits.  A shape that needs more scratch
 * (65536 + ceil(N/128) * (K/512) * M * 512 bytes) is rejected with MKB_E_UNSUPPORTED.
 *   - The call itself calls no allocator.  The first call on each device looks up the array's
 *     device address (cudaGetSymbolAddress): make that first call with the device current and
 *     before any stream capture begins.
 *   - All calls on a device share the one array.  Calls that may overlap on the GPU (different
 *     streams, or two threads) race on it; order them on one stream.
 *   - The 8 MiB become resident when the first call loads the library's tensor-memory kernel module
 *     (CUDA loads modules lazily); that call also sets the kernel's shared-memory attribute and
 *     queries its occupancy.  A host that has committed all device memory must make it before.
 *   - mkb_gemv_static_status reads, and clears, the status word of the built-in scratch: non-zero
 *     when a bounded wait inside one of the calls since the last reading expired (the results of that
 *     call are not valid).  It synchronises with the device: call it outside stream captures.  It has
 *     no counterpart in the reference either.
 */
int64_t mkb_gemv_static_scratch_bytes(void);
int mkb_gemv_static(const void* x, const uint8_t* packed, const void* scales, const void* bias, void* y,
                    int M, int N, int K, int group,
                    int64_t packed_row_stride, int64_t scale_row_stride,
                    float grid_minimum, void* stream);
int mkb_gemv_static_status(int* status);

/*
 * The matvec with the randomised Hadamard rotation of its input fused into the activation load:
 *   y = mkb_gemv(S(x * signs), ...),  S the normalised (normalize != 0) Walsh-Hadamard transform of width K.
 * Replaces the pair the reference runs for a rotated layer: the pre-hook's transform
 * (src/mlkit/conversion/model_transforms.py:189-196 calling src/mlkit/kernels/hadamard.py:21-136) as
 * launches of its own, then the packed matvec.  Every CTA transforms the (at most 64 KB of fp32) activations
 * in shared memory with the butterflies of mkb_hadamard and rounds them to fp16 as that call stores them, so
 * the result equals mkb_hadamard followed by mkb_gemv bit for bit; no rotated activation is written to
 * or read from global memory.
 * signs: int8 [K] of +1 / -1, 16-byte aligned, or null for the plain transform.
 * Covers what the streaming matvec covers (fp16 activations and scales; INT2/4/8 on the integer grid with
 * groups of 128, 3- and 4-bit tables with groups of 64 or 128) when K is a power of two >= 512 and
 * M * K * 4 <= 65536 (K = 4096: M <= 4); anything else returns MKB_E_UNSUPPORTED and the caller runs
 * mkb_hadamard, then mkb_gemv.  Widths with an odd factor (14336 = 28 * 512) are not covered.
 */
int mkb_gemv_hadamard(const void* x, const int8_t* signs, const uint8_t* packed, const void* scales,
                      const float* lut, const void* bias, void* y,
                      int M, int N, int K, int group, int bits, int lut_len,
                      int x_dtype, int scale_dtype,
                      int64_t packed_row_stride, int64_t scale_row_stride,
                      int integer_grid, float grid_minimum, int normalize, void* stream);

/*
 * Fused dequantise + GEMM for more activation rows than the matvec takes:
 *   y[m,n] = sum_k x[m,k] * fp16(lut[code[n,k]] * scale[n, k / 128]) (+ bias[n]),  1 <= M <= 128.
 * Replaces the dense route the reference takes above eight rows, which reconstructs the whole weight
 * in global memory and hands it to a library GEMM (PackedLinear.forward,
 * src/mlkit/inference/packed_linear.py:153-154 with the `weight` property at :110-130).  The weights
 * are rounded to fp16 exactly as that reconstruction rounds them, products are accumulated in fp32
 * on the tensor cores (tcgen05.mma, weights through tensor memory), the result is rounded once.
 * Covers symmetric INT4 on the integer grid -8..7 (bits = 4, lut_len = 16, integer_grid = 1,
 * grid_minimum = -8, zeros = null), fp16 activations and scales, group = 128, K a multiple of 128,
 * x and packed 16-byte aligned; anything else returns MKB_E_UNSUPPORTED and the caller keeps the
 * dense route.  Argument meaning as for mkb_gemv_ws.
 * workspace: device memory of at least mkb_gemm_workspace_bytes(M, N, K) bytes, 16-byte aligned,
 *         ZERO-FILLED ONCE before its first use; the kernel leaves it ready for the next call.  Calls
 *         that may overlap on the GPU need workspaces of their own.
 * mkb_gemm_status reads the workspace's status word (synchronises with the device): non-zero when
 * a bounded wait inside a call that used this workspace expired (its results are not valid).
 */
int64_t mkb_gemm_workspace_bytes(int M, int N, int K);
int mkb_gemm(const void* x, const uint8_t* packed, const void* scales, const float* lut,
             const void* zeros, const void* bias, void* y,
             int M, int N, int K, int group, int bits, int lut_len,
             int x_dtype, int scale_dtype,
             int64_t packed_row_stride, int64_t scale_row_stride,
             int integer_grid, float grid_minimum,
             void* workspace, int64_t workspace_bytes, void* stream);
int mkb_gemm_status(const void* workspace, int* status);

/*
 * Unpack and dequantise a packed weight:
 *   codes_out[n,k] = code (uint8), w_out[n,k] = lut[code] * scale (+ zero) rounded once to out_dtype.
 * Either output may be null.  The multiply and the add are separate IEEE binary32 operations,
 * so the result equals the reference reconstruction bit for bit.
 *
 * Replaces `decode` / `decode_rows` (src/mlkit/kernels/packed_linear.py:229-313), the tensor route
 * `unpack` + `decode_scaled` that `PackedLinear.weight` takes for layouts without whole words
 * (src/mlkit/inference/packed_linear.py:110-143; src/mlkit/quantization/codecs/scaled.py:53-61) and
 * `unpack` itself (src/mlkit/quantization/operations/bit_packing.py:80-99).
 *
 * The stream is read as one flat run of N*K codes (rows need not start on a byte); scales and zeros
 * are [N, ceil(K/group)] with row stride scale_row_stride.  bits in 1..8.
 */
int mkb_dequant(const uint8_t* packed, const void* scales, const float* lut, const void* zeros,
                void* w_out, uint8_t* codes_out,
                int64_t N, int64_t K, int group, int bits, int lut_len,
                int scale_dtype, int out_dtype, int64_t scale_row_stride, void* stream);

/*
 * Decode selected rows of a packed weight (embedding lookup through a packed output head):
 *   out[i,:] = dequantised row rows[i], i < count, in out_dtype.
 * Replaces `PackedEmbedding.forward` (src/mlkit/inference/packed_linear.py:274-287).
 * Rows must hold whole bytes (K*bits % 8 == 0).
 */
int mkb_dequant_rows(const uint8_t* packed, const void* scales, const float* lut, const void* zeros,
                     const int64_t* rows, void* out,
                     int64_t count, int64_t N, int64_t K, int group, int bits, int lut_len,
                     int scale_dtype, int out_dtype, int64_t scale_row_stride, void* stream);

/*
 * Round-to-nearest encoding with one fp16 scale per row group (absolute maximum, symmetric), and
 * packing, in one launch:
 *   scale[n,j] = fp16(max(max_k |w[n,k]| over group j, 1e-12) * reciprocal)   (clamped to [2^-24, 65504])
 *   code[n,k]  = round_half_even(w / scale) clamped to [grid_low, grid_high], minus grid_low    (integer_grid)
 *              = index of the nearest level, a tie taking the lower one                        (otherwise)
 *   packed     = the little-endian bit stream of the codes (bit_packing.py:13-77)
 * `reciprocal` is fp32(1) / fp32(max |level|); the division w / scale is IEEE binary32.  codes_out
 * (uint8 [N,K]) may be null.  A trailing partial group gets its own scale.  group * bits and K * bits
 * must be multiples of 8 (groups and rows end on bytes).  weight_dtype is MKB_F16/BF16/F32.
 *
 * Replaces the fused encode the reference runs on CUDA (src/mlkit/kernels/scalar_encode.py:65-146)
 * and the tensor route it must equal (src/mlkit/quantization/formats/grouped_scaling.py:288-392,
 * scale_storage.py:11-26), followed by `pack` (src/mlkit/quantization/operations/bit_packing.py:13-77).
 */
int mkb_rtn_encode(const void* weight, const float* levels, uint8_t* packed, void* scales, uint8_t* codes_out,
                   int64_t N, int K, int group, int bits, int level_count, int integer_grid,
                   float grid_low, float grid_high, float reciprocal, int weight_dtype, void* stream);

/*
 * Structured orthogonal transform of activation rows, fused:
 *   y[m,:] = (B kron H_pow2)(x[m,:] * signs), W = factor * pow2,
 * H the Sylvester-ordered Walsh-Hadamard butterflies in ascending stride in fp32, scaled by
 * fp32(1)/fp32(sqrt(pow2)); B (row-major [factor,factor] fp32, may be null when factor == 1) mixes
 * the `factor` blocks:  y[f',p] = sum_f B[f',f] * h[f,p].  With inverse != 0 the transposed
 * basis is applied and the signs multiply the result instead of the input.
 * x and y have element type dtype and may alias; signs (int8 +1/-1) may be null.
 *
 * Replaces `hadamard_pass`/`transform` (src/mlkit/kernels/hadamard.py:21-136) and the tensor
 * route around it, `structured_transform` / `randomized_transform`
 * (src/mlkit/quantization/operations/orthogonal_transforms.py:101-118), as invoked by the
 * rotation pre-hook (src/mlkit/conversion/model_transforms.py:189-196).
 * pow2 is a power of two; W*4 bytes (+ factor^2*4) must fit shared memory (W <= 49152).
 */
int mkb_hadamard(const void* x, const int8_t* signs, const float* basis, void* y,
                 int64_t M, int W, int factor, int pow2, int dtype, int inverse, int normalize,
                 void* stream);

/*
 * Operators between the packed matvecs of a Llama-style decode step (fp16 storage, fp32 arithmetic).
 * They have no counterpart in the reference, which leaves the decoder block to the `transformers`
 * modules and their compilation (src/mlkit/inference/optimization.py:86-99); here each is one launch so
 * that the tensor-parallel decode step of this library is a short, graph-capturable chain.
 *
 * mkb_add_rmsnorm: residual[m,:] += delta[m,:] (delta may be null), normed = rms_norm(residual) * weight.
 * mkb_rope_append: qkv[m] = [q_heads | kv_heads | kv_heads] x head_dim; rotates q and k in place
 *     (rotate-half pairing, angle positions[m] * theta^(-2i/head_dim)) and stores k, v at
 *     cache[m, kv_head, positions[m], :]; caches are [M, kv_heads, capacity, head_dim].
 * mkb_attention_decode: out[m, head, :] = softmax(q . K[0..positions[m]] * scale) V, grouped-query,
 *     head_dim 128.  With at most 8 query heads per key-value head it runs on the tensor cores, one
 *     CTA per (m, key-value head), the softmax weights rounded to fp16 for the second product.
 * mkb_silu_mul: out[m, i] = silu(gate_up[m, i]) * gate_up[m, I + i].
 */
int mkb_add_rmsnorm(void* residual, const void* delta, const void* weight, void* normed,
                    int M, int H, float eps, void* stream);
int mkb_rope_append(void* qkv, const int* positions, void* k_cache, void* v_cache,
                    int M, int q_heads, int kv_heads, int head_dim, int capacity, float theta, void* stream);
int mkb_attention_decode(const void* qkv, const int* positions, const void* k_cache, const void* v_cache,
                         void* out, int M, int q_heads, int kv_heads, int head_dim, int capacity,
                         float scale, void* stream);
/* mkb_rope_append and mkb_attention_decode in one launch, for at most 8 query heads per key-value
 * head and head_dim 128: every CTA rotates the new key of its key-value head, appends key and value
 * to the caches at positions[m], rotates its query heads in registers (qkv itself is left
 * unrotated) and attends over positions 0..positions[m].  `positions` is read before the kernel waits for
 * its predecessor in the stream (the rotation table is formed meanwhile), so it must not be written by the
 * kernel launched immediately before this call; the same holds for mkb_attention_decode. */
int mkb_rope_attention_decode(const void* qkv, const int* positions, void* k_cache, void* v_cache, void* out,
                              int M, int q_heads, int kv_heads, int head_dim, int capacity, float theta,
                              float scale, void* stream);
int mkb_silu_mul(const void* gate_up, void* out, int M, int I, void* stream);
/* Greedy pick over a shard of the vocabulary: best[m] (uint64) = key(max_i logits[m, i]) << 32 |
 * (0xffffffff - (argmax index + offset)), key a monotone map of the fp16 value to an unsigned word, so
 * that the unsigned maximum of the ranks' words is the global pick and, on a tie, the smallest token.
 * Ranks exchange these 8 bytes per sequence instead of their logits.  logits are fp16 [M, width] with
 * row stride row_stride.  No counterpart in the reference, which leaves sampling to `transformers`. */
int mkb_argmax(const void* logits, void* best, int M, int64_t width, int64_t row_stride, int64_t offset, void* stream);
/* positions[m] must lie in [0, capacity).  The kernels above never turn a position outside that range
 * into an address: they clamp it, leave the caches untouched and raise a device-wide status word.
 * mkb_decode_status reads and clears that word (non-zero: some launch since the last reading saw such
 * a position and its results are not valid).  It synchronises with the device: call it outside
 * stream captures. */
int mkb_decode_status(int* status);

/*
 * One-shot all-reduce over peer memory for the row-parallel linears (o, down) of the tensor-parallel
 * decode step, fused with the residual add and RMS norm that consume the sum.  No counterpart in the
 * reference (it has no multi-GPU path); it replaces the library all-reduce that a Megatron-style
 * sharding of src/mlkit/inference/packed_linear.py:145-179 would call after each row-parallel layer.
 *
 * Every rank allocates one exchange buffer (mkb_peer_alloc, mkb_peer_buffer_bytes(rows, H, world)
 * bytes, rows <= 8: a 2 KB header of counters and a status word, then 2 x world slots of rows x H / 2
 * packets of 8 bytes: two fp16 values and a 32-bit flag), exports it (64-byte handle), and opens the
 * buffers of all other ranks of the node.  A reduction of a partial [M, H] is ONE kernel,
 * mkb_peer_reduce_add_rmsnorm: CTA m writes row m of the partial, as packets whose flag is the number of
 * the reduction, into this rank's slot on every rank with plain stores over NVLink (data and flag in one
 * store: no fence, no second message), polls (bounded) the packets of all ranks in its own buffer, adds
 * them in rank order in fp32, rounds to
 * fp16, and then residual += sum, normed = rmsnorm(residual) * weight; `reduced`, when not null,
 * receives the sum.  All ranks must issue the same sequence of reductions.  `peers` is a DEVICE
 * array of `world` buffer pointers (entry `rank` is the rank's own buffer).  A wait that expires sets
 * a status word (mkb_peer_status), later waits are skipped, the kernels finish; nothing hangs.
 */
int64_t mkb_peer_buffer_bytes(int rows, int H, int world);
int mkb_peer_alloc(int64_t bytes, void** buffer);
int mkb_peer_free(void* buffer);
int mkb_peer_export(void* buffer, void* handle64);
int mkb_peer_open(const void* handle64, void** buffer);
int mkb_peer_close(void* buffer);
int mkb_peer_reduce_add_rmsnorm(const void* partial, void* const* peers, void* own, void* residual,
                                const void* weight, void* normed, void* reduced, int M, int H, int rows,
                                int world, int rank, float eps, void* stream);
int mkb_peer_status(const void* own, int* status);
/* Polls of one flag before a wait gives up (default 60 million, of the order of half a minute;
 * ranks are separate processes and may be seconds apart).  Synchronous; call it outside captures. */
int mkb_peer_set_poll_limit(void* own, int64_t polls);
/* CTAs that share one row of a reduction on this buffer: 0 (default) lets the call choose from the world size
 * and the rows (up to 4: one SM sustains only a few tens of GB/s of remote stores, so a launch aims at about four
 * pushing CTAs, more with eight ranks),
 * a power of two up to 8 fixes it.  Host-side state of the library, kept until mkb_peer_free. */
int mkb_peer_set_split(void* own, int split);

#ifdef __cplusplus
}
#endif
#endif /* MLKIT_B200_H */
