/*
 * texelator_b200 -- C ABI of the BC4 weight-linear operator for NVIDIA B200 (sm_100a).
 *
 * This is the drop-in boundary for the functions the reference binds with pybind11 in
 * texelator/cuda/extension.cpp:7-48 (implemented there by texelator/cuda/texelator_cuda.cu).
 * Plain pointers and sizes only: no torch types cross this interface.  Device pointers are raw
 * CUDA device addresses, `stream` is a cudaStream_t passed as void*.
 *
 * Every function returns TX_OK (0) or a negative TX_E* code; tx_last_error() returns the message
 * of the last failure on the calling thread (the reference raises TORCH_CHECK exceptions with the
 * same meaning; the Python wrapper turns a non-zero status into RuntimeError).
 *
 * Threading: like the reference, a handle is not safe for concurrent use from several host
 * threads, and setters are plain field writes.  All launches of one process on one device share
 * a per-device activation scratch (multi-token decode), so tx_linear calls on the same device must
 * be ordered on one stream (or otherwise serialised) with respect to each other.
 */
#ifndef TEXELATOR_B200_H
#define TEXELATOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TX_OK 0
#define TX_EINVAL (-1)       /* bad argument (shape, dtype, null handle, ...) */
#define TX_ECUDA (-2)        /* a CUDA runtime call failed */
#define TX_EUNSUPPORTED (-3) /* feature not available on this device/build */
#define TX_ESTATE (-4)       /* handle not in a state that allows the call */

/* activation / bias element types (the reference accepts fp16 or bf16: texelator_cuda.cu:1332-1335).  tx_linear
 * computes both; the entry points with no reference counterpart (fused, single-token, static-scratch) and the
 * TX_DECODE_ALU_EXACT / TX_DECODE_TEXTURE paths are bf16 only.  A handle's bias must have the activations'
 * type ("input and bias dtypes must match", texelator_cuda.cu:1449). */
#define TX_DTYPE_F16 0
#define TX_DTYPE_BF16 1

/* decode paths for tokens < prefill_threshold */
#define TX_DECODE_ALU_MMA 0   /* in-register palette interpolation feeding mma.sync (default) */
#define TX_DECODE_ALU_EXACT 1 /* per-weight bf16(pal*scale) with fp32 FMA, the reference's arithmetic */
#define TX_DECODE_TEXTURE 2   /* signed-BC4 texture object + tex2Dgather, if the device offers it */

/* palettes a payload can be encoded against */
#define TX_PALETTE_SOFTWARE 0 /* exact BC4-SNORM values rounded once to fp32 (default) */
#define TX_PALETTE_HARDWARE 1 /* what NVIDIA texture units return (the reference's published models) */

/* tx_dequant output selectors */
#define TX_DEQUANT_PALETTE_F32 0 /* unscaled palette value per weight, fp32 [M,K] */
#define TX_DEQUANT_SCALED_F32 1  /* pal * scale_m, fp32 [M,K] */
#define TX_DEQUANT_SCALED_BF16 2 /* bf16(pal * scale_m) [M,K] -- the matrix the operator multiplies by */

const char *tx_last_error(void);

/* Library / device facts: out[0]=ABI version, out[1]=compiled sm arch (100), out[2]=SM count of
 * `device`, out[3]=1 if signed-BC4 texture views can be created on it, else 0. */
int tx_runtime_info(int device, int64_t out[4]);

/* pack_encoded(blocks, scales, bias) -> handle: texelator_cuda.cu:1260-1327 (extension.cpp:28-29).
 * `blocks`: host, M * K/16 * 8 bytes, row-major BC4 blocks (encoder.py:105-117); `scales`: host,
 * M floats; `bias_dev`: optional device pointer to M elements of `bias_dtype` (copied).  K is
 * derived as 16 * nbytes / (8*M).  Copies are complete when the call returns.  `blocks` and
 * `scales` may also be device pointers (the copies use cudaMemcpyDefault), which lets a caller that
 * encodes on the GPU pack without a round trip through host memory. */
int tx_pack_encoded(const uint8_t *blocks, size_t nbytes, const float *scales, int M,
                    const void *bias_dev, int bias_dtype, int device, uint64_t *out_handle);

/* Tensor-parallel variant (no counterpart in the reference, which is single-GPU): packs rows
 * [row_begin,row_end) and 16-column blocks [kblock_begin,kblock_end) of a full M x K matrix.
 * `scales` and `bias_dev` are indexed with the full-matrix row numbers. */
int tx_pack_encoded_shard(const uint8_t *blocks, size_t nbytes, const float *scales, int M, int K,
                          int row_begin, int row_end, int kblock_begin, int kblock_end,
                          const void *bias_dev, int bias_dtype, int device, uint64_t *out_handle);

/* linear(handle, x) -> y: texelator_cuda.cu:1329-1469 (extension.cpp:30).  `x` is a contiguous
 * device [tokens, K] array, `y` a device [tokens, M] array the caller allocated (the reference
 * allocates with at::empty); both of `dtype`.  Asynchronous on `stream`.
 * TX_DTYPE_BF16: y = bf16(sum_k pal * scale_m * x + bias) (texelator_bc4_bf16_kernel, :141-199, rounds the weight
 * to bf16 first; this build does not, which is inside the operator's tolerance).  TX_DTYPE_F16: the fp16 twin
 * (texelator_bc4_kernel, :94-139, un-rounded weight, fp32 accumulation, one fp16 rounding; for tokens >=
 * prefill_threshold the reference goes through fp16(pal*scale) and cuBLAS, :996-1046): the same kernels, the
 * fp16 activations are the tensor-core operand as they are.
 * Token groups below the threshold read the matrix once for all rows (the reference launches one grid row per
 * token, :1438-1468); for groups and for short prompts on matrices with few rows K may be cut into ranges whose
 * fp32 sums a second kernel adds in a fixed order (results repeat bit for bit; they can differ in the last bit
 * from the same rows taken one at a time).  All calls on one device share one activation scratch and one
 * partial-sum scratch: order them on one stream. */
int tx_linear(uint64_t handle, const void *x, void *y, int tokens, int dtype, void *stream);

/* No counterpart in the reference.  The result of tx_linear for a small token group (1..32 tokens,
 * tokens * K <= 262144 with K rounded up to 128, one shared-memory pass; every CTA sums whole rows here, while
 * tx_linear may cut K into ranges, so the two can differ in the last bit of an output), but the fp16 activation
 * scratch of the multi-token decode kernel is a fixed array inside the library image instead of
 * memory from cudaMalloc, and the call allocates nothing on the device.  Meant for hosts that cannot
 * allocate when they need the linear (all memory owned by their own pool, a thread that must
 * not take the allocator lock).  Larger requests fail with TX_EINVAL.  The first
 * call on a device looks the array's address up (cudaGetSymbolAddress); make that call before any
 * stream capture.  Every call on a device uses the same array: calls that overlap on the GPU race. */
int tx_linear_static_scratch(uint64_t handle, const void *x, void *y, int tokens, int dtype, void *stream);

/* No counterpart in the reference (its decode loop leaves these steps to PyTorch kernels between the
 * linears, texelator/cli.py:189-219).  Decode linear with its neighbours fused into the same launch:
 *   norm_weight != NULL : r = bf16(x + delta) (delta may be NULL), a = bf16(rmsnorm(r, eps) * norm_weight)
 *                         feeds the linear; r is also stored to residual_out when that is non-NULL
 *                         (it must not overlap x, delta or y: one thread block stores it while the others
 *                         still read their copy of the row).  K <= 18432.
 *   swiglu != 0         : the handle's rows are (gate, up) pairs -- in every group of 16 rows, rows 0-7
 *                         are gate rows and rows 8-15 the matching up rows -- and
 *                         y[t, 8*g + i] = silu(lin[16*g + i]) * lin[16*g + 8 + i]; y is [tokens, M/2].
 * Rounding points are those of the separate steps (bf16 after the add, after the norm, after each
 * linear output, after the product).  At most 2 tokens with tokens * K <= 36864; TX_DECODE_ALU_MMA only. */
int tx_linear_fused(uint64_t handle, const void *x, const void *delta, const void *norm_weight, float eps, void *residual_out,
                    int swiglu, void *y, int tokens, int dtype, void *stream);

/* No counterpart in the reference.  One token through the single-token decode kernel with the two
 * extras a decode loop uses (the handle must be on TX_DECODE_ALU_MMA with the software palette and no
 * low-mode block; tx_linear_single_info tells):
 *   x / staged       the token as bf16 [K], or in the staged form tx_aux_add_rmsnorm_single wrote for this
 *                    K (exactly one of the two is non-NULL); results are bit-identical either way;
 *   y / y_partial    bf16 [M] (or [M/2] with swiglu, rows paired as in tx_linear_fused), or `splits` fp32
 *                    vectors y_partial[s * partial_stride + m]: row sums of the s-th of `splits` equal K
 *                    ranges, scale (and, in split 0, bias) applied, not rounded.  Their sum in split order
 *                    is the linear's output; tx_aux_add_rmsnorm_single consumes them.  K-split work items
 *                    spread matrices with few rows over all SMs.  `splits` must divide ceil(K/128).
 * The kernel hands the tensor cores the masked index fields themselves and applies the endpoints to
 * per-block sums, so it executes fewer instructions per weight than the general kernel, but staging a bf16
 * token costs it more: it pays off when the token arrives staged.
 * tx_linear_single_info: out[0] = 1 if the handle qualifies, out[1] = number of splits this library
 * would choose for it on this device, out[2] = bytes of the staged form of one token of this K. */
int tx_linear_single(uint64_t handle, const void *x, const void *staged, int swiglu, void *y, float *y_partial, int splits,
                     size_t partial_stride, void *stream);
int tx_linear_single_info(uint64_t handle, int64_t out[3]);

/* set_lookahead: texelator_cuda.cu:1471-1478.  k in {1,2,3,4,6,8}: 1 KiB weight requests each
 * warp keeps in flight (the reference: texture requests in flight). */
int tx_set_lookahead(uint64_t handle, int lookahead);
/* set_prefill: texelator_cuda.cu:1480-1488.  threshold >= 1; tile_rows >= 16 and % 16 == 0. */
int tx_set_prefill(uint64_t handle, int threshold, int tile_rows);
/* set_prefill_backend: texelator_cuda.cu:1490-1503.  0..4: streamed small-batch path in token
 * groups; 5..9: tensor-core tile candidates (rows x tokens per CTA: 128x256, 256x256, 128x128, 128x64,
 * 128x192; see tx_kernel_info). */
int tx_set_prefill_backend(uint64_t handle, int backend);
/* New: choose the decode path (TX_DECODE_*). TX_DECODE_TEXTURE fails with TX_EUNSUPPORTED when
 * BC4 texture views are unavailable, and with TX_ESTATE when the hardware palette differs from
 * the software palette (the reference's palette-hash gate, tuning.py:38-41). */
int tx_set_decode_path(uint64_t handle, int path);

/* handle_info: texelator_cuda.cu:1505-1512 -> [M, K, threshold, tile_rows, backend,
 * pipelined_supported, graphics_supported]; the last two report [decode_path, lookahead + 16*palette]
 * here (the reference's two flags describe kernels that do not exist in this build). */
int tx_handle_info(uint64_t handle, int64_t out[7]);

/* *_kernel_info(): texelator_cuda.cu:1514-1536, cutlass_texture_mainloop.cu:251-267 ->
 * [numRegs, staticSmem, localBytes, maxThreads, dynamicSmem, tileM, tileN, tileK, activeBlocks/SM]
 * for backend id 0 (decode GEMV) and 5..9 (prefill tile candidates). */
int tx_kernel_info(int backend, int64_t out[9]);

/* free: texelator_cuda.cu:1538.  The caller synchronises first (runtime.py:268-271). */
int tx_free(uint64_t handle);

/* palette_probe(): texelator_cuda.cu:1540-1595.  Measures the texture unit's BC4 palette:
 * out_host[(e1+127)*255 + (e0+127)][selector], 65025*8 floats.  TX_EUNSUPPORTED when the device
 * cannot create signed-BC4 texture views. */
int tx_palette_probe(int device, float *out_host);
/* Same table produced by this library's ALU decoder from the same probe blocks. */
int tx_software_palette(int device, float *out_host);
/* New: the ALU decoder's table for TX_PALETTE_HARDWARE (closed form of the texture-unit palette; its
 * SHA-256 is the hash the reference publishes, WINDOWS_VALIDATION.md:13-14). */
int tx_hardware_palette(int device, float *out_host);
/* New: declare which palette the handle's payload was encoded against (TX_PALETTE_*).  All decode
 * paths follow it.  With TX_PALETTE_HARDWARE the texture decode path passes the palette gate on
 * devices whose texture unit reproduces that table. */
int tx_set_palette(uint64_t handle, int palette);

/* encode: the reference's offline encoder for one matrix, texelator/encoder.py:34-102 (endpoint_opt), :23-31
 * (nearest), :105-117 (pack_blocks) and :137-145 (row scales) -- there a chain of PyTorch tensor operations,
 * here two kernels whose output is byte-identical to it.  All pointers are device pointers: `weight` fp32
 * [M, K] row-major, `hdiag` fp32 [K] (the activation second moments E[x_k^2] that weight the error),
 * `lut` fp32 [255, 255, 8] = palette[e1 + 127][e0 + 127][selector]; writes M * K / 2 bytes of row-major BC4
 * blocks (the .bc4 file content) and M fp32 row scales (the .scales.f32 content), which tx_pack_encoded
 * accepts as they are.  Asynchronous on `stream`. */
int tx_encode(const float *weight, const float *hdiag, const float *lut, int M, int K, uint8_t *blocks_out, float *scales_out,
              void *stream);

/* New: exact decode of the packed device copy (TX_DEQUANT_*), for bit-exact checks against the
 * encoder's palette.  `out` is a device [M,K] array. */
int tx_dequant(uint64_t handle, void *out, int what, void *stream);

/* New: copies the BC4 blocks back out of the device layout into host row-major order
 * (round-trip check of the packed copy). `out_host` holds M*K/2 bytes. */
int tx_unpack_blocks(uint64_t handle, uint8_t *out_host);

/* New: device status word.  Kernels never spin without a limit; when a bounded wait of the tensor-core
 * prefill kernel runs out it records a positive code (1..5 = producer, TMA, A-ready, X-ready,
 * accumulator wait) here and returns early.  Synchronises the device; returns the code (0 = healthy)
 * or a negative TX_E* value; `clear` resets it. */
int tx_kernel_status(int device, int clear);

/* Decode-loop glue around the linears (no counterpart in the reference, which leaves these steps to
 * Hugging Face / PyTorch: texelator/cli.py:189-219).  All tensors bf16 on the device, fp32 arithmetic,
 * asynchronous on `stream`.
 *   add_rmsnorm      : h += delta (delta may be null); y = rmsnorm(h) * weight, per token row
 *   rope_append      : rotate q and k of one token in place (rotate-half), append k and v to the
 *                      caches [kv_heads, max_len, head_dim] at *position (device int64)
 *   attention_decode : one query per head over cache positions 0..*position, grouped-query; `scratch`
 *                      holds q_heads * ceil(max_len/128) * (head_dim+2) floats; head_dim must be 128
 *   attention_step   : rope_append + attention_decode of one token in one call (q is rotated on the
 *                      fly, qkv is left untouched): one launch over 64-key splits of the cache and a small
 *                      dependent launch that merges them (TEXELATOR_B200_ATTENTION_MERGE=inline: one launch,
 *                      the last split's CTA merges); `scratch` holds q_heads * ceil(max_len/64) * 132
 *                      floats; head_dim 128; long caches are walked in 64-key chunks per CTA.  `position` and
 *                      the cache rows below it are read before the kernel waits for the launch in front of it
 *                      (they overlap that launch's tail): they must be complete when that launch starts, as they
 *                      are in a decode loop, where earlier steps wrote them
 *   silu_mul         : out[t,i] = silu(gate_up[t,i]) * gate_up[t,intermediate+i]                     */
int tx_aux_add_rmsnorm(void *h, const void *delta, const void *weight, void *y, int tokens, int hidden, float eps, void *stream);
/* add_rmsnorm for one token with the extras of tx_linear_single: delta may come as `splits` fp32 partial
 * vectors (partials[s * partial_stride + i], added in split order, rounded to bf16, then added to h), and
 * the normalised row may also (or only: y may be NULL then) be written in staged form to `staged`
 * (tx_linear_single_info out[2] bytes for K = hidden). */
int tx_aux_add_rmsnorm_single(void *h, const void *delta, const float *partials, int splits, size_t partial_stride, const void *weight,
                              void *y, void *staged, int hidden, float eps, void *stream);
/* Tensor parallelism, one token: the all-reduce of a row-parallel linear's partial output fused into the
 * residual add + RMSNorm that consumes it.  Every rank stores `partial` [hidden] into all ranks' inboxes
 * over peer memory, publishes an epoch flag, waits (bounded; a wait that runs out records 32 in the
 * status word read by tx_kernel_status) for the flags of all ranks and sums the inbox rows in rank order
 * (fp32, one bf16 rounding, identical bits on every rank); then h += sum, y = rmsnorm(h) * weight.
 * peer_inboxes[r] / peer_flags[r]: rank r's inbox (2 * world * hidden bf16, zero-initialised flags of
 * 2 * world uint32) as addressable from this rank; `epoch_word`: a zero-initialised uint32 in this rank's
 * memory that the kernel advances.  All ranks must make the same sequence of calls.  No reference
 * counterpart (the reference is single-GPU). */
int tx_aux_allreduce_add_rmsnorm(void *h, const void *partial, const void *weight, void *y, int hidden, float eps,
                                 void *const *peer_inboxes, void *const *peer_flags, int rank, int world, void *epoch_word,
                                 void *stream);
/* Tensor parallelism, one token, second generation of the exchange (no reference counterpart).  Every rank
 * owns an inbox of 2 * world * (hidden / 4) 16-byte packets in peer-mapped memory (zero-initialised) and an
 * epoch word (uint32, zero-initialised).  A packet {two bf16, epoch, two bf16, epoch} is written with one
 * 16-byte store and is complete for a reader once both flag words show the current epoch.
 *   tx_linear_single_push       the row-parallel linear (tx_linear_single rules; M = hidden) sends its bf16
 *                               partial row into the inboxes of all ranks from its epilogue, tile by tile, while
 *                               the rest of its weights still stream;
 *   tx_aux_peer_reduce_rmsnorm  world >= 1: polls (bounded; code 32 in the status word when a poll runs out)
 *                               the packets of all ranks in this rank's `inbox`, adds them in rank order (fp32,
 *                               one bf16 rounding, identical bits on every rank), h += sum, y / staged =
 *                               rmsnorm(h) * weight, and advances the epoch word.  world == 0: no exchange,
 *                               h += delta (may be NULL): the same kernel as a multi-SM add_rmsnorm.
 *                               Runs as one thread-block cluster of up to eight CTAs.
 *   tx_aux_peer_best_token      vocabulary-parallel output head: every rank sends (its best score, its token +
 *                               token_offset) to all ranks' token inboxes (2 * world packets, own epoch word);
 *                               next_token (int64) = the token of the highest score, lowest rank on ties.
 * All ranks must make the same sequence of calls; peer_inboxes[r] is rank r's inbox as addressable here. */
int tx_linear_single_push(uint64_t handle, const void *x, const void *staged, void *const *peer_inboxes, int rank, int world,
                          void *epoch_word, void *stream);
int tx_aux_peer_reduce_rmsnorm(void *h, const void *delta, const void *weight, void *y, void *staged, int hidden, float eps,
                               const void *inbox, int world, void *epoch_word, void *stream);
int tx_aux_peer_best_token(const float *local_score, const void *local_token, long long token_offset, void *const *peer_inboxes, int rank,
                           int world, void *epoch_word, void *next_token, void *stream);
int tx_aux_rope_append(void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                       void *v_cache, int q_heads, int kv_heads, int head_dim, int max_len, void *stream);
int tx_aux_attention_decode(const void *qkv, const void *k_cache, const void *v_cache, const void *position, float *scratch,
                            void *out, int q_heads, int kv_heads, int head_dim, int max_len, float scale, void *stream);
int tx_aux_attention_step(const void *qkv, const float *cos_table, const float *sin_table, const void *position, void *k_cache,
                          void *v_cache, float *scratch, void *out, int q_heads, int kv_heads, int head_dim, int max_len,
                          float scale, void *stream);
int tx_aux_silu_mul(const void *gate_up, void *out, int tokens, int intermediate, void *stream);
/* Batched decode (one token of each of `sequences` sequences per step; no reference counterpart, the reference
 * serves a batch as tokens of one GEMV launch, texelator_cuda.cu:1438-1468, and leaves attention to PyTorch).
 *   attention_step_batch : attention_step for every sequence in one launch.  qkv [sequences, (q_heads + 2 kv_heads) *
 *                          head_dim], positions int64 [sequences], caches [sequences, kv_heads, max_len, head_dim],
 *                          out [sequences, q_heads * head_dim]; `scratch` holds `sequences` times the floats of
 *                          attention_step; sequences * kv_heads <= 4096.
 *   silu_mul_pairs       : silu_mul for gate/up rows stored as alternating groups of eight (the row order the
 *                          SwiGLU-fused linear takes): out[t, 8j + e] = silu(gu[t, 16j + e]) * gu[t, 16j + 8 + e]. */
int tx_aux_attention_step_batch(const void *qkv, const float *cos_table, const float *sin_table, const void *positions, void *k_cache,
                                void *v_cache, float *scratch, void *out, int sequences, int q_heads, int kv_heads, int head_dim,
                                int max_len, float scale, void *stream);
int tx_aux_silu_mul_pairs(const void *gate_up, void *out, int tokens, int intermediate, void *stream);

/* Number of this library's kernels launched by the calling process since load (all threads). */
int64_t tx_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TEXELATOR_B200_H */
