/*
 * emmyq — C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * This is the boundary a host program binds instead of the reference's
 * compiled-program runtime for the quantized linear operator.  Conventions,
 * kept from the reference's runtime boundary (crates/emmy-runtime-py/src/lib.rs:168-361,
 * crates/emmy-runtime/ARCHITECTURE.md:216-227):
 *   - every pointer is a DEVICE pointer that the caller owns and keeps alive
 *     and unwritten until the work queued on `stream` has finished; nothing
 *     here frees or retains caller memory;
 *   - all work is enqueued on the caller's stream (`stream` is a
 *     cudaStream_t passed as void*; NULL is the legacy default stream);
 *   - nothing allocates: scratch memory is sized by a *_workspace_bytes()
 *     query and handed in by the caller;
 *   - every entry point returns an int status, EQ_OK (0) or a negative
 *     EQ_ERR_* code; nothing aborts or throws across the boundary;
 *     eq_last_error() gives the calling thread's last message.
 *
 * Tensor names and layouts are the checkpoint's own
 * (emmy/compiler/loader/quant.py:99-133, 136-144, 1120-1194):
 *   AWQ   qweight int32 [K, N/8] (nibble order 0,2,4,6,1,3,5,7), qzeros int32 [K/G, N/8], scales f16 [K/G, N]
 *   GPTQ  qweight int32 [K/8, N] (sequential down K), qzeros int32 [K/G, N/8] (zero = stored + 1),
 *         scales f16 [K/G, N], g_idx int32 [K] (optional)
 *   CT    compressed-tensors int4: GPTQ's layout once transposed (see EQ_W4_CT), zero = stored, scales usually bf16
 *   FP8   weight u8 e4m3fn [N, K], weight_scale f32 [N] (multiplier)
 *   NVFP4 weight u8 [N, K/2] (low nibble = even k), weight_scale u8 e4m3 [N, K/16], weight_scale_2 f32 [1]
 * K = in features, N = out features, G = group size, y[M,N] = x[M,K] @ W[K,N].
 */
#ifndef EMMYQ_H
#define EMMYQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    EQ_OK = 0,
    EQ_ERR_BAD_ARG = -1,     /* null pointer, non-positive extent, unknown enum */
    EQ_ERR_BAD_ALIGN = -2,   /* pointer or extent not aligned as the kernel needs */
    EQ_ERR_UNSUPPORTED = -3, /* a shape / group size / dtype this build has no kernel for */
    EQ_ERR_CUDA = -4,        /* a CUDA runtime call or launch failed */
    EQ_ERR_NCCL = -5,
    EQ_ERR_TIMEOUT = -6,     /* a bounded device-side wait ran out */
    EQ_ERR_WORKSPACE = -7    /* workspace missing or too small */
};

/* Packed-int4 family (emmy/compiler/loader/quant.py:86-133).  EQ_W4_CT is compressed-tensors' pack-quantized int4 AFTER its
 * three tensors have been transposed into GPTQ's orientation (weight_packed [N, K/8] -> [K/8, N], weight_zero_point
 * [N/8, K/G] -> [K/G, N/8], weight_scale [N, K/G] -> [K/G, N]): GPTQ's sequential nibble order, zero point as stored. */
enum { EQ_W4_AWQ = 0, EQ_W4_GPTQ = 1, EQ_W4_CT = 2 };
enum { EQ_F16 = 0, EQ_BF16 = 1, EQ_F32 = 2 };     /* element types of activations / outputs / scales */

/* Library version (major*10000 + minor*100 + patch) and message of the calling thread's last failure. */
int eq_version(void);
const char* eq_last_error(void);
const char* eq_status_name(int status);

/* ------------------------------------------------------------------ decode (bit-exact) */

/* int32 words -> uint8 nibbles in [0,15], eight per word, in logical order.
 * along_rows = 0: out[r, 8c+i] (AWQ qweight, both families' qzeros); 1: out[8r+i, c] (GPTQ qweight).
 * Replaces unpack_int4 (emmy/compiler/loader/quant.py:515-530). */
int eq_unpack_int4(int fmt, int along_rows, const int32_t* words, int64_t rows, int64_t cols, uint8_t* out, void* stream);

/* Packed int4 linear -> value matrix, (q - (z + bias)) * s computed exactly in f32 and rounded ONCE to out_dtype.
 * g_idx may be NULL (group of row k is k / G).  G = -1 means one group.  scale_dtype is EQ_F16 or EQ_BF16.
 * transpose = 0 writes W[K, N]; 1 writes the HF orientation W[N, K].
 * Replaces dequantize_packed_int4 (emmy/compiler/loader/quant.py:533-555) followed by the eager cast
 * (emmy/compiler/trace/huggingface.py:2908-2910). */
int eq_dequant_w4(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales, int scale_dtype,
                  const int32_t* g_idx, int64_t K, int64_t N, int64_t G, int out_dtype, int transpose, void* out,
                  void* stream);

/* e4m3 weight [N, K] times a multiplier scale [scale_rows, scale_cols] whose extents divide N and K
 * (1x1 per tensor, Nx1 per output channel, 2-D blocks) -> out_dtype [N, K].
 * Replaces decode_f8 + dequantize (emmy/compiler/dtype.py:236-238, emmy/compiler/loader/quant.py:147-170). */
int eq_dequant_fp8(const uint8_t* bits, const float* scale, int64_t N, int64_t K, int64_t scale_rows,
                   int64_t scale_cols, int out_dtype, void* out, void* stream);

/* NVFP4 weight -> out_dtype [N, K]: e2m1 value times f32(f16(e4m3(scale) * scale_2)).
 * Replaces dequantize_nvfp4 (emmy/compiler/loader/quant.py:173-197). */
int eq_dequant_nvfp4(const uint8_t* packed, const uint8_t* scale_bits, const float* scale_2, int64_t N, int64_t K,
                     int out_dtype, void* out, void* stream);

/* Native MXFP4 (gpt-oss experts): blocks uint8 [N, K/32, 16] (a byte = the even value in its low nibble, the odd one in its
 * high nibble; the e2m1 value table of NVFP4), scales uint8 [N, K/32] (a power of two, exponent biased by 127).
 * out[n, k] = F4[code] * 2^(scale - 127), exact (infinity at the largest exponents), [N, K] in out_dtype: the stored
 * orientation; the reference's decode_mxfp4 returns its transpose (emmy/compiler/loader/quant.py:477-496).  Decoder
 * only: an MXFP4 linear is not part of this library. */
int eq_dequant_mxfp4(const uint8_t* blocks, const uint8_t* scales, int64_t N, int64_t K, int out_dtype, void* out, void* stream);

/* ------------------------------------------------------------------ load-time repack (W4) */

/* The reference binds checkpoint bytes verbatim and lets its compiler pick a folded or source layout per weight
 * (emmy/compiler/loader/binder.py:19-131, emmy/compiler/pipeline/passes/tile/_layout.py:47-65).  Here the
 * load-time step re-tiles the int4 words once into the order the tensor-core fragments read:
 *   wq  u8  [N/16][K/128][1088 B]          one record per 16 columns x 128 input rows: two 16x64 nibble tiles
 *                                          (512 B each; a lane of a warp owns 16 B, its four words are four k16
 *                                          steps) followed by 64 B of that group's scales (dtype kept) and zero
 *                                          points (family bias added, 0..16), one 8-byte entry per column pair
 *   perm int32 [K + 4]                     row order, used only when g_idx is not constant on aligned G-blocks:
 *                                          row k' of the repacked weight is input feature perm[k'] (rows sorted by
 *                                          group); the four trailing words are status words of the repack itself
 * With g_idx the scale/zero rows are gathered so that repacked group index is k' / G.
 * Requires K % 128 == 0, N % 16 == 0, G % 128 == 0 (or G = -1), every group holding exactly G rows. */
int eq_w4_repack_sizes(int64_t K, int64_t N, int64_t G, size_t* wq_bytes, size_t* perm_bytes);
/* *uses_perm (host int) is set to 1 when `perm` must be passed to the linear call; the call synchronizes the
 * stream once to read that flag.  `perm` may be NULL when g_idx is NULL. */
int eq_w4_repack(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales, const int32_t* g_idx,
                 int64_t K, int64_t N, int64_t G, void* wq, int32_t* perm, int* uses_perm, void* stream);
/* The experts of an MoE layer in one call: E stacked weights (qweight [E, ...], qzeros [E, ...], scales [E, K/G, N], each
 * expert in its checkpoint layout, no g_idx) -> E repacked blobs back to back (eq_w4_repack_sizes bytes each), the layout
 * eq_moe_w4a16 takes.  Two launches for the whole stack, no host synchronization (the reference stacks expert weights at
 * load the same way, emmy/compiler/trace/huggingface.py:2110-2141). */
int eq_w4_repack_stack(int fmt, const int32_t* qweight, const int32_t* qzeros, const void* scales, int64_t E, int64_t K, int64_t N,
                       int64_t G, void* wq, void* stream);
/* Inverse view for round-trip checks: repacked blob -> uint8 nibbles [K, N] in repacked row order. */
int eq_w4_unpack_repacked(const void* wq, int64_t K, int64_t N, uint8_t* out, void* stream);

/* ------------------------------------------------------------------ W4A16 linear */

/* Scratch for eq_w4a16_linear: a 256-byte header whose first word is the status word, then f32 words (the partial
 * sums of the split-K kernels; at M = 1 the sixteen-word hand-overs between neighbouring CTAs of the GEMV) and one
 * arrival counter per 16-column tile (up to 256 rows of sums), plus, for M > 16, room for a column-gathered copy of x
 * (used when the weight carries a row permutation).  The buffer must be zero the first time it is used; every call
 * leaves the words it used zero again, so it can be reused by calls on one stream (calls on different streams need
 * different buffers). */
size_t eq_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K);
/* y[M, N] = x[M, K] @ W on repacked weights; x and y are act_dtype (EQ_F16 or EQ_BF16), f32 accumulation.
 * The operator the reference spells as int4 decode algebra in front of a LinearOp
 * (emmy/compiler/loader/quant.py:1235-1435) and evaluates eagerly as dequantize + F.linear
 * (emmy/compiler/trace/huggingface.py:2877-2920).  perm is NULL unless eq_w4_repack asked for it.
 * Needs K % 128 == 0, N % 16 == 0, G % 128 == 0 (or G = -1); x and wq 16-byte aligned.
 * M <= 24 runs the bandwidth kernels (any K: shapes whose activations do not fit shared memory run a split-K form
 * through the workspace, and from 17 rows on such shapes take the next path); above that the tcgen05 kernel, which
 * dequantises into shared memory. */
int eq_w4a16_linear(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N, int64_t G,
                    const void* x, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                    void* stream);
/* The device-side waits (the tensor-path kernel's pipeline barriers, the GEMV's wait for a neighbour's sixteen words)
 * are bounded; one that runs out sets the status word at the start of the workspace and the affected outputs are
 * undefined.  The linear itself never clears the word: it stays set over later calls until this call, which
 * synchronizes the stream, reads the word, clears it if it was set and returns EQ_ERR_TIMEOUT in that case (the
 * reference's counterpart is the host-side hung-launch deadline, crates/emmy-runtime/src/cuda.rs:1401-1451). */
int eq_w4a16_status(const void* workspace, int64_t M, int64_t N, void* stream);

/* gate / up + SwiGLU in one call: h[M, I] = act(silu(x W_gate)) * (x W_up), wq the repacked [gate | up] weight (the two
 * projections concatenated along N: K x 2I), with the eager form's roundings (both projections, the silu and the product
 * each rounded to the activation dtype; emmy/compiler/trace/huggingface.py:1663-1669).  M > 16 runs the tensor path with
 * the activation in the GEMM's epilogue (the [M, 2I] intermediate never exists in memory; needs perm == NULL and a
 * 16-byte aligned h); M <= 16 runs the linear into scratch and an elementwise pass.  One of the fused forms the
 * reference's compiler realizes around its linears (tests/compiler/realization/cases/fused/gate-up-*.json).
 * The workspace starts like eq_w4a16_linear's (zero on first use, left zero; eq_w4a16_status(workspace, M, 2 * I) reads
 * its status word). */
size_t eq_w4a16_gate_up_workspace_bytes(int64_t M, int64_t I, int64_t K);
int eq_w4a16_gate_up_swiglu(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t I, int64_t G, const void* x,
                            int64_t M, int act_dtype, void* h, void* workspace, size_t workspace_bytes, void* stream);

/* eq_w4a16_linear for hosts that cannot hand over scratch memory.  (No counterpart in the reference: its runtime
 * owns all device memory itself.)  Some callers of this library run where device allocation is off limits: a
 * serving engine that has already given every byte to its KV-cache pool and forbids cudaMalloc afterwards, code on
 * a latency-critical decode path where an allocation would synchronize the device, or a plug-in loaded into a
 * process whose allocator it may not touch.  This variant takes inputs and outputs only.  The workspace of
 * eq_w4a16_linear (status word, hand-over words of the M = 1 kernel, partial sums and arrival counters of the split-K
 * kernel that serves very large K) is one array built into the library (about 2 MiB, present on every GPU that loads
 * the library until the process exits), which limits it to M <= 16 rows and N <= 32768 columns; larger calls are
 * refused with EQ_ERR_UNSUPPORTED and should use eq_w4a16_linear.  It calls no allocating routine.
 * The first call on each device looks up the array's device address (the device must be current); make that call
 * before starting a stream capture.  The array starts out zero, every kernel leaves the words it used zero again,
 * and all calls share it, so two calls that overlap on the GPU (different streams, or different threads without
 * ordering) race: keep calls on one device ordered.  After a call that failed the array is cleared before its next
 * use. */
int eq_w4a16_linear_noalloc(const void* wq, int scale_dtype, const int32_t* perm, int64_t K, int64_t N, int64_t G,
                            const void* x, int64_t M, int act_dtype, void* y, void* stream);
/* eq_w4a16_status for the built-in array of the current device (no counterpart in the reference). */
int eq_w4a16_noalloc_status(void* stream);

/* ------------------------------------------------------------------ FP8-E4M3 W8A8 linear */

/* Dynamic per-token activation quantize: scale[m] = max(amax_k |x[m,k]|, 1e-12) / 448 (f32), q = e4m3 (round to
 * nearest even, saturating to +-448) of x / scale with an f32 division.  x is [M, K] of in_dtype (EQ_F16, EQ_BF16 or
 * EQ_F32), q is [M, K] bytes, scale [M] f32.  Bit-exact with the rule the reference spells into its graphs
 * (_spell_dynamic_activation, emmy/compiler/loader/quant.py:1655-1735).  Applied to a weight's rows it is the
 * per-output-channel weight quantizer. */
int eq_quant_fp8_per_token(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, void* stream);

/* Scratch of eq_fp8_linear: the quantized activations, their scales and a status word. */
size_t eq_fp8_workspace_bytes(int64_t M, int64_t K);
/* y[M, N] = (sum_k q_x[m,k] q_w[n,k]) * s_x[m] * s_w[n] in act_dtype (EQ_F16 or EQ_BF16), f32 accumulation.
 * weight: e4m3 bits [N, K] as the checkpoint stores them, weight_scale: f32 [N] multiplier.  The activation is
 * quantized per token inside the call.  Every M runs on tcgen05: M <= 16 a weight-streaming tile with the operands' roles
 * swapped (weight tiles as the MMA's A operand), larger M the 128- and 256-row tiles.
 * The operator the reference spells as FP8 decode + dynamic activation round trip in front of a LinearOp
 * (emmy/compiler/loader/quant.py:1581-1768) and runs natively with both scales hoisted
 * (tests/compiler/passes/test_fp8_mma.py:111-120).  Needs K % 128 == 0, N % 16 == 0; workspace 256-byte aligned. */
int eq_fp8_linear(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, int64_t M,
                  int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* The same with a STATIC activation scale: q = e4m3(x / input_scale) for every token (input_scale: device f32 [1], the
 * checkpoint's `input_scale` / `activation_scale`), y = (sum q_x q_w) * input_scale * s_w[n].  The static FP8 activation
 * the reference spells for `activation_scheme: static` checkpoints (emmy/compiler/loader/quant.py:1818-1905). */
int eq_fp8_linear_static(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, const float* input_scale,
                         int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* RMSNorm -> quantize -> linear with the norm inside the quantize kernel (one of the fused forms the reference's compiler
 * realizes around its linears, tests/compiler/realization/cases/fused/norm-linear-*.json): y = fp8_linear(h) with
 * h = dtype(dtype(x * rsqrt(mean(x^2) + eps)) * gamma), the model's RMSNorm (the normalised value is rounded to the
 * activation dtype before gamma multiplies it); gamma: [K] in act_dtype.  The normalised row is never written to memory.
 * Same workspace and status as eq_fp8_linear. */
int eq_fp8_linear_rmsnorm(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, const void* gamma,
                          float eps, int64_t M, int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* Synchronizes the stream and returns EQ_ERR_TIMEOUT if a bounded pipeline wait of the last eq_fp8_linear call on
 * this workspace ran out (same role as eq_w4a16_status). */
int eq_fp8_status(const void* workspace, int64_t M, int64_t K, void* stream);

/* Block-scaled FP8 (the official 128 x 128 weight-block form): weight e4m3 [N, K], weight_scale f32 [N/128, K/128]
 * (the checkpoint's `weight_scale_inv`, a multiplier: emmy/compiler/loader/quant.py:136-144), activations quantized per
 * token and per 128 elements of K (emmy/compiler/loader/quant.py:1581-1593, 1655-1717):
 * y[m, n] = sum_kb (sum_{k in kb} q_x q_w) * s_x[m, kb] * s_w[n / 128, kb].  Needs K % 128 == 0, N % 128 == 0. */
int eq_quant_fp8_per_group(const void* x, int64_t M, int64_t K, int in_dtype, uint8_t* q, float* scale, void* stream);
size_t eq_fp8_block_workspace_bytes(int64_t M, int64_t K);
int eq_fp8_block_linear(const uint8_t* weight, const float* weight_scale, int64_t N, int64_t K, const void* x, int64_t M,
                        int act_dtype, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* Synchronizes the stream; EQ_ERR_TIMEOUT if a bounded pipeline wait of the tensor path (M > 16) ran out. */
int eq_fp8_block_status(const void* workspace, int64_t M, int64_t K, void* stream);

/* ------------------------------------------------------------------ NVFP4 W4A4 linear */

/* The input scale calibrated on the sample itself: max(amax |x|, 1e-12) / (6 * 448), computed in f64 and rounded to
 * f32 (emmy/compiler/loader/synthesize.py:181-183; the same rule gives weight_scale_2 in quantize_nvfp4,
 * emmy/compiler/loader/quant.py:221-226).  scale2: device f32 [1]; scratch_u32: device uint32 [1]. */
int eq_nvfp4_global_scale(const void* x, int64_t M, int64_t K, int in_dtype, float* scale2, unsigned int* scratch_u32,
                          void* stream);
/* The NVFP4 weight quantizer, bit-exact with quantize_nvfp4 (emmy/compiler/loader/quant.py:206-237): scale_2 =
 * max(amax, 1e-12) / (6 * 448) for the whole tensor, one e4m3 scale per 16 elements along K stored relative to it
 * (block amax / 6 / scale_2), codes = e2m1 (round to nearest even code, saturating at 6) of value / f16(scale *
 * scale_2), zero where that fused scale is zero.  values: [N, K] of in_dtype (EQ_F32, EQ_F16 or EQ_BF16); packed:
 * [N, K/2] bytes (low nibble = even k); scale_bits: [N, K/16]; scale_2: device f32 [1]; scratch_u32: device uint32 [1].
 * Needs K % 16 == 0.  (The reference's limit |values| <= 6 * 65504 for an f16 fused scale is the caller's to keep.) */
int eq_quant_nvfp4_weight(const void* values, int64_t N, int64_t K, int in_dtype, uint8_t* packed, uint8_t* scale_bits,
                          float* scale_2, unsigned int* scratch_u32, void* stream);
/* Static-scale NVFP4 activation quantize, bit-exact with the algebra the reference spells
 * (_spell_static_fp4_quantize, emmy/compiler/loader/quant.py:1968-2139; pinned by _static_quantize_ref,
 * tests/compiler/loader/test_quant.py:1776-1784).  codes: [M, K/2] bytes (low nibble = even k); scale_bits: optional
 * plain e4m3 scales [M, K/16]; scale_tiled: optional scales in the tensor core's atom order (size from
 * eq_nvfp4_tiled_scale_bytes).  input_scale: device f32 [1]. */
int eq_quant_nvfp4_act(const void* x, int64_t M, int64_t K, int in_dtype, const float* input_scale, uint8_t* codes,
                       uint8_t* scale_bits, uint8_t* scale_tiled, void* stream);
/* Load-time re-tiling of a checkpoint's weight_scale [rows, K/16] into 512-byte atoms: [row block of 128][64
 * elements of K][512 B], scale of (row r, block i) at byte (r % 32) * 16 + (r / 32) * 4 + i; rows padded to 128 with
 * zeros.  (The reference binds these bytes verbatim, emmy/compiler/loader/binder.py:124-130; here the scale-factor
 * copy into tensor memory wants this order.)  Needs K % 64 == 0. */
size_t eq_nvfp4_tiled_scale_bytes(int64_t rows, int64_t K);
int eq_nvfp4_tile_scales(const uint8_t* scale_bits, int64_t rows, int64_t K, uint8_t* tiled, void* stream);
/* The weight's scales for eq_nvfp4_linear: the layout above, followed (256-byte aligned) by the same atoms grouped for
 * the prefill kernel's 224-row column tiles ([tile of 224 rows][two row blocks][64 elements of K][512 B], rows past the
 * tile zero).  `tiled` must be 256-byte aligned. */
size_t eq_nvfp4_weight_scale_bytes(int64_t N, int64_t K);
int eq_nvfp4_tile_weight_scales(const uint8_t* scale_bits, int64_t N, int64_t K, uint8_t* tiled, void* stream);
/* y[M, N] = input_scale * weight_scale_2 * sum_blocks s_x s_w sum_k c_x c_w in act_dtype: the native block-scaled
 * product (tcgen05.mma kind::mxf4nvf4).  weight: packed e2m1 [N, K/2] as stored; weight_scale_tiled: from
 * eq_nvfp4_tile_weight_scales; weight_scale_2, input_scale: device f32 [1].  The activation is quantized inside the call.
 * The operator the reference spells as NVFP4 decode + static activation quantize in front of a LinearOp
 * (emmy/compiler/loader/quant.py:2142-2209, 1968-2139).  Needs K % 256 == 0, N % 8 == 0. */
size_t eq_nvfp4_workspace_bytes(int64_t M, int64_t K);
int eq_nvfp4_linear(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N,
                    int64_t K, const void* x, const float* input_scale, int64_t M, int act_dtype, void* y, void* workspace,
                    size_t workspace_bytes, void* stream);
/* RMSNorm -> static quantize -> linear with the norm inside the quantize kernel (as eq_fp8_linear_rmsnorm): gamma [K] in
 * act_dtype; input_scale is the calibrated global scale of the NORMALISED activations. */
int eq_nvfp4_linear_rmsnorm(const uint8_t* weight, const uint8_t* weight_scale_tiled, const float* weight_scale_2, int64_t N, int64_t K,
                            const void* x, const void* gamma, float eps, const float* input_scale, int64_t M, int act_dtype, void* y,
                            void* workspace, size_t workspace_bytes, void* stream);
int eq_nvfp4_status(const void* workspace, int64_t M, int64_t K, void* stream);

/* ------------------------------------------------------------------ MoE on W4A16 experts */

/* Router: softmax in f32 over logits [T, E], top-k with ties to the lowest expert id, picked probabilities
 * renormalised when renorm != 0.  ids int32 [T, k] and scores f32 [T, k] come out sorted by ascending expert id per
 * row, the order the combine adds them in.  Follows the router of emmy/serving/native/prepare.py:424-463 (contract
 * of the fused router in emmy/serving/gen_runner.py:3175-3197).  E <= 1024, k <= 16. */
int eq_moe_route(const float* logits, int64_t T, int64_t E, int64_t topk, int renorm, int32_t* ids, float* scores, void* stream);

/* Scratch of the MoE calls for T tokens (for eq_moe_experts_w4a16: T = rows, topk = 1). */
size_t eq_moe_workspace_bytes(int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I);

/* Grouped expert FFN over R rows: row r reads activation row src_row[r] of x (src_row NULL: row r) and belongs to
 * expert expert_ids[r]; out[r] = down_e( silu(gate_e(x_r)) * up_e(x_r) ) in act_dtype.  wq_gate_up / wq_down: the
 * experts' repacked int4 weights (eq_w4_repack) stacked expert-major; gate_up is K = H, N = 2 I (gate columns then up
 * columns), down is K = I, N = H.  The expert algebra of ExpertFFN.forward (emmy/compiler/trace/huggingface.py:1663-1669)
 * over the row lists the reference builds with a stable argsort and a host read of the counts
 * (emmy/serving/gen_runner.py:276-283, 3359-3479); here counts, offsets and row blocks stay on the device.
 * This is also the local step of expert-parallel serving: the rows are the tokens received from all ranks. */
int eq_moe_experts_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t H, int64_t I, int64_t G,
                         const void* x, const int32_t* src_row, const int32_t* expert_ids, int64_t R, int act_dtype, void* out,
                         void* workspace, size_t workspace_bytes, void* stream);

/* y[t] = dtype( sum_j f32(dtype(score[t, j])) * f32(out_rows[t k + j]) ): products and sum in f32 in the stored pick
 * order, one rounding (combine_routed_experts, emmy/serving/gen_runner.py:235-287). */
int eq_moe_combine(const void* out_rows, const float* scores, int64_t T, int64_t topk, int64_t H, int act_dtype, void* y, void* stream);

/* Whole routed layer on one device: route (renormalised top-k), grouped expert FFN, combine. */
int eq_moe_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E, int64_t topk, int64_t H, int64_t I, int64_t G,
                 const void* x, const float* router_logits, int64_t T, int act_dtype, void* y, void* workspace, size_t workspace_bytes,
                 void* stream);
/* Synchronizes the stream; EQ_ERR_BAD_ARG if the last call met an expert id outside [0, E) (such rows are dropped). */
int eq_moe_status(const void* workspace, int64_t T, int64_t E, int64_t topk, int64_t H, int64_t I, void* stream);

/* ------------------------------------------------------------------ expert-parallel MoE over peer memory */

/* Experts sharded E_local per rank over `world` GPUs of one node.  The token exchange of the reference's expert
 * sharding is different: every rank keeps a slice of EVERY expert's intermediate axis and the partial outputs meet in
 * one all-reduce (emmy/compiler/trace/huggingface.py:1071-1124, emmy/serving/vllm_model_gen.py:986-991; the host-side
 * split is pinned by tests/serving/test_expert_sharding.py:49-165); it has no token exchange.  Here whole experts are
 * sharded and the kernels move the tokens: rows are stored into the owner's receive buffer
 * and results stored back into the token's rank over NVLink peer mappings, ordered by epoch flags.  Every pointer
 * below is a device address valid ON THE CALLING RANK (its own buffer, or a peer's buffer mapped into this
 * process, e.g. through CUDA IPC or torch symmetric memory); entry r describes rank r's buffers. */
#define EQ_EP_MAX_RANKS 8
typedef struct eq_ep_peers {
    int32_t world, rank;
    int64_t cap;                          /* a rank's receive buffer holds world * cap rows (shared by the sources) */
    void* recv_x[EQ_EP_MAX_RANKS];        /* [world * cap][H] activation rows in expert order, written by the sources */
    int32_t* recv_meta[EQ_EP_MAX_RANKS];  /* [world * cap][2]: source rank, return slot (pick index at the source) */
    int32_t* recv_count[EQ_EP_MAX_RANKS]; /* [world sources][world destinations][E_local]: every rank's pick counts */
    void* back[EQ_EP_MAX_RANKS];          /* [T_max * topk][H]: expert outputs in the owner's pick order */
    uint32_t* flags[EQ_EP_MAX_RANKS];     /* [3][world] uint32 (counts, rows, results), zero before the first call */
} eq_ep_peers;

size_t eq_ep_moe_workspace_bytes(int64_t world, int64_t cap, int64_t E_local, int64_t H, int64_t I);
/* One routed layer on this rank's T tokens (ids / scores as eq_moe_route returns them, over all E_local * world
 * experts).  Collective: every rank of the group calls it the same number of times.  epoch = 0 keeps the call counter
 * in the workspace on the device (one increment per call on every rank), which makes the whole layer replayable from
 * a captured CUDA graph; a non-zero epoch is taken as given and must grow by one per call, starting at 1, the same on
 * all ranks (do not mix the two forms on one set of buffers).  The workspace is local, zero on first use.  Waits on
 * peers are bounded (about one second). */
int eq_ep_moe_w4a16(const void* wq_gate_up, const void* wq_down, int scale_dtype, int64_t E_local, int64_t topk, int64_t H,
                    int64_t I, int64_t G, const void* x, const int32_t* ids, const float* scores, int64_t T, int act_dtype,
                    void* y, const eq_ep_peers* peers, uint32_t epoch, void* workspace, size_t workspace_bytes, void* stream);
/* EQ_ERR_TIMEOUT when a peer did not arrive in time, EQ_ERR_UNSUPPORTED when a rank was sent more than world * cap rows. */
int eq_ep_moe_status(const void* workspace, int64_t world, int64_t cap, int64_t E_local, int64_t H, int64_t I, void* stream);

/* ---- sum of a row-parallel linear's partial results over peer memory ------------------------------------------
 * The reference completes a rank's partial sums by a reduction over the tensor-parallel group
 * (emmy/serving/vllm_model_gen.py:986-991, vLLM's tensor_model_parallel_all_reduce).  This is that reduction for small
 * results (decode steps), done by one kernel over NVLink peer mappings in one round: every rank pushes its partial into
 * every peer's receive buffer, flags it, waits (bounded, about a second) for the peers' pieces and adds the world's
 * partials in rank order in f32, rounded once -- all ranks end with bit-identical y.  Pointers as in eq_ep_peers: device
 * addresses valid on the calling rank, entry r describing rank r's buffers. */
typedef struct eq_ar_peers {
    int32_t world, rank;
    int64_t cap;                       /* values (2 bytes each) a call may carry at most; a multiple of 8 */
    int64_t max_blocks;                /* ceil(cap / 2048) */
    void* recv[EQ_EP_MAX_RANKS];       /* [2 slots][world sources][cap] values, written by the sources */
    uint32_t* flags[EQ_EP_MAX_RANKS];  /* [2 slots][world sources][max_blocks] uint32, zero before the first call */
} eq_ar_peers;
size_t eq_peer_allreduce_recv_bytes(int64_t world, int64_t cap);
size_t eq_peer_allreduce_flag_bytes(int64_t world, int64_t cap);
size_t eq_peer_allreduce_state_bytes(void);
/* y[count] = sum over ranks of partial[count] (f16 or bf16, f32 sum, one rounding).  Collective: every rank of the group
 * calls it the same number of times with the same count.  `state` is local device memory of
 * eq_peer_allreduce_state_bytes(), zero on first use (status word, the call counter -- kept on the device, so the call
 * replays from a captured CUDA graph -- and a block counter).  partial and y must not be the receive buffers. */
int eq_peer_allreduce(const eq_ar_peers* peers, const void* partial, int64_t count, int dtype, void* y, void* state, void* stream);
/* Synchronizes the stream; EQ_ERR_TIMEOUT if a peer's piece did not arrive in time (y is undefined then). */
int eq_peer_allreduce_status(const void* state, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EMMYQ_H */
