/*
 * scratchy_cuda.h — C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * This is the boundary a `cuda` target of the reference project binds through a
 * thin `extern "C"` shim: every entry point takes plain pointers and sizes, an
 * explicit CUDA stream (passed as `void*`, i.e. a `cudaStream_t`), returns an
 * `int32_t` status (0 = OK, negative = error), never throws, never aborts and
 * allocates nothing on the step path.  All device pointers must be 16-byte
 * aligned unless stated otherwise.  One caller thread drives one stream; the
 * library keeps no global mutable state besides the per-device context, and a
 * context serves one host thread at a time (a call parks its variant's options
 * in the context while it runs): give each worker thread its own context.
 *
 * Each declaration cites the reference interface it replaces (paths relative to
 * the reference project's root).
 */
#ifndef SCRATCHY_CUDA_H_
#define SCRATCHY_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define SCR_OK              0
#define SCR_E_ARG          -1   /* null pointer / bad enum                              */
#define SCR_E_SHAPE        -2   /* shape violates the preset's law (K % group, ...)     */
#define SCR_E_ALIGN        -3   /* pointer not 16-byte aligned                          */
#define SCR_E_DTYPE        -4   /* unsupported bits / group size / dtype                */
#define SCR_E_CUDA         -5   /* a CUDA runtime call or a kernel launch failed        */
#define SCR_E_WORKSPACE    -6   /* workspace missing or too small                       */
#define SCR_E_UNSUPPORTED  -7   /* valid request this build does not implement          */
#define SCR_E_TIMEOUT      -8   /* a bounded device-side wait ran out                   */
#define SCR_E_COMM         -9   /* tensor-parallel communicator error                   */

typedef struct scr_ctx scr_ctx;

/* Human-readable name of a status code. */
const char* scr_status_string(int32_t status);
/* Detail text of the last error recorded on this context (empty string if none). */
const char* scr_last_error(const scr_ctx* ctx);

/* ---- lifecycle ----------------------------------------------------------
 * Replaces the Metal target's device bring-up behind `Worker::init_device`
 * (crates/serving/engine/src/worker.rs:50-84).  `scr_cuda_init` makes `device`
 * current, checks that it is an sm_100 part and records its SM count. */
int32_t scr_cuda_init(int32_t device, scr_ctx** out);
int32_t scr_cuda_destroy(scr_ctx* ctx);
/* Number of kernels this context has launched since creation (bench accounting). */
int64_t scr_launch_count(const scr_ctx* ctx);
/* Health probe, the device-side half of `Executor::check_health`
 * (crates/serving/engine/src/executor.rs:454): every wait inside the tensor-core kernels is
 * bounded; one that runs out records a code in a device word instead of hanging.  This call
 * synchronises `stream`, reads and clears the word and returns SCR_E_TIMEOUT if it was set
 * (`code` receives the raw value; may be NULL), or SCR_E_ARG if the word holds a device-side
 * argument check of the decode-step operators (a token id, position, slot or block id out of
 * range).  Not for the step path. */
int32_t scr_device_status(scr_ctx* ctx, void* stream, int32_t* code);

/* ---- MLX affine int4 (groups of 32, 64 or 128): load-time repack ------------
 * Replaces `MetalAffineQuantOps::load` (crates/targets/metal/src/layers_quant.rs:289-345)
 * + `load_layered_linear_affine_quant` (crates/targets/metal/src/loaders.rs:96-116): the
 * checkpoint tensors of `AffineQuantLinear` (crates/models/quantization/src/layers_quant.rs:33-52)
 *   w       U32  [N, K/8]   element i of a word at bits [4i, 4i+4)
 *   scales  F16 or BF16 [N, K/group]   (`scale_dtype`: the model's SCALE_DTYPE the loader pins,
 *   biases  F16 or BF16 [N, K/group]    crates/targets/metal/src/layers_quant.rs:238-285)
 * already resident on the device, are rewritten once into the kernels' streaming
 * layout (`dst`, `scr_affine_b4_repack_size` bytes, 128-byte aligned).  F16 scales and biases —
 * what every mlx-community 4-bit checkpoint ships — are narrowed to the bf16 activation type here,
 * exactly as the reference narrows them before it multiplies (`TAct::from_f32(scale.to_f32())`,
 * crates/targets/metal/src/cpu_reference.rs:63-68,90-92), so the kernels see one layout.
 * Validation follows layers_quant.rs:310-338: bits == 4, K % group == 0; group is 32, 64 or 128, the
 * sizes the reference's lowering admits (crates/compiler/subtile/src/lower.rs:112-127; SCR_E_DTYPE otherwise).
 * Every forward entry point takes the three; two things are built for groups of 64 and 128 only and answer
 * SCR_E_UNSUPPORTED at 32: the norm-in end of `scr_linear_affine_b4_ends` and the matvec tape. */
int32_t scr_affine_b4_repack_size(int32_t N, int32_t K, int32_t group, size_t* bytes);
/* The reference's `DType` discriminants (crates/tensors/src/dtype.rs:7-16). */
#define SCR_DTYPE_F16  0
#define SCR_DTYPE_BF16 1
int32_t scr_affine_b4_repack(scr_ctx* ctx, const uint32_t* w, const uint16_t* scales,
                             const uint16_t* biases, int32_t scale_dtype, int32_t N, int32_t K,
                             int32_t group, void* dst, void* stream);

/* Test hook: dequantise the *repacked* buffer back to dense bf16 [N, K] with the very
 * device code the matvec and the GEMM use.  Must equal, bit for bit,
 * `affine_dequant_b4_to_dtype` (crates/models/quantization/src/affine.rs:35-196). */
int32_t scr_affine_b4_dequant_dump(scr_ctx* ctx, const void* packed, int32_t N, int32_t K,
                                   int32_t group, uint16_t* w_bf16, void* stream);
/* The quantized token embedding, `AffineQuantEmbedding` (crates/models/quantization/src/layers_quant.rs:105-150;
 * `Instruction::AffineEmbed`, kernel `affine_embed_b4`, crates/targets/metal/shaders/quantized_dequantize.metal:82-157):
 *   out[i, :] (bf16) = dequant(table[ids[i], :])        gather and dequantisation in one pass
 * with the dequantisation of the matrix path, bit for bit.  `packed` is a table [vocab, hidden] repacked by
 * `scr_affine_b4_repack` — the buffer a tied lm_head multiplies with (`scr_linear_affine_b4` with N = vocab,
 * K = hidden), as the reference shares one buffer triple between the two layers.  An id >= vocab records a code
 * (`scr_device_status` reports SCR_E_ARG) and yields a row of zeros. */
int32_t scr_affine_b4_embed(scr_ctx* ctx, const void* packed, const uint32_t* ids, int32_t n_ids,
                            int32_t vocab, int32_t hidden, int32_t group, uint16_t* out_bf16, void* stream);

/* ---- MLX affine int4: forward ---------------------------------------------
 * Replaces the `MetalStep::AffineQmm(AffineMatmul{input, output, layer, n, k, group_size,
 * bits, ..})` step (crates/targets/metal/src/tape/step.rs:456-470) and its M-bucket
 * kernel pickers (crates/targets/metal/src/tape/quantized.rs:130-157,403-426,563-595):
 *   y[M,N] (bf16) = x[M,K] (bf16) @ dequant(W)[N,K]^T, f32 accumulation, one rounding,
 * the contraction of `cpu_reference::affine_qmm_t_b4` (crates/targets/metal/src/cpu_reference.rs:107-137).
 * The kernel is chosen from M (matvec for M <= 16, tensor-core GEMM above).
 * `bias_bf16` (may be NULL) is the linear's own bias [N], the `{prefix}.bias` tensor the loader
 * takes (crates/targets/metal/src/layers_quant.rs:318-351): it is added in f32 before the one
 * rounding, as the reference's matvec epilogue does (the `QmvEnds.bias` end,
 * crates/targets/metal/src/tape/step.rs:472-482, shaders/quantized_qmv.metal:104-112).
 * `workspace` may be NULL when `scr_linear_workspace_size` reports 0 bytes. */
#define SCR_KIND_AFFINE_B4   0
#define SCR_KIND_FP8_DYNAMIC 1
int32_t scr_linear_workspace_size(int32_t kind, int32_t M, int32_t N, int32_t K, size_t* bytes);
int32_t scr_linear_affine_b4(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                             int32_t M, int32_t N, int32_t K, int32_t group,
                             const uint16_t* bias_bf16, uint16_t* y_bf16,
                             void* workspace, size_t workspace_bytes, void* stream);
/* Up to 4 independent linears over the SAME activations — q, k, v of a layer; gate and up — as ONE launch: what the
 * reference gets by fusing the projections at load time (`load_rows_concat`, crates/targets/metal/src/layers_quant.rs:363-450)
 * without re-laying the weights.  Every member keeps its own packed buffer (`packed[i]`, [N[i], K]) and its own output
 * (`y[i]`, [M, N[i]] bf16); all share K, the group size and x.  Same bits per member as `scr_linear_affine_b4`.  Up to
 * 16 tokens one matvec launch runs over all members' rows; above, the members run one after the other (`workspace` as
 * for `scr_linear_affine_b4` at the largest member). */
int32_t scr_linear_affine_b4_group(scr_ctx* ctx, int32_t count, const void* const* packed, const uint16_t* x_bf16,
                                   int32_t M, const int32_t* N, int32_t K, int32_t group, uint16_t* const* y_bf16,
                                   void* workspace, size_t workspace_bytes, void* stream);
/* The fused gate/up projection with its activation, the `FusedGateUpSiluMul` end of the reference's
 * matvec (`QmvEnds`, crates/targets/metal/src/tape/step.rs:472-482; golden cpu_golden.rs:211-219):
 *   out[M, N2/2] (bf16) = silu(bf16(x @ gate^T)) * bf16(x @ up^T)
 * for a matrix of N2 rows that holds, per block of 16 rows, 8 gate rows then the 8 up rows of the
 * same channels (the Python mirror's `load_rows_interleave8`).  One launch; M <= 16 only
 * (SCR_E_UNSUPPORTED above: run `scr_linear_affine_b4` and `scr_silu_mul_pairs8_bf16`). */
int32_t scr_linear_affine_b4_silu_mul(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                                      int32_t M, int32_t N2, int32_t K, int32_t group,
                                      uint16_t* out_bf16, void* stream);

/* The one-row matvec with the ends the reference folds around it — `QmvEnds {norm, bias, scale, residual}`
 * (crates/targets/metal/src/tape/step.rs:472-498; shader crates/targets/metal/shaders/quantized_qmv.metal:60-112) — and,
 * on the output side, the gate/up pairing of `scr_linear_affine_b4_silu_mul`.  Up to 16 tokens (SCR_E_UNSUPPORTED above).
 *   norm_gain != NULL   x is the INPUT of an RMSNorm whose gain this is: every CTA normalises the rows into shared
 *                       memory as it loads them, with the arithmetic and summation order of `scr_rmsnorm_bf16`
 *                       (cpu_golden.rs:25-37), so the result is the bits of that operator followed by the plain linear
 *                       (the reference's fused kernel keeps x * gain in f32 instead, one rounding away from its own
 *                       unfused path).  Up to 8 tokens and M * K * 2 <= 20 KiB.
 *   bias, scale         sum + bias[n], then * scale, in f32 before the one rounding (scale 0 is read as 1)
 *   residual            y is the residual stream: y <- bf16(y + bf16(sum)), the bits of the separate add
 *                       (`fused_add_rmsnorm`'s residual, cpu_golden.rs:171-200)
 *   silu_pairs          the gate/up pairing (N = fused rows, y is [M, N/2]); excludes bias, scale and residual
 *   norm_row_scale      with `norm_gain`, which arithmetic the norm-in end uses.  0: the normalised row is formed and rounded
 *                       to bf16 exactly as `scr_rmsnorm_bf16` stores it, then dotted — the bits of the two separate operators,
 *                       at the price of every CTA finishing the row's sum of squares before its first product.  Non-zero: the
 *                       reference matvec's own form (crates/targets/metal/tests/affine_qmv_ends_test.rs:6-9, "dots x (.) gain
 *                       and scales the row by 1 / rms(x), so it skips the normed row's rounding"): the dot runs over
 *                       bf16(x * (gain + offset)) and the finished f32 sum is multiplied by 1 / sqrt(mean(x^2) + eps) before
 *                       the bias — as close to the exact W . rmsnorm(x) as the norm followed by the matvec is (the reference
 *                       test's bound: one rounding of the output plus 2 ulp of the row's sum of |terms|), not its bits. */
typedef struct scr_qmv_ends {
    const uint16_t* norm_gain;     /* [K] bf16 or NULL */
    float norm_eps;
    float norm_gain_offset;        /* rmsnorm(x, gain + offset) (`RowNorm.offset`) */
    const uint16_t* bias;          /* [N] bf16 or NULL */
    float scale;
    int32_t residual;
    int32_t silu_pairs;
    int32_t norm_row_scale;
} scr_qmv_ends;
int32_t scr_linear_affine_b4_ends(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16, int32_t M,
                                  int32_t N, int32_t K, int32_t group, const scr_qmv_ends* ends,
                                  uint16_t* y_bf16, void* stream);

/* The o / down projection with the residual add and the following RMSNorm folded in (the reference's
 * `QmvEnds` residual end, step.rs:472-482, and `fused_add_rmsnorm`, cpu_golden.rs:171-200), one launch:
 *   residual[M,N] <- bf16(residual + bf16(x @ W^T));  normed[M,N] <- rmsnorm(residual, gain, eps)
 * The last CTA to finish normalises the rows (partial sums of squares are added in CTA order:
 * deterministic).  `scratch`: SCR_ENDS_SCRATCH_BYTES of device memory, zeroed once by the caller before
 * the first call and left zeroed; calls that may overlap on the GPU need their own.  M <= 16 only
 * (SCR_E_UNSUPPORTED above: run `scr_linear_affine_b4` and `scr_fused_add_rmsnorm_bf16`); N % 8 == 0. */
#define SCR_ENDS_SCRATCH_BYTES 65536
int32_t scr_linear_affine_b4_residual_rmsnorm(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                                              int32_t M, int32_t N, int32_t K, int32_t group,
                                              uint16_t* residual, const uint16_t* gain, float eps,
                                              uint16_t* normed, void* scratch, size_t scratch_bytes,
                                              void* stream);

/* ---- a tape of matvecs in one launch ----------------------------------------
 * The reference runs a decode step as a tape of operators that is fixed at build time
 * (crates/targets/metal/src/tape/step.rs: one `Step` per dispatch, encoded back to back into one
 * command buffer).  `scr_affine_b4_tape_create` takes the int4 linears of such a tape — for each its
 * repacked matrix, x [max_rows, K] and y [max_rows, N] (bf16, device, fixed for the life of the
 * tape) and up to three earlier jobs it must wait for — and `scr_linear_affine_b4_tape` runs all of
 * them, M <= max_rows <= 16 rows each, inside ONE persistent kernel: y_j = x_j @ W_j^T in tape
 * order, a job starting once the jobs in dep[] have stored their outputs.  The caller names every
 * dependency: the producer of a job's x, and — when a buffer is reused — the earlier readers and
 * writers of its y.  Results are deterministic (fixed summation order) and within the matvec's
 * tolerance of `scr_linear_affine_b4`; create allocates and synchronises (load time), the run call
 * allocates nothing and can be captured in a CUDA graph.  A matrix repacked after create needs a
 * new tape.  Runs of one tape must not overlap on the GPU. */
typedef struct scr_tape scr_tape;
typedef struct scr_tape_linear {
    const void* packed;     /* scr_affine_b4_repack output */
    const uint16_t* x;      /* [max_rows, K] bf16 */
    uint16_t* y;            /* [max_rows, N] bf16 */
    int32_t N, K, group;
    int32_t dep[3];         /* indices of earlier jobs, -1 = none */
} scr_tape_linear;
int32_t scr_affine_b4_tape_create(scr_ctx* ctx, const scr_tape_linear* jobs, int32_t n_jobs,
                                  int32_t max_rows, scr_tape** out);
int32_t scr_linear_affine_b4_tape(scr_ctx* ctx, scr_tape* tape, int32_t M, void* stream);
int32_t scr_tape_destroy(scr_tape* tape);

/* ---- fp8-dynamic-per-channel: load-time repack ----------------------------
 * Replaces the `load_layered_fp8...` loaders the reference's codegen names but no live
 * target implements (Metal refuses fp8: crates/targets/metal/compiler/src/steps_from_tape.rs:2009).
 * Payload of `Fp8Linear` (crates/layers/src/layers.rs:179-191): `w_e4m3` FP8 E4M3 [N,K],
 * `w_scale` F32 [N] (per output channel).  `dst` receives the tiled layout the kernels
 * stream (`scr_fp8_repack_size` bytes, 128-byte aligned; the scales are copied into it). */
int32_t scr_fp8_repack_size(int32_t N, int32_t K, size_t* bytes);
int32_t scr_fp8_repack(scr_ctx* ctx, const uint8_t* w_e4m3, const float* w_scale, int32_t N,
                       int32_t K, void* dst, void* stream);

/* ---- fp8-dynamic-per-channel: per-token activation quantisation -----------
 * Replaces the shared W8A8 activation-quantise chain `fp8_quantize_descriptors`
 * (backends/spyre/crates/ktir/ktir-superdsc/src/emit/ktir_matmul_fp8.rs:123-322,430-531):
 *   a_scale[m] = min(max(absmax(x[m,:]) * (1/448), 1/448^2), 448);  x_q = e4m3(clip(x / a_scale, +-448))
 * with the reference encoder's rounding (backends/spyre/crates/ktir/ktir-core/src/codec.rs:1023-1070).
 * `act` is an opaque activation pack of `scr_fp8_act_size(M, K)` bytes that several
 * linears reading the same activation may share (the reference shares one quantise
 * across q/k/v and gate/up: ktir_matmul_fp8.rs:47-100). */
int32_t scr_fp8_act_size(int32_t M, int32_t K, size_t* bytes);
int32_t scr_fp8_quant_per_token(scr_ctx* ctx, const uint16_t* x_bf16, int32_t M, int32_t K,
                                void* act, void* stream);
/* RMSNorm fused with the quantisation: the activation pack of a W8A8 linear straight from the residual
 * stream (the reference quantises on the norm side for its W4A8 path,
 * crates/targets/metal/src/shaders/norm_w4a8_quant.h:1-12; norm golden cpu_golden.rs:25-37).  The codes and
 * a_scale are those `scr_fp8_quant_per_token` computes from bf16(rmsnorm(x)); `normed_bf16` (may be NULL)
 * receives that bf16 row as well, for consumers that are not quantised linears. */
int32_t scr_rmsnorm_fp8_quant(scr_ctx* ctx, const uint16_t* x_bf16, const uint16_t* gain, float eps,
                              int32_t M, int32_t K, void* act, uint16_t* normed_bf16, void* stream);
/* Test hook: unpack an activation pack to plain x_q [M,K] bytes and a_scale [M]. */
int32_t scr_fp8_act_unpack(scr_ctx* ctx, const void* act, int32_t M, int32_t K, uint8_t* xq,
                           float* a_scale, void* stream);
/* Test hook: the device e4m3 encoder on `count` f32 values (codec.rs:1023-1070). */
int32_t scr_e4m3_encode(scr_ctx* ctx, const float* v, int64_t count, uint8_t* out, void* stream);

/* ---- fp8-dynamic-per-channel: forward -------------------------------------
 * Replaces the arity-3 fp8 matmul body (ktir_matmul_fp8.rs:633-720; program
 * backends/spyre/kernels/matmul_fp8.py:46-82):
 *   y[m,n] (bf16) = ((sum_k x_q[m,k] * w_q[n,k]) * a_scale[m]) * w_scale[n],  f32 accumulation.
 * `scr_linear_fp8` consumes an activation pack; `scr_linear_fp8_dynamic` is the whole
 * generated Linear (quantise, then contract) and needs a workspace that holds the pack.  For
 * M <= 4 (and M*K <= 16 KiB of codes) the matvec quantises the activations itself — same x_q and
 * a_scale bits, one launch, the workspace is not touched.  `bias_bf16` (may be NULL) is the linear's
 * own bias [N] (`{prefix}.bias`; the q/k/v projections of Qwen2.5 carry one), added in f32 to the
 * dequantised sum before the one rounding. */
int32_t scr_linear_fp8(scr_ctx* ctx, const void* packed, const void* act, int32_t M, int32_t N,
                       int32_t K, const uint16_t* bias_bf16, uint16_t* y_bf16, void* workspace,
                       size_t workspace_bytes, void* stream);
int32_t scr_linear_fp8_dynamic(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16, int32_t M,
                               int32_t N, int32_t K, const uint16_t* bias_bf16, uint16_t* y_bf16,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ---- tensor parallel: row-parallel partials --------------------------------
 * A row-parallel linear (o, down) holds a K-slice of the weight and yields a `Partial`
 * (crates/compiler/subtile/src/tensor_parallel.rs:508-625): these variants write the UNROUNDED
 * f32 sums [M,N] instead of bf16, the caller all-reduces them over the ranks (the reference's
 * meaning: a sum in rank order, tensor_parallel.rs:1350-1362) and rounds once with
 * `scr_partial_to_bf16`.  Same arguments otherwise as `scr_linear_affine_b4` / `scr_linear_fp8`. */
int32_t scr_linear_affine_b4_partial(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                                     int32_t M, int32_t N, int32_t K, int32_t group, float* y_f32,
                                     void* workspace, size_t workspace_bytes, void* stream);
int32_t scr_linear_fp8_partial(scr_ctx* ctx, const void* packed, const void* act, int32_t M,
                               int32_t N, int32_t K, float* y_f32, void* workspace,
                               size_t workspace_bytes, void* stream);
/* The whole row-parallel fp8 linear in one call: quantise this rank's K-slice per token (inside the
 * matvec for M <= 4, where no pack is written), contract, f32 partials out. */
int32_t scr_linear_fp8_dynamic_partial(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                                       int32_t M, int32_t N, int32_t K, float* y_f32,
                                       void* workspace, size_t workspace_bytes, void* stream);
int32_t scr_partial_to_bf16(scr_ctx* ctx, const float* in, int64_t count, uint16_t* out_bf16,
                            void* stream);

/* ---- the operators either side of the linears in one decode step -----------
 * bf16 activations, f32 arithmetic.  Each replaces the device instruction whose host golden
 * is the cited function of crates/targets/metal/src/cpu_golden.rs ("Mirrors
 * `Instruction::<Name>` (CUDA) and Metal `KernelId::<Name>`").  Row strides `ld_*` are in
 * elements, so q / k / v may be column slices of one fused projection output.  Token ids,
 * positions, slots and block ids are checked on the device: an out-of-range value records a
 * code that `scr_device_status` reports as SCR_E_ARG, and the access is skipped. */
/* `embed` (cpu_golden.rs:114-124): out[i,:] = table[ids[i],:].  hidden % 8 == 0. */
int32_t scr_embed_bf16(scr_ctx* ctx, const uint32_t* ids, int32_t n_ids, const uint16_t* table,
                       int32_t vocab, int32_t hidden, uint16_t* out, void* stream);
/* `rmsnorm` (cpu_golden.rs:25-37) over `rows` rows: out = x * (1/sqrt(mean(x^2)+eps)) * weight. */
int32_t scr_rmsnorm_bf16(scr_ctx* ctx, const uint16_t* x, const uint16_t* weight, uint16_t* out,
                         int32_t rows, int32_t hidden, float eps, void* stream);
/* `fused_add_rmsnorm` (cpu_golden.rs:171-200): residual += delta in place (stored as bf16), out =
 * rmsnorm(residual as stored).  `out` may be `delta` (the reference writes the norm there). */
int32_t scr_fused_add_rmsnorm_bf16(scr_ctx* ctx, uint16_t* residual, const uint16_t* delta,
                                   const uint16_t* weight, uint16_t* out, int32_t rows,
                                   int32_t hidden, float eps, void* stream);
/* `fused_gate_up_silu_mul` (cpu_golden.rs:211-219): out[r,i] = gate[r,i]/(1+exp(-gate[r,i])) * up[r,i];
 * gate and up have row stride ld_in (halves of one fused gate/up output), out is dense [rows, inter]. */
int32_t scr_silu_mul_bf16(scr_ctx* ctx, const uint16_t* gate, const uint16_t* up, int64_t ld_in,
                          uint16_t* out, int32_t rows, int32_t inter, void* stream);
/* The same on a fused gate/up output whose columns interleave gate and up in runs of 8 (8 gate
 * columns, then the 8 up columns of the same channels) — the row order `scr_linear_affine_b4_silu_mul`
 * expects of its matrix; used above 16 tokens, where that fused epilogue is not available. */
int32_t scr_silu_mul_pairs8_bf16(scr_ctx* ctx, const uint16_t* gate_up, int64_t ld_in, uint16_t* out,
                                 int32_t rows, int32_t inter, void* stream);
/* `rope_append` (cpu_golden.rs:289-362): NeoX pairing, f32 cos/sin tables [max_pos, head_dim]
 * (first half of each row read); q_out = rotated q (may be q itself); rotated k and unrotated v
 * go to global slot slot_mapping[t] of the paged caches [num_blocks, num_kv_heads, block_size,
 * head_dim] (crates/targets/metal/src/paged_kv_layout.rs:74-115).  The stored bf16 values are
 * exactly the bf16 roundings of the golden's f32 results. */
int32_t scr_rope_append_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q, const uint16_t* k,
                             int64_t ld_k, const uint16_t* v, int64_t ld_v,
                             const uint32_t* positions, const uint32_t* slot_mapping,
                             const float* cos_table, const float* sin_table, int32_t max_pos,
                             uint16_t* q_out, int64_t ld_qo, uint16_t* cache_k, uint16_t* cache_v,
                             int32_t num_blocks, int32_t num_tokens, int32_t num_q_heads,
                             int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                             void* stream);
/* `attention_via_cache` (cpu_golden.rs:386-460): one query token per sequence over the paged
 * cache through block_table [batch, max_blocks_per_seq] and seq_used_k [batch]; softmax with
 * inv_sum = 1/(sum_exp + 1e-6); seq_used_k == 0 yields zeros.  head_dim 64 or 128, up to 8
 * query heads per kv head.  block_table and seq_used_k are runtime bindings the host writes before
 * the step (the reference's `BlockTable` / `SeqUsedK`): the kernel reads them, and streams every
 * cache block except each sequence's last one, while the previous kernels of the stream may still
 * be running — those kernels may produce q and the cache slot of token seq_used_k - 1 (what
 * `scr_rope_append_bf16` does in a decode step), nothing else this call reads. */
int32_t scr_attention_via_cache_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q,
                                     const uint16_t* cache_k, const uint16_t* cache_v,
                                     int32_t num_blocks, const uint32_t* block_table,
                                     const uint32_t* seq_used_k, uint16_t* out, int64_t ld_o,
                                     int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                     int32_t head_dim, int32_t block_size,
                                     int32_t max_blocks_per_seq, float attn_scale, void* stream);
/* `rope_append` (cpu_golden.rs:289-362) followed by `attention_via_cache` (cpu_golden.rs:386-460) as
 * ONE launch for a decode step: q, k, v are the unrotated outputs of the QKV projection (one token
 * per sequence); the kernel rotates q in registers, rotates k and stores it and v into the cache
 * slot of token seq_used_k[b] - 1 of sequence b (block block_table[b][(seq_used_k[b]-1) /
 * block_size], i.e. the slot the reference's slot_mapping names for that token), and attends over
 * the seq_used_k[b] tokens including it.  q is left unrotated.  The cache contents and `out` are
 * the same bits as the two separate calls give.  Needs block_size a multiple of 16 (<= 256);
 * SCR_E_UNSUPPORTED otherwise — call the two operators separately then. */
int32_t scr_rope_attention_via_cache_bf16(scr_ctx* ctx, const uint16_t* q, int64_t ld_q,
                                          const uint16_t* k, int64_t ld_k, const uint16_t* v,
                                          int64_t ld_v, const uint32_t* positions,
                                          const float* cos_table, const float* sin_table,
                                          int32_t max_pos, uint16_t* cache_k, uint16_t* cache_v,
                                          int32_t num_blocks, const uint32_t* block_table,
                                          const uint32_t* seq_used_k, uint16_t* out, int64_t ld_o,
                                          int32_t batch, int32_t num_q_heads, int32_t num_kv_heads,
                                          int32_t head_dim, int32_t block_size,
                                          int32_t max_blocks_per_seq, float attn_scale,
                                          void* stream);
/* Greedy sampling (crates/targets/metal/tests/argmax_split_test.rs:24-33): per row the id of the
 * largest value, the smallest id among equal ones, NaN never. */
int32_t scr_argmax_bf16(scr_ctx* ctx, const uint16_t* logits, int64_t ld, int32_t rows,
                        int32_t width, uint32_t* out, void* stream);

/* ---- tensor parallel: the exchange step of a decode layer ---------------------
 * `SubOp::AllReduce` after a row-parallel linear (crates/compiler/subtile/src/tensor_parallel.rs:
 * 1342-1393): the ranks' f32 partials are summed in rank order 0..W-1 and rounded once.  For decode
 * sizes this is one kernel per rank over NVLink peer memory (every rank stores its partials into a
 * slot it owns on every rank, publishes a flag, waits — bounded — for the others, sums): the result
 * is the rank-ordered sum bit for bit on every rank.  One process per GPU: each creates its
 * communicator (the buffer is allocated here, once), the host exchanges the 64-byte handles by any
 * means (the Python mirror uses torch.distributed) and every rank connects.  All ranks must issue
 * the same sequence of all-reduce calls.  `count` <= `max_elems`, both multiples of 4. */
#define SCR_TP_HANDLE_BYTES 64
typedef struct scr_tp_comm scr_tp_comm;
int32_t scr_tp_comm_create(scr_ctx* ctx, int32_t world, int32_t rank, int64_t max_elems,
                           scr_tp_comm** out, uint8_t* handle_out /* SCR_TP_HANDLE_BYTES */);
int32_t scr_tp_comm_connect(scr_tp_comm* comm, const uint8_t* handles /* world x SCR_TP_HANDLE_BYTES */);
/* The same for ranks that are THREADS OF ONE PROCESS — how the reference's executor drives its ranks
 * (crates/serving/worker/src/threadpool.rs:1-16, crates/serving/worker/src/parallel.rs:103-150): an IPC handle
 * opens only in another process, so such ranks exchange raw device pointers.  Every rank reads its own
 * `scr_tp_comm_base`; each then calls `scr_tp_comm_connect_local` with all `world` bases and the devices they
 * live on, its own device current (peer access is enabled here). */
int32_t scr_tp_comm_base(scr_tp_comm* comm, void** base);
int32_t scr_tp_comm_connect_local(scr_tp_comm* comm, void* const* peer_bases /* world */,
                                  const int32_t* peer_devices /* world */);
/* Failure detection, the device half of the executor's health check (crates/serving/engine/src/executor.rs:454):
 * a kernel of this communicator polls at most `polls` times for a peer's data, then records a code in the
 * context's status word (`scr_device_status` reports SCR_E_TIMEOUT) and runs to its end — nothing hangs, the
 * call's results are garbage, the call counter still advances and the next call works.  While the status word
 * is set every bounded wait on this context gives up early, so read (and thereby clear) it with
 * `scr_device_status` once per step, after the host has synchronised on the step's result anyway. */
int32_t scr_tp_comm_set_wait_limit(scr_tp_comm* comm, uint32_t polls);
/* y_bf16 and/or y_f32 receive the reduced [count] values (either may be NULL, not both). */
int32_t scr_tp_allreduce_partial(scr_tp_comm* comm, const float* partial, int64_t count,
                                 uint16_t* y_bf16, float* y_f32, void* stream);
/* The other collective of the reference's placement lattice, `SubOp::AllGather{cols}`
 * (crates/compiler/subtile/src/tensor_parallel.rs:1363-1386): an N-split projection (the vocabulary head) restores
 * its full width.  Every rank passes its [rows, lc] bf16 column block; every rank receives
 *   y[rows, cols] = the ranks' blocks side by side in absolute rank order, cropped to `cols`
 * (world * lc >= cols: a padded last block's tail is cut off).  One launch over peer memory; a block holds at most
 * 2 * min(max_elems, 524288) values.  Counts as one call in the communicator's call sequence. */
int32_t scr_tp_allgather_cols(scr_tp_comm* comm, const uint16_t* local_bf16, int64_t rows, int64_t lc,
                              int64_t cols, uint16_t* y_bf16, void* stream);
int32_t scr_tp_comm_destroy(scr_tp_comm* comm);
/* A row-parallel fp8-dynamic linear and its all-reduce as ONE launch, for decode sizes: the matvec's
 * epilogue stores its f32 partial sums straight into every rank's receive buffer over NVLink, and
 * each CTA then sums the ranks' copies of its own rows in rank order and rounds once
 *   y[M,N] (bf16) = round( sum over ranks r, in order, of  x_r[M,K_r] @ W_r^T ).
 * Same bits as `scr_linear_fp8_dynamic_partial` followed by `scr_tp_allreduce_partial`.  Every rank
 * calls it with the same M and N, in the same order as its other calls on `comm`; M * N <= the
 * communicator's max_elems.  Covers what the self-quantising matvec covers (M <= 4 and M * K16 <=
 * 14 KiB); SCR_E_UNSUPPORTED otherwise — run the two calls then. */
int32_t scr_linear_fp8_dynamic_allreduce(scr_tp_comm* comm, const void* packed, const uint16_t* x_bf16,
                                         int32_t M, int32_t N, int32_t K, uint16_t* y_bf16, void* stream);

/* No counterpart in the reference.  The same linear as `scr_linear_fp8_dynamic` for callers
 * that cannot allocate device memory on the step path (an arena-owning runtime, code inside a
 * no-allocation region, an FFI shim that owns only inputs and outputs): the activation pack
 * lives in a fixed 8 MiB device array built into the library, so no workspace is passed and
 * nothing is allocated.  Requests whose pack exceeds 8 MiB return SCR_E_WORKSPACE.  The first
 * call on a device resolves the array's address; make it before any stream capture, with the
 * context's device current.  All calls share the array (it keeps the last call's contents), so
 * calls that overlap on the GPU race: serialise them. */
int32_t scr_linear_fp8_dynamic_static(scr_ctx* ctx, const void* packed, const uint16_t* x_bf16,
                                      int32_t M, int32_t N, int32_t K, uint16_t* y_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SCRATCHY_CUDA_H_ */
