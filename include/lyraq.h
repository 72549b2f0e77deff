/*
 * lyraq — C ABI of the B200 (sm_100a) quantized-linear path.
 *
 * Every entry point takes plain device pointers and sizes, is asynchronous on the CUDA
 * stream it is given (passed as void*, i.e. a cudaStream_t; NULL = the default stream),
 * allocates nothing, never throws and returns a lyraq_status_t.  Unsupported shapes are
 * refused with an error code before anything is launched; nothing is silently skipped.
 * Tensor element types are named by lyraq_dtype_t.  "rows" is batch*sequence, flattened.
 *
 * Each declaration names the reference interface (file:line within lyraDiff's source
 * tree) that it replaces.
 */
#ifndef LYRAQ_H_
#define LYRAQ_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define LYRAQ_API __attribute__((visibility("default")))
#else
#define LYRAQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    LYRAQ_OK = 0,
    LYRAQ_ERR_INVALID_ARG = 1,    /* null pointer, bad enum, misaligned pointer */
    LYRAQ_ERR_UNSUPPORTED = 2,    /* shape outside what the kernels cover */
    LYRAQ_ERR_CUDA = 3,           /* a CUDA runtime/driver call failed */
    LYRAQ_ERR_DEVICE_TIMEOUT = 4, /* a bounded wait inside a kernel ran out (see lyraq_last_status) */
    LYRAQ_ERR_WORKSPACE = 5       /* workspace missing or too small */
} lyraq_status_t;

typedef enum {
    LYRAQ_F16 = 0,
    LYRAQ_BF16 = 1,
    LYRAQ_F32 = 2,
    LYRAQ_S32 = 3,
    LYRAQ_E4M3 = 4 /* FP8 e4m3 codes, one byte each (only where an entry point says so) */
} lyraq_dtype_t;

/* How the activation scale of an INT8 quantize / GEMM is given. */
typedef enum {
    LYRAQ_SCALE_PER_TENSOR = 0,       /* one fp32 scalar on the device */
    LYRAQ_SCALE_PER_TOKEN = 1,        /* fp32 [rows], precomputed */
    LYRAQ_SCALE_PER_TOKEN_DYNAMIC = 2 /* fp32 [rows], computed by the kernel as amax/127 and written out */
} lyraq_scale_mode_t;

/* Epilogue flags of the GEMMs (bit set). */
enum {
    LYRAQ_EPI_NONE = 0,
    LYRAQ_EPI_GELU_TANH = 1, /* tanh-GELU after bias (and after beta*residual, as cuBLASLt orders it) */
    LYRAQ_EPI_ROUND_EACH = 2 /* W4A4 entry points only: round to the output type after the accumulate, after the bias,
                              * after the GELU and after the residual, i.e. the bits the reference gets from its GEMM
                              * followed by separate 16-bit kernels (invokeFusedBiasAndGelu, invokeFusedBiasAndResidual,
                              * src/lyradiff/kernels/flux_single_transformer_block/flux_single_transformer_kernels.cu:68-134;
                              * the bias add of fuseBiasRmsNormAndRope, kernels/rope/flux_apply_rope.cu:203-205).
                              * Without it the epilogue rounds once. */
};

LYRAQ_API const char* lyraq_version(void);
LYRAQ_API const char* lyraq_status_string(int status);

/* Reads (and clears) the device-side status word of the current device after synchronising
 * `stream`: LYRAQ_OK, or LYRAQ_ERR_DEVICE_TIMEOUT with *detail (may be NULL) = which wait gave up.
 * The reference has no counterpart: its kernels have no bounded waits. */
LYRAQ_API int lyraq_last_status(void* stream, uint32_t* detail);

/* Text of the last CUDA runtime / driver error that made an entry point return LYRAQ_ERR_CUDA (which call, the
 * error string and name).  Process-wide, for diagnostics.  The reference prints such errors to its log
 * (check_cuda_error, src/lyradiff/utils/cuda_utils.h:62-90); this is the same information as a string. */
LYRAQ_API const char* lyraq_last_cuda_error(void);

/* Debug / measurement hook (no counterpart in the reference): every kernel of the library is launched so that it may
 * begin while the kernel before it on the stream is still draining (programmatic dependent launch: the kernel's
 * set-up overlaps its predecessor's tail, and it waits for the predecessor's completion before it first touches
 * global memory).  on = 0 launches them as ordinary stream-ordered kernels instead; on = 1 (default) restores it. */
LYRAQ_API int lyraq_debug_set_dependent_launch(int on);

/* Test / sweep hook: force the tile configuration of the dense GEMMs.  0 = automatic (default); 2561 = one CTA,
 * 128 x 256 tile; 1281 = one CTA, 128 x 128; 2562 = CTA pair, 256 x 256.  Process-wide, not thread-safe.
 * No counterpart in the reference API; it plays the role of choosing a tactic by hand, which the reference does
 * through CutlassGemmConfig (src/lyradiff/kernels/cutlass_extensions/include/cutlass_extensions/gemm_configs.h:101-130). */
LYRAQ_API int lyraq_debug_force_gemm_tile(int code);

/* Test hook for the bounded waits (process-wide, not thread-safe): with skip_loads != 0 the attention kernel's producer
 * issues no copy, so every consumer's wait runs out after wait_limit_ms (0 = the default of 2 s) -- the non-faulting way
 * to run the path a timed-out wait takes: the kernel records LYRAQ_ERR_DEVICE_TIMEOUT in the status word, raises its
 * block-wide abort flag, all roles leave, tensor memory is freed and the kernel returns without having written anything.
 * (0, 0) restores normal operation.  It has no counterpart in the reference, whose kernels have no bounded waits. */
LYRAQ_API int lyraq_debug_attention_wait_test(int skip_loads, unsigned int wait_limit_ms);

/* Test / sweep hook for the row kernels (quantize, LayerNorm, AdaLN, GEGLU): the most 16-byte vectors one thread
 * holds (4 or 6, default 6) before a row is given to a team twice as large.  Process-wide, not thread-safe.
 * No counterpart in the reference, whose kernels fix columns-per-thread per supported width
 * (src/lyradiff/kernels/quant_kernels/layer_norm_int8.cu:558-617). */
LYRAQ_API int lyraq_debug_set_row_vectors_per_thread(int max_vpt);

/* Test hook: some calls have kernels of their own beside the general row kernel -- AdaLN over rows of 3072 elements with
 * a quantized output (the FLUX form; one warp per row); bias + GEGLU -> int8 and the int8 quantize with a static or a
 * given per-token scale (no row statistic, so no row loop); the dynamically scaled int8 quantize and LayerNorm -> int8
 * over rows of 320, 640 or 1280 columns (8, 16 or 32 lanes per row).  All give the general kernel's bytes except the
 * short-row LayerNorm, which differs in the order of its two fp32 sums.  on = 0 sends those calls through the general
 * row kernel instead, so that a test can compare the two; on = 1 (default) restores it.  Process-wide, not thread-safe.
 * It has no counterpart in the reference (one kernel each: src/lyradiff/kernels/norms/layer_norm.cu:405-484,
 * src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.cu:189-290). */
LYRAQ_API int lyraq_debug_set_special_row_kernels(int on);

/* ------------------------------------------------------------------ activation quantizers */

/* INT8 SmoothQuant activation quantize: q = sat_s8(rne(float(x)*pre[c] / s)).
 * Replaces invokeSqInputQuant<T> (src/lyradiff/kernels/quant_kernels/quant_kernels.h:9-17;
 * kernels quant_kernels.cu:51-115).  pre_quant_scale may be NULL (= ones).
 * scale_mode PER_TENSOR / PER_TOKEN read `scale`; PER_TOKEN_DYNAMIC writes `scale` [rows].
 * dim must be a multiple of 8 and at most 16384. */
LYRAQ_API int lyraq_quant_int8(int8_t* dst, const void* src, int src_dtype, const float* pre_quant_scale,
                     float* scale, int scale_mode, size_t rows, size_t dim, void* stream);

/* Per-tensor static-scale conversion to e4m3: dst = e4m3_rne_satfinite(float(src) * r),
 * r = 1/scale[0] if invert_scale else scale[0].
 * Replaces invokeCudaD2DScaleCpyConvert<Tin, __nv_fp8_e4m3> (src/lyradiff/utils/memory_utils.h:74;
 * kernel memory_utils.cu:431-446). */
LYRAQ_API int lyraq_quant_fp8(uint8_t* dst, const void* src, int src_dtype, const float* scale, int invert_scale,
                    size_t n, void* stream);

/* scale[0] = max(scale[0], max|w| / 448).  The caller zeroes scale[0] first, as the reference does.
 * Replaces invokeGetFP8WeightScale (src/lyradiff/kernels/lora/load_lora.cu:49-54,109-113). */
LYRAQ_API int lyraq_fp8_amax_scale(float* scale, const void* w, int w_dtype, size_t n, void* stream);

/* FP8 weight quantize in one call, all on `stream` and without a host round trip: scale[0] = max|w| / 448, then
 * qw = e4m3(w / scale[0]).  What MACROLoadFP8WeightFromCache does with a memset, invokeGetFP8WeightScale and
 * invokeCudaD2DScaleCpyConvert (src/lyradiff/utils/common_macro_def.h:76-92), and what a LoRA swap repeats for every
 * merged weight (src/lyradiff/interface/IFLoraWeight.h:80-128). */
LYRAQ_API int lyraq_weight_quant_fp8(uint8_t* qw, float* scale, const void* w, int w_dtype, size_t n, void* stream);

/* INT4 activation quantize, groups of 64 along K: v = float(x)/smooth[c]; s = max|v|/7; q = sat_s4(rne(v/s)).
 * q: packed [m, k/2] bytes (even element in the low nibble), q_scale: fp32 [m, k/64].
 * Replaces the quantize half of invokeFusedQuantizeAndLoraDownSimple
 * (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:6-17; kernel w4a4_gemm.cu:769-954).
 * smooth may be NULL (= ones).  If lora_down (bf16/f16 [32, k], same type as x) and lora_act
 * (fp32 [m, 32]) are both non-NULL, lora_act = x * lora_down^T is also produced (deterministic,
 * overwritten not accumulated).  k must be a multiple of 64. */
LYRAQ_API int lyraq_quant_int4_g64(uint8_t* q, float* q_scale, float* lora_act, const void* x, int x_dtype,
                         const float* smooth, const void* lora_down, size_t m, size_t k, void* stream);

/* ------------------------------------------------------------------ load-time weight quantizers */

/* Per-output-channel INT8 weight quantize: w' = w/pre[c]; s_w[n] = amax_n/127; q = sat_s8(rne(w'/s_w)).
 * Replaces invokeGetINT8WeightScale<T> (src/lyradiff/kernels/quant_kernels/quant_kernels.cu:173-223,270-312).
 * pre_quant_scale may be NULL. */
LYRAQ_API int lyraq_weight_quant_int8(float* w_scale, int8_t* qw, const void* w, int w_dtype, const float* pre_quant_scale,
                            size_t d_out, size_t d_in, void* stream);

/* INT4 group-64 weight quantize into the layout W4A4GemmWeight holds
 * (src/lyradiff/layers/w4a4_gemm_block/W4A4GemmWeight.h:8-45): packed [n, k/2], scales [n, k/64]
 * of scale_dtype (LYRAQ_F32 or LYRAQ_F16).  The reference has no device quantizer for this format. */
LYRAQ_API int lyraq_weight_quant_int4_g64(uint8_t* qw, void* w_scale, int scale_dtype, const void* w, int w_dtype,
                                size_t n, size_t k, void* stream);

/* ------------------------------------------------------------------ fused producers */

/* AdaLN-Zero modulation y = LN(x)*(1+scale_b)+shift_b (eps, no affine), x [B,S,D], scale/shift [B,D].
 * Replaces invokeLayerNormWithShiftAndScale<T> (src/lyradiff/kernels/norms/layer_norm.h:19; kernel
 * layer_norm.cu:405-484), fused with the quantize pass that follows it in the reference
 * (memory_utils.cu:431-446 / quant_kernels.cu:93-115).  Any of the three outputs may be NULL:
 *   y     [B*S, D] of dtype                       (the un-quantized result)
 *   q8    int8 [B*S, D] with q8_scale fp32 [B*S]  (dynamic per-token, amax/127; pre_quant_scale optional)
 *   qf8   e4m3 [B*S, D] with f8_scale fp32 [1]    (static per-tensor, dst = y / f8_scale[0])
 * D must be a multiple of 8 and at most 16384. */
LYRAQ_API int lyraq_adaln_quant(void* y, int8_t* q8, float* q8_scale, uint8_t* qf8, const float* f8_scale,
                      const void* x, const void* scale, const void* shift, int dtype,
                      const float* pre_quant_scale, size_t B, size_t S, size_t D, double eps, void* stream);

/* lyraq_adaln_quant with two e4m3 outputs of the same modulated row, each with its own static scale: in the FLUX
 * single-stream block the AdaLN output feeds both to_qkv and proj_mlp, whose calibrated input scales differ, and the
 * reference quantizes it twice (FluxSingleAttentionFP8Processor.cc:155 and FluxSingleTransformerFP8Block.cc:216 of
 * src/lyradiff/layers/...).  y (the 16-bit result) may be NULL. */
LYRAQ_API int lyraq_adaln_quant_fp8x2(void* y, uint8_t* qa, const float* scale_a, uint8_t* qb, const float* scale_b,
                                      const void* x, const void* scale, const void* shift, int dtype, size_t B, size_t S,
                                      size_t D, double eps, void* stream);

/* (residual + bias +) LayerNorm(gamma, beta) -> int8 with a static scalar scale.
 * Replaces invokeLayerNormInt8O<T> and invokeFusedResidualBiasLayerNormInt8O<T>
 * (src/lyradiff/kernels/quant_kernels/layer_norm_int8.h:9-38; launchers layer_norm_int8.cu:558-679).
 * residual/bias may be NULL; when residual is given, sum_out (dtype [rows, dim], may alias x) receives x+residual+bias. */
LYRAQ_API int lyraq_ln_quant_int8(int8_t* dst, void* sum_out, const void* x, const void* residual, const void* bias,
                        const void* gamma, const void* beta, int dtype, const float* pre_quant_scale,
                        const float* input_quant_scale, size_t rows, size_t dim, double eps, void* stream);

/* bias + GEGLU (tanh-GELU) -> int8: h [rows, 2*dim] -> dst [rows, dim], static scalar scale.
 * Replaces invokeFusedAddBiasGegluInt8O<T> (src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.h:13-21;
 * kernels ffn_kernels_int8.cu:15-187).  bias ([2*dim]) may be NULL. */
LYRAQ_API int lyraq_geglu_quant_int8(int8_t* dst, const void* h, const void* bias, int dtype, const float* pre_quant_scale,
                           const float* input_quant_scale, size_t rows, size_t dim, void* stream);

/* ------------------------------------------------------------------ GEMMs (tcgen05, accumulators in TMEM) */

/* Operation codes for lyraq_workspace_bytes. */
enum {
    LYRAQ_OP_GEMM_INT8 = 0,
    LYRAQ_OP_GEMM_FP8 = 1,
    LYRAQ_OP_GEMM_W4A4 = 2,
    LYRAQ_OP_LINEAR_INT8 = 3,
    LYRAQ_OP_LINEAR_FP8 = 4,
    LYRAQ_OP_LINEAR_W4A4 = 5,
    LYRAQ_OP_LINEAR_W4A4_LORA = 6
};

/* Bytes of workspace an operation needs for (m, n, k).  0 for the bare GEMMs (no split-K; the call is kept so that
 * callers written against the reference's getWorkspaceSize, int8_gemm_template.h:683-692, keep working); for the
 * LINEAR_* layer forwards below, the size of the quantized activation plus its scales. */
LYRAQ_API size_t lyraq_workspace_bytes(int op, int m, int n, int k);

/* INT8 W8A8: C[m,n] = T( T(float(sum_k A[m,k]*B[n,k]) * (alpha_col[n]*alpha_row)) + bias[n] ).
 * A int8 [m,k] row-major, B int8 [n,k] (K contiguous), int32 accumulation (exact), alpha_col fp32 [n],
 * alpha_row fp32 [1] or [m] (row_scale_mode PER_TENSOR / PER_TOKEN), bias of c_dtype [n] or NULL.
 * c_dtype F16/BF16/F32, or S32 to get the raw accumulators (scales and bias ignored).
 * Replaces cublasMMWrapper::runGemmInt8 (src/lyradiff/utils/cublasMMWrapper.h:368-385) ->
 * SmoothQuantGemmPlugin<T>::RunGemm (layers/gemm_utils/SmoothQuantGemm.cc:108-163) ->
 * CutlassInt8GemmRunner<T>::gemm (kernels/cutlass_kernels/int8_gemm/int8_gemm_template.h:643-672).
 * k must be a multiple of 16; A and B 16-byte aligned; C 16-byte aligned. */
LYRAQ_API int lyraq_gemm_int8(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row,
                    int row_scale_mode, void* C, int c_dtype, const void* bias, int m, int n, int k,
                    void* workspace, size_t workspace_bytes, void* stream);

/* lyraq_gemm_int8 with the residual add that follows the feed-forward output linear of the SDXL INT8 blocks fused in:
 * C[m,n] = T( T( T(acc * (alpha_col[n]*alpha_row)) + R[m,n] ) + bias[n] ), every step rounded to T as the reference's
 * separate kernel does (fusedBiasResidualAdd, src/lyradiff/kernels/basic_transformer/basic_transformer_kernels.cu:183-215,
 * called at layers/basic_transformer/BasicTransformerInt8Block.cc:824-845).  R of c_dtype [m,n] or NULL; C may alias R.
 * c_dtype F16/BF16/F32. */
LYRAQ_API int lyraq_gemm_int8_residual(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row,
                                       int row_scale_mode, void* C, int c_dtype, const void* bias, const void* residual,
                                       int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream);

/* FP8 e4m3: Y[m,n] = T( epi( alpha*s_x[0]*s_w[0] * sum_k X[m,k]*W[n,k] + beta*R[m,n] + bias[n] ) ),
 * fp32 accumulation, epi = identity or tanh-GELU (epilogue flags), bias/R of c_dtype or NULL.
 * Replaces cublasMMWrapper::GemmWithResidualAndBias for __nv_fp8_e4m3
 * (src/lyradiff/utils/cublasMMWrapper.h:300-317, .cc:1104-1276), in its only calling form
 * (OP_T, OP_N, n, m, k, W, k, s_w, X, k, s_x, Y, n, bias, R, alpha, beta, is_gelu). */
LYRAQ_API int lyraq_gemm_fp8(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, int c_dtype,
                   const void* bias, const void* residual, float alpha, float beta, int epilogue,
                   int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream);

/* FP8 GEMM with the block's gate and residual fused in: Y[m,n] = T( T( T(s_w*s_x*acc + bias[n]) * gate[b,n] ) + R[m,n] ),
 * b = m / rows_per_batch, every step rounded to T as the reference's separate kernel does.  Replaces
 * GemmWithResidualAndBias followed by invokeFusedGateAndResidual<T>
 * (src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:262-303;
 * kernel flux_single_transformer_kernels.cu:43-65).  gate of type T [batches, n]; R of type T [m,n] or NULL; Y may alias R.
 * When m spans several batch entries rows_per_batch must be a multiple of 256 (LYRAQ_ERR_UNSUPPORTED otherwise: use
 * lyraq_gemm_fp8 + lyraq_gate_residual). */
LYRAQ_API int lyraq_gemm_fp8_gate(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, int c_dtype,
                                  const void* bias, const void* gate, const void* residual, int rows_per_batch, int m, int n,
                                  int k, void* workspace, size_t workspace_bytes, void* stream);

/* lyraq_gemm_fp8 with the activation quantize of the NEXT FP8 linear fused into the epilogue:
 * Yq[m,n] = e4m3_rne_satfinite( float( T( epi(...) ) ) / y_scale[0] ), T = dtype (the type of bias and residual, and the
 * type the reference would have stored Y in).  Replaces the sequence GemmWithResidualAndBias -> (GELU kernel) ->
 * invokeCudaD2DScaleCpyConvert that the FLUX FP8 blocks run between two chained linears
 * (src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:227-281,
 * src/lyradiff/layers/flux_attn_post_processor/FluxAttnPostFP8Processor.cc:146-195): the 16-bit Y never goes to memory. */
LYRAQ_API int lyraq_gemm_fp8_quant(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, uint8_t* Yq,
                                   const float* y_scale, int dtype, const void* bias, const void* residual, float alpha,
                                   float beta, int epilogue, int m, int n, int k, void* workspace, size_t workspace_bytes,
                                   void* stream);

/* lyraq_gemm_fp8_quant whose e4m3 output is a column window of a wider matrix: row m of the result starts at
 * Yq + m * ldy (ldy >= n bytes, a multiple of 16 for the fast path).  This is how the MLP activation lands next to the
 * attention output in the [tokens, 15360] input of proj_out without the 16-bit concat the reference builds
 * (invokeFusedCatAndGelu + invokeCudaD2DScaleCpyConvert,
 * src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:245-260).  residual must be
 * NULL when ldy != n. */
LYRAQ_API int lyraq_gemm_fp8_quant_ld(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, uint8_t* Yq,
                                      size_t ldy, const float* y_scale, int dtype, const void* bias, const void* residual,
                                      float alpha, float beta, int epilogue, int m, int n, int k, void* workspace,
                                      size_t workspace_bytes, void* stream);

/* W4A4, groups of 64 along K: D[m,n] = T( epi( sum_g (float(sum_{k in g} a*b) * sa[m,g]) * sb[n,g]
 *                                              + lora_act[m,:] . lora_up[n,:] + bias[n] ) + R[m,n] ).
 * A packed int4 [m,k/2], B packed int4 [n,k/2], sa fp32 [m,k/64], sb [n,k/64] of sb_dtype (F32 or F16),
 * exact int32 per group, fp32 across groups in order g = 0..k/64-1.  lora_act [m,32] and lora_up (c_dtype, [n,32])
 * may both be NULL; lora_act_dtype is F32 (the down projection as lyraq_quant_int4_g64 wrote it; it is rounded to
 * c_dtype on the way in, which replaces the invokeCudaD2DcpyConvert of W4A4Gemm.cc:143) or c_dtype (already converted,
 * as the reference's caller passes it).  bias, R of c_dtype or NULL.
 * Replaces invokeFusedW4A4GemmAndLoraUp (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:19-30; kernels
 * w4a4_gemm.cu:227-767) and the bias/GELU/residual kernels that follow it
 * (kernels/flux_single_transformer_block/flux_single_transformer_kernels.cu:68-134); with LYRAQ_EPI_ROUND_EACH in
 * `epilogue`, T(.) is applied after every step as those kernels do: T(T(epi(T(T(sum + lora) + bias))) + R). */
LYRAQ_API int lyraq_gemm_w4a4(const uint8_t* A, const uint8_t* B, const float* sa, const void* sb, int sb_dtype,
                    void* D, int c_dtype, const void* lora_act, int lora_act_dtype, const void* lora_up,
                    const void* bias, const void* residual, int epilogue, int m, int n, int k,
                    void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ between the linears of a FLUX block
 * (the callers either side of the quantized-linear path) */

/* QK RMSNorm + rotary embedding on the packed QKV projection: qkv [batch, seq, 3, heads, head_dim] (q heads, k heads,
 * v heads), scale [2, head_dim] (q then k), rope [batch * seq, head_dim / 2, 2, 2]; q and k heads are normalised
 * (fp32 statistics, eps), scaled and rotated with every step rounded to T as the reference does, v heads are copied
 * (skipped when out == qkv).  head_dim 64 or 128.  Replaces invokeFusedRmsNormAndRope<T>
 * (src/lyradiff/kernels/rope/flux_apply_rope.h:20-30; kernel flux_apply_rope.cu:8-76). */
LYRAQ_API int lyraq_rmsnorm_rope(void* out, const void* qkv, const void* scale, const void* rope, int dtype, double eps,
                                 size_t batch, size_t seq_len, int heads, int head_dim, void* stream);

/* The QKV projection of a FLUX block with lyraq_rmsnorm_rope fused into its epilogue: Y[m, 0 .. n) (row pitch ldy
 * elements) = X W^T * (s_x s_w) + bias, rounded to T, and then, for the q and k heads (columns below 2 * heads * 128), the
 * RMSNorm with qk_norm [2, 128] and the rotation rope [m, 64, 2, 2] of row m, each step rounded as lyraq_rmsnorm_rope rounds
 * it; the bits equal those of lyraq_gemm_fp8 followed by lyraq_rmsnorm_rope in place.  n = 3 * heads * 128, 16-bit Y.
 * Replaces the pair of calls in FluxSingleTransformerFP8Block.cc:224-250 and FluxAttentionFP8Processor.cc (the to_qkv GEMM,
 * then invokeFusedRmsNormAndRope, src/lyradiff/kernels/rope/flux_apply_rope.h:20-30) with one launch and one pass
 * over the projection. */
LYRAQ_API int lyraq_gemm_fp8_qk_rope(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, size_t ldy,
                                     int c_dtype, const void* bias, const void* qk_norm, const void* rope, int heads, int head_dim,
                                     double eps, int m, int n, int k, void* stream);

/* Attention of the FLUX blocks over the packed projection qkv [batch, seq, 3, heads, head_dim] (q heads, k heads, v heads,
 * as lyraq_rmsnorm_rope leaves them): out[b, s, h, :] = softmax(q k^T * softmax_scale) v, no mask, head_dim 128, fp32
 * scores and accumulation on tcgen05, probabilities rounded to the 16-bit type for the second product.  The result is
 * rounded to `dtype` and written to out [batch, seq, heads * head_dim] with row pitch out_ld elements -- or, with
 * out_dtype LYRAQ_E4M3, quantized from that rounded value with 1 / out_scale[0] as lyraq_quant_fp8 does, straight into
 * the input of the FP8 linear that follows (a column window of a wider matrix when out_ld > heads * head_dim).  With
 * out2 != NULL the rows [split, seq) of every batch go to out2 (row s - split, pitch out2_ld, scale out2_scale) and only
 * rows [0, split) to out: the text and image parts of a joint sequence feed different linears.
 * Replaces FlashAttention2Layer<T>::forward (src/lyradiff/layers/flash_attn2/flash_attn2.cu:59-118, called at
 * layers/flux_single_attention_processor/FluxSingleAttentionFP8Processor.cc:213 and
 * layers/flux_attention_processor/FluxAttentionFP8Processor.cc:274) and the e4m3 cast of its output
 * (FluxSingleTransformerFP8Block.cc:254, FluxAttnPostFP8Processor.cc:135,168). */
LYRAQ_API int lyraq_attention(void* out, int out_dtype, size_t out_ld, const float* out_scale, void* out2, size_t out2_ld,
                              const float* out2_scale, size_t split, const void* qkv, int dtype, size_t batch, size_t seq_len,
                              int heads, int head_dim, float softmax_scale, void* stream);

/* e4m3 quantize of src [rows, cols] (static per-tensor scale, 1/scale[0] applied) into a column window of an e4m3
 * matrix with row pitch dst_ld bytes: the attention output's share of the proj_out input.  Same arithmetic as
 * lyraq_quant_fp8 (invokeCudaD2DScaleCpyConvert, src/lyradiff/utils/memory_utils.h:74). */
LYRAQ_API int lyraq_quant_fp8_2d(uint8_t* dst, size_t dst_ld, const void* src, int src_dtype, const float* scale, size_t rows,
                                 size_t cols, void* stream);

/* out = T(T(y * gate[b, :]) + x) with y, x, out [batch, seq, dim] and gate [batch, dim].  Replaces
 * invokeFusedGateAndResidual<T> (src/lyradiff/kernels/flux_single_transformer_block/flux_single_transformer_kernels.cu:43-65,
 * 152-160). */
LYRAQ_API int lyraq_gate_residual(void* out, const void* y, const void* gate, const void* x, int dtype, size_t batch,
                                  size_t seq_len, size_t dim, void* stream);

/* LoRA hot-swap on a 16-bit weight: weight[i] = T(weight[i] + T(lora[i] * T(alpha))), i < n, in place; every step rounds to
 * T as the reference's 16-bit operators do.  The FP8 layers follow it with lyraq_weight_quant_fp8 on the merged weight
 * (FP8LoraWeight<T>::load_lora, src/lyradiff/interface/IFLoraWeight.h:104-116).  Replaces invokeLoadLora<T>
 * (src/lyradiff/kernels/lora/load_lora.h; kernel load_lora.cu:6-14). */
LYRAQ_API int lyraq_load_lora(void* weight, const void* lora, int dtype, float alpha, size_t n, void* stream);

/* ------------------------------------------------------------------ quantized-Linear layer forwards
 * Activation quantize + GEMM of one linear on `stream`; the quantized activation lives in `workspace`
 * (lyraq_workspace_bytes(LYRAQ_OP_LINEAR_*, m, n, k) bytes, 16-byte aligned, owned by the caller, free for reuse
 * once the call's work on `stream` has finished).  x, Y, bias and residual all have element type `dtype`. */

/* FP8 linear: x -> e4m3 with the static per-tensor scale x_scale[0], then lyraq_gemm_fp8 (alpha = 1).
 * Replaces the invokeCudaD2DScaleCpyConvert + GemmWithResidualAndBias pair the FLUX FP8 blocks run per linear
 * (src/lyradiff/layers/flux_single_transformer_block/FluxSingleTransformerFP8Block.cc:216-243, :254-281). */
LYRAQ_API int lyraq_linear_fp8_forward(void* Y, const void* x, int dtype, const float* x_scale, const uint8_t* W,
                                       const float* w_scale, const void* bias, const void* residual, float beta, int epilogue,
                                       int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream);

/* INT8 SmoothQuant linear: x -> int8 (scale_mode as in lyraq_quant_int8; PER_TOKEN_DYNAMIC keeps the computed scales in
 * the workspace), then lyraq_gemm_int8 with bias.  Replaces the invokeSqInputQuant + runGemmInt8 pair of the SDXL INT8
 * block (src/lyradiff/layers/basic_transformer/BasicTransformerInt8Block.cc:427-441). */
LYRAQ_API int lyraq_linear_int8_forward(void* Y, const void* x, int dtype, const float* pre_quant_scale, const float* input_scale,
                                        int scale_mode, const int8_t* W, const float* w_scale, const void* bias, int m, int n,
                                        int k, void* workspace, size_t workspace_bytes, void* stream);

/* W4A4 linear: x -> int4 group-64 (with the smoothing vector), then lyraq_gemm_w4a4 with bias / GELU / residual.
 * Replaces W4A4Gemm<T>::forward (src/lyradiff/layers/w4a4_gemm_block/W4A4Gemm.cc:113-169) without its low-rank branch
 * (lyraq_w4a4_lora_forward has it). */
LYRAQ_API int lyraq_w4a4_forward(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W, const void* w_scale,
                                 int w_scale_dtype, const void* bias, const void* residual, int epilogue, int m, int n, int k,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* The whole of W4A4Gemm<T>::forward (src/lyradiff/layers/w4a4_gemm_block/W4A4Gemm.cc:113-169), low-rank branch
 * included: int4 group-64 quantize of x plus act = x * lora_down^T (fp32, [m, 32]), then the W4A4 GEMM with
 * T(act) * lora_up^T added after the last group, then bias / GELU / residual.  lora_down [32, k] and lora_up [n, 32] have
 * the type of x and D.  Workspace: lyraq_workspace_bytes(LYRAQ_OP_LINEAR_W4A4_LORA, m, n, k). */
LYRAQ_API int lyraq_w4a4_lora_forward(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W,
                                      const void* w_scale, int w_scale_dtype, const void* lora_down, const void* lora_up,
                                      const void* bias, const void* residual, int epilogue, int m, int n, int k,
                                      void* workspace, size_t workspace_bytes, void* stream);

/* lyraq_w4a4_forward without a workspace argument and without any allocation: the packed activation and its group
 * scales are kept in a fixed 16 MiB array inside the library's device image (lyraq_static_scratch_bytes()), which a GPU
 * holds from the moment the array is first used there until the process exits.  Meant for hosts that may not allocate device memory and
 * have no scratch pointer to pass (an asynchronous enqueue hook, a plug-in interface with inputs and outputs only, a
 * process whose memory pool belongs to another framework).  It has no counterpart in the reference, whose layers
 * always draw their buffers from the context's allocator.
 *   - m * k / 2 + 4 * m * (k / 64) (each rounded up to 256) must fit in the array; larger problems get
 *     LYRAQ_ERR_WORKSPACE and nothing is launched.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress).  CUDA loads device images
 *     lazily by default, so that look-up is when the driver creates the array -- its one allocation, which may
 *     synchronise the device and can fail with LYRAQ_ERR_CUDA if the memory pool is exhausted.  Make that first call
 *     outside any stream capture and outside the latency-critical path, or call lyraq_static_scratch_bytes() once per
 *     device at start-up, which does the same look-up (CUDA_MODULE_LOADING=EAGER moves it to context creation).
 *     After that no call allocates or frees anything.
 *   - Every call reuses the same array, which keeps the previous call's contents; nothing in it needs clearing
 *     because the quantizer rewrites all of it that the GEMM reads.  Calls whose GPU work overlaps race on it:
 *     issue them on one stream.
 * Arguments and results are those of lyraq_w4a4_forward. */
LYRAQ_API int lyraq_w4a4_forward_static(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W,
                                        const void* w_scale, int w_scale_dtype, const void* bias, const void* residual,
                                        int epilogue, int m, int n, int k, void* stream);

/* Size in bytes of the fixed scratch array behind lyraq_w4a4_forward_static (no counterpart in the reference).  When a
 * device is present the call also resolves the array's address on the current device: the start-up warm-up of that
 * entry point.  A failure of the look-up is not reported here; the first forward reports it. */
LYRAQ_API size_t lyraq_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
#endif /* LYRAQ_H_ */
