// Runs the reference's call forms through include/lyradiff_shim.h on real device buffers.
//
// Every function below calls ONE shim function with the argument order the reference's layers use (the file:line of the
// call site is given) and is exported with plain C types so that a test can drive it through ctypes and compare the
// result with the same operation issued through the C ABI directly.  A swapped argument in a forwarding template shows
// up as different bits.  Built by tests/test_gpu_shim.py with g++ against liblyraq.so; no device code here.
#include <string>

#include "lyradiff_shim.h"

using namespace lyradiff;

namespace {
std::string g_error;

template<typename F> int guarded(F&& f)
{
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}
}  // namespace

#define EXPORT extern "C" __attribute__((visibility("default")))

EXPORT const char* shim_last_error() { return g_error.c_str(); }

// ---- SDXL INT8 path (fp16)
// BasicTransformerInt8Block.cc:427-441: invokeSqInputQuant(dst, src, pre, scale, quant_mode, batch, seq, dim, stream)
EXPORT int shim_sq_input_quant(int8_t* dst, const half* src, const float* pre, const float* scale, int per_token, size_t batch,
                               size_t seq, size_t dim, cudaStream_t s)
{
    return guarded([&] { invokeSqInputQuant<half>(dst, src, pre, scale, QuantMode::useSmoothQuant(per_token != 0, true), batch, seq, dim, s); });
}

// BasicTransformerInt8Block.cc:395-408
EXPORT int shim_layer_norm_int8o(int8_t* dst, const half* src, const half* gamma, const half* beta, const float* pre,
                                 const float* scale, size_t batch, size_t channels, size_t hidden, cudaStream_t s, double eps)
{
    return guarded([&] { invokeLayerNormInt8O<half>(dst, src, gamma, beta, pre, scale, QuantMode::useSmoothQuant(), batch, channels, hidden, s, eps); });
}

// BasicTransformerInt8Block.cc:770-790
EXPORT int shim_residual_bias_layer_norm_int8o(int8_t* dst, half* dst2, const half* src, const half* residual, const half* bias,
                                               const half* gamma, const half* beta, const float* pre, const float* scale,
                                               size_t batch, size_t channels, size_t hidden, cudaStream_t s, double eps)
{
    return guarded([&] {
        invokeFusedResidualBiasLayerNormInt8O<half>(dst, dst2, src, residual, bias, gamma, beta, pre, scale, QuantMode::useSmoothQuant(),
                                                    batch, channels, hidden, s, eps);
    });
}

// BasicTransformerInt8Block.cc:811-822: (dst, hidden_states, bias, pre, scale, seq_len, dim, batch_size, stream)
EXPORT int shim_add_bias_geglu_int8o(int8_t* dst, const half* hidden, const half* bias, const float* pre, const float* scale,
                                     int seq_len, int dim, int batch, cudaStream_t s, int v2)
{
    return guarded([&] {
        if (v2) {
            invokeFusedAddBiasGegluInt8OV2<half>(dst, hidden, bias, pre, scale, seq_len, dim, batch, s);
        } else {
            invokeFusedAddBiasGegluInt8O<half>(dst, hidden, bias, pre, scale, seq_len, dim, batch, s);
        }
    });
}

// quant_kernels.h:30-37
EXPORT int shim_get_int8_weight_scale(float* new_scale, int8_t* qw, const half* w, const float* pre, size_t d_out, size_t d_in,
                                      cudaStream_t s)
{
    return guarded([&] { invokeGetINT8WeightScale<half>(new_scale, qw, w, pre, d_out, d_in, s); });
}

// cublasMMWrapper.h:354-385: profileGemmInt8(maxM, n, k); runGemmInt8(A, B, alphaCol, alphaRow, C, m, n, k, workspace, stream)
EXPORT int shim_run_gemm_int8(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row, half* C, int m, int n,
                              int k, char* workspace, cudaStream_t s, int per_token)
{
    return guarded([&] {
        QuantGemmWrapper w(s, LYRAQ_F16);
        w.profileGemmInt8(16384, n, k);
        w.runGemmInt8(A, B, alpha_col, alpha_row, C, m, n, k, workspace, s, per_token != 0);
    });
}

// BasicTransformerInt8Block.cc:824-845 folded into the GEMM
EXPORT int shim_run_gemm_int8_bias_residual(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row, half* C,
                                            const half* bias, const half* residual, int m, int n, int k, cudaStream_t s)
{
    return guarded([&] {
        QuantGemmWrapper w(s, LYRAQ_F16);
        w.runGemmInt8BiasResidual(A, B, alpha_col, alpha_row, C, bias, residual, m, n, k, nullptr, s);
    });
}

// ---- FLUX FP8 path (bf16)
// FluxSingleTransformerFP8Block.cc:216: invokeCudaD2DScaleCpyConvert(dst, src, scale, true, size, stream)
EXPORT int shim_d2d_scale_cpy_convert(__nv_fp8_e4m3* dst, const __nv_bfloat16* src, const float* scale, int invert, size_t n,
                                      cudaStream_t s)
{
    return guarded([&] { invokeCudaD2DScaleCpyConvert<__nv_bfloat16, __nv_fp8_e4m3>(dst, src, scale, invert != 0, n, s); });
}

// IFLoraWeight.h:95-128: scale, then load_lora
EXPORT int shim_get_fp8_weight_scale(float* scale, const __nv_bfloat16* w, size_t n, cudaStream_t s)
{
    return guarded([&] { invokeGetFP8WeightScale<__nv_bfloat16>(scale, w, n, s); });
}
EXPORT int shim_load_lora(__nv_bfloat16* dst, const __nv_bfloat16* src, size_t n, float alpha, cudaStream_t s)
{
    return guarded([&] { invokeLoadLora<__nv_bfloat16>(dst, src, n, alpha, s); });
}

// AdaFP8LayerNorm.cc:188-198: (dst, src, scale, shift, batch, seq, dim, stream)
EXPORT int shim_layer_norm_shift_scale(__nv_bfloat16* dst, const __nv_bfloat16* src, const __nv_bfloat16* scale,
                                       const __nv_bfloat16* shift, size_t batch, size_t seq, size_t dim, cudaStream_t s)
{
    return guarded([&] { invokeLayerNormWithShiftAndScale<__nv_bfloat16>(dst, src, scale, shift, batch, seq, dim, s); });
}
EXPORT int shim_layer_norm_shift_scale_fp8o(__nv_fp8_e4m3* dst8, const float* in_scale, __nv_bfloat16* dst, const __nv_bfloat16* src,
                                            const __nv_bfloat16* scale, const __nv_bfloat16* shift, size_t batch, size_t seq,
                                            size_t dim, cudaStream_t s)
{
    return guarded([&] { invokeLayerNormWithShiftAndScaleFp8O<__nv_bfloat16>(dst8, in_scale, dst, src, scale, shift, batch, seq, dim, s); });
}

// FluxSingleAttentionFP8Processor.cc:183: (out, in, scale, rope, eps, batch, seq, heads, head_dim, stream)
EXPORT int shim_rmsnorm_rope(__nv_bfloat16* out, const __nv_bfloat16* in, const __nv_bfloat16* scale, const __nv_bfloat16* rope,
                             float eps, int batch, int seq, int heads, int head_dim, cudaStream_t s)
{
    return guarded([&] { invokeFusedRmsNormAndRope<__nv_bfloat16>(out, in, scale, rope, eps, batch, seq, heads, head_dim, s); });
}

// FluxSingleTransformerFP8Block.cc:296: (out, input, gate, residual, batch, seq, dim, stream)
EXPORT int shim_gate_residual(__nv_bfloat16* out, const __nv_bfloat16* in, const __nv_bfloat16* gate, const __nv_bfloat16* residual,
                              int batch, int seq, int dim, cudaStream_t s)
{
    return guarded([&] { invokeFusedGateAndResidual<__nv_bfloat16>(out, in, gate, residual, batch, seq, dim, s); });
}

// FluxSingleTransformerFP8Block.cc:227-243: GemmWithResidualAndBias(OP_T, OP_N, n_out, m_tokens, k, W, k, s_w, X, k, s_x, Y,
// n_out, bias, residual, alpha, beta, is_gelu)
EXPORT int shim_gemm_fp8(int n_out, int m_tokens, int k, const __nv_fp8_e4m3* W, const float* w_scale, const __nv_fp8_e4m3* X,
                         const float* x_scale, __nv_bfloat16* Y, const __nv_bfloat16* bias, const __nv_bfloat16* residual, float alpha,
                         float beta, int is_gelu, cudaStream_t s, int bad_layout)
{
    return guarded([&] {
        QuantGemmWrapper w(s, LYRAQ_BF16);
        w.GemmWithResidualAndBias(bad_layout ? CUBLAS_OP_N : CUBLAS_OP_T, CUBLAS_OP_N, n_out, m_tokens, k, W, k, w_scale, X, k, x_scale, Y,
                                  n_out, bias, residual, alpha, beta, is_gelu != 0);
    });
}

// ---- FLUX W4A4 path (bf16)
// W4A4Gemm.cc:138-148 (the reference passes group_num where group_dim is declared; both are ignored)
EXPORT int shim_quantize_lora_down(float* C, uint32_t* q, float* q_scale, const void* A, const void* lora_down, const float* smooth,
                                   int m, int rank, int k, int group_num, cudaStream_t s)
{
    return guarded([&] { invokeFusedQuantizeAndLoraDownSimple(C, q, q_scale, A, lora_down, smooth, m, rank, k, group_num, s); });
}

// W4A4Gemm.cc:152-164
EXPORT int shim_w4a4_gemm_lora_up(void* D, const void* A, const void* B, const void* lora_act, const void* lora_up, const float* sa,
                                  const float* sb, int m, int n, int k, int rank, int groups, cudaStream_t s)
{
    return guarded([&] { invokeFusedW4A4GemmAndLoraUp(D, A, B, lora_act, lora_up, sa, sb, m, n, k, rank, groups, s); });
}

// W4A4GemmWeight<T>::loadWeights (W4A4GemmWeight.cc:60-82) + W4A4Gemm<T>::forward (W4A4Gemm.cc:113-169)
EXPORT int shim_w4a4_layer_from_bins(__nv_bfloat16* out, const __nv_bfloat16* in, size_t m, size_t d_out, size_t d_in, const char* prefix,
                                     int file_type, cudaStream_t s)
{
    return guarded([&] {
        W4A4GemmWeight<__nv_bfloat16> w(d_out, d_in, 32, false, 64, LyraQuantType::INT4_W4A4, nullptr);
        w.loadWeights(prefix, (FtCudaDataType)file_type);
        W4A4Gemm<__nv_bfloat16> layer(d_out, d_in, s);
        layer.forward(out, in, m, &w);
        layer.forward(out, in, m, &w);  // the kept scratch is reused
        lyraq_detail::cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");  // the weights die with this scope
    });
}
