// Quantized-Linear layer forwards: the activation quantizer and the GEMM of one linear, chained on one stream, with
// the quantized activation (and its scales) held in caller-provided workspace.  These are what the reference's layers
// do around every quantized linear with buffers from their allocator; here the caller owns the buffer.
#include "common.cuh"

namespace lyraq {

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Workspace layouts (offsets are multiples of 256 bytes):
//   LINEAR_FP8  : e4m3 activation [m, k]
//   LINEAR_INT8 : int8 activation [m, k] | fp32 per-token scales [m]
//   LINEAR_W4A4 : packed int4 activation [m, k/2] | fp32 group scales [m, k/64]
//   LINEAR_W4A4_LORA : the same, then the fp32 low-rank activation [m, 32]
size_t linear_workspace_bytes(int op, size_t m, size_t k)
{
    switch (op) {
        case LYRAQ_OP_LINEAR_FP8: return align_up(m * k, 256);
        case LYRAQ_OP_LINEAR_INT8: return align_up(m * k, 256) + align_up(4 * m, 256);
        case LYRAQ_OP_LINEAR_W4A4: return align_up(m * k / 2, 256) + align_up(4 * m * (k / 64), 256);
        case LYRAQ_OP_LINEAR_W4A4_LORA:
            return align_up(m * k / 2, 256) + align_up(4 * m * (k / 64), 256) + align_up(4 * m * 32, 256);
        default: return 0;
    }
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {

size_t lyraq_workspace_bytes(int op, int m, int n, int k)
{
    (void)n;
    if (m <= 0 || k <= 0) {
        return 0;
    }
    return linear_workspace_bytes(op, (size_t)m, (size_t)k);
}

int lyraq_linear_fp8_forward(void* Y, const void* x, int dtype, const float* x_scale, const uint8_t* W, const float* w_scale,
                             const void* bias, const void* residual, float beta, int epilogue, int m, int n, int k,
                             void* workspace, size_t workspace_bytes, void* stream)
{
    if (m < 0 || n < 0 || k < 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    if (workspace == nullptr || workspace_bytes < linear_workspace_bytes(LYRAQ_OP_LINEAR_FP8, (size_t)m, (size_t)k) ||
        !aligned16(workspace)) {
        return LYRAQ_ERR_WORKSPACE;
    }
    uint8_t* qx = static_cast<uint8_t*>(workspace);
    int      st = lyraq_quant_fp8(qx, x, dtype, x_scale, 1, (size_t)m * (size_t)k, stream);
    if (st != LYRAQ_OK) {
        return st;
    }
    return lyraq_gemm_fp8(qx, x_scale, W, w_scale, Y, dtype, bias, residual, 1.0f, beta, epilogue, m, n, k, nullptr, 0, stream);
}

int lyraq_linear_int8_forward(void* Y, const void* x, int dtype, const float* pre_quant_scale, const float* input_scale,
                              int scale_mode, const int8_t* W, const float* w_scale, const void* bias, int m, int n, int k,
                              void* workspace, size_t workspace_bytes, void* stream)
{
    if (m < 0 || n < 0 || k < 0 || scale_mode < LYRAQ_SCALE_PER_TENSOR || scale_mode > LYRAQ_SCALE_PER_TOKEN_DYNAMIC) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    if (workspace == nullptr || workspace_bytes < linear_workspace_bytes(LYRAQ_OP_LINEAR_INT8, (size_t)m, (size_t)k) ||
        !aligned16(workspace)) {
        return LYRAQ_ERR_WORKSPACE;
    }
    if (scale_mode != LYRAQ_SCALE_PER_TOKEN_DYNAMIC && input_scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    int8_t* qx     = static_cast<int8_t*>(workspace);
    float*  tokens = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + align_up((size_t)m * (size_t)k, 256));
    float*  scale  = (scale_mode == LYRAQ_SCALE_PER_TOKEN_DYNAMIC) ? tokens : const_cast<float*>(input_scale);
    int     st     = lyraq_quant_int8(qx, x, dtype, pre_quant_scale, scale, scale_mode, (size_t)m, (size_t)k, stream);
    if (st != LYRAQ_OK) {
        return st;
    }
    const int row_mode = (scale_mode == LYRAQ_SCALE_PER_TENSOR) ? LYRAQ_SCALE_PER_TENSOR : LYRAQ_SCALE_PER_TOKEN;
    return lyraq_gemm_int8(qx, W, w_scale, scale, row_mode, Y, dtype, bias, m, n, k, nullptr, 0, stream);
}

int lyraq_w4a4_forward(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W, const void* w_scale,
                       int w_scale_dtype, const void* bias, const void* residual, int epilogue, int m, int n, int k,
                       void* workspace, size_t workspace_bytes, void* stream)
{
    if (m < 0 || n < 0 || k < 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    if (k == 0 || (k & 63) != 0) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (workspace == nullptr || workspace_bytes < linear_workspace_bytes(LYRAQ_OP_LINEAR_W4A4, (size_t)m, (size_t)k) ||
        !aligned16(workspace)) {
        return LYRAQ_ERR_WORKSPACE;
    }
    uint8_t* q  = static_cast<uint8_t*>(workspace);
    float*   qs = reinterpret_cast<float*>(q + align_up((size_t)m * (size_t)k / 2, 256));
    int      st = lyraq_quant_int4_g64(q, qs, nullptr, x, dtype, smooth, nullptr, (size_t)m, (size_t)k, stream);
    if (st != LYRAQ_OK) {
        return st;
    }
    return lyraq_gemm_w4a4(q, W, qs, w_scale, w_scale_dtype, D, dtype, nullptr, LYRAQ_F32, nullptr, bias, residual, epilogue, m, n, k,
                           nullptr, 0, stream);
}

int lyraq_w4a4_lora_forward(void* D, const void* x, int dtype, const float* smooth, const uint8_t* W, const void* w_scale,
                            int w_scale_dtype, const void* lora_down, const void* lora_up, const void* bias,
                            const void* residual, int epilogue, int m, int n, int k, void* workspace, size_t workspace_bytes,
                            void* stream)
{
    if (m < 0 || n < 0 || k < 0 || lora_down == nullptr || lora_up == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    if (k == 0 || (k & 63) != 0) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (workspace == nullptr || workspace_bytes < linear_workspace_bytes(LYRAQ_OP_LINEAR_W4A4_LORA, (size_t)m, (size_t)k) ||
        !aligned16(workspace)) {
        return LYRAQ_ERR_WORKSPACE;
    }
    uint8_t* q   = static_cast<uint8_t*>(workspace);
    float*   qs  = reinterpret_cast<float*>(q + align_up((size_t)m * (size_t)k / 2, 256));
    float*   act = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(qs) + align_up(4 * (size_t)m * (size_t)(k / 64), 256));
    int      st  = lyraq_quant_int4_g64(q, qs, act, x, dtype, smooth, lora_down, (size_t)m, (size_t)k, stream);
    if (st != LYRAQ_OK) {
        return st;
    }
    return lyraq_gemm_w4a4(q, W, qs, w_scale, w_scale_dtype, D, dtype, act, LYRAQ_F32, lora_up, bias, residual, epilogue, m, n, k, nullptr,
                           0, stream);
}

}  // extern "C"
