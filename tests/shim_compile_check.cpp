// Compile-only check: the reference's call forms resolve against the shim header.
#include "lyradiff_shim.h"

using namespace lyradiff;

void sdxl_int8_call_sites(int8_t* q, half* h, const float* f, float* fo, char* ws, cudaStream_t s)
{
    QuantMode qm = QuantMode::useSmoothQuant(false, true);
    invokeSqInputQuant<half>(q, h, f, f, qm, 2, 4096, 640, s);
    invokeLayerNormInt8O<half>(q, h, h, h, f, f, qm, 2, 4096, 640, s);
    invokeFusedResidualBiasLayerNormInt8O<half>(q, h, h, h, h, h, h, f, f, qm, 2, 4096, 640, s, 1e-5);
    invokeFusedAddBiasGegluInt8O<half>(q, h, h, f, f, 4096, 2560, 2, s);
    invokeGetINT8WeightScale<half>(fo, q, h, f, 5120, 640, s);
    QuantGemmWrapper w(s, LYRAQ_F16);
    w.profileGemmInt8(16384, 5120, 640);
    w.runGemmInt8(q, q, f, f, h, 8192, 5120, 640, ws, s);
}

void flux_fp8_call_sites(__nv_fp8_e4m3* q8, __nv_bfloat16* b, const float* f, float* fo, cudaStream_t s)
{
    invokeCudaD2DScaleCpyConvert<__nv_bfloat16, __nv_fp8_e4m3>(q8, b, f, true, 4608 * 3072, s);
    invokeGetFP8WeightScale<__nv_bfloat16>(fo, b, 9216 * 3072, s);
    invokeLoadLora<__nv_bfloat16>(b, b, 9216 * 3072, 0.8f, s);                         // IFLoraWeight.h:108
    invokeLayerNormWithShiftAndScale<__nv_bfloat16>(b, b, b, b, 1, 4608, 3072, s);
    invokeLayerNormWithShiftAndScaleFp8O<__nv_bfloat16>(q8, f, nullptr, b, b, b, 1, 4608, 3072, s);
    invokeFusedRmsNormAndRope<__nv_bfloat16>(b, b, b, b, 1e-6f, 1, 4608, 24, 128, s);   // FluxSingleAttentionFP8Processor.cc:183
    invokeFusedGateAndResidual<__nv_bfloat16>(b, b, b, b, 1, 4608, 3072, s);           // FluxSingleTransformerFP8Block.cc:296
    QuantGemmWrapper w(s, LYRAQ_BF16);
    w.GemmWithResidualAndBias(CUBLAS_OP_T, CUBLAS_OP_N, 12288, 4608, 3072, q8, 3072, f, q8, 3072, f, b, 12288, b, nullptr, 1.0f,
                              0.0f, true);
}

void flux_w4a4_call_sites(void* d, uint32_t* q, float* sc, const void* a, const float* f, cudaStream_t s)
{
    invokeFusedQuantizeAndLoraDownSimple(nullptr, q, sc, a, nullptr, f, 4608, 32, 3072, 64, s);
    invokeFusedW4A4GemmAndLoraUp(d, q, a, nullptr, nullptr, sc, f, 4608, 9216, 3072, 32, 48, s);
}
