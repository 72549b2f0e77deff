/*
 * C++ shim: the reference's layer-level function names and argument lists, forwarded to the lyraq C ABI.
 *
 * A maintainer of the reference who wants its quantized layers to run on B200 includes this header in
 * place of the kernel headers named below and links liblyraq.so; the layer code (BasicTransformerInt8Block,
 * FluxSingleTransformerFP8Block, W4A4Gemm, AdaFP8LayerNorm, ...) compiles unchanged.  Everything is inline
 * and header-only.  Like the reference's functions these return void and report failure by throwing
 * (std::runtime_error here; the reference throws its own exception type or a string literal); unlike
 * the reference nothing is silently skipped for an unsupported width.
 */
#ifndef LYRADIFF_SHIM_H_
#define LYRADIFF_SHIM_H_

#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "lyraq.h"

namespace lyradiff {

namespace lyraq_detail {
template<typename T> struct DType;
template<> struct DType<half> { static constexpr int value = LYRAQ_F16; };
template<> struct DType<__nv_bfloat16> { static constexpr int value = LYRAQ_BF16; };
template<> struct DType<float> { static constexpr int value = LYRAQ_F32; };
template<> struct DType<int32_t> { static constexpr int value = LYRAQ_S32; };

inline void check(int status, const char* what)
{
    if (status != LYRAQ_OK) {
        throw std::runtime_error(std::string(what) + ": " + lyraq_status_string(status));
    }
}
}  // namespace lyraq_detail

/* Flags describing a quantization scheme; same member names as the reference's QuantMode
 * (src/lyradiff/utils/quantization.h:9-274), only the members the hot path reads. */
class QuantMode {
public:
    using BaseType = std::uint32_t;
    explicit constexpr QuantMode(BaseType value) noexcept: value_(value) {}
    constexpr QuantMode() noexcept: value_(0) {}
    static constexpr QuantMode none() noexcept { return QuantMode(0); }
    static constexpr QuantMode activations() noexcept { return QuantMode(1u << 2); }
    static constexpr QuantMode perChannelScaling() noexcept { return QuantMode(1u << 3); }
    static constexpr QuantMode perTokenScaling() noexcept { return QuantMode(1u << 4); }
    static constexpr QuantMode int8Weights() noexcept { return QuantMode(1u << 1); }
    static constexpr QuantMode useSmoothQuant(bool per_token = false, bool per_channel = false) noexcept
    {
        return QuantMode((1u << 1) | (1u << 2) | (per_token ? (1u << 4) : 0u) | (per_channel ? (1u << 3) : 0u));
    }
    constexpr bool hasPerTokenScaling() const noexcept { return (value_ & (1u << 4)) != 0; }
    constexpr bool hasPerChannelScaling() const noexcept { return (value_ & (1u << 3)) != 0; }
    constexpr bool hasActivations() const noexcept { return (value_ & (1u << 2)) != 0; }
    constexpr BaseType value() const noexcept { return value_; }

private:
    BaseType value_;
};

/* src/lyradiff/kernels/quant_kernels/quant_kernels.h:9-17 */
template<typename T>
inline void invokeSqInputQuant(int8_t* dst, const T* src, const float* pre_quant_scale, const float* input_quant_scale,
                               QuantMode quant_mode, size_t batch_size, size_t seq_len, size_t dim, cudaStream_t stream)
{
    lyraq_detail::check(lyraq_quant_int8(dst, src, lyraq_detail::DType<T>::value, pre_quant_scale,
                                         const_cast<float*>(input_quant_scale),
                                         quant_mode.hasPerTokenScaling() ? LYRAQ_SCALE_PER_TOKEN : LYRAQ_SCALE_PER_TENSOR,
                                         batch_size * seq_len, dim, stream),
                        "invokeSqInputQuant");
}

/* src/lyradiff/kernels/quant_kernels/quant_kernels.h:30-37 */
template<typename T>
inline void invokeGetINT8WeightScale(float* new_weight_scale, int8_t* quantized_weight, const T* weight,
                                     const float* pre_quant_scale, const size_t d_out, const size_t d_in,
                                     cudaStream_t stream = 0)
{
    lyraq_detail::check(lyraq_weight_quant_int8(new_weight_scale, quantized_weight, weight, lyraq_detail::DType<T>::value,
                                                pre_quant_scale, d_out, d_in, stream),
                        "invokeGetINT8WeightScale");
}

/* src/lyradiff/kernels/quant_kernels/layer_norm_int8.h:9-20 */
template<typename T>
inline void invokeLayerNormInt8O(int8_t* dst, const T* src, const T* gamma, const T* beta, const float* pre_quant_scale,
                                 const float* input_quant_scale, QuantMode, size_t batch_size, size_t channels,
                                 size_t nhiddens, cudaStream_t stream, const double eps = 1e-6)
{
    lyraq_detail::check(lyraq_ln_quant_int8(dst, nullptr, src, nullptr, nullptr, gamma, beta, lyraq_detail::DType<T>::value,
                                            pre_quant_scale, input_quant_scale, batch_size * channels, nhiddens, eps, stream),
                        "invokeLayerNormInt8O");
}

/* src/lyradiff/kernels/quant_kernels/layer_norm_int8.h:22-38 */
template<typename T>
inline void invokeFusedResidualBiasLayerNormInt8O(int8_t* dst, T* dst2, const T* src, const T* residual, const T* bias,
                                                  const T* gamma, const T* beta, const float* pre_quant_scale,
                                                  const float* input_quant_scale, QuantMode, size_t batch_size,
                                                  size_t channels, size_t nhiddens, cudaStream_t stream,
                                                  const double eps = 1e-6)
{
    lyraq_detail::check(lyraq_ln_quant_int8(dst, dst2, src, residual, bias, gamma, beta, lyraq_detail::DType<T>::value,
                                            pre_quant_scale, input_quant_scale, batch_size * channels, nhiddens, eps, stream),
                        "invokeFusedResidualBiasLayerNormInt8O");
}

/* src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.h:13-21 (and the V2 twin :23-31, same arithmetic) */
template<typename T>
inline void invokeFusedAddBiasGegluInt8O(int8_t* dst, const T* hidden_states, const T* bias, const float* pre_quant_scale,
                                         const float* input_quant_scale, const int seq_len, const int dim,
                                         const int batch_size, cudaStream_t stream)
{
    lyraq_detail::check(lyraq_geglu_quant_int8(dst, hidden_states, bias, lyraq_detail::DType<T>::value, pre_quant_scale,
                                               input_quant_scale, (size_t)seq_len * (size_t)batch_size, (size_t)dim, stream),
                        "invokeFusedAddBiasGegluInt8O");
}
template<typename T>
inline void invokeFusedAddBiasGegluInt8OV2(int8_t* dst, const T* hidden_states, const T* bias, const float* pre_quant_scale,
                                           const float* input_quant_scale, const int seq_len, const int dim,
                                           const int batch_size, cudaStream_t stream)
{
    invokeFusedAddBiasGegluInt8O<T>(dst, hidden_states, bias, pre_quant_scale, input_quant_scale, seq_len, dim, batch_size,
                                    stream);
}

/* src/lyradiff/utils/memory_utils.h:74 — only the conversions to e4m3 are on the hot path */
template<typename T_IN, typename T_OUT>
inline void invokeCudaD2DScaleCpyConvert(T_OUT* tgt, const T_IN* src, const float* scale, bool invert_scale,
                                         const size_t size, cudaStream_t stream)
{
    static_assert(std::is_same<T_OUT, __nv_fp8_e4m3>::value, "lyraq covers the e4m3 destination only");
    lyraq_detail::check(lyraq_quant_fp8(reinterpret_cast<uint8_t*>(tgt), src, lyraq_detail::DType<T_IN>::value, scale,
                                        invert_scale ? 1 : 0, size, stream),
                        "invokeCudaD2DScaleCpyConvert");
}

/* src/lyradiff/kernels/lora/load_lora.cu:109-113 */
template<typename T> inline void invokeGetFP8WeightScale(float* scale, const T* weight, const size_t size, cudaStream_t stream)
{
    lyraq_detail::check(lyraq_fp8_amax_scale(scale, weight, lyraq_detail::DType<T>::value, size, stream),
                        "invokeGetFP8WeightScale");
}

/* src/lyradiff/kernels/norms/layer_norm.h:19 — un-fused form (writes dst only) */
template<typename T>
inline void invokeLayerNormWithShiftAndScale(T* dst, const T* src, const T* scale, const T* shift, size_t batch_size,
                                             size_t seq_len, size_t dim, cudaStream_t stream, const double eps = 1e-6)
{
    lyraq_detail::check(lyraq_adaln_quant(dst, nullptr, nullptr, nullptr, nullptr, src, scale, shift,
                                          lyraq_detail::DType<T>::value, nullptr, batch_size, seq_len, dim, eps, stream),
                        "invokeLayerNormWithShiftAndScale");
}

/* New on this path (the reference runs layer_norm.cu:405-484 and then memory_utils.cu:431-446 as two passes):
 * AdaLN modulation with the e4m3 quantize of the FP8 GEMM that follows fused in.  dst may be null. */
template<typename T>
inline void invokeLayerNormWithShiftAndScaleFp8O(__nv_fp8_e4m3* dst_fp8, const float* fp8_input_scale, T* dst, const T* src,
                                                 const T* scale, const T* shift, size_t batch_size, size_t seq_len,
                                                 size_t dim, cudaStream_t stream, const double eps = 1e-6)
{
    lyraq_detail::check(lyraq_adaln_quant(dst, nullptr, nullptr, reinterpret_cast<uint8_t*>(dst_fp8), fp8_input_scale, src,
                                          scale, shift, lyraq_detail::DType<T>::value, nullptr, batch_size, seq_len, dim, eps,
                                          stream),
                        "invokeLayerNormWithShiftAndScaleFp8O");
}

/* src/lyradiff/kernels/rope/flux_apply_rope.h:20-30 */
template<typename T>
inline void invokeFusedRmsNormAndRope(T* out, const T* input, const T* scale, const T* rope_emb, float eps, int batch_size,
                                      int seq_len, int head_num, int head_dim, cudaStream_t stream)
{
    lyraq_detail::check(lyraq_rmsnorm_rope(out, input, scale, rope_emb, lyraq_detail::DType<T>::value, (double)eps,
                                           (size_t)batch_size, (size_t)seq_len, head_num, head_dim, stream),
                        "invokeFusedRmsNormAndRope");
}

/* src/lyradiff/kernels/flux_single_transformer_block/flux_single_transformer_kernels.cu:152-160 */
template<typename T>
inline void invokeFusedGateAndResidual(T* out, const T* input, const T* gate, const T* residual, int batch_size, int seq_len,
                                       int dim, cudaStream_t stream)
{
    lyraq_detail::check(lyraq_gate_residual(out, input, gate, residual, lyraq_detail::DType<T>::value, (size_t)batch_size,
                                            (size_t)seq_len, (size_t)dim, stream),
                        "invokeFusedGateAndResidual");
}

/* src/lyradiff/kernels/lora/load_lora.h:9-10 (kernel load_lora.cu:6-14): dst += src * T(alpha) in T arithmetic. */
template<typename T>
inline void invokeLoadLora(T* dst, const T* src, size_t size, float alpha, cudaStream_t stream = 0)
{
    lyraq_detail::check(lyraq_load_lora(dst, src, lyraq_detail::DType<T>::value, alpha, size, stream), "invokeLoadLora");
}

/* src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:6-17.  A is bf16 [m,k]; B (lora_down) bf16 [32,k]; n is the LoRA rank. */
inline void invokeFusedQuantizeAndLoraDownSimple(float* Cptr, uint32_t* quantized_input, float* quantized_scale,
                                                 const void* Aptr, const void* Bptr, const float* Smoothptr, int m, int n,
                                                 int k, int group_dim = 64, cudaStream_t stream = 0)
{
    (void)n;
    (void)group_dim;  /* the reference's kernel hard-codes 64 whatever is passed (W4A4Gemm.cc:138-148) */
    lyraq_detail::check(lyraq_quant_int4_g64(reinterpret_cast<uint8_t*>(quantized_input), quantized_scale, Cptr, Aptr,
                                             LYRAQ_BF16, Smoothptr, Bptr, (size_t)m, (size_t)k, stream),
                        "invokeFusedQuantizeAndLoraDownSimple");
}

/* src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.h:19-30.  D bf16 [m,n]; LoraA bf16 [m,lora_k]; LoraB bf16 [n,lora_k]. */
inline void invokeFusedW4A4GemmAndLoraUp(void* Dptr, const void* Aptr, const void* Bptr, const void* LoraAptr,
                                         const void* LoraBptr, const float* AweightScale, const float* BweightScale, int m,
                                         int n, int k, int lora_k, int groups, cudaStream_t stream)
{
    (void)lora_k;
    (void)groups;
    lyraq_detail::check(lyraq_gemm_w4a4(static_cast<const uint8_t*>(Aptr), static_cast<const uint8_t*>(Bptr), AweightScale,
                                        BweightScale, LYRAQ_F32, Dptr, LYRAQ_BF16, LoraAptr, LYRAQ_BF16,
                                        LoraBptr, nullptr, nullptr, LYRAQ_EPI_NONE, m, n, k, nullptr, 0, stream),
                        "invokeFusedW4A4GemmAndLoraUp");
}

/* Element type of a raw .bin weight file (src/lyradiff/utils/cuda_utils.h:37-43) and the quantization levels the torch
 * ops are constructed with (:45-55; only the levels this library runs are named). */
enum FtCudaDataType { FP32 = 0, FP16 = 1, BF16 = 2, INT8 = 3, FP8 = 4 };
enum class LyraQuantType { NONE = 0, FP8_W8A8 = 1, FP8_W8A8_FULL = 2, INT4_W4A4 = 7, INT4_W4A4_FULL = 8 };

namespace lyraq_detail {
inline void cuda_check(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
}
template<typename T> inline T from_float(float v);
template<> inline float from_float<float>(float v) { return v; }
template<> inline half from_float<half>(float v) { return __float2half(v); }
template<> inline __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

/* Reads `count` elements of file type `file_type` from a raw .bin file into device memory as T (the reference's
 * loadWeightFromBin<T>, src/lyradiff/utils/memory_utils.cu: same-type files are copied, other types converted). */
template<typename T>
inline void load_bin(T* dst, size_t count, const std::string& path, FtCudaDataType file_type)
{
    const size_t esz = file_type == FP32 ? 4 : (file_type == INT8 || file_type == FP8) ? 1 : 2;
    std::vector<unsigned char> raw(count * esz);
    FILE* f = std::fopen(path.c_str(), "rb");
    if (f == nullptr) {
        throw std::runtime_error("cannot open " + path);
    }
    const size_t got = std::fread(raw.data(), 1, raw.size(), f);
    std::fclose(f);
    if (got != raw.size()) {
        throw std::runtime_error(path + ": file is shorter than the tensor it should hold");
    }
    std::vector<T> host(count);
    for (size_t i = 0; i < count; ++i) {
        float v;
        if (file_type == FP32) {
            v = reinterpret_cast<const float*>(raw.data())[i];
        } else if (file_type == FP16) {
            v = __half2float(reinterpret_cast<const half*>(raw.data())[i]);
        } else if (file_type == BF16) {
            v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(raw.data())[i]);
        } else {
            v = (float)reinterpret_cast<const signed char*>(raw.data())[i];
        }
        host[i] = from_float<T>(v);
    }
    cuda_check(cudaMemcpy(dst, host.data(), count * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy(load_bin)");
}
template<> inline void load_bin<int8_t>(int8_t* dst, size_t count, const std::string& path, FtCudaDataType)
{
    std::vector<int8_t> raw(count);
    FILE* f = std::fopen(path.c_str(), "rb");
    if (f == nullptr) {
        throw std::runtime_error("cannot open " + path);
    }
    const size_t got = std::fread(raw.data(), 1, raw.size(), f);
    std::fclose(f);
    if (got != raw.size()) {
        throw std::runtime_error(path + ": file is shorter than the tensor it should hold");
    }
    cuda_check(cudaMemcpy(dst, raw.data(), count, cudaMemcpyHostToDevice), "cudaMemcpy(load_bin)");
}
}  // namespace lyraq_detail

/* The weights of one W4A4 linear, with the reference's member names, sizes and file names
 * (src/lyradiff/layers/w4a4_gemm_block/W4A4GemmWeight.h:8-45, W4A4GemmWeight.cc:48-82): packed int4 weight [d_out, d_in / 2]
 * (even element in the low nibble), fp32 group scales [d_out, d_in / 64], the rank-32 low-rank factors, the smoothing
 * vector and an optional bias.  The object owns its device buffers once mallocWeights() or loadWeights() has run. */
template<typename T>
class W4A4GemmWeight {
public:
    int8_t* packed_weight = nullptr;
    float*  weight_scale  = nullptr;
    T*      lora_up       = nullptr;
    T*      lora_down     = nullptr;
    T*      bias          = nullptr;
    float*  smooth        = nullptr;

    W4A4GemmWeight() = default;
    W4A4GemmWeight(size_t d_out, size_t d_in, size_t lora_rank = 32, bool has_bias = false, size_t group_size = 64,
                   LyraQuantType = LyraQuantType::NONE, void* /*allocator*/ = nullptr):
        d_out_(d_out), d_in_(d_in), lora_rank_(lora_rank), group_size_(group_size), group_num_(d_in / group_size), has_bias_(has_bias)
    {
        if (lora_rank != 32 || group_size != 64 || d_in % 64 != 0) {
            throw std::runtime_error("W4A4GemmWeight: rank 32 and groups of 64 only (as the reference's kernels)");
        }
    }
    W4A4GemmWeight(const W4A4GemmWeight&)            = delete;
    W4A4GemmWeight& operator=(const W4A4GemmWeight&) = delete;
    virtual ~W4A4GemmWeight()
    {
        if (is_maintain_buffer) {
            cudaFree(packed_weight);
            cudaFree(weight_scale);
            cudaFree(lora_up);
            cudaFree(lora_down);
            cudaFree(smooth);
            cudaFree(bias);
        }
    }

    virtual void mallocWeights()
    {
        if (!is_maintain_buffer) {
            lyraq_detail::cuda_check(cudaMalloc(&packed_weight, d_out_ * d_in_ / 2), "cudaMalloc(packed_weight)");
            lyraq_detail::cuda_check(cudaMalloc(&weight_scale, d_out_ * group_num_ * sizeof(float)), "cudaMalloc(weight_scale)");
            lyraq_detail::cuda_check(cudaMalloc(&lora_up, d_out_ * lora_rank_ * sizeof(T)), "cudaMalloc(lora_up)");
            lyraq_detail::cuda_check(cudaMalloc(&lora_down, d_in_ * lora_rank_ * sizeof(T)), "cudaMalloc(lora_down)");
            lyraq_detail::cuda_check(cudaMalloc(&smooth, d_in_ * sizeof(float)), "cudaMalloc(smooth)");
            if (has_bias_) {
                lyraq_detail::cuda_check(cudaMalloc(&bias, d_out_ * sizeof(T)), "cudaMalloc(bias)");
            }
        }
        is_maintain_buffer = true;
    }

    /* <prefix>packed_weight.bin, weight_scale.bin, lora_up.bin, lora_down.bin, smooth.bin, bias.bin */
    virtual void loadWeights(const std::string prefix, FtCudaDataType model_file_type)
    {
        mallocWeights();
        lyraq_detail::load_bin<int8_t>(packed_weight, d_out_ * d_in_ / 2, prefix + "packed_weight.bin", INT8);
        lyraq_detail::load_bin<float>(weight_scale, d_out_ * group_num_, prefix + "weight_scale.bin", FP32);
        lyraq_detail::load_bin<T>(lora_up, d_out_ * lora_rank_, prefix + "lora_up.bin", model_file_type);
        lyraq_detail::load_bin<T>(lora_down, d_in_ * lora_rank_, prefix + "lora_down.bin", model_file_type);
        lyraq_detail::load_bin<float>(smooth, d_in_, prefix + "smooth.bin", FP32);
        if (has_bias_) {
            lyraq_detail::load_bin<T>(bias, d_out_, prefix + "bias.bin", model_file_type);
        }
    }

    size_t d_out() const { return d_out_; }
    size_t d_in() const { return d_in_; }
    size_t group_num() const { return group_num_; }
    bool   has_bias() const { return has_bias_; }

protected:
    bool is_maintain_buffer = false;

private:
    size_t d_out_ = 0, d_in_ = 0, lora_rank_ = 32, group_size_ = 64, group_num_ = 0;
    bool   has_bias_ = true;
};

/* W4A4Gemm<T>::forward (src/lyradiff/layers/w4a4_gemm_block/W4A4Gemm.cc:113-169) on raw pointers: int4 quantize + low-rank
 * down projection, grouped GEMM + low-rank up projection -> output [m, d_out] of T, no bias (the reference's layers add it
 * afterwards).  The layer keeps its scratch (quantized input, scales, low-rank activation) between calls and grows it
 * when m grows, as the reference's allocateBuffer does. */
template<typename T>
class W4A4Gemm {
public:
    W4A4Gemm(size_t d_out, size_t d_in, cudaStream_t stream = 0): d_out_(d_out), d_in_(d_in), stream_(stream) {}
    W4A4Gemm(const W4A4Gemm&)            = delete;
    W4A4Gemm& operator=(const W4A4Gemm&) = delete;
    ~W4A4Gemm() { cudaFree(workspace_); }

    void forward(T* output, const T* input, size_t m, const W4A4GemmWeight<T>* weights)
    {
        const size_t need = lyraq_workspace_bytes(LYRAQ_OP_LINEAR_W4A4_LORA, (int)m, (int)d_out_, (int)d_in_);
        if (need > workspace_bytes_) {
            cudaFree(workspace_);
            workspace_ = nullptr;
            workspace_bytes_ = 0;
            lyraq_detail::cuda_check(cudaMalloc(&workspace_, need), "cudaMalloc(W4A4Gemm workspace)");
            workspace_bytes_ = need;
        }
        lyraq_detail::check(lyraq_w4a4_lora_forward(output, input, lyraq_detail::DType<T>::value, weights->smooth,
                                                    reinterpret_cast<const uint8_t*>(weights->packed_weight), weights->weight_scale,
                                                    LYRAQ_F32, weights->lora_down, weights->lora_up, nullptr, nullptr, LYRAQ_EPI_NONE,
                                                    (int)m, (int)d_out_, (int)d_in_, workspace_, workspace_bytes_, stream_),
                            "W4A4Gemm::forward");
    }

private:
    size_t       d_out_, d_in_;
    cudaStream_t stream_;
    void*        workspace_       = nullptr;
    size_t       workspace_bytes_ = 0;
};

/* The two quantized entry points of cublasMMWrapper (src/lyradiff/utils/cublasMMWrapper.h:300-317 and :354-385),
 * as a small class that the layers can hold where they hold `cublas_wrapper_`. */
class QuantGemmWrapper {
public:
    explicit QuantGemmWrapper(cudaStream_t stream = 0, int c_dtype = LYRAQ_BF16): stream_(stream), c_dtype_(c_dtype) {}
    void setStream(cudaStream_t stream) { stream_ = stream; }
    void setOutputType(int c_dtype) { c_dtype_ = c_dtype; }

    /* The reference times 168 CUTLASS tactics per shape here (layers/gemm_utils/GemmProfiler.cc:78-127); the tcgen05
     * kernel picks its tile from the shape, so there is nothing to profile. */
    void profileGemmInt8(int, int, int) {}
    size_t getInt8WorkspaceSize(int m, int n, int k) const { return lyraq_workspace_bytes(0, m, n, k); }

    void runGemmInt8(const int8_t* A, const int8_t* B, const float* alphaCol, const float* alphaRow, void* C, int m, int n,
                     int k, char* workspace, cudaStream_t stream, bool per_token = false) const
    {
        lyraq_detail::check(lyraq_gemm_int8(A, B, alphaCol, alphaRow,
                                            per_token ? LYRAQ_SCALE_PER_TOKEN : LYRAQ_SCALE_PER_TENSOR, C, c_dtype_, nullptr,
                                            m, n, k, workspace, 0, stream),
                            "runGemmInt8");
    }

    /* runGemmInt8 followed by invokeFusedBiasResidualAdd<T>(dst, gemm_out, residual, bias, ...) in one launch
     * (BasicTransformerInt8Block.cc:824-845); C may be the residual buffer itself. */
    void runGemmInt8BiasResidual(const int8_t* A, const int8_t* B, const float* alphaCol, const float* alphaRow, void* C,
                                 const void* bias, const void* residual, int m, int n, int k, char* workspace,
                                 cudaStream_t stream, bool per_token = false) const
    {
        lyraq_detail::check(lyraq_gemm_int8_residual(A, B, alphaCol, alphaRow,
                                                     per_token ? LYRAQ_SCALE_PER_TOKEN : LYRAQ_SCALE_PER_TENSOR, C, c_dtype_,
                                                     bias, residual, m, n, k, workspace, 0, stream),
                            "runGemmInt8BiasResidual");
    }

    /* Called by the reference only as (OP_T, OP_N, n_out, m_tokens, k, W, k, s_w, X, k, s_x, Y, n_out, bias, R, alpha,
     * beta, is_gelu): Y[m_tokens, n_out] = X W^T.  Any other layout is refused. */
    void GemmWithResidualAndBias(cublasOperation_t transa, cublasOperation_t transb, const int m, const int n, const int k,
                                 const __nv_fp8_e4m3* A, const int lda, const float* a_scale, const __nv_fp8_e4m3* B,
                                 const int ldb, const float* b_scale, void* C, const int ldc, const void* bias,
                                 const void* Residual, float alpha = 1.0f, float beta = 1.0f, const bool is_gelu = false) const
    {
        if (transa != CUBLAS_OP_T || transb != CUBLAS_OP_N || lda != k || ldb != k || ldc != m) {
            throw std::runtime_error("GemmWithResidualAndBias(e4m3): only the (OP_T, OP_N, lda=ldb=k, ldc=m) form is supported");
        }
        lyraq_detail::check(lyraq_gemm_fp8(reinterpret_cast<const uint8_t*>(B), b_scale, reinterpret_cast<const uint8_t*>(A),
                                           a_scale, C, c_dtype_, bias, Residual, alpha, beta,
                                           is_gelu ? LYRAQ_EPI_GELU_TANH : LYRAQ_EPI_NONE, n, m, k, nullptr, 0, stream_),
                            "GemmWithResidualAndBias(e4m3)");
    }

private:
    cudaStream_t stream_;
    int          c_dtype_;
};

}  // namespace lyradiff

#endif /* LYRADIFF_SHIM_H_ */
