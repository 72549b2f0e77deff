// torch custom classes with the reference's names and signatures (namespace `lyradiff`, src/lyradiff/th_op/pybind.cc:9-96):
//   torch.classes.lyradiff.LyraDiffCommonContext()
//   torch.classes.lyradiff.FluxSingleTransformerBlockOp(inference_dtype, embedding_dim, embedding_head_num,
//                                                       embedding_head_dim, mlp_scale, quant_level)
//   torch.classes.lyradiff.FluxTransformerBlockOp(... same ...)
//   torch.classes.lyradiff.FluxTransformer2DModelOp(inference_dtype, input_channels, num_layers, num_single_layers,
//                                                   attention_head_dim, num_attention_heads, pooled_projection_dim,
//                                                   joint_attention_dim, guidance_embeds, quant_level)
// with initialize / forward / reload_model_from_state_dict / reload_model_from_bin / load_lora_by_name / clear_lora.
// quant_level 1, 2 (FP8) and 7, 8 (INT4 W4A4; the double-stream block keeps net.2 in FP8, as the reference does).
// Host code only: every device operation is a call into the C ABI of liblyraq.so (include/lyraq.h) on torch's current
// stream (attention included: lyraq_attention), plus one ATen library call per block (addmm for the 16-bit modulation
// linear of quant_level 1).  torch supplies device memory, the stream and the class registry; nothing here computes.
// The data flow is the one documented in lyradiff_b200/flux_blocks.py, which is the Python twin of this file.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <cmath>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/lyraq.h"

namespace {

using at::Tensor;

void check(int status, const char* what)
{
    TORCH_CHECK(status == LYRAQ_OK, what, " failed: ", lyraq_status_string(status),
                status == LYRAQ_ERR_CUDA ? lyraq_last_cuda_error() : "");
}

void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dt_code(at::ScalarType t)
{
    TORCH_CHECK(t == at::kBFloat16 || t == at::kHalf, "only bf16 and fp16 are supported");
    return t == at::kBFloat16 ? LYRAQ_BF16 : LYRAQ_F16;
}

at::ScalarType parse_dtype(const std::string& s)
{
    TORCH_CHECK(s == "bf16" || s == "fp16", "inference_dtype must be 'bf16' or 'fp16'");
    return s == "bf16" ? at::kBFloat16 : at::kHalf;
}

const void* ptr(const Tensor& t) { return t.defined() ? t.data_ptr() : nullptr; }

// A weight that takes part in LoRA hot-swap (LoraWeight<T> and its subclasses, src/lyradiff/interface/IFLoraWeight.h:15-133).
struct LoraTarget {
    virtual void load_lora(const Tensor& lora, double scale) = 0;
    virtual void clear_lora()                                = 0;
    virtual ~LoraTarget()                                    = default;
};

// w = T(w + T(lora * T(scale))) on the device copy `w` of a 16-bit weight
void merge_lora(Tensor& w, const Tensor& lora, double scale, at::ScalarType dt)
{
    TORCH_CHECK(lora.numel() == w.numel(), "lora weight has ", lora.numel(), " elements, the layer's weight ", w.numel());
    Tensor l = lora.to(w.device(), dt).contiguous();
    check(lyraq_load_lora(w.data_ptr(), l.data_ptr(), dt_code(dt), (float)scale, (size_t)w.numel(), stream()), "lyraq_load_lora");
}

// One FP8 linear as MACROLoadFP8WeightFromCache leaves it (src/lyradiff/utils/common_macro_def.h:76-92): e4m3 weight with
// its amax / 448 scale, bias, static input scale and a host copy of the 16-bit weight that every LoRA merge starts from
// (FP8LoraWeight<T>, IFLoraWeight.h:81-133).
struct Fp8Weight: LoraTarget {
    Tensor         qweight, w_scale, bias, input_scale, weight_h;
    int64_t        n = 0, k = 0;
    at::ScalarType dt = at::kBFloat16;
    bool           loaded_lora = false;

    void quantize(const Tensor& w)
    {
        check(lyraq_weight_quant_fp8(qweight.data_ptr<uint8_t>(), w_scale.data_ptr<float>(), w.data_ptr(), dt_code(dt),
                                     (size_t)w.numel(), stream()),
              "lyraq_weight_quant_fp8");
    }

    void load(const Tensor& weight, const Tensor& b, const Tensor& in_scale, const at::Device& dev, at::ScalarType dt_)
    {
        dt       = dt_;
        Tensor w = weight.to(dev, dt).contiguous();
        n        = w.size(0);
        k        = w.size(1);
        weight_h = w.to(at::kCPU);
        qweight  = at::empty({n, k}, w.options().dtype(at::kByte));
        w_scale  = at::empty({1}, w.options().dtype(at::kFloat));
        quantize(w);
        bias        = b.to(dev, dt).contiguous();
        input_scale = in_scale.to(dev, at::kFloat).reshape({1}).contiguous();
        loaded_lora = false;
    }

    void load_lora(const Tensor& lora, double scale) override
    {
        Tensor w = weight_h.to(qweight.device());
        merge_lora(w, lora, scale, dt);
        quantize(w);
        loaded_lora = true;
    }

    void clear_lora() override
    {
        if (loaded_lora) {
            quantize(weight_h.to(qweight.device()));
            loaded_lora = false;
        }
    }
};

Tensor fp8_gemm(const Fp8Weight& w, const Tensor& xq, int64_t m, at::ScalarType dt)
{
    Tensor y = at::empty({m, w.n}, xq.options().dtype(dt));
    check(lyraq_gemm_fp8(xq.data_ptr<uint8_t>(), w.input_scale.data_ptr<float>(), w.qweight.data_ptr<uint8_t>(),
                         w.w_scale.data_ptr<float>(), y.data_ptr(), dt_code(dt), ptr(w.bias), nullptr, 1.0f, 0.0f, LYRAQ_EPI_NONE,
                         (int)m, (int)w.n, (int)w.k, nullptr, 0, stream()),
          "lyraq_gemm_fp8");
    return y;
}

// out = gate * (x_q W^T * s + bias) + residual, in the GEMM's epilogue where a tile cannot straddle two batch entries.
Tensor fp8_gemm_gate_residual(const Fp8Weight& w, const Tensor& xq, const Tensor& gate, const Tensor& residual, int64_t batch,
                              int64_t seq, at::ScalarType dt)
{
    const int64_t m   = batch * seq;
    Tensor        out = at::empty_like(residual);
    if (batch == 1 || seq % 256 == 0) {
        check(lyraq_gemm_fp8_gate(xq.data_ptr<uint8_t>(), w.input_scale.data_ptr<float>(), w.qweight.data_ptr<uint8_t>(),
                                  w.w_scale.data_ptr<float>(), out.data_ptr(), dt_code(dt), ptr(w.bias), gate.data_ptr(),
                                  residual.data_ptr(), (int)seq, (int)m, (int)w.n, (int)w.k, nullptr, 0, stream()),
              "lyraq_gemm_fp8_gate");
        return out;
    }
    Tensor y = fp8_gemm(w, xq, m, dt);
    check(lyraq_gate_residual(out.data_ptr(), y.data_ptr(), gate.data_ptr(), residual.data_ptr(), dt_code(dt), (size_t)batch,
                              (size_t)seq, (size_t)w.n, stream()),
          "lyraq_gate_residual");
    return out;
}

// One W4A4 linear with its rank-32 LoRA branch, from the tensors W4A4GemmWeight<T>::loadWeights reads
// (src/lyradiff/layers/w4a4_gemm_block/W4A4GemmWeight.cc:62-79; the reference's state-dict loader for this layer is
// empty, so its .bin names serve as keys).
struct W4Weight {
    Tensor  packed, w_scale, smooth, lora_down, lora_up, bias, workspace;
    int64_t n = 0, k = 0;
    int     epilogue = LYRAQ_EPI_ROUND_EACH;

    void load(const c10::Dict<std::string, Tensor>& sd, const std::string& name, int64_t n_, int64_t k_, bool has_bias, bool gelu,
              const at::Device& dev, at::ScalarType dt)
    {
        n         = n_;
        k         = k_;
        packed    = sd.at(name + "packed_weight").to(dev).contiguous().view(at::kByte).reshape({n, k / 2});
        w_scale   = sd.at(name + "weight_scale").to(dev).contiguous().reshape({n, k / 64});
        if (w_scale.scalar_type() != at::kFloat && w_scale.scalar_type() != at::kHalf) {
            w_scale = w_scale.to(at::kFloat);
        }
        smooth    = sd.at(name + "smooth").to(dev, at::kFloat).contiguous();
        lora_down = sd.at(name + "lora_down").to(dev, dt).contiguous().reshape({32, k});
        lora_up   = sd.at(name + "lora_up").to(dev, dt).contiguous().reshape({n, 32});
        if (has_bias) {
            bias = sd.at(name + "bias").to(dev, dt).contiguous();
        }
        epilogue = LYRAQ_EPI_ROUND_EACH | (gelu ? LYRAQ_EPI_GELU_TANH : 0);
    }

    // the whole of W4A4Gemm<T>::forward with the roundings of the 16-bit kernels that follow it in the reference
    Tensor run(const Tensor& x, int64_t m, const Tensor& residual, at::ScalarType dt)
    {
        const size_t need = lyraq_workspace_bytes(LYRAQ_OP_LINEAR_W4A4_LORA, (int)m, (int)n, (int)k);
        if (!workspace.defined() || (size_t)workspace.numel() < need) {
            workspace = at::empty({(int64_t)need}, x.options().dtype(at::kByte));
        }
        Tensor y = at::empty({m, n}, x.options().dtype(dt));
        check(lyraq_w4a4_lora_forward(y.data_ptr(), x.data_ptr(), dt_code(dt), smooth.data_ptr<float>(), packed.data_ptr<uint8_t>(),
                                      w_scale.data_ptr(), w_scale.scalar_type() == at::kHalf ? LYRAQ_F16 : LYRAQ_F32,
                                      lora_down.data_ptr(), lora_up.data_ptr(), ptr(bias), ptr(residual), epilogue, (int)m, (int)n,
                                      (int)k, workspace.data_ptr(), (size_t)workspace.numel(), stream()),
              "lyraq_w4a4_lora_forward");
        return y;
    }
};

struct Modulation: LoraTarget {
    bool           fp8 = false;
    Fp8Weight      q;
    Tensor         w, b, weight_h;  // the 16-bit linear of quant_level 1 / 7 (LoraWeightV2<T>, IFLoraWeight.h:40-78)
    at::ScalarType dt16        = at::kBFloat16;
    bool           loaded_lora = false;

    void load(const c10::Dict<std::string, Tensor>& sd, const std::string& name, bool full, const at::Device& dev, at::ScalarType dt)
    {
        fp8 = full;
        if (full) {
            q.load(sd.at(name + ".weight"), sd.at(name + ".bias"), sd.at(name + "_input_scale"), dev, dt);
        } else {
            dt16        = dt;
            w           = sd.at(name + ".weight").to(dev, dt).contiguous();
            b           = sd.at(name + ".bias").to(dev, dt).contiguous();
            weight_h    = w.to(at::kCPU);
            loaded_lora = false;
        }
    }

    void load_lora(const Tensor& lora, double scale) override
    {
        if (fp8) {
            q.load_lora(lora, scale);
            return;
        }
        w.copy_(weight_h);
        merge_lora(w, lora, scale, dt16);
        loaded_lora = true;
    }

    void clear_lora() override
    {
        if (fp8) {
            q.clear_lora();
        } else if (loaded_lora) {
            w.copy_(weight_h);
            loaded_lora = false;
        }
    }

    // linear(temb) -> `chunks` contiguous [B, D] tensors (AdaFP8LayerNorm<T>::forward, AdaFP8LayerNorm.cc:96-160)
    std::vector<Tensor> run(const Tensor& temb, int64_t chunks, at::ScalarType dt) const
    {
        Tensor msa;
        if (fp8) {
            Tensor tq = at::empty(temb.sizes(), temb.options().dtype(at::kByte));
            check(lyraq_quant_fp8(tq.data_ptr<uint8_t>(), temb.data_ptr(), dt_code(dt), q.input_scale.data_ptr<float>(), 1,
                                  (size_t)temb.numel(), stream()),
                  "lyraq_quant_fp8");
            msa = fp8_gemm(q, tq, temb.size(0), dt);
        } else {
            msa = at::addmm(b, temb, w.t());
        }
        std::vector<Tensor> out;
        for (auto& c : msa.chunk(chunks, 1)) {
            out.push_back(c.contiguous());
        }
        return out;
    }
};

// One raw array of loadWeightFromBin (src/lyradiff/utils/memory_utils.cu:295-364): file `<path><key>.bin`; kind 'T' = a 16-bit
// tensor stored in the model file type (fp32 or fp16), 'f' = fp32 scales, 'i' = int8 (packed int4 weights).  A missing or
// short file raises (the reference logs a warning and leaves the weight uninitialised).
struct BinFile {
    std::string          key;
    std::vector<int64_t> shape;
    char                 kind;
};

Tensor read_bin(const std::string& path, const BinFile& f, bool file_fp16)
{
    const at::ScalarType st = f.kind == 'i' ? at::kChar : (f.kind == 'f' || !file_fp16) ? at::kFloat : at::kHalf;
    Tensor               t  = at::empty(f.shape, at::TensorOptions().dtype(st).device(at::kCPU));
    const std::string    fn = path + f.key + ".bin";
    const size_t         bytes = (size_t)t.numel() * t.element_size();
    FILE*                fp    = std::fopen(fn.c_str(), "rb");
    TORCH_CHECK(fp != nullptr, "weight file missing: ", fn);
    const size_t got = std::fread(t.data_ptr(), 1, bytes, fp);
    std::fclose(fp);
    TORCH_CHECK(got == bytes, "weight file too small: ", fn);
    return t;
}

void fp8_linear_files(std::vector<BinFile>& v, const std::string& name, int64_t n, int64_t k)
{
    v.push_back({name + ".weight", {n, k}, 'T'});
    v.push_back({name + ".bias", {n}, 'T'});
    v.push_back({name + "_input_scale", {1}, 'f'});
}

void w4a4_linear_files(std::vector<BinFile>& v, const std::string& name, int64_t n, int64_t k, bool has_bias)
{
    v.push_back({name + "packed_weight", {n, k / 2}, 'i'});
    v.push_back({name + "weight_scale", {n, k / 64}, 'f'});
    v.push_back({name + "lora_up", {n, 32}, 'T'});
    v.push_back({name + "lora_down", {32, k}, 'T'});
    v.push_back({name + "smooth", {k}, 'f'});
    if (has_bias) {
        v.push_back({name + "bias", {n}, 'T'});
    }
}

void modulation_files(std::vector<BinFile>& v, const std::string& name, int64_t chunks, int64_t D, bool fp8)
{
    v.push_back({name + ".weight", {chunks * D, D}, 'T'});
    v.push_back({name + ".bias", {chunks * D}, 'T'});
    if (fp8) {
        v.push_back({name + "_input_scale", {1}, 'f'});
    }
}

// The `device` argument of reload_model_from_state_dict says where the state dict's tensors live ("cpu" or "cuda...": the
// reference picks the memcpy kind from it, FluxSingleTransformerBlockOp.h:261-264, and its Python wrappers pass "cpu"); the
// weights always go to the current CUDA device.
at::Device target_device(const std::string& device)
{
    TORCH_CHECK(device == "cpu" || device.rfind("cuda", 0) == 0, "device must be 'cpu' or 'cuda[:n]' (where the state dict's tensors are)");
    return at::Device(at::kCUDA, at::cuda::current_device());
}

void check_inputs(std::initializer_list<Tensor> ts, at::ScalarType dt)
{
    for (const Tensor& t : ts) {
        TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == dt,
                    "inputs must be contiguous CUDA tensors of the inference dtype");
    }
}

// FlashAttention2Layer<T>::forward of the reference (layers/flash_attn2/flash_attn2.cu:59-118) on the packed, normalised
// and rotated projection qkv [B, S, 3, H, Dh]: lyraq_attention.  `out` is [B * rows, ld] in the inference type or, when
// `scale` is given, e4m3 codes for the FP8 linear that follows (the reference's separate cast pass); with `out2` the rows
// from `split` on of every batch go there (text and image parts of a joint sequence).
void attention(const Tensor& qkv, int64_t B, int64_t S, int64_t H, int64_t Dh, at::ScalarType dtype, uint8_t* out, int64_t ld,
               const Tensor* scale, uint8_t* out2 = nullptr, int64_t ld2 = 0, const Tensor* scale2 = nullptr, int64_t split = 0)
{
    const int dtc = dt_code(dtype);
    check(lyraq_attention(out, scale != nullptr ? LYRAQ_E4M3 : dtc, (size_t)ld, scale != nullptr ? scale->data_ptr<float>() : nullptr,
                          out2, (size_t)ld2, scale2 != nullptr ? scale2->data_ptr<float>() : nullptr, (size_t)split, qkv.data_ptr(),
                          dtc, (size_t)B, (size_t)S, (int)H, (int)Dh, 1.0f / std::sqrt((float)Dh), stream()),
          "lyraq_attention");
}

}  // namespace

struct LyraDiffCommonContext: torch::CustomClassHolder {
    LyraDiffCommonContext() = default;
};

// A block's modulation computed ahead of the block on another stream (the whole-model forward does that: it depends on temb
// alone): the tensors and the event recorded behind them.  take() makes the current stream wait for the event and tells the
// caching allocator that the tensors are used on this stream too.
struct AheadModulation {
    std::vector<std::vector<Tensor>>       parts;  // single block: one list of 3; double block: image list of 6, text list of 6
    std::shared_ptr<at::cuda::CUDAEvent>   event;
    void take() const
    {
        auto cur = at::cuda::getCurrentCUDAStream();
        event->block(cur);
        for (const auto& list : parts) {
            for (const Tensor& t : list) {
                c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), cur);
            }
        }
    }
};

struct BlockBase: torch::CustomClassHolder {
    at::ScalarType dtype;
    int64_t        dim, heads, head_dim, mlp_scale, quant_level;
    bool           loaded = false;

    BlockBase(const std::string& inference_dtype, int64_t embedding_dim, int64_t embedding_head_num, int64_t embedding_head_dim,
              int64_t mlp_scale_, int64_t quant_level_):
        dtype(parse_dtype(inference_dtype)), dim(embedding_dim), heads(embedding_head_num), head_dim(embedding_head_dim),
        mlp_scale(mlp_scale_), quant_level(quant_level_)
    {
        TORCH_CHECK(quant_level == 1 || quant_level == 2 || quant_level == 7 || quant_level == 8, "quant_level ", quant_level,
                    ": only 1, 2 (FP8) and 7, 8 (INT4 W4A4) are built here; the 16-bit level 0 (the reference's default) and FP8 "
                    "weight-only level 3 stay with the reference's own library");
        TORCH_CHECK(heads * head_dim == dim, "embedding_dim must equal embedding_head_num * embedding_head_dim");
    }
    // one lock per op object, held for the whole call, as the reference's ops do (FluxSingleTransformerBlockOp.h:67,231)
    std::mutex lock;

    void initialize(const c10::intrusive_ptr<LyraDiffCommonContext>&) {}

    virtual void                               load_state_dict(const std::string& prefix, const c10::Dict<std::string, Tensor>& sd,
                                                               const std::string& device) = 0;
    virtual std::vector<BinFile>               bin_files()                                = 0;
    virtual std::map<std::string, LoraTarget*> lora_table()                               = 0;

    void reload_model_from_state_dict(const std::string& prefix, const c10::Dict<std::string, Tensor>& sd, const std::string& device)
    {
        std::lock_guard<std::mutex> g(lock);
        load_state_dict(prefix, sd, device);
    }

    // *BlockWeight<T>::loadWeights: one raw file `<model_path><key>.bin` per tensor, keys as in the state dict; model_dtype
    // "fp32" or "fp16" is the file type of the 16-bit tensors (FluxSingleTransformerBlockOp.h:229-248).
    void reload_model_from_bin(const std::string& model_path, const std::string& model_dtype)
    {
        TORCH_CHECK(model_dtype == "fp32" || model_dtype == "fp16", "wrong model_dtype");
        c10::Dict<std::string, Tensor> sd;
        for (const BinFile& f : bin_files()) {
            sd.insert(f.key, read_bin(model_path, f, model_dtype == "fp16"));
        }
        std::lock_guard<std::mutex> g(lock);
        load_state_dict("", sd, "cuda");
    }

    // IFLoraWeight<T>::loadLoraByName (IFLoraWeight.h:150-173): the names are the path to one linear; a path that leads
    // nowhere is reported and skipped, as the reference does.
    void load_lora_by_name(const std::vector<std::string>& names, const Tensor& weight, double scale)
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::string key;
        for (const std::string& n : names) {
            key += (key.empty() ? "" : "/") + n;
        }
        std::lock_guard<std::mutex> g(lock);
        auto                        table = lora_table();
        auto                        it    = table.find(key);
        if (it == table.end()) {
            TORCH_WARN("lora name cannot find weights to load: ", key);
            return;
        }
        it->second->load_lora(weight, scale);
    }

    void clear_lora()
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::lock_guard<std::mutex> g(lock);
        for (auto& kv : lora_table()) {
            kv.second->clear_lora();
        }
    }
};

// FluxSingleTransformerBlockOp (th_op/flux_single_transformer_block/FluxSingleTransformerBlockOp.h:287-315)
struct FluxSingleTransformerBlockOp: BlockBase {
    using BlockBase::BlockBase;
    Fp8Weight  qkv, mlp, out;
    W4Weight   qkv4, mlp4, out4_attn, out4_mlp;  // quant_level 7 / 8
    Modulation norm;
    Tensor     qk_scale;

    bool   int4() const { return quant_level == 7 || quant_level == 8; }
    Tensor forward_int4(const Tensor& hidden, const Tensor& rope, const std::vector<Tensor>& mod);

    std::vector<BinFile> bin_files() override
    {
        std::vector<BinFile> v;
        modulation_files(v, "norm.linear", 3, dim, quant_level == 2 || quant_level == 8);
        v.push_back({"attn.norm_q.weight", {head_dim}, 'T'});
        v.push_back({"attn.norm_k.weight", {head_dim}, 'T'});
        if (int4()) {
            w4a4_linear_files(v, "attn.to_qkv.", 3 * dim, dim, true);
            w4a4_linear_files(v, "proj_mlp.", mlp_scale * dim, dim, true);
            w4a4_linear_files(v, "proj_out.linears.0.", dim, dim, true);
            w4a4_linear_files(v, "proj_out.linears.1.linear.", dim, mlp_scale * dim, false);
        } else {
            fp8_linear_files(v, "attn.to_qkv", 3 * dim, dim);
            fp8_linear_files(v, "proj_mlp", mlp_scale * dim, dim);
            fp8_linear_files(v, "proj_out", dim, (mlp_scale + 1) * dim);
        }
        return v;
    }

    // names as the reference's lora_layer_map / lora_weight_map nest them (FluxSingleTransformerFP8BlockWeight.cc:33,80-89,
    // FluxSingleAttentionFP8ProcessorWeight.cc:51-54, AdaFP8LayerNormWeight.cc:47-51); the W4A4 linears have no hot-swap
    // in the reference either
    std::map<std::string, LoraTarget*> lora_table() override
    {
        std::map<std::string, LoraTarget*> t{{"norm/linear", &norm}};
        if (!int4()) {
            t["attn/to_qkv"] = &qkv;
            t["proj_mlp"]    = &mlp;
            t["proj_out"]    = &out;
        }
        return t;
    }

    void load_state_dict(const std::string& prefix, const c10::Dict<std::string, Tensor>& sd, const std::string& device) override
    {
        const at::Device dev = target_device(device);
        auto g = [&](const std::string& n) { return sd.at(prefix + n); };
        const bool fp8_modulation = quant_level == 2 || quant_level == 8;
        if (int4()) {
            // keys of FluxSingleTransformerInt4BlockWeight.cc:79-83 and FluxSingleAttentionInt4ProcessorWeight.cc:73-78
            qkv4.load(sd, prefix + "attn.to_qkv.", 3 * dim, dim, true, false, dev, dtype);
            mlp4.load(sd, prefix + "proj_mlp.", mlp_scale * dim, dim, true, true, dev, dtype);
            out4_attn.load(sd, prefix + "proj_out.linears.0.", dim, dim, true, false, dev, dtype);
            out4_mlp.load(sd, prefix + "proj_out.linears.1.linear.", dim, mlp_scale * dim, false, false, dev, dtype);
        } else {
            qkv.load(g("attn.to_qkv.weight"), g("attn.to_qkv.bias"), g("attn.to_qkv_input_scale"), dev, dtype);
            mlp.load(g("proj_mlp.weight"), g("proj_mlp.bias"), g("proj_mlp_input_scale"), dev, dtype);
            out.load(g("proj_out.weight"), g("proj_out.bias"), g("proj_out_input_scale"), dev, dtype);
            TORCH_CHECK(qkv.n == 3 * dim && mlp.n == mlp_scale * dim && out.k == (mlp_scale + 1) * dim,
                        "weight shapes do not match the block's dimensions");
        }
        c10::Dict<std::string, Tensor> sub;
        for (const char* n : {"norm.linear.weight", "norm.linear.bias"}) {
            sub.insert(n, g(n));
        }
        if (fp8_modulation) {
            sub.insert("norm.linear_input_scale", g("norm.linear_input_scale"));
        }
        norm.load(sub, "norm.linear", fp8_modulation, dev, dtype);
        qk_scale = at::cat({g("attn.norm_q.weight").reshape({-1}), g("attn.norm_k.weight").reshape({-1})}).to(dev, dtype).contiguous();
        loaded = true;
    }

    std::vector<Tensor> modulation(const Tensor& temb) { return norm.run(temb, 3, dtype); }

    Tensor forward(const Tensor& hidden, const Tensor& rope, const Tensor& temb) { return forward_with(hidden, rope, temb, nullptr); }

    Tensor forward_with(const Tensor& hidden, const Tensor& rope, const Tensor& temb, const AheadModulation* ahead)
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::lock_guard<std::mutex> guard(lock);
        check_inputs({hidden, rope, temb}, dtype);
        const int64_t B = hidden.size(0), S = hidden.size(1), D = hidden.size(2), T = B * S;
        TORCH_CHECK(D == dim && temb.size(0) == B && temb.size(1) == D && rope.numel() == T * head_dim * 2, "shape mismatch");
        const int  dtc  = dt_code(dtype);
        if (ahead != nullptr) {
            ahead->take();
        }
        auto       mod  = ahead != nullptr ? ahead->parts[0] : norm.run(temb, 3, dtype);  // shift, scale, gate
        if (int4()) {
            return forward_int4(hidden, rope, mod);
        }
        const auto opt8 = hidden.options().dtype(at::kByte);
        Tensor     nq = at::empty({T, D}, opt8), mq = at::empty({T, D}, opt8);
        check(lyraq_adaln_quant_fp8x2(nullptr, nq.data_ptr<uint8_t>(), qkv.input_scale.data_ptr<float>(), mq.data_ptr<uint8_t>(),
                                      mlp.input_scale.data_ptr<float>(), hidden.data_ptr(), mod[1].data_ptr(), mod[0].data_ptr(),
                                      dtc, (size_t)B, (size_t)S, (size_t)D, 1e-6, stream()),
              "lyraq_adaln_quant_fp8x2");
        Tensor q3 = fp8_gemm(qkv, nq, T, dtype);
        check(lyraq_rmsnorm_rope(q3.data_ptr(), q3.data_ptr(), qk_scale.data_ptr(), rope.data_ptr(), dtc, 1e-6, (size_t)B, (size_t)S,
                                 (int)heads, (int)head_dim, stream()),
              "lyraq_rmsnorm_rope");
        // the attention output leaves the kernel as e4m3 in the first column window of proj_out's [T, (mlp_scale + 1) D] input
        const int64_t ld = (mlp_scale + 1) * D;
        Tensor cat8 = at::empty({T, ld}, opt8);
        attention(q3, B, S, heads, head_dim, dtype, cat8.data_ptr<uint8_t>(), ld, &out.input_scale);
        check(lyraq_gemm_fp8_quant_ld(mq.data_ptr<uint8_t>(), mlp.input_scale.data_ptr<float>(), mlp.qweight.data_ptr<uint8_t>(),
                                      mlp.w_scale.data_ptr<float>(), cat8.data_ptr<uint8_t>() + D, (size_t)ld,
                                      out.input_scale.data_ptr<float>(), dtc, ptr(mlp.bias), nullptr, 1.0f, 0.0f,
                                      LYRAQ_EPI_GELU_TANH, (int)T, (int)mlp.n, (int)mlp.k, nullptr, 0, stream()),
              "lyraq_gemm_fp8_quant_ld");
        return fp8_gemm_gate_residual(out, cat8, mod[2], hidden, B, S, dtype);
    }
};

// FluxSingleTransformerInt4Block<T>::forward (layers/flux_single_transformer_block/FluxSingleTransformerInt4Block.cc:198-322):
// every linear a W4A4 linear with its LoRA branch; proj_out is two of them, summed through the second one's residual.
Tensor FluxSingleTransformerBlockOp::forward_int4(const Tensor& hidden, const Tensor& rope, const std::vector<Tensor>& mod)
{
    const int64_t B = hidden.size(0), S = hidden.size(1), D = hidden.size(2), T = B * S;
    const int     dtc = dt_code(dtype);
    Tensor norm16 = at::empty({T, D}, hidden.options());
    check(lyraq_adaln_quant(norm16.data_ptr(), nullptr, nullptr, nullptr, nullptr, hidden.data_ptr(), mod[1].data_ptr(),
                            mod[0].data_ptr(), dtc, nullptr, (size_t)B, (size_t)S, (size_t)D, 1e-6, stream()),
          "lyraq_adaln_quant");
    Tensor q3 = qkv4.run(norm16, T, Tensor(), dtype);
    check(lyraq_rmsnorm_rope(q3.data_ptr(), q3.data_ptr(), qk_scale.data_ptr(), rope.data_ptr(), dtc, 1e-6, (size_t)B, (size_t)S,
                             (int)heads, (int)head_dim, stream()),
          "lyraq_rmsnorm_rope");
    Tensor attn = at::empty({T, D}, hidden.options());
    attention(q3, B, S, heads, head_dim, dtype, static_cast<uint8_t*>(attn.data_ptr()), D, nullptr);
    Tensor act  = mlp4.run(norm16, T, Tensor(), dtype);
    Tensor h1   = out4_attn.run(attn, T, Tensor(), dtype);
    Tensor h    = out4_mlp.run(act, T, h1, dtype);
    Tensor out  = at::empty_like(hidden);
    check(lyraq_gate_residual(out.data_ptr(), h.data_ptr(), mod[2].data_ptr(), hidden.data_ptr(), dtc, (size_t)B, (size_t)S, (size_t)D,
                              stream()),
          "lyraq_gate_residual");
    return out;
}

// FluxTransformerBlockOp (th_op/flux_transformer_block/FluxTransformerBlockOp.h:187-237)
struct FluxTransformerBlockOp: BlockBase {
    using BlockBase::BlockBase;
    bool int4() const { return quant_level == 7 || quant_level == 8; }
    struct Stream {
        Fp8Weight  qkv, out, ff1, ff2;
        W4Weight   qkv4, out4, ff14;  // quant_level 7 / 8: to_qkv, to_out and net.0.proj are W4A4 linears; net.2 stays FP8
        Modulation norm;
        Tensor     qk_scale;
    } img, txt;

    void load_stream(Stream& s, const std::string& prefix, const c10::Dict<std::string, Tensor>& sd, const at::Device& dev,
                     const std::string& norm, const std::string& qkv, const std::string& out, const std::string& nq,
                     const std::string& nk, const std::string& ff)
    {
        auto g = [&](const std::string& n) { return sd.at(prefix + n); };
        auto lin = [&](Fp8Weight& w, const std::string& n) { w.load(g(n + ".weight"), g(n + ".bias"), g(n + "_input_scale"), dev, dtype); };
        const bool fp8_modulation = quant_level == 2 || quant_level == 8;
        if (int4()) {
            // keys of FluxAttentionInt4ProcessorWeight.cc:63-66 and FluxAttnPostInt4ProcessorWeight.cc:94-96
            s.qkv4.load(sd, prefix + qkv + ".", 3 * dim, dim, true, false, dev, dtype);
            s.out4.load(sd, prefix + out + ".", dim, dim, true, false, dev, dtype);
            s.ff14.load(sd, prefix + ff + ".net.0.proj.", 4 * dim, dim, true, true, dev, dtype);
        } else {
            lin(s.qkv, qkv);
            lin(s.out, out);
            lin(s.ff1, ff + ".net.0.proj");
        }
        lin(s.ff2, ff + ".net.2");
        c10::Dict<std::string, Tensor> sub;
        sub.insert("m.weight", g(norm + ".linear.weight"));
        sub.insert("m.bias", g(norm + ".linear.bias"));
        if (fp8_modulation) {
            sub.insert("m_input_scale", g(norm + ".linear_input_scale"));
        }
        s.norm.load(sub, "m", fp8_modulation, dev, dtype);
        s.qk_scale = at::cat({g(nq).reshape({-1}), g(nk).reshape({-1})}).to(dev, dtype).contiguous();
    }

    std::vector<BinFile> bin_files() override
    {
        std::vector<BinFile> v;
        const char*          names[2][6] = {{"norm1", "attn.to_qkv", "attn.to_out.0", "attn.norm_q.weight", "attn.norm_k.weight", "ff"},
                                            {"norm1_context", "attn.to_added_qkv", "attn.to_add_out", "attn.norm_added_q.weight",
                                             "attn.norm_added_k.weight", "ff_context"}};
        for (auto& s : names) {
            const std::string norm = s[0], qkv = s[1], out = s[2], ff = s[5];
            modulation_files(v, norm + ".linear", 6, dim, quant_level == 2 || quant_level == 8);
            v.push_back({s[3], {head_dim}, 'T'});
            v.push_back({s[4], {head_dim}, 'T'});
            if (int4()) {
                w4a4_linear_files(v, qkv + ".", 3 * dim, dim, true);
                w4a4_linear_files(v, out + ".", dim, dim, true);
                w4a4_linear_files(v, ff + ".net.0.proj.", 4 * dim, dim, true);
            } else {
                fp8_linear_files(v, qkv, 3 * dim, dim);
                fp8_linear_files(v, out, dim, dim);
                fp8_linear_files(v, ff + ".net.0.proj", 4 * dim, dim);
            }
            fp8_linear_files(v, ff + ".net.2", dim, 4 * dim);
        }
        return v;
    }

    // FluxTransformerFP8BlockWeight.cc:41-45, FluxAttentionFP8ProcessorWeight.cc:91-108, FluxAttnPostFP8ProcessorWeight.cc:58-64
    std::map<std::string, LoraTarget*> lora_table() override
    {
        std::map<std::string, LoraTarget*> t{{"norm1/linear", &img.norm}, {"norm1_context/linear", &txt.norm},
                                             {"ff/net.2", &img.ff2}, {"ff_context/net.2", &txt.ff2}};
        if (!int4()) {
            t["attn/to_qkv"]           = &img.qkv;
            t["attn/to_out.0"]         = &img.out;
            t["attn/to_added_qkv"]     = &txt.qkv;
            t["attn/to_add_out"]       = &txt.out;
            t["ff/net.0.proj"]         = &img.ff1;
            t["ff_context/net.0.proj"] = &txt.ff1;
        }
        return t;
    }

    void load_state_dict(const std::string& prefix, const c10::Dict<std::string, Tensor>& sd, const std::string& device) override
    {
        const at::Device dev = target_device(device);
        load_stream(img, prefix, sd, dev, "norm1", "attn.to_qkv", "attn.to_out.0", "attn.norm_q.weight", "attn.norm_k.weight", "ff");
        load_stream(txt, prefix, sd, dev, "norm1_context", "attn.to_added_qkv", "attn.to_add_out", "attn.norm_added_q.weight",
                    "attn.norm_added_k.weight", "ff_context");
        loaded = true;
    }

    Tensor adaln16(const Tensor& x, const Tensor& scale, const Tensor& shift)
    {
        Tensor y = at::empty_like(x);
        check(lyraq_adaln_quant(y.data_ptr(), nullptr, nullptr, nullptr, nullptr, x.data_ptr(), scale.data_ptr(), shift.data_ptr(),
                                dt_code(dtype), nullptr, (size_t)x.size(0), (size_t)x.size(1), (size_t)x.size(2), 1e-6, stream()),
              "lyraq_adaln_quant");
        return y;
    }

    Tensor pre_attention(Stream& s, const Tensor& x, const std::vector<Tensor>& mod)
    {
        const int64_t B = x.size(0), S = x.size(1), D = x.size(2);
        if (int4()) {
            return s.qkv4.run(adaln16(x, mod[1], mod[0]).view({B * S, D}), B * S, Tensor(), dtype);
        }
        Tensor nq = at::empty({B * S, D}, x.options().dtype(at::kByte));
        check(lyraq_adaln_quant(nullptr, nullptr, nullptr, nq.data_ptr<uint8_t>(), s.qkv.input_scale.data_ptr<float>(), x.data_ptr(),
                                mod[1].data_ptr(), mod[0].data_ptr(), dt_code(dtype), nullptr, (size_t)B, (size_t)S, (size_t)D, 1e-6,
                                stream()),
              "lyraq_adaln_quant");
        return fp8_gemm(s.qkv, nq, B * S, dtype);
    }

    Tensor post_attention(Stream& s, const Tensor& x, const Tensor& attn, const std::vector<Tensor>& mod)
    {
        const int64_t B = x.size(0), S = x.size(1), D = x.size(2), T = B * S;
        const int     dtc  = dt_code(dtype);
        const auto    opt8 = x.options().dtype(at::kByte);
        if (int4()) {
            // FluxAttnPostInt4Processor<T>::forward: W4A4 to_out and net.0.proj with the reference's 16-bit bias / GELU
            // kernels as rounding steps of their epilogues, then the e4m3 quantize and the FP8 net.2 with gate + residual
            Tensor ao = s.out4.run(attn, T, Tensor(), dtype);
            Tensor h  = at::empty_like(x);
            check(lyraq_gate_residual(h.data_ptr(), ao.data_ptr(), mod[2].data_ptr(), x.data_ptr(), dtc, (size_t)B, (size_t)S,
                                      (size_t)D, stream()),
                  "lyraq_gate_residual");
            Tensor n2  = adaln16(h, mod[4], mod[3]);
            Tensor f1  = s.ff14.run(n2.view({T, D}), T, Tensor(), dtype);
            Tensor f1q = at::empty({T, s.ff14.n}, opt8);
            check(lyraq_quant_fp8(f1q.data_ptr<uint8_t>(), f1.data_ptr(), dtc, s.ff2.input_scale.data_ptr<float>(), 1,
                                  (size_t)f1.numel(), stream()),
                  "lyraq_quant_fp8");
            return fp8_gemm_gate_residual(s.ff2, f1q, mod[5], h, B, S, dtype);
        }
        Tensor h  = fp8_gemm_gate_residual(s.out, attn, mod[2], x, B, S, dtype);  // attn: e4m3 codes from the attention kernel
        Tensor nq = at::empty({T, D}, opt8);
        check(lyraq_adaln_quant(nullptr, nullptr, nullptr, nq.data_ptr<uint8_t>(), s.ff1.input_scale.data_ptr<float>(), h.data_ptr(),
                                mod[4].data_ptr(), mod[3].data_ptr(), dtc, nullptr, (size_t)B, (size_t)S, (size_t)D, 1e-6, stream()),
              "lyraq_adaln_quant");
        Tensor f1 = at::empty({T, s.ff1.n}, opt8);
        check(lyraq_gemm_fp8_quant(nq.data_ptr<uint8_t>(), s.ff1.input_scale.data_ptr<float>(), s.ff1.qweight.data_ptr<uint8_t>(),
                                   s.ff1.w_scale.data_ptr<float>(), f1.data_ptr<uint8_t>(), s.ff2.input_scale.data_ptr<float>(), dtc,
                                   ptr(s.ff1.bias), nullptr, 1.0f, 0.0f, LYRAQ_EPI_GELU_TANH, (int)T, (int)s.ff1.n, (int)s.ff1.k,
                                   nullptr, 0, stream()),
              "lyraq_gemm_fp8_quant");
        return fp8_gemm_gate_residual(s.ff2, f1, mod[5], h, B, S, dtype);
    }

    std::vector<std::vector<Tensor>> modulation(const Tensor& temb) { return {img.norm.run(temb, 6, dtype), txt.norm.run(temb, 6, dtype)}; }

    std::vector<Tensor> forward(const Tensor& hidden, const Tensor& encoder, const Tensor& rope, const Tensor& temb)
    {
        return forward_with(hidden, encoder, rope, temb, nullptr);
    }

    std::vector<Tensor> forward_with(const Tensor& hidden, const Tensor& encoder, const Tensor& rope, const Tensor& temb,
                                     const AheadModulation* ahead)
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::lock_guard<std::mutex> guard(lock);
        check_inputs({hidden, encoder, rope, temb}, dtype);
        const int64_t B = hidden.size(0), S = hidden.size(1), D = hidden.size(2), E = encoder.size(1), tot = S + E;
        TORCH_CHECK(D == dim && encoder.size(0) == B && encoder.size(2) == D && temb.size(0) == B && temb.size(1) == D &&
                        rope.numel() == B * tot * head_dim * 2,
                    "shape mismatch");
        if (ahead != nullptr) {
            ahead->take();
        }
        auto   mod_i = ahead != nullptr ? ahead->parts[0] : img.norm.run(temb, 6, dtype);
        auto   mod_t = ahead != nullptr ? ahead->parts[1] : txt.norm.run(temb, 6, dtype);
        Tensor qi = pre_attention(img, hidden, mod_i).view({B, S, 3 * D});
        Tensor qt = pre_attention(txt, encoder, mod_t).view({B, E, 3 * D});
        // joint sequence [B, E + S, 3, H, Dh], text first (invokeFusedRmsNormCatAndRope, flux_apply_rope.cu:78-156)
        Tensor joint = at::empty({B, tot, 3 * D}, hidden.options());
        Tensor r     = rope.view({B, tot, head_dim * 2});
        const int dtc = dt_code(dtype);
        for (int64_t b = 0; b < B; ++b) {
            check(lyraq_rmsnorm_rope(joint[b].slice(0, 0, E).data_ptr(), qt[b].data_ptr(), txt.qk_scale.data_ptr(),
                                     r[b].slice(0, 0, E).data_ptr(), dtc, 1e-6, 1, (size_t)E, (int)heads, (int)head_dim, stream()),
                  "lyraq_rmsnorm_rope");
            check(lyraq_rmsnorm_rope(joint[b].slice(0, E, tot).data_ptr(), qi[b].data_ptr(), img.qk_scale.data_ptr(),
                                     r[b].slice(0, E, tot).data_ptr(), dtc, 1e-6, 1, (size_t)S, (int)heads, (int)head_dim, stream()),
                  "lyraq_rmsnorm_rope");
        }
        // one attention over the joint sequence; its text rows and image rows leave as the inputs of the two to_out linears
        // (e4m3 with each linear's input scale; the 16-bit type for the W4A4 linears, which quantize their own input)
        const auto opt_a = int4() ? hidden.options() : hidden.options().dtype(at::kByte);
        Tensor attn_t = at::empty({B * E, D}, opt_a), attn_i = at::empty({B * S, D}, opt_a);
        attention(joint, B, tot, heads, head_dim, dtype, static_cast<uint8_t*>(attn_t.data_ptr()), D,
                  int4() ? nullptr : &txt.out.input_scale, static_cast<uint8_t*>(attn_i.data_ptr()), D,
                  int4() ? nullptr : &img.out.input_scale, E);
        Tensor out_i  = post_attention(img, hidden, attn_i, mod_i);
        Tensor out_t  = post_attention(txt, encoder, attn_t, mod_t);
        return {out_i, out_t};
    }
};

// ---------------------------------------------------------------------------------------------------------------------
// FluxTransformer2DModelOp (th_op/pybind.cc:13-44, th_op/flux_transformer_2d_model/FluxTransformer2DModelOp.cc:65-154):
// FluxTransformer2DModel<T>::transformer_forward (models/flux_transformer_2d_model/FluxTransformer2DModel.cc:230-515).  The
// quantized blocks are the classes above; what the reference runs in 16 bits through cuBLAS (the three small embedders,
// x_embedder, context_embedder, norm_out.linear, proj_out) runs through ATen matmuls, library code on both sides.
struct Linear16: LoraTarget {
    Tensor         w, b, weight_h;
    at::ScalarType dt = at::kBFloat16;
    bool           loaded_lora = false;

    void load(const c10::Dict<std::string, Tensor>& sd, const std::string& name, const at::Device& dev, at::ScalarType dt_)
    {
        dt          = dt_;
        w           = sd.at(name + ".weight").to(dev, dt).contiguous();
        b           = sd.at(name + ".bias").to(dev, dt).contiguous();
        weight_h    = w.to(at::kCPU);
        loaded_lora = false;
    }
    Tensor run(const Tensor& x) const { return at::addmm(b, x, w.t()); }
    void   load_lora(const Tensor& lora, double scale) override
    {
        w.copy_(weight_h);
        merge_lora(w, lora, scale, dt);
        loaded_lora = true;
    }
    void clear_lora() override
    {
        if (loaded_lora) {
            w.copy_(weight_h);
            loaded_lora = false;
        }
    }
};

// TimestepEmbeddingBlock<T>::forward (layers/timestep_embedding_block/TimestepEmbeddingBlock.cc): linear_1 -> T(h + bias)
// -> SiLU -> linear_2 + bias
struct Mlp16 {
    Linear16 l1, l2;
    void load(const c10::Dict<std::string, Tensor>& sd, const std::string& prefix, const at::Device& dev, at::ScalarType dt)
    {
        l1.load(sd, prefix + "linear_1", dev, dt);
        l2.load(sd, prefix + "linear_2", dev, dt);
    }
    Tensor run(const Tensor& x) const { return l2.run(at::silu(at::matmul(x, l1.w.t()) + l1.b)); }
};

struct FluxTransformer2DModelOp: torch::CustomClassHolder {
    at::ScalarType dtype;
    int64_t        in_ch, n_double, n_single, head_dim, heads, dim, pooled_dim, joint_dim, quant_level;
    bool           loaded = false;
    std::mutex     lock;
    std::vector<c10::intrusive_ptr<FluxTransformerBlockOp>>       dbl;
    std::vector<c10::intrusive_ptr<FluxSingleTransformerBlockOp>> sgl;
    Linear16 x_embedder, context_embedder, proj_out, norm_out;
    Mlp16    timestep_embedder, guidance_embedder, text_embedder;
    Tensor   exponents;  // the frequency table of TimeProjection<T>, fp32 [128], on the device

    FluxTransformer2DModelOp(const std::string& inference_dtype, int64_t input_channels, int64_t num_layers,
                             int64_t num_single_layers, int64_t attention_head_dim, int64_t num_attention_heads,
                             int64_t pooled_projection_dim, int64_t joint_attention_dim, bool guidance_embeds, int64_t quant_level_):
        dtype(parse_dtype(inference_dtype)), in_ch(input_channels), n_double(num_layers), n_single(num_single_layers),
        head_dim(attention_head_dim), heads(num_attention_heads), dim(attention_head_dim * num_attention_heads),
        pooled_dim(pooled_projection_dim), joint_dim(joint_attention_dim), quant_level(quant_level_)
    {
        TORCH_CHECK(guidance_embeds, "the model is built with the guidance embedder, as the reference's C++ model is");
        for (int64_t i = 0; i < n_double; ++i) {
            dbl.push_back(c10::make_intrusive<FluxTransformerBlockOp>(inference_dtype, dim, heads, head_dim, 6, quant_level));
        }
        for (int64_t i = 0; i < n_single; ++i) {
            sgl.push_back(c10::make_intrusive<FluxSingleTransformerBlockOp>(inference_dtype, dim, heads, head_dim, 4, quant_level));
        }
    }

    void initialize(const c10::intrusive_ptr<LyraDiffCommonContext>&) {}

    void load(const c10::Dict<std::string, Tensor>& sd, const std::string& device)
    {
        const at::Device dev = target_device(device);
        x_embedder.load(sd, "x_embedder", dev, dtype);
        context_embedder.load(sd, "context_embedder", dev, dtype);
        proj_out.load(sd, "proj_out", dev, dtype);
        norm_out.load(sd, "norm_out.linear", dev, dtype);
        timestep_embedder.load(sd, "time_text_embed.timestep_embedder.", dev, dtype);
        guidance_embedder.load(sd, "time_text_embed.guidance_embedder.", dev, dtype);
        text_embedder.load(sd, "time_text_embed.text_embedder.", dev, dtype);
        // TimeProjection<T>(256, flip_sin_to_cos = true, downscale_freq_shift = 0) (layers/time_proj/TimeProjection.cc:39-51):
        // exponents exp(-ln(10000) * i / 128) in fp32 on the host, copied to the device once
        std::vector<float> table(128);
        const float        factor = -std::log(10000.0f) / 128.0f;
        for (int i = 0; i < 128; ++i) {
            table[i] = std::exp(factor * (float)i);
        }
        exponents = at::from_blob(table.data(), {128}, at::TensorOptions().dtype(at::kFloat)).to(dev);
        for (int64_t i = 0; i < n_double; ++i) {
            dbl[i]->reload_model_from_state_dict("transformer_blocks." + std::to_string(i) + ".", sd, device);
        }
        for (int64_t i = 0; i < n_single; ++i) {
            sgl[i]->reload_model_from_state_dict("single_transformer_blocks." + std::to_string(i) + ".", sd, device);
        }
        loaded = true;
    }

    // keys of FluxTransformer2DModelWeight<T>::loadWeightsFromCache (FluxTransformer2DModelWeight.cc:297-337)
    void reload_transformer_model_from_state_dict(const c10::Dict<std::string, Tensor>& weights, const std::string& device)
    {
        std::lock_guard<std::mutex> g(lock);
        load(weights, device);
    }

    // FluxTransformer2DModelWeight<T>::loadWeights (FluxTransformer2DModelWeight.cc:239-275): raw `<model_path><key>.bin` files
    void reload_transformer_model(const std::string& model_path, const std::string& model_dtype)
    {
        TORCH_CHECK(model_dtype == "fp32" || model_dtype == "fp16", "wrong model_dtype");
        std::string path = model_path;
        if (!path.empty() && path.back() != '/') {
            path += "/";
        }
        std::vector<BinFile> files;
        auto lin = [&](const std::string& name, int64_t n, int64_t k) {
            files.push_back({name + ".weight", {n, k}, 'T'});
            files.push_back({name + ".bias", {n}, 'T'});
        };
        lin("x_embedder", dim, in_ch);
        lin("context_embedder", dim, joint_dim);
        lin("proj_out", in_ch, dim);
        lin("norm_out.linear", 2 * dim, dim);
        for (const char* e : {"timestep_embedder", "guidance_embedder", "text_embedder"}) {
            const std::string p = std::string("time_text_embed.") + e + ".";
            lin(p + "linear_1", dim, std::string(e) == "text_embedder" ? pooled_dim : 256);
            lin(p + "linear_2", dim, dim);
        }
        for (int64_t i = 0; i < n_double; ++i) {
            for (BinFile f : dbl[i]->bin_files()) {
                f.key = "transformer_blocks." + std::to_string(i) + "." + f.key;
                files.push_back(f);
            }
        }
        for (int64_t i = 0; i < n_single; ++i) {
            for (BinFile f : sgl[i]->bin_files()) {
                f.key = "single_transformer_blocks." + std::to_string(i) + "." + f.key;
                files.push_back(f);
            }
        }
        c10::Dict<std::string, Tensor> sd;
        for (const BinFile& f : files) {
            sd.insert(f.key, read_bin(path, f, model_dtype == "fp16"));
        }
        std::lock_guard<std::mutex> g(lock);
        load(sd, "cpu");
    }

    // FluxTransformer2DModelWeight.cc:34-97,160-175: blocks under transformer_blocks_<i> / single_transformer_blocks_<j>, the
    // embedders under time_text_embed, then norm_out, x_embedder, context_embedder, proj_out
    std::map<std::string, LoraTarget*> lora_table()
    {
        std::map<std::string, LoraTarget*> t{{"x_embedder", &x_embedder}, {"context_embedder", &context_embedder},
                                             {"proj_out", &proj_out}, {"norm_out/linear", &norm_out}};
        auto mlp = [&](const std::string& name, Mlp16& m) {
            t["time_text_embed/" + name + "/linear_1"] = &m.l1;
            t["time_text_embed/" + name + "/linear_2"] = &m.l2;
        };
        mlp("timestep_embedder", timestep_embedder);
        mlp("guidance_embedder", guidance_embedder);
        mlp("text_embedder", text_embedder);
        for (int64_t i = 0; i < n_double; ++i) {
            for (auto& kv : dbl[i]->lora_table()) {
                t["transformer_blocks_" + std::to_string(i) + "/" + kv.first] = kv.second;
            }
        }
        for (int64_t i = 0; i < n_single; ++i) {
            for (auto& kv : sgl[i]->lora_table()) {
                t["single_transformer_blocks_" + std::to_string(i) + "/" + kv.first] = kv.second;
            }
        }
        return t;
    }

    void load_lora_by_name(const std::vector<std::string>& names, const Tensor& weight, double scale)
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::string key;
        for (const std::string& n : names) {
            key += (key.empty() ? "" : "/") + n;
        }
        std::lock_guard<std::mutex> g(lock);
        auto                        table = lora_table();
        auto                        it    = table.find(key);
        if (it == table.end()) {
            TORCH_WARN("lora name cannot find weights to load: ", key);
            return;
        }
        it->second->load_lora(weight, scale);
    }

    void clear_lora()
    {
        TORCH_CHECK(loaded, "weights not loaded");
        std::lock_guard<std::mutex> g(lock);
        for (auto& kv : lora_table()) {
            kv.second->clear_lora();
        }
    }

    // kernel kernels/time_proj/time_proj_kernels.cu:70-97: fp32 sin / cos of exponent * value, cast to T, cosine half first;
    // device work only, so a forward can be captured into a CUDA graph
    Tensor time_projection(double value) const
    {
        Tensor a = exponents * (float)value;
        return at::cat({at::cos(a), at::sin(a)}).to(dtype).reshape({1, 256});
    }

    Tensor transformer_forward(const Tensor& hidden_states, const Tensor& encoder_hidden_states, const Tensor& rope_emb,
                               const Tensor& pooled_projection, double timestep, double guidance,
                               const c10::optional<std::vector<Tensor>>& controlnet_block_samples,
                               const c10::optional<std::vector<Tensor>>& controlnet_single_block_samples,
                               const c10::optional<bool>&                controlnet_blocks_repeat)
    {
        TORCH_CHECK(loaded, "weights not loaded");
        check_inputs({hidden_states, encoder_hidden_states, rope_emb, pooled_projection}, dtype);
        TORCH_CHECK(!controlnet_single_block_samples.has_value() || controlnet_single_block_samples->empty(),
                    "controlnet_single_block_samples currently needs to be 0");  // FluxTransformer2DModel.cc:252
        std::lock_guard<std::mutex> guard(lock);
        const int64_t B = hidden_states.size(0), S = hidden_states.size(1), E = encoder_hidden_states.size(1);

        // conditioning vector, SiLU'd as the blocks expect it (add3Tensor2dAndSilu: src1 + src2 + src3 in T, then SiLU)
        Tensor t_emb = timestep_embedder.run(time_projection(timestep));
        Tensor g_emb = guidance_embedder.run(time_projection(guidance));
        Tensor p_emb = text_embedder.run(pooled_projection);
        Tensor temb  = at::silu((p_emb + g_emb) + t_emb).contiguous();

        Tensor h = x_embedder.run(hidden_states.view({B * S, in_ch})).view({B, S, dim});
        Tensor c = context_embedder.run(encoder_hidden_states.view({B * E, joint_dim})).view({B, E, dim});

        // Every block's modulation linear depends on temb alone (an M = B product that streams 56-113 MB of weights): all of
        // them are issued on a second stream now and each block waits only for its own event, so that memory-bound work
        // overlaps the tensor-bound GEMMs of the blocks in front of it.
        std::vector<AheadModulation> ahead((size_t)(n_double + n_single));
        const auto                   main_stream = at::cuda::getCurrentCUDAStream();
        const auto                   side_stream = at::cuda::getStreamFromPool(false, main_stream.device_index());
        {
            at::cuda::CUDAEvent ready;
            ready.record(main_stream);
            ready.block(side_stream);
            c10::cuda::CUDACachingAllocator::recordStream(temb.storage().data_ptr(), side_stream);
            c10::cuda::CUDAStreamGuard on_side(side_stream);
            for (int64_t i = 0; i < n_double + n_single; ++i) {
                AheadModulation& a = ahead[(size_t)i];
                if (i < n_double) {
                    a.parts = dbl[i]->modulation(temb);
                } else {
                    a.parts = {sgl[i - n_double]->modulation(temb)};
                }
                a.event = std::make_shared<at::cuda::CUDAEvent>();
                a.event->record(side_stream);
            }
        }

        const std::vector<Tensor> samples = controlnet_block_samples.value_or(std::vector<Tensor>{});
        const bool    repeat   = controlnet_blocks_repeat.value_or(false);
        const int64_t interval = samples.empty() ? 0 : (n_double - 1) / (int64_t)samples.size() + 1;
        for (int64_t i = 0; i < n_double; ++i) {
            auto out = dbl[i]->forward_with(h, c, rope_emb, temb, &ahead[(size_t)i]);
            h        = out[0];
            c        = out[1];
            if (!samples.empty()) {
                Tensor res = (repeat ? samples[i % (int64_t)samples.size()] : samples[i / interval]).contiguous();
                TORCH_CHECK(res.numel() == h.numel() && res.scalar_type() == dtype && res.is_cuda(), "controlnet sample mismatch");
                check(lyraq_load_lora(h.data_ptr(), res.data_ptr(), dt_code(dtype), 1.0f, (size_t)h.numel(), stream()),
                      "lyraq_load_lora");  // the reference adds it with invokeLoadLora too (FluxTransformer2DModel.cc:389)
            }
        }
        Tensor x = at::cat({c, h}, 1);
        for (int64_t i = 0; i < n_single; ++i) {
            x = sgl[i]->forward_with(x, rope_emb, temb, &ahead[(size_t)(n_double + i)]);
        }
        {
            at::cuda::CUDAEvent joined;  // the second stream joins again (needed when the forward is being captured into a graph)
            joined.record(side_stream);
            joined.block(main_stream);
        }
        h = x.slice(1, E, E + S).contiguous();

        // norm_out: AdaLayerNorm<T>(dim, 2, switch_scale = true): scale first, then shift
        Tensor msa    = norm_out.run(temb);
        auto   parts  = msa.chunk(2, 1);
        Tensor scale  = parts[0].contiguous(), shift = parts[1].contiguous();
        Tensor normed = at::empty_like(h);
        check(lyraq_adaln_quant(normed.data_ptr(), nullptr, nullptr, nullptr, nullptr, h.data_ptr(), scale.data_ptr(), shift.data_ptr(),
                                dt_code(dtype), nullptr, (size_t)B, (size_t)S, (size_t)dim, 1e-6, stream()),
              "lyraq_adaln_quant");
        return proj_out.run(normed.view({B * S, dim})).view({B, S, in_ch});
    }
};

// The shared methods live in BlockBase; they are bound through lambdas on the concrete class, since the class registry
// takes `self` from the member pointer's class and BlockBase itself is not registered.
template<class Op>
void register_block(torch::Library& m, const char* name, int64_t default_mlp_scale)
{
    using Self = c10::intrusive_ptr<Op>;
    // argument names and defaults of th_op/pybind.cc:66-96 (mlp_scale 6 for the double-stream block, 4 for the single one)
    m.class_<Op>(name)
        .def(torch::init<std::string, int64_t, int64_t, int64_t, int64_t, int64_t>(), "init",
             {torch::arg("inference_dtype") = "bf16", torch::arg("embedding_dim") = 3072, torch::arg("embedding_head_num") = 24,
              torch::arg("embedding_head_dim") = 128, torch::arg("mlp_scale") = default_mlp_scale, torch::arg("quant_level") = 0})
        .def("initialize", [](const Self& self, const c10::intrusive_ptr<LyraDiffCommonContext>& ctx) { self->initialize(ctx); })
        .def("forward", &Op::forward)
        .def("reload_model_from_state_dict", [](const Self& self, const std::string& prefix, const c10::Dict<std::string, Tensor>& sd,
                                                const std::string& device) { self->reload_model_from_state_dict(prefix, sd, device); })
        .def("reload_model_from_bin",
             [](const Self& self, const std::string& path, const std::string& dtype) { self->reload_model_from_bin(path, dtype); })
        .def("load_lora_by_name", [](const Self& self, const std::vector<std::string>& names, const Tensor& w,
                                     double scale) { self->load_lora_by_name(names, w, scale); })
        .def("clear_lora", [](const Self& self) { self->clear_lora(); });
}

TORCH_LIBRARY(lyradiff, m)
{
    m.class_<LyraDiffCommonContext>("LyraDiffCommonContext").def(torch::init<>());
    register_block<FluxSingleTransformerBlockOp>(m, "FluxSingleTransformerBlockOp", 4);
    register_block<FluxTransformerBlockOp>(m, "FluxTransformerBlockOp", 6);
    m.class_<FluxTransformer2DModelOp>("FluxTransformer2DModelOp")
        .def(torch::init<std::string, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, bool, int64_t>(), "init",
             {torch::arg("inference_dtype") = "bf16", torch::arg("input_channels") = 64, torch::arg("num_layers") = 19,
              torch::arg("num_single_layers") = 38, torch::arg("attention_head_dim") = 128, torch::arg("num_attention_heads") = 24,
              torch::arg("pooled_projection_dim") = 768, torch::arg("joint_attention_dim") = 4096,
              torch::arg("guidance_embeds") = true, torch::arg("quant_level") = 0})
        .def("initialize", &FluxTransformer2DModelOp::initialize)
        .def("transformer_forward", &FluxTransformer2DModelOp::transformer_forward, "transformer_forward",
             {torch::arg("hidden_states"), torch::arg("encoder_hidden_states"), torch::arg("rope_emb"),
              torch::arg("pooled_projection"), torch::arg("timestep"), torch::arg("guidance"),
              torch::arg("controlnet_block_samples") = c10::nullopt, torch::arg("controlnet_single_block_samples") = c10::nullopt,
              torch::arg("controlnet_blocks_repeat") = false})
        .def("reload_transformer_model", &FluxTransformer2DModelOp::reload_transformer_model)
        .def("load_lora_by_name", &FluxTransformer2DModelOp::load_lora_by_name)
        .def("clear_lora", &FluxTransformer2DModelOp::clear_lora)
        .def("reload_transformer_model_from_state_dict", &FluxTransformer2DModelOp::reload_transformer_model_from_state_dict);
}
