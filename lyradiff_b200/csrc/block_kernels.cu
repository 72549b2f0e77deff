// The element-wise kernels that sit between the quantized linears of a FLUX single-stream block:
//   - QK RMSNorm + rotary embedding on the packed QKV projection (the attention's input),
//   - e4m3 quantize of a [rows, cols] tensor into a column window of a wider e4m3 matrix (the concat in front of
//     proj_out, so that attention output and MLP activation are never concatenated in 16-bit form),
//   - gate * y + residual (the block's output).
// All are HBM-bound streaming kernels with 16-byte accesses; arithmetic follows the reference's rounding steps.
#include "common.cuh"

namespace lyraq {

// One thread owns 8 consecutive elements of one head; the head_dim / 8 threads of a head (8 or 16 consecutive lanes)
// reduce the sum of squares with shuffles.  Reference: fuseRmsNormAndRope
// (src/lyradiff/kernels/rope/flux_apply_rope.cu:8-76): inv = rsqrt(mean(x^2) + eps) in fp32; t = T(x * inv);
// t = T(t * scale); out.x = T(T(t.x * r0.x) + T(t.y * r0.y)); out.y = T(T(t.x * r1.x) + T(t.y * r1.y)); V heads are copied.
template<typename T, int LANES>
__global__ void __launch_bounds__(256) rmsnorm_rope_kernel(T* out, const T* qkv, const T* scale, const T* rope, float eps,
                                                           size_t tokens, int seq_len, int heads)
{
    using P2 = Pair<T>;
    grid_launch_dependents();
    grid_dependency_wait();
    constexpr int kHeadDim   = LANES * 8;
    const size_t  vec_per_tok = (size_t)3 * heads * LANES;
    const size_t  total      = tokens * vec_per_tok;
    const size_t  stride     = (size_t)gridDim.x * blockDim.x;
    const bool    in_place   = (out == qkv);
    // total is a multiple of LANES and so is the block size: the lanes of a head stay together in every iteration.  A warp
    // may hold a V head next to a Q/K head, and the tail of the last iteration may leave lanes without work, so every
    // lane of the warp takes part in the shuffles (lanes without a Q/K head reduce zeros) and only the loads, the
    // arithmetic and the store are predicated.
    const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t iters = (total + stride - 1) / stride;
    for (size_t it = 0; it < iters; ++it) {
        const size_t vi     = first + it * stride;
        const bool   active = vi < total;
        const size_t tok    = active ? vi / vec_per_tok : 0;
        const int    rem    = active ? (int)(vi - tok * vec_per_tok) : 0;
        const int    head   = rem / LANES;          // 0 .. 3 * heads - 1: q heads, k heads, v heads
        const int    part   = rem - head * LANES;   // which 8 elements of the head
        const bool   is_v   = head >= 2 * heads;
        const bool   load   = active && !(is_v && in_place);
        const bool   rotate = active && !is_v;
        Vec16        x      = {};
        if (load) {
            // an ordered plain load, not the read-only (.nc) path: with out == qkv this kernel writes what it reads
            const uint4 raw = ld_u32x4(reinterpret_cast<const uint4*>(qkv + (vi << 3)));
            x.w[0] = raw.x;
            x.w[1] = raw.y;
            x.w[2] = raw.z;
            x.w[3] = raw.w;
        }
        float f[8];
        unpack8<T>(x, f);
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            ss = fmaf(f[j], f[j], ss);
        }
#pragma unroll
        for (int m = LANES / 2; m > 0; m >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, m);
        }
        if (rotate) {
            const float inv = rsqrtf(ss / (float)kHeadDim + eps);
            const Vec16 sc  = ld_nc_16_keep(scale + (head >= heads ? kHeadDim : 0) + part * 8);
            // rope: [tokens, head_dim / 2, 2, 2]; this thread's 4 pairs are 16 consecutive values
            const T*    rp  = rope + (tok * (size_t)kHeadDim * 2) + part * 16;
            const Vec16 r0  = ld_nc_16_keep(rp);
            const Vec16 r1  = ld_nc_16_keep(rp + 8);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t t = P2::from_f32(f[2 * j] * inv, f[2 * j + 1] * inv);
                t          = P2::mul(t, sc.w[j]);
                // pair j uses rope values 4j .. 4j+3 = (r0.x, r0.y, r1.x, r1.y): two words of r0 (j < 2) or r1
                const uint32_t ra = (j < 2) ? r0.w[2 * j] : r1.w[2 * (j - 2)];        // (rope0.x, rope0.y)
                const uint32_t rb = (j < 2) ? r0.w[2 * j + 1] : r1.w[2 * (j - 2) + 1];  // (rope1.x, rope1.y)
                const float2 pa = P2::to_f32(P2::mul(t, ra));  // (T(t.x r0.x), T(t.y r0.y))
                const float2 pb = P2::to_f32(P2::mul(t, rb));
                x.w[j]          = P2::from_f32(pa.x + pa.y, pb.x + pb.y);  // fp32 sum of two T values, rounded once = T add
            }
        }
        if (load) {
            st_16(out + (vi << 3), x);
        }
    }
}

// dst[r, col0 + c] = e4m3(src[r, c] / scale) for a [rows, cols] source into a matrix with row pitch dst_ld bytes.
template<typename T>
__global__ void __launch_bounds__(256) fp8_cast_2d_kernel(uint8_t* dst, size_t dst_ld, const T* src, const float* scale,
                                                          size_t rows, int cols)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const float  r       = 1.0f / ld_f32(scale);
    const int    vec_row = cols >> 3;
    const size_t total   = rows * (size_t)vec_row;
    const size_t stride  = (size_t)gridDim.x * blockDim.x;
    for (size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; vi < total; vi += stride) {
        const size_t row = vi / vec_row;
        const int    c   = (int)(vi - row * vec_row) << 3;
        float        v[8];
        unpack8<T>(ld_nc_16(src + (vi << 3)), v);
        const uint32_t w0 = f32x2_to_e4m3x2(v[0] * r, v[1] * r) | (f32x2_to_e4m3x2(v[2] * r, v[3] * r) << 16);
        const uint32_t w1 = f32x2_to_e4m3x2(v[4] * r, v[5] * r) | (f32x2_to_e4m3x2(v[6] * r, v[7] * r) << 16);
        st_8(dst + row * dst_ld + c, w0, w1);
    }
}

// out = T(T(y * gate[b]) + x): fuseGateAndResidual (src/lyradiff/kernels/flux_single_transformer_block/
// flux_single_transformer_kernels.cu:43-65).
template<typename T>
__global__ void __launch_bounds__(256) gate_residual_kernel(T* out, const T* y, const T* gate, const T* x, size_t rows,
                                                            int rows_per_batch, int dim)
{
    using P2 = Pair<T>;
    grid_launch_dependents();
    grid_dependency_wait();
    const int    vec_row = dim >> 3;
    const size_t total   = rows * (size_t)vec_row;
    const size_t stride  = (size_t)gridDim.x * blockDim.x;
    for (size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; vi < total; vi += stride) {
        const size_t row = vi / vec_row;
        const int    c   = (int)(vi - row * vec_row) << 3;
        const Vec16  a   = ld_nc_16(y + (vi << 3));
        const Vec16  r   = ld_nc_16(x + (vi << 3));
        const Vec16  g   = ld_nc_16_keep(gate + (row / (size_t)rows_per_batch) * (size_t)dim + c);
        Vec16        o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o.w[j] = P2::add(P2::mul(a.w[j], g.w[j]), r.w[j]);
        }
        st_16(out + (vi << 3), o);
    }
}

// w[i] = T(w[i] + T(lora[i] * T(alpha))), each step in T's own arithmetic: loadLora<T>
// (src/lyradiff/kernels/lora/load_lora.cu:6-14).  n8 vectors of 8 elements, then a scalar tail.
template<typename T>
__global__ void __launch_bounds__(256) load_lora_kernel(T* w, const T* lora, size_t n, float alpha)
{
    using P2 = Pair<T>;
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t a2     = P2::from_f32(alpha, alpha);
    const size_t   n8     = n >> 3;
    const size_t   stride = (size_t)gridDim.x * blockDim.x;
    const size_t   tid    = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t vi = tid; vi < n8; vi += stride) {
        Vec16       o = *reinterpret_cast<const Vec16*>(w + (vi << 3));  // plain load: this kernel writes w
        const Vec16 l = ld_nc_16(lora + (vi << 3));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o.w[j] = P2::add(o.w[j], P2::mul(l.w[j], a2));
        }
        st_16(w + (vi << 3), o);
    }
    for (size_t i = (n8 << 3) + tid; i < n; i += stride) {
        const T t = from_f32<T>(to_f32(lora[i]) * to_f32(from_f32<T>(alpha)));  // exact product of two T values, one rounding
        w[i]      = from_f32<T>(to_f32(w[i]) + to_f32(t));
    }
}

static unsigned stream_grid(size_t nvec)
{
    size_t       g   = (nvec + 255) / 256;
    const size_t cap = 148 * 8;
    if (g > cap) {
        g = cap;
    }
    return g == 0 ? 1u : (unsigned)g;
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {

int lyraq_rmsnorm_rope(void* out, const void* qkv, const void* scale, const void* rope, int dtype, double eps, size_t batch,
                       size_t seq_len, int heads, int head_dim, void* stream)
{
    if (batch * seq_len == 0) {
        return LYRAQ_OK;
    }
    if (out == nullptr || qkv == nullptr || scale == nullptr || rope == nullptr || heads <= 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(out) || !aligned16(qkv) || !aligned16(scale) || !aligned16(rope)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((head_dim != 64 && head_dim != 128) || seq_len > 0x7fffffffu || (dtype != LYRAQ_BF16 && dtype != LYRAQ_F16)) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    const size_t   tokens = batch * seq_len;
    const size_t   nvec   = tokens * 3 * (size_t)heads * (size_t)(head_dim / 8);
    const unsigned grid   = stream_grid(nvec);
    cudaStream_t   s      = (cudaStream_t)stream;
    cudaError_t    e;
    if (dtype == LYRAQ_BF16) {
        using T = __nv_bfloat16;
        e = (head_dim == 128) ? launch_kernel(rmsnorm_rope_kernel<T, 16>, grid, 256u, (size_t)0, s, 1u, (T*)out, (const T*)qkv,
                                              (const T*)scale, (const T*)rope, (float)eps, tokens, (int)seq_len, heads)
                              : launch_kernel(rmsnorm_rope_kernel<T, 8>, grid, 256u, (size_t)0, s, 1u, (T*)out, (const T*)qkv,
                                              (const T*)scale, (const T*)rope, (float)eps, tokens, (int)seq_len, heads);
    } else {
        using T = __half;
        e = (head_dim == 128) ? launch_kernel(rmsnorm_rope_kernel<T, 16>, grid, 256u, (size_t)0, s, 1u, (T*)out, (const T*)qkv,
                                              (const T*)scale, (const T*)rope, (float)eps, tokens, (int)seq_len, heads)
                              : launch_kernel(rmsnorm_rope_kernel<T, 8>, grid, 256u, (size_t)0, s, 1u, (T*)out, (const T*)qkv,
                                              (const T*)scale, (const T*)rope, (float)eps, tokens, (int)seq_len, heads);
    }
    return cuda_status(e, "cudaLaunchKernelEx(rmsnorm_rope_kernel)");
}

int lyraq_quant_fp8_2d(uint8_t* dst, size_t dst_ld, const void* src, int src_dtype, const float* scale, size_t rows,
                       size_t cols, void* stream)
{
    if (rows * cols == 0) {
        return LYRAQ_OK;
    }
    if (dst == nullptr || src == nullptr || scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 7u) != 0 || (dst_ld & 7u) != 0 || dst_ld < cols) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((cols & 7u) != 0 || cols > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    const unsigned grid = stream_grid(rows * (cols >> 3));
    cudaError_t    e;
    if (src_dtype == LYRAQ_BF16) {
        e = launch_kernel(fp8_cast_2d_kernel<__nv_bfloat16>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, dst, dst_ld,
                          (const __nv_bfloat16*)src, scale, rows, (int)cols);
    } else if (src_dtype == LYRAQ_F16) {
        e = launch_kernel(fp8_cast_2d_kernel<__half>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, dst, dst_ld,
                          (const __half*)src, scale, rows, (int)cols);
    } else {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    return cuda_status(e, "cudaLaunchKernelEx(fp8_cast_2d_kernel)");
}

int lyraq_gate_residual(void* out, const void* y, const void* gate, const void* x, int dtype, size_t batch, size_t seq_len,
                        size_t dim, void* stream)
{
    if (batch * seq_len * dim == 0) {
        return LYRAQ_OK;
    }
    if (out == nullptr || y == nullptr || gate == nullptr || x == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(out) || !aligned16(y) || !aligned16(gate) || !aligned16(x)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((dim & 7u) != 0 || dim > 0x7fffffffu || seq_len > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    const size_t   rows = batch * seq_len;
    const unsigned grid = stream_grid(rows * (dim >> 3));
    cudaError_t    e;
    if (dtype == LYRAQ_BF16) {
        using T = __nv_bfloat16;
        e = launch_kernel(gate_residual_kernel<T>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, (T*)out, (const T*)y,
                          (const T*)gate, (const T*)x, rows, (int)seq_len, (int)dim);
    } else if (dtype == LYRAQ_F16) {
        using T = __half;
        e = launch_kernel(gate_residual_kernel<T>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, (T*)out, (const T*)y,
                          (const T*)gate, (const T*)x, rows, (int)seq_len, (int)dim);
    } else {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    return cuda_status(e, "cudaLaunchKernelEx(gate_residual_kernel)");
}

int lyraq_load_lora(void* weight, const void* lora, int dtype, float alpha, size_t n, void* stream)
{
    if (n == 0) {
        return LYRAQ_OK;
    }
    if (weight == nullptr || lora == nullptr || !aligned16(weight) || !aligned16(lora)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    const unsigned grid = stream_grid((n + 7) / 8);
    cudaError_t    e;
    if (dtype == LYRAQ_BF16) {
        using T = __nv_bfloat16;
        e = launch_kernel(load_lora_kernel<T>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, (T*)weight, (const T*)lora, n, alpha);
    } else if (dtype == LYRAQ_F16) {
        using T = __half;
        e = launch_kernel(load_lora_kernel<T>, grid, 256u, (size_t)0, (cudaStream_t)stream, 1u, (T*)weight, (const T*)lora, n, alpha);
    } else {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    return cuda_status(e, "cudaLaunchKernelEx(load_lora_kernel)");
}

}  // extern "C"
