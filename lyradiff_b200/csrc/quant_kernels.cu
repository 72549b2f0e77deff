// Activation / weight quantizers and the fused LayerNorm, AdaLN and GEGLU producers.
//
// All of them are HBM-bound row kernels: a team of 32..256 threads owns one row, reads it once
// with 16-byte loads into registers, reduces what it must (sum, sum of squares, amax) with warp
// shuffles (plus one shared-memory hop when the team spans several warps), and writes the
// quantized row once with 8- or 16-byte stores.  Nothing is staged through global memory.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

int device_sm_count();  // gemm_dense.cu
unsigned int* status_word_ptr();  // api.cu
int launch_lora_down(float* act, const void* x, const void* down, int dtype, size_t m, size_t k, cudaStream_t stream);
int launch_quant_int4_lora_down(uint8_t* q, float* q_scale, float* act, const void* x, const void* down, const float* smooth, int dtype,
                                size_t m, size_t k, cudaStream_t stream);  // lora_down.cu

enum RowMode { ROW_PLAIN = 0, ROW_ADALN = 1, ROW_LN = 2, ROW_GEGLU = 3 };

struct RowParams {
    // inputs
    const void*  x;            // [rows, in_cols]
    const void*  residual;     // LN: [rows, dim] or null
    const void*  bias;         // LN: [dim]; GEGLU: [2*dim]; or null
    const void*  gamma;        // LN
    const void*  beta;         // LN
    const void*  ada_scale;    // AdaLN: [B, dim]
    const void*  ada_shift;    // AdaLN: [B, dim]
    const float* pre;          // [dim] or null
    const float* f8_scale;     // [1]
    // outputs
    void*    y;                // [rows, dim] of T or null
    void*    sum_out;          // LN with residual: [rows, dim] of T or null
    int8_t*  q8;               // [rows, dim] or null
    float*   q8_scale;         // in (static/per-token) or out (dynamic)
    uint8_t* qf8;              // [rows, dim] or null
    uint8_t* qf8b;             // second e4m3 output with its own scale (same y, another consumer), or null
    const float* f8_scale_b;   // [1]
    int      scale_mode;
    int      f8_invert;
    size_t   rows;
    int      dim;
    int      in_cols;
    int      rows_per_batch;   // AdaLN: S
    float    eps;
    int      tpr;              // threads per row (32, 64, 128 or 256)
};

template<bool IS_MAX> __device__ __forceinline__ float warp_reduce(float v)
{
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float o = __shfl_xor_sync(0xffffffffu, v, m);
        v             = IS_MAX ? fmaxf(v, o) : v + o;
    }
    return v;
}

// Reduction over the tpr threads of a team (tpr is a multiple of 32; a warp belongs to one team).
// Every thread of the team must call it.
template<bool IS_MAX> __device__ __forceinline__ float team_reduce(float v, int tpr, float* red)
{
    v = warp_reduce<IS_MAX>(v);
    if (tpr == 32) {
        return v;
    }
    const int warp  = threadIdx.x >> 5;
    const int wpt   = tpr >> 5;
    const int first = (warp / wpt) * wpt;
    if ((threadIdx.x & 31) == 0) {
        red[warp] = v;
    }
    // only the warps of this team meet: named barrier 1 + team index, tpr participants
    asm volatile("bar.sync %0, %1;" ::"r"(1 + first / wpt), "r"(tpr) : "memory");
    float r = red[first];
    for (int i = 1; i < wpt; ++i) {
        r = IS_MAX ? fmaxf(r, red[first + i]) : r + red[first + i];
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + first / wpt), "r"(tpr) : "memory");
    return r;
}

// Bias + GEGLU on eight columns: h and g are the value and gate halves of the projection at columns c .. c + 7, bias
// (or null) has 2 * dim entries.  Returns T(T(h + b_h) * T(g' * T(cdf(g')))) with g' = T(g + b_g): the products and the
// cube in T, the cdf in fp32 and rounded to T, as GeluActivation<half2> does in the reference
// (src/lyradiff/kernels/quant_kernels/ffn_kernels_int8.cu:189-290).  Both GEGLU kernels below call this, so they
// leave the same bits.
template<typename T> __device__ __forceinline__ Vec16 geglu_vec(Vec16 h, Vec16 g, const T* bias, int dim, int c)
{
    using P2 = Pair<T>;
    if (bias != nullptr) {
        const Vec16 bh = ld_nc_16_keep(bias + c);
        const Vec16 bg = ld_nc_16_keep(bias + dim + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h.w[j] = P2::add(h.w[j], bh.w[j]);
            g.w[j] = P2::add(g.w[j], bg.w[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t cube = P2::mul(g.w[j], P2::mul(g.w[j], g.w[j]));
        const float2   gf   = P2::to_f32(g.w[j]);
        const float2   cf   = P2::to_f32(cube);
        const float    c0   = 0.5f * (1.0f + tanh_approx(0.7978845608028654f * (gf.x + 0.044715f * cf.x)));
        const float    c1   = 0.5f * (1.0f + tanh_approx(0.7978845608028654f * (gf.y + 0.044715f * cf.y)));
        const uint32_t act  = P2::mul(g.w[j], P2::from_f32(c0, c1));
        h.w[j]              = P2::mul(h.w[j], act);
    }
    return h;
}

// The row lives in registers as fp32 (f[i][0..7] = the i-th 16-byte vector of this thread); every step the
// reference evaluates in T is done on packed pairs with the type's native single-rounding add / multiply.
template<typename T, int VPT, int MODE>
__global__ void __launch_bounds__(256, (VPT <= 4 && MODE != ROW_LN && MODE != ROW_GEGLU) ? 3 : (VPT <= 6) ? 2 : 1)
row_quant_kernel(const RowParams p)
{
    using P2 = Pair<T>;
    __shared__ float red[8];

    grid_launch_dependents();
    grid_dependency_wait();
    const int    tpr    = p.tpr;
    const int    team   = threadIdx.x / tpr;
    const int    tlane  = threadIdx.x - team * tpr;
    const int    nvec   = p.dim >> 3;
    const size_t stride = (size_t)gridDim.x * (256 / tpr);  // rows advance by the number of teams in the grid

    // The grid is sized to what is resident at once; every team walks over rows row0, row0 + stride, ... and
    // fetches the next row's vectors (and, for LayerNorm + residual or GEGLU, the second operand's) before it
    // starts on the current one, so the load latency is spent computing.
    constexpr bool kSecond = (MODE == ROW_LN || MODE == ROW_GEGLU);
    Vec16 nx[VPT];
    Vec16 nx2[kSecond ? VPT : 1];
    auto prefetch = [&](size_t r) {
        const T* xr = reinterpret_cast<const T*>(p.x) + r * (size_t)p.in_cols;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vi = tlane + i * tpr;
            if (vi < nvec) {
                nx[i] = ld_nc_16(xr + (vi << 3));
                if (MODE == ROW_GEGLU) {
                    nx2[kSecond ? i : 0] = ld_nc_16(xr + p.dim + (vi << 3));
                }
                if (MODE == ROW_LN && p.residual != nullptr) {
                    nx2[kSecond ? i : 0] = ld_nc_16(reinterpret_cast<const T*>(p.residual) + r * (size_t)p.dim + (vi << 3));
                }
            }
        }
    };

    size_t row = (size_t)blockIdx.x * (256 / tpr) + team;
    if (row < p.rows) {
        prefetch(row);
    }
    for (; row < p.rows; row += stride) {
    const bool live = true;
    // the row in fp32 as packed pairs: f[i][q] = elements (2q, 2q + 1) of this thread's i-th vector.  All fp32 steps
    // below run as .f32x2 instructions (IEEE rounding per lane, so the results equal the scalar ones bit for bit) and
    // keep the summation order of the scalar formulation.
    float2     f[VPT][4];

    // ---- take the prefetched row (and, per mode, pre-combine in T arithmetic); start fetching the next one
    Vec16 cur[VPT];
    Vec16 cur2[kSecond ? VPT : 1];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        cur[i] = nx[i];
        if (kSecond) {
            cur2[kSecond ? i : 0] = nx2[kSecond ? i : 0];
        }
    }
    if (row + stride < p.rows) {
        prefetch(row + stride);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vi = tlane + i * tpr;
        if (live && vi < nvec) {
            const int c = vi << 3;
            Vec16     h = cur[i];
            if (MODE == ROW_LN && p.residual != nullptr) {
                // h = T(T(x + residual) + bias)
                const Vec16 r = cur2[kSecond ? i : 0];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    h.w[j] = P2::add(h.w[j], r.w[j]);
                }
                if (p.bias != nullptr) {
                    const Vec16 b = ld_nc_16_keep(reinterpret_cast<const T*>(p.bias) + c);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        h.w[j] = P2::add(h.w[j], b.w[j]);
                    }
                }
                if (p.sum_out != nullptr) {
                    st_16(reinterpret_cast<T*>(p.sum_out) + row * (size_t)p.dim + c, h);
                }
            }
            if (MODE == ROW_GEGLU) {
                h = geglu_vec<T>(h, cur2[kSecond ? i : 0], reinterpret_cast<const T*>(p.bias), p.dim, c);
            }
            if ((MODE == ROW_PLAIN || MODE == ROW_GEGLU) && p.y != nullptr) {
                st_16(reinterpret_cast<T*>(p.y) + row * (size_t)p.dim + c, h);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[i][j] = P2::to_f32(h.w[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[i][j] = make_float2(0.0f, 0.0f);
            }
        }
    }

    // ---- row statistics (fp32), then normalise and modulate (T arithmetic)
    if (MODE == ROW_ADALN || MODE == ROW_LN) {
        // four independent partial sums per pass: a single running sum would be one long dependency chain
        // partial sums over elements (0,1)+(4,5) and (2,3)+(6,7) of every vector, as four scalar chains would keep them
        float2 sa = make_float2(0.0f, 0.0f), sb = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            sa = add_f32x2(sa, add_f32x2(f[i][0], f[i][2]));
            sb = add_f32x2(sb, add_f32x2(f[i][1], f[i][3]));
        }
        float s          = team_reduce<false>((sa.x + sa.y) + (sb.x + sb.y), tpr, red);
        const float mean = s / (float)p.dim;
        const float2 nm  = make_float2(-mean, -mean);
        float2       qa  = make_float2(0.0f, 0.0f), qb = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vi = tlane + i * tpr;
            if (vi < nvec) {
                const float2 d0 = add_f32x2(f[i][0], nm), d2 = add_f32x2(f[i][2], nm);
                const float2 d1 = add_f32x2(f[i][1], nm), d3 = add_f32x2(f[i][3], nm);
                qa              = fma_f32x2(d0, d0, fma_f32x2(d2, d2, qa));
                qb              = fma_f32x2(d1, d1, fma_f32x2(d3, d3, qb));
            }
        }
        float m2         = team_reduce<false>((qa.x + qa.y) + (qb.x + qb.y), tpr, red);
        const float var  = fmaxf(m2 / (float)p.dim, 0.0f);
        const float rstd = 1.0f / sqrtf(var + p.eps);  // IEEE sqrt and divide: within one ulp of the exact value

        const size_t brow  = (MODE == ROW_ADALN) ? (row / (size_t)p.rows_per_batch) : 0;
        const T*     mul_v = (MODE == ROW_ADALN) ? reinterpret_cast<const T*>(p.ada_scale) + brow * (size_t)p.dim
                                                 : reinterpret_cast<const T*>(p.gamma);
        const T*     add_v = (MODE == ROW_ADALN) ? reinterpret_cast<const T*>(p.ada_shift) + brow * (size_t)p.dim
                                                 : reinterpret_cast<const T*>(p.beta);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int vi = tlane + i * tpr;
            if (live && vi < nvec) {
                const int   c = vi << 3;
                const Vec16 a = ld_nc_16_keep(mul_v + c);
                const Vec16 b = ld_nc_16_keep(add_v + c);
                Vec16       y;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // x_hat rounded to T; m = T(scale + 1) | gamma; y = T(T(m * x_hat) + shift)
                    const float2   xn = mul_f32x2(add_f32x2(f[i][j], nm), make_float2(rstd, rstd));
                    const uint32_t xh = P2::from_f32(xn.x, xn.y);
                    const uint32_t m  = (MODE == ROW_ADALN) ? P2::add(a.w[j], P2::one()) : a.w[j];
                    y.w[j]            = P2::add(P2::mul(m, xh), b.w[j]);
                    f[i][j]           = P2::to_f32(y.w[j]);
                }
                if (p.y != nullptr) {
                    st_16(reinterpret_cast<T*>(p.y) + row * (size_t)p.dim + c, y);
                }
            }
        }
    }

    // ---- int8 scale: q = sat_s8(rne((float(y) * pre[c]) / s)); the e4m3 output uses y before the pre factor
    float s8 = 1.0f;
    float f8r = 0.0f;
    if (p.qf8 != nullptr) {
        const float s = ld_f32(p.f8_scale);
        f8r           = p.f8_invert ? 1.0f / s : s;
    }
    float f8rb = 0.0f;
    if (p.qf8b != nullptr) {
        f8rb = 1.0f / ld_f32(p.f8_scale_b);
    }
    const bool dynamic = (p.scale_mode == LYRAQ_SCALE_PER_TOKEN_DYNAMIC);
    if (p.q8 != nullptr) {
        if (dynamic) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int vi = tlane + i * tpr;
                float2 g[4];
                if (p.pre != nullptr && live && vi < nvec) {
                    const float4 p0 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + (vi << 3)));
                    const float4 p1 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + (vi << 3) + 4));
                    g[0] = mul_f32x2(f[i][0], make_float2(p0.x, p0.y));
                    g[1] = mul_f32x2(f[i][1], make_float2(p0.z, p0.w));
                    g[2] = mul_f32x2(f[i][2], make_float2(p1.x, p1.y));
                    g[3] = mul_f32x2(f[i][3], make_float2(p1.z, p1.w));
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        g[j] = f[i][j];
                    }
                }
                amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(g[0].x), fabsf(g[0].y)), fmaxf(fabsf(g[1].x), fabsf(g[1].y))),
                                         fmaxf(fmaxf(fabsf(g[2].x), fabsf(g[2].y)), fmaxf(fabsf(g[3].x), fabsf(g[3].y)))));
            }
            amax = team_reduce<true>(amax, tpr, red);
            s8   = (amax == 0.0f) ? 1.0f : amax / 127.0f;
            if (live && tlane == 0) {
                p.q8_scale[row] = s8;
            }
        } else if (p.scale_mode == LYRAQ_SCALE_PER_TOKEN) {
            s8 = live ? ld_f32(p.q8_scale + row) : 1.0f;
        } else {
            s8 = ld_f32(p.q8_scale);
        }
    }
    const float r8 = 1.0f / s8;

    // ---- quantized outputs, one 16-byte vector of the row at a time
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int vi = tlane + i * tpr;
        if (live && vi < nvec) {
            const size_t off = row * (size_t)p.dim + (vi << 3);
            if (p.qf8 != nullptr) {
                const float2 r2 = make_float2(f8r, f8r);
                const float2 e0 = mul_f32x2(f[i][0], r2), e1 = mul_f32x2(f[i][1], r2);
                const float2 e2 = mul_f32x2(f[i][2], r2), e3 = mul_f32x2(f[i][3], r2);
                const uint32_t w0 = f32x2_to_e4m3x2(e0.x, e0.y) | (f32x2_to_e4m3x2(e1.x, e1.y) << 16);
                const uint32_t w1 = f32x2_to_e4m3x2(e2.x, e2.y) | (f32x2_to_e4m3x2(e3.x, e3.y) << 16);
                st_8(p.qf8 + off, w0, w1);
            }
            if (p.qf8b != nullptr) {
                const float2 r2 = make_float2(f8rb, f8rb);
                const float2 e0 = mul_f32x2(f[i][0], r2), e1 = mul_f32x2(f[i][1], r2);
                const float2 e2 = mul_f32x2(f[i][2], r2), e3 = mul_f32x2(f[i][3], r2);
                const uint32_t w0 = f32x2_to_e4m3x2(e0.x, e0.y) | (f32x2_to_e4m3x2(e1.x, e1.y) << 16);
                const uint32_t w1 = f32x2_to_e4m3x2(e2.x, e2.y) | (f32x2_to_e4m3x2(e3.x, e3.y) << 16);
                st_8(p.qf8b + off, w0, w1);
            }
            if (p.q8 != nullptr) {
                if (p.pre != nullptr) {
                    const float4 p0 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + (vi << 3)));
                    const float4 p1 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + (vi << 3) + 4));
                    f[i][0] = mul_f32x2(f[i][0], make_float2(p0.x, p0.y));
                    f[i][1] = mul_f32x2(f[i][1], make_float2(p0.z, p0.w));
                    f[i][2] = mul_f32x2(f[i][2], make_float2(p1.x, p1.y));
                    f[i][3] = mul_f32x2(f[i][3], make_float2(p1.z, p1.w));
                }
                uint32_t w0, w1;
                if (dynamic) {
                    quant8_s8_inrange(f[i], s8, r8, w0, w1);
                } else {
                    quant8_s8(f[i], s8, r8, w0, w1);
                }
                st_8(p.q8 + off, w0, w1);
            }
        }
    }
    }  // rows of this team
}

// Grid = the blocks that are resident at once (occupancy x SMs), or fewer when the rows do not fill them.
template<typename K> static int launch_row_variant(K kernel, const RowParams& p, size_t needed, cudaStream_t stream)
{
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0) != cudaSuccess || per_sm <= 0) {
        return cuda_status(cudaGetLastError(), "cudaOccupancyMaxActiveBlocksPerMultiprocessor(row_quant_kernel)");
    }
    const int sms = device_sm_count();
    if (sms <= 0) {
        return LYRAQ_ERR_CUDA;
    }
    const size_t resident = (size_t)per_sm * (size_t)sms;
    const size_t grid     = needed < resident ? needed : resident;
    return cuda_status(launch_kernel(kernel, (unsigned)grid, 256u, (size_t)0, stream, 1u, p), "cudaLaunchKernelEx(row_quant_kernel)");
}

// Most 16-byte vectors a thread may hold before the team is doubled (4 or 6; sweepable through the debug hook).
static int g_row_max_vpt = 6;
static int g_special_rows_on = 1;   // test hook: 0 sends every call through the general row kernel

// Picks the team size and launches.  dim is a multiple of 8 and <= 16384.  The smallest team (32..256 threads) that
// keeps at most six 16-byte vectors per thread is used, so narrow rows need no cross-warp reduction and every thread
// has several independent loads in flight; only rows wider than 12288 elements use eight vectors per thread.
template<typename T, int MODE> static int launch_row(RowParams p, cudaStream_t stream)
{
    const int nvec = p.dim >> 3;
    int       tpr  = 32;
    while (tpr < 256 && (nvec + tpr - 1) / tpr > g_row_max_vpt) {
        tpr <<= 1;
    }
    p.tpr                = tpr;
    const int    vpt     = (nvec + tpr - 1) / tpr;
    const size_t per_cta = 256 / tpr;
    const size_t needed  = (p.rows + per_cta - 1) / per_cta;
    if (needed == 0) {
        return LYRAQ_OK;
    }
    if (vpt <= 4) {
        return launch_row_variant(row_quant_kernel<T, 4, MODE>, p, needed, stream);
    }
    if (vpt <= 6) {
        return launch_row_variant(row_quant_kernel<T, 6, MODE>, p, needed, stream);
    }
    if (vpt <= 8) {
        return launch_row_variant(row_quant_kernel<T, 8, MODE>, p, needed, stream);
    }
    return LYRAQ_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// AdaLN + e4m3 quantize of rows of 3072 elements, the form the FLUX blocks use, optionally with the int8 output and its
// per-token dynamic scale (then y replaces x in the registers and a last pass quantizes it).  One warp owns a row:
// the row stays in registers as the 12 sixteen-byte vectors each lane loaded (vector lane + 32 j), statistics are reduced
// with shuffles only -- no shared memory, no block barrier, and three times the rows in flight of the general kernel.  The arithmetic is row_quant_kernel's, step for step,
// including the order of the fp32 sums: there two warps share a row and a thread sums vectors t + 64 i, so lane l here
// plays thread l (its even j) and thread l + 32 (its odd j), reduces the two halves separately and adds them as the general
// kernel adds its two warps.  The results are the same bits.
#ifndef ADALN_OUT_UNROLL
#define ADALN_OUT_UNROLL 4
#endif
#ifndef ADALN_PER_SM
#define ADALN_PER_SM 2
#endif
template<typename T, bool HAS_Y, bool HAS_B, bool HAS_Q8>
__global__ void __launch_bounds__(256, ADALN_PER_SM) adaln3072_e4m3_kernel(const RowParams p)
{
    using P2 = Pair<T>;
    constexpr int kVec = 12;             // 16-byte vectors per lane
    constexpr int kDim = 3072;
    constexpr int kOutGroup = ADALN_OUT_UNROLL;    // output vectors whose scale / shift loads may be in flight together (register budget)
    grid_launch_dependents();
    grid_dependency_wait();
    const int    lane   = threadIdx.x & 31;
    const size_t stride = (size_t)gridDim.x * 8;
    size_t       row    = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);

    const float f8r  = (!HAS_Q8 || p.qf8 != nullptr) ? 1.0f / ld_f32(p.f8_scale) : 0.0f;
    const float f8rb = HAS_B ? 1.0f / ld_f32(p.f8_scale_b) : 0.0f;
    const bool  has_f8 = !HAS_Q8 || p.qf8 != nullptr;
    for (; row < p.rows; row += stride) {
        // twelve independent loads per lane; the other warps of the SM (two blocks of eight) work while they are in flight
        Vec16 cur[kVec];
        {
            const T* xr = reinterpret_cast<const T*>(p.x) + row * (size_t)kDim;
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
                cur[j] = ld_nc_16(xr + ((lane + 32 * j) << 3));
            }
        }
        // ---- mean: per played thread, partial sums over elements (0,1)+(4,5) and (2,3)+(6,7) of its vectors in order
        float2 sa[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)}, sb[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const float2 f0 = P2::to_f32(cur[j].w[0]), f1 = P2::to_f32(cur[j].w[1]), f2 = P2::to_f32(cur[j].w[2]), f3 = P2::to_f32(cur[j].w[3]);
            sa[j & 1] = add_f32x2(sa[j & 1], add_f32x2(f0, f2));
            sb[j & 1] = add_f32x2(sb[j & 1], add_f32x2(f1, f3));
        }
        float s0 = (sa[0].x + sa[0].y) + (sb[0].x + sb[0].y), s1 = (sa[1].x + sa[1].y) + (sb[1].x + sb[1].y);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, m);
            s1 += __shfl_xor_sync(0xffffffffu, s1, m);
        }
        const float  mean = (s0 + s1) / (float)kDim;
        const float2 nm   = make_float2(-mean, -mean);
        // ---- variance, the same way
        float2 qa[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)}, qb[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const float2 d0 = add_f32x2(P2::to_f32(cur[j].w[0]), nm), d2 = add_f32x2(P2::to_f32(cur[j].w[2]), nm);
            const float2 d1 = add_f32x2(P2::to_f32(cur[j].w[1]), nm), d3 = add_f32x2(P2::to_f32(cur[j].w[3]), nm);
            qa[j & 1] = fma_f32x2(d0, d0, fma_f32x2(d2, d2, qa[j & 1]));
            qb[j & 1] = fma_f32x2(d1, d1, fma_f32x2(d3, d3, qb[j & 1]));
        }
        float v0 = (qa[0].x + qa[0].y) + (qb[0].x + qb[0].y), v1 = (qa[1].x + qa[1].y) + (qb[1].x + qb[1].y);
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            v0 += __shfl_xor_sync(0xffffffffu, v0, m);
            v1 += __shfl_xor_sync(0xffffffffu, v1, m);
        }
        const float  var  = fmaxf((v0 + v1) / (float)kDim, 0.0f);
        const float  rstd = 1.0f / sqrtf(var + p.eps);
        const float2 rs2  = make_float2(rstd, rstd);
        // ---- x_hat rounded to T; m = T(scale + 1); y = T(T(m * x_hat) + shift); e4m3 of float(y) / scale
        const size_t brow  = row / (size_t)p.rows_per_batch;
        const T*     mul_v = reinterpret_cast<const T*>(p.ada_scale) + brow * (size_t)kDim;
        const T*     add_v = reinterpret_cast<const T*>(p.ada_shift) + brow * (size_t)kDim;
        float        amax  = 0.0f;
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            if (j % kOutGroup == 0) {
                asm volatile("" ::: "memory");   // keeps the scale / shift loads of later groups from being hoisted up here
            }
            const int   c = (lane + 32 * j) << 3;
            const Vec16 a = ld_nc_16_keep(mul_v + c);
            const Vec16 b = ld_nc_16_keep(add_v + c);
            Vec16  y;
            float2 e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2   xn = mul_f32x2(add_f32x2(P2::to_f32(cur[j].w[k]), nm), rs2);
                const uint32_t xh = P2::from_f32(xn.x, xn.y);
                const uint32_t m  = P2::add(a.w[k], P2::one());
                y.w[k]            = P2::add(P2::mul(m, xh), b.w[k]);
                e[k]              = P2::to_f32(y.w[k]);
            }
            const size_t off = row * (size_t)kDim + c;
            if (HAS_Y) {
                st_16(reinterpret_cast<T*>(p.y) + off, y);
            }
            if (has_f8) {
                const float2 r2 = make_float2(f8r, f8r);
                const float2 e0 = mul_f32x2(e[0], r2), e1 = mul_f32x2(e[1], r2), e2 = mul_f32x2(e[2], r2), e3 = mul_f32x2(e[3], r2);
                st_8(p.qf8 + off, f32x2_to_e4m3x2(e0.x, e0.y) | (f32x2_to_e4m3x2(e1.x, e1.y) << 16),
                     f32x2_to_e4m3x2(e2.x, e2.y) | (f32x2_to_e4m3x2(e3.x, e3.y) << 16));
            }
            if (HAS_Q8) {
                cur[j] = y;   // x is no longer needed: the row's y waits here for its scale
                amax   = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(e[0].x), fabsf(e[0].y)), fmaxf(fabsf(e[1].x), fabsf(e[1].y))),
                                           fmaxf(fmaxf(fabsf(e[2].x), fabsf(e[2].y)), fmaxf(fabsf(e[3].x), fabsf(e[3].y)))));
            }
            if (HAS_B) {
                const float2 r2 = make_float2(f8rb, f8rb);
                const float2 e0 = mul_f32x2(e[0], r2), e1 = mul_f32x2(e[1], r2), e2 = mul_f32x2(e[2], r2), e3 = mul_f32x2(e[3], r2);
                st_8(p.qf8b + off, f32x2_to_e4m3x2(e0.x, e0.y) | (f32x2_to_e4m3x2(e1.x, e1.y) << 16),
                     f32x2_to_e4m3x2(e2.x, e2.y) | (f32x2_to_e4m3x2(e3.x, e3.y) << 16));
            }
        }
        if (HAS_Q8) {
            // ---- int8 with the row's own scale: s = amax / 127 (1 for an all-zero row), q = sat_s8(rne(float(y) / s))
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            }
            const float s8 = (amax == 0.0f) ? 1.0f : amax / 127.0f;
            const float r8 = 1.0f / s8;
            if (lane == 0) {
                p.q8_scale[row] = s8;
            }
#pragma unroll
            for (int j = 0; j < kVec; ++j) {
                const float2 f[4] = {P2::to_f32(cur[j].w[0]), P2::to_f32(cur[j].w[1]), P2::to_f32(cur[j].w[2]), P2::to_f32(cur[j].w[3])};
                uint32_t     w0, w1;
                quant8_s8_inrange(f, s8, r8, w0, w1);
                st_8(p.q8 + row * (size_t)kDim + ((lane + 32 * j) << 3), w0, w1);
            }
        }
    }
}

template<typename T, bool HAS_Y, bool HAS_B, bool HAS_Q8> static int launch_adaln3072(const RowParams& p, cudaStream_t stream)
{
    return launch_row_variant(adaln3072_e4m3_kernel<T, HAS_Y, HAS_B, HAS_Q8>, p, (p.rows + 7) / 8, stream);
}

// AdaLN over rows of 3072 with an e4m3 output (the FLUX form), or with the dynamically scaled int8 output and optionally e4m3
// beside it, has a kernel of its own; it reproduces the general kernel's bits for the general kernel's default team shape,
// so it steps aside when the debug hook has changed that shape.
template<typename T> static bool adaln_fast_path(const RowParams& p, cudaStream_t stream, int& status)
{
    if (g_special_rows_on == 0 || p.dim != 3072 || p.pre != nullptr || g_row_max_vpt != 6 || (p.qf8 != nullptr && p.f8_invert == 0)) {
        return false;
    }
    if (p.q8 != nullptr) {
        if (p.scale_mode != LYRAQ_SCALE_PER_TOKEN_DYNAMIC || p.qf8b != nullptr) {
            return false;
        }
        status = p.y != nullptr ? launch_adaln3072<T, true, false, true>(p, stream) : launch_adaln3072<T, false, false, true>(p, stream);
        return true;
    }
    if (p.qf8 == nullptr) {
        return false;
    }
    if (p.y != nullptr) {
        status = p.qf8b != nullptr ? launch_adaln3072<T, true, true, false>(p, stream) : launch_adaln3072<T, true, false, false>(p, stream);
    } else {
        status = p.qf8b != nullptr ? launch_adaln3072<T, false, true, false>(p, stream) : launch_adaln3072<T, false, false, false>(p, stream);
    }
    return true;
}

// Bias + GEGLU -> int8 with a static scale has no row statistic, so it needs no team and no row loop: this kernel gives
// every thread GEGLU_UNITS independent 8-column vectors (consecutive threads take consecutive vectors; all loads go out
// before the first is used), with more warps resident than the row kernel can afford.  The per-vector arithmetic is the
// row kernel's (geglu_vec, the smoothing multiply, quant8_s8), so the bytes are the same.
constexpr int GEGLU_UNITS = 2;
template<typename T, bool GEGLU>
__global__ void __launch_bounds__(256, 4) geglu_int8_flat_kernel(const RowParams p, uint32_t total)
{
    using P2 = Pair<T>;
    grid_launch_dependents();
    grid_dependency_wait();
    const uint32_t nvec  = (uint32_t)p.dim >> 3;
    const uint32_t first = blockIdx.x * (256u * GEGLU_UNITS) + threadIdx.x;
    const T*       x     = reinterpret_cast<const T*>(p.x);
    Vec16          h[GEGLU_UNITS], g[GEGLU ? GEGLU_UNITS : 1];
    uint32_t       row[GEGLU_UNITS], col[GEGLU_UNITS];
#pragma unroll
    for (int u = 0; u < GEGLU_UNITS; ++u) {
        const uint32_t idx = first + (uint32_t)u * 256u;
        row[u]             = idx / nvec;
        col[u]             = (idx - row[u] * nvec) << 3;
        if (idx < total) {
            const T* xr = x + (size_t)row[u] * (size_t)p.in_cols + col[u];
            h[u]        = ld_nc_16(xr);
            if (GEGLU) {
                g[GEGLU ? u : 0] = ld_nc_16(xr + p.dim);
            }
        }
    }
    const bool  per_token = !GEGLU && p.scale_mode == LYRAQ_SCALE_PER_TOKEN;
    const float s_tensor  = per_token ? 1.0f : ld_f32(p.q8_scale);
#pragma unroll
    for (int u = 0; u < GEGLU_UNITS; ++u) {
        if (first + (uint32_t)u * 256u < total) {
            const float s8 = per_token ? ld_f32(p.q8_scale + row[u]) : s_tensor;
            const float r8 = 1.0f / s8;
            const Vec16 a  = GEGLU ? geglu_vec<T>(h[u], g[GEGLU ? u : 0], reinterpret_cast<const T*>(p.bias), p.dim, (int)col[u]) : h[u];
            float2      f[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[j] = P2::to_f32(a.w[j]);
            }
            if (p.pre != nullptr) {
                const float4 p0 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + col[u]));
                const float4 p1 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + col[u] + 4));
                f[0] = mul_f32x2(f[0], make_float2(p0.x, p0.y));
                f[1] = mul_f32x2(f[1], make_float2(p0.z, p0.w));
                f[2] = mul_f32x2(f[2], make_float2(p1.x, p1.y));
                f[3] = mul_f32x2(f[3], make_float2(p1.z, p1.w));
            }
            uint32_t w0, w1;
            quant8_s8(f, s8, r8, w0, w1);
            st_8(p.q8 + (size_t)row[u] * (size_t)p.dim + col[u], w0, w1);
        }
    }
}

template<typename T> static bool geglu_fast_path(const RowParams& p, cudaStream_t stream, int& status)
{
    const size_t total = p.rows * (size_t)(p.dim >> 3);
    if (g_special_rows_on == 0 || p.q8 == nullptr || p.y != nullptr || p.qf8 != nullptr || p.qf8b != nullptr ||
        p.scale_mode != LYRAQ_SCALE_PER_TENSOR || total >= (1ull << 31)) {
        return false;
    }
    const unsigned grid = (unsigned)((total + 256u * GEGLU_UNITS - 1) / (256u * GEGLU_UNITS));
    status = cuda_status(launch_kernel(geglu_int8_flat_kernel<T, true>, grid, 256u, (size_t)0, stream, 1u, p, (uint32_t)total),
                         "cudaLaunchKernelEx(geglu_int8_flat_kernel)");
    return true;
}

// The SmoothQuant quantize with a static or a given per-token scale has no row statistic either: the same flat kernel
// without the GEGLU step, for any row width.
template<typename T> static bool quant_flat_path(const RowParams& p, cudaStream_t stream, int& status)
{
    const size_t total = p.rows * (size_t)(p.dim >> 3);
    if (g_special_rows_on == 0 || p.q8 == nullptr || p.y != nullptr || p.qf8 != nullptr || p.qf8b != nullptr ||
        p.scale_mode == LYRAQ_SCALE_PER_TOKEN_DYNAMIC || total >= (1ull << 31)) {
        return false;
    }
    const unsigned grid = (unsigned)((total + 256u * GEGLU_UNITS - 1) / (256u * GEGLU_UNITS));
    status = cuda_status(launch_kernel(geglu_int8_flat_kernel<T, false>, grid, 256u, (size_t)0, stream, 1u, p, (uint32_t)total),
                         "cudaLaunchKernelEx(geglu_int8_flat_kernel<plain>)");
    return true;
}

// LayerNorm -> int8 (static scale; optionally x + residual + bias first, with the sum stored) for rows of 320, 640 or 1280 columns, the widths of the SDXL and SD 1.5
// transformer blocks (640 columns = 80 vectors = 2.5 per lane of a warp: the general kernel leaves lanes idle).  8, 16 or
// 32 lanes own a row with exactly five vectors each, so a warp works on four, two or one rows at once with every lane busy, the
// two reductions are xor-butterflies inside the lane group, and with no row loop state to carry twice as many warps are
// resident as in the general kernel.  Same formulas as the general kernel (mean and variance in fp32, x_hat rounded to T,
// T(T(gamma * x_hat) + beta), smoothing multiply, quant8_s8); only the order of the fp32 sums differs.
template<typename T, int LANES_LOG2, bool HAS_RES>
__global__ void __launch_bounds__(256, 4) ln_int8_short_kernel(const RowParams p)
{
    using P2 = Pair<T>;
    constexpr int VPL   = 5;
    constexpr int LANES = 1 << LANES_LOG2;
    constexpr int RPW   = 32 / LANES;  // rows per warp
    grid_launch_dependents();
    grid_dependency_wait();
    const int    lane   = threadIdx.x & 31;
    const int    sub    = lane & (LANES - 1);
    const size_t stride = (size_t)gridDim.x * 8 * RPW;
    const T*     gamma  = reinterpret_cast<const T*>(p.gamma);
    const T*     beta   = reinterpret_cast<const T*>(p.beta);
    const float  s8     = ld_f32(p.q8_scale);
    const float  r8     = 1.0f / s8;
    for (size_t wrow = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW; wrow < p.rows; wrow += stride) {
        const size_t row  = wrow + (size_t)(lane >> LANES_LOG2);
        const bool   live = row < p.rows;  // the shuffles below need every lane, so a lane without a row works on zeros
        const T*     xr   = reinterpret_cast<const T*>(p.x) + row * (size_t)p.dim;
        Vec16        v[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            if (live) {
                v[i] = ld_nc_16(xr + ((sub + LANES * i) << 3));
            } else {
                v[i].w[0] = v[i].w[1] = v[i].w[2] = v[i].w[3] = 0u;
            }
        }
        if (HAS_RES) {
            // h = T(T(x + residual) + bias), stored as the block's new hidden state and normalised in place of x
            const T* rr = reinterpret_cast<const T*>(p.residual) + row * (size_t)p.dim;
            Vec16    r[VPL];
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                if (live) {
                    r[i] = ld_nc_16(rr + ((sub + LANES * i) << 3));
                } else {
                    r[i].w[0] = r[i].w[1] = r[i].w[2] = r[i].w[3] = 0u;
                }
            }
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                const int c = (sub + LANES * i) << 3;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[i].w[j] = P2::add(v[i].w[j], r[i].w[j]);
                }
                if (p.bias != nullptr) {
                    const Vec16 bv = ld_nc_16_keep(reinterpret_cast<const T*>(p.bias) + c);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[i].w[j] = P2::add(v[i].w[j], bv.w[j]);
                    }
                }
                if (live && p.sum_out != nullptr) {
                    st_16(reinterpret_cast<T*>(p.sum_out) + row * (size_t)p.dim + c, v[i]);
                }
            }
        }
        // the row stays packed in T (20 registers); each of the three passes converts on the fly
        float2 sa = make_float2(0.0f, 0.0f), sb = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            sa = add_f32x2(sa, add_f32x2(P2::to_f32(v[i].w[0]), P2::to_f32(v[i].w[2])));
            sb = add_f32x2(sb, add_f32x2(P2::to_f32(v[i].w[1]), P2::to_f32(v[i].w[3])));
        }
        float sum = (sa.x + sa.y) + (sb.x + sb.y);
#pragma unroll
        for (int m = LANES / 2; m > 0; m >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, m);
        }
        const float  mean = sum / (float)p.dim;
        const float2 nm   = make_float2(-mean, -mean);
        float2       qa   = make_float2(0.0f, 0.0f), qb = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const float2 d0 = add_f32x2(P2::to_f32(v[i].w[0]), nm), d2 = add_f32x2(P2::to_f32(v[i].w[2]), nm);
            const float2 d1 = add_f32x2(P2::to_f32(v[i].w[1]), nm), d3 = add_f32x2(P2::to_f32(v[i].w[3]), nm);
            qa              = fma_f32x2(d0, d0, fma_f32x2(d2, d2, qa));
            qb              = fma_f32x2(d1, d1, fma_f32x2(d3, d3, qb));
        }
        float m2 = (qa.x + qa.y) + (qb.x + qb.y);
#pragma unroll
        for (int m = LANES / 2; m > 0; m >>= 1) {
            m2 += __shfl_xor_sync(0xffffffffu, m2, m);
        }
        const float  var  = fmaxf(m2 / (float)p.dim, 0.0f);
        const float  rstd = 1.0f / sqrtf(var + p.eps);
        const float2 rs   = make_float2(rstd, rstd);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int   c = (sub + LANES * i) << 3;
            const Vec16 a = ld_nc_16_keep(gamma + c);
            const Vec16 b = ld_nc_16_keep(beta + c);
            float2      y[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2   xn = mul_f32x2(add_f32x2(P2::to_f32(v[i].w[j]), nm), rs);
                const uint32_t xh = P2::from_f32(xn.x, xn.y);
                y[j]              = P2::to_f32(P2::add(P2::mul(a.w[j], xh), b.w[j]));
            }
            if (p.pre != nullptr) {
                const float4 p0 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + c));
                const float4 p1 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + c + 4));
                y[0] = mul_f32x2(y[0], make_float2(p0.x, p0.y));
                y[1] = mul_f32x2(y[1], make_float2(p0.z, p0.w));
                y[2] = mul_f32x2(y[2], make_float2(p1.x, p1.y));
                y[3] = mul_f32x2(y[3], make_float2(p1.z, p1.w));
            }
            uint32_t w0, w1;
            quant8_s8(y, s8, r8, w0, w1);
            if (live) {
                st_8(p.q8 + row * (size_t)p.dim + c, w0, w1);
            }
        }
    }
}

// The SmoothQuant int8 quantize (static, given per-token, or dynamic per-token scale) in the same short-row form.  The
// maximum of a row does not depend on the order it is taken in and the rest is per element, so the bytes and the scales
// are the general kernel's.
template<typename T, int LANES_LOG2>
__global__ void __launch_bounds__(256, 4) quant_int8_short_kernel(const RowParams p)
{
    using P2 = Pair<T>;
    constexpr int VPL   = 5;
    constexpr int LANES = 1 << LANES_LOG2;
    constexpr int RPW   = 32 / LANES;
    grid_launch_dependents();
    grid_dependency_wait();
    const int    lane    = threadIdx.x & 31;
    const int    sub     = lane & (LANES - 1);
    const size_t stride  = (size_t)gridDim.x * 8 * RPW;
    const bool   dynamic = (p.scale_mode == LYRAQ_SCALE_PER_TOKEN_DYNAMIC);
    for (size_t wrow = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW; wrow < p.rows; wrow += stride) {
        const size_t row  = wrow + (size_t)(lane >> LANES_LOG2);
        const bool   live = row < p.rows;
        const T*     xr   = reinterpret_cast<const T*>(p.x) + row * (size_t)p.dim;
        // the row stays packed in T (20 registers); the maximum pass and the quantize pass each convert a vector and apply
        // the smoothing factors as they go
        Vec16 v[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            if (live) {
                v[i] = ld_nc_16(xr + ((sub + LANES * i) << 3));
            } else {
                v[i].w[0] = v[i].w[1] = v[i].w[2] = v[i].w[3] = 0u;
            }
        }
        auto smoothed = [&](int i, float2 (&g)[4]) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                g[j] = P2::to_f32(v[i].w[j]);
            }
            if (p.pre != nullptr) {
                const int    c  = (sub + LANES * i) << 3;
                const float4 p0 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + c));
                const float4 p1 = ld_f32x4(reinterpret_cast<const float4*>(p.pre + c + 4));
                g[0] = mul_f32x2(g[0], make_float2(p0.x, p0.y));
                g[1] = mul_f32x2(g[1], make_float2(p0.z, p0.w));
                g[2] = mul_f32x2(g[2], make_float2(p1.x, p1.y));
                g[3] = mul_f32x2(g[3], make_float2(p1.z, p1.w));
            }
        };
        float s8;
        if (dynamic) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < VPL; ++i) {
                float2 g[4];
                smoothed(i, g);
                amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(g[0].x), fabsf(g[0].y)), fmaxf(fabsf(g[1].x), fabsf(g[1].y))),
                                         fmaxf(fmaxf(fabsf(g[2].x), fabsf(g[2].y)), fmaxf(fabsf(g[3].x), fabsf(g[3].y)))));
            }
#pragma unroll
            for (int m = LANES / 2; m > 0; m >>= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
            }
            s8 = (amax == 0.0f) ? 1.0f : amax / 127.0f;
            if (live && sub == 0) {
                p.q8_scale[row] = s8;
            }
        } else if (p.scale_mode == LYRAQ_SCALE_PER_TOKEN) {
            s8 = live ? ld_f32(p.q8_scale + row) : 1.0f;
        } else {
            s8 = ld_f32(p.q8_scale);
        }
        const float r8 = 1.0f / s8;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            float2 g[4];
            smoothed(i, g);
            uint32_t w0, w1;
            if (dynamic) {
                quant8_s8_inrange(g, s8, r8, w0, w1);
            } else {
                quant8_s8(g, s8, r8, w0, w1);
            }
            if (live) {
                st_8(p.q8 + row * (size_t)p.dim + ((sub + LANES * i) << 3), w0, w1);
            }
        }
    }
}

template<typename T> static bool quant_fast_path(const RowParams& p, cudaStream_t stream, int& status)
{
    if (g_special_rows_on == 0 || (p.dim != 320 && p.dim != 640 && p.dim != 1280) || p.q8 == nullptr || p.y != nullptr ||
        p.qf8 != nullptr || p.qf8b != nullptr) {
        return false;
    }
    if (p.dim == 1280) {
        status = launch_row_variant(quant_int8_short_kernel<T, 5>, p, (p.rows + 7) / 8, stream);
    } else if (p.dim == 640) {
        status = launch_row_variant(quant_int8_short_kernel<T, 4>, p, (p.rows + 15) / 16, stream);
    } else {
        status = launch_row_variant(quant_int8_short_kernel<T, 3>, p, (p.rows + 31) / 32, stream);
    }
    return true;
}

template<typename T> static bool ln_fast_path(const RowParams& p, cudaStream_t stream, int& status)
{
    if (g_special_rows_on == 0 || (p.dim != 320 && p.dim != 640 && p.dim != 1280) || p.q8 == nullptr || p.y != nullptr ||
        p.qf8 != nullptr || p.qf8b != nullptr || p.scale_mode != LYRAQ_SCALE_PER_TENSOR) {
        return false;
    }
    const bool res = p.residual != nullptr;
    if (p.dim == 1280) {
        status = res ? launch_row_variant(ln_int8_short_kernel<T, 5, true>, p, (p.rows + 7) / 8, stream)
                     : launch_row_variant(ln_int8_short_kernel<T, 5, false>, p, (p.rows + 7) / 8, stream);
    } else if (p.dim == 640) {
        status = res ? launch_row_variant(ln_int8_short_kernel<T, 4, true>, p, (p.rows + 15) / 16, stream)
                     : launch_row_variant(ln_int8_short_kernel<T, 4, false>, p, (p.rows + 15) / 16, stream);
    } else {
        status = res ? launch_row_variant(ln_int8_short_kernel<T, 3, true>, p, (p.rows + 31) / 32, stream)
                     : launch_row_variant(ln_int8_short_kernel<T, 3, false>, p, (p.rows + 31) / 32, stream);
    }
    return true;
}

template<int MODE> static int dispatch_row(int dtype, const RowParams& p, cudaStream_t stream)
{
    if (p.dim <= 0 || (p.dim & 7) != 0 || p.dim > 16384) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (MODE == ROW_ADALN) {
        int status = LYRAQ_OK;
        if ((dtype == LYRAQ_F16 && adaln_fast_path<__half>(p, stream, status)) ||
            (dtype == LYRAQ_BF16 && adaln_fast_path<__nv_bfloat16>(p, stream, status))) {
            return status;
        }
    }
    if (MODE == ROW_PLAIN) {
        int status = LYRAQ_OK;
        if ((dtype == LYRAQ_F16 && quant_flat_path<__half>(p, stream, status)) ||
            (dtype == LYRAQ_BF16 && quant_flat_path<__nv_bfloat16>(p, stream, status))) {
            return status;
        }
        if ((dtype == LYRAQ_F16 && quant_fast_path<__half>(p, stream, status)) ||
            (dtype == LYRAQ_BF16 && quant_fast_path<__nv_bfloat16>(p, stream, status))) {
            return status;
        }
    }
    if (MODE == ROW_LN) {
        int status = LYRAQ_OK;
        if ((dtype == LYRAQ_F16 && ln_fast_path<__half>(p, stream, status)) ||
            (dtype == LYRAQ_BF16 && ln_fast_path<__nv_bfloat16>(p, stream, status))) {
            return status;
        }
    }
    if (MODE == ROW_GEGLU) {
        int status = LYRAQ_OK;
        if ((dtype == LYRAQ_F16 && geglu_fast_path<__half>(p, stream, status)) ||
            (dtype == LYRAQ_BF16 && geglu_fast_path<__nv_bfloat16>(p, stream, status))) {
            return status;
        }
    }
    if (dtype == LYRAQ_F16) {
        return launch_row<__half, MODE>(p, stream);
    }
    if (dtype == LYRAQ_BF16) {
        return launch_row<__nv_bfloat16, MODE>(p, stream);
    }
    return LYRAQ_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// Flat per-tensor e4m3 conversion (no row structure): 8 elements per thread per step.
template<typename T>
__global__ void __launch_bounds__(256) fp8_cast_kernel(uint8_t* dst, const T* src, const float* scale, int invert, size_t n)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const float  s      = ld_f32(scale);
    const float  r      = invert ? 1.0f / s : s;
    const size_t nvec   = n >> 3;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    // four independent 16-byte loads in flight per thread and step
    size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; vi + 3 * stride < nvec; vi += 4 * stride) {
        Vec16 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            x[u] = ld_nc_16(src + ((vi + u * stride) << 3));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float v[8];
            unpack8<T>(x[u], v);
            const uint32_t w0 = f32x2_to_e4m3x2(v[0] * r, v[1] * r) | (f32x2_to_e4m3x2(v[2] * r, v[3] * r) << 16);
            const uint32_t w1 = f32x2_to_e4m3x2(v[4] * r, v[5] * r) | (f32x2_to_e4m3x2(v[6] * r, v[7] * r) << 16);
            st_8(dst + ((vi + u * stride) << 3), w0, w1);
        }
    }
    for (; vi < nvec; vi += stride) {
        float v[8];
        unpack8<T>(ld_nc_16(src + (vi << 3)), v);
        const uint32_t w0 = f32x2_to_e4m3x2(v[0] * r, v[1] * r) | (f32x2_to_e4m3x2(v[2] * r, v[3] * r) << 16);
        const uint32_t w1 = f32x2_to_e4m3x2(v[4] * r, v[5] * r) | (f32x2_to_e4m3x2(v[6] * r, v[7] * r) << 16);
        st_8(dst + (vi << 3), w0, w1);
    }
    // tail (n not a multiple of 8)
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
        const size_t i = (nvec << 3) + threadIdx.x;
        dst[i]         = (uint8_t)(f32x2_to_e4m3x2(to_f32(src[i]) * r, 0.0f) & 0xff);
    }
}

// The same conversion with the source staged through shared memory: one bulk asynchronous copy per block brings its
// 32 KB chunk in (no registers held while it is in flight), so six resident blocks keep 192 KB per SM outstanding and a
// tensor of up to 148 * 6 chunks (29 MB of 16-bit input) is read in a single wave with a single round trip to DRAM.
constexpr int kBulkElems = 16384;
constexpr int kBulkSmem  = kBulkElems * 2 + 16;
template<typename T>
__global__ void __launch_bounds__(256) fp8_cast_bulk_kernel(uint8_t* dst, const T* src, const float* scale, int invert, size_t n,
                                                            unsigned int* status)
{
    extern __shared__ __align__(128) uint8_t cast_smem[];
    const uint32_t data       = sm100::smem_u32(cast_smem);
    const uint32_t bar        = data + kBulkElems * 2;
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(cast_smem + kBulkElems * 2 + 8);
    const size_t   e0         = (size_t)blockIdx.x * kBulkElems;
    const size_t   n8         = n & ~(size_t)7;
    const uint32_t elems      = (uint32_t)((n8 - e0 < (size_t)kBulkElems) ? (n8 - e0) : (size_t)kBulkElems);
    grid_launch_dependents();
    if (threadIdx.x == 0) {
        sm100::mbar_init(bar, 1);
        *abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
    grid_dependency_wait();
    if (threadIdx.x == 0 && elems != 0) {
        sm100::mbar_arrive_expect_tx(bar, elems * 2u);
        sm100::bulk_load(data, src + e0, elems * 2u, bar);
    }
    const float s = ld_f32(scale);
    const float r = invert ? 1.0f / s : s;
    if (elems != 0) {
        if (!sm100::mbar_wait(bar, 0u, abort_flag)) {
            if (threadIdx.x == 0) {
                report_timeout(status, 0x3100u);
            }
            return;
        }
        const uint32_t nv = elems >> 3;
#pragma unroll 4
        for (uint32_t v = threadIdx.x; v < nv; v += 256) {
            float v8[8];
            unpack8<T>(*reinterpret_cast<const Vec16*>(cast_smem + (size_t)v * 16), v8);
            const uint32_t w0 = f32x2_to_e4m3x2(v8[0] * r, v8[1] * r) | (f32x2_to_e4m3x2(v8[2] * r, v8[3] * r) << 16);
            const uint32_t w1 = f32x2_to_e4m3x2(v8[4] * r, v8[5] * r) | (f32x2_to_e4m3x2(v8[6] * r, v8[7] * r) << 16);
            st_8(dst + e0 + ((size_t)v << 3), w0, w1);
        }
    }
    // tail (n not a multiple of 8): the last block
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x < (n & 7)) {
        const size_t i = n8 + threadIdx.x;
        dst[i]         = (uint8_t)(f32x2_to_e4m3x2(to_f32(src[i]) * r, 0.0f) & 0xff);
    }
}

// max|w|/448 folded into scale[0] with an integer atomicMax on the (non-negative) float bits.
template<typename T> __global__ void __launch_bounds__(256) fp8_amax_kernel(float* scale, const T* src, size_t n)
{
    __shared__ float red[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t     nvec   = n >> 3;
    const size_t     stride = (size_t)gridDim.x * blockDim.x;
    float            amax   = 0.0f;
    for (size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += stride) {
        float v[8];
        unpack8<T>(ld_nc_16(src + (vi << 3)), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            amax = fmaxf(amax, fabsf(v[j]));
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < (n & 7)) {
        amax = fmaxf(amax, fabsf(to_f32(src[(nvec << 3) + threadIdx.x])));
    }
    amax = team_reduce<true>(amax, 256, red);
    if (threadIdx.x == 0) {
        // |w|/448 is monotone in |w|, so dividing the block maximum equals the maximum of the quotients.
        atomicMax(reinterpret_cast<int*>(scale), __float_as_int(amax / 448.0f));
    }
}

// ---------------------------------------------------------------------------------------------
// INT4 group-64 quantize: 8 consecutive threads own one group of 64 values, 8 values each.
template<typename T, typename ST>
__global__ void __launch_bounds__(256)
int4_g64_kernel(uint32_t* q, ST* q_scale, const T* x, const float* smooth, size_t rows, int k)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t nvec_total = rows * (size_t)(k >> 3);
    const size_t stride     = (size_t)gridDim.x * blockDim.x;
    const int    vec_per_row = k >> 3;
    // the loop bound is rounded up to a multiple of 8 threads so that shuffles stay converged
    for (size_t base = (size_t)blockIdx.x * blockDim.x; base < nvec_total; base += stride) {
        const size_t vi   = base + threadIdx.x;
        const bool   live = vi < nvec_total;
        float        v[8];
        if (live) {
            unpack8<T>(ld_nc_16(x + (vi << 3)), v);
            if (smooth != nullptr) {
                const int    c  = (int)(vi % vec_per_row) << 3;
                const float4 s0 = ld_f32x4(reinterpret_cast<const float4*>(smooth + c));
                const float4 s1 = ld_f32x4(reinterpret_cast<const float4*>(smooth + c + 4));
                v[0] /= s0.x; v[1] /= s0.y; v[2] /= s0.z; v[3] /= s0.w;
                v[4] /= s1.x; v[5] /= s1.y; v[6] /= s1.z; v[7] /= s1.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = 0.0f;
            }
        }
        float          s;
        const uint32_t w = int4_g64_quantize8(v, s);
        if (live) {
            q[vi] = w;
            if ((threadIdx.x & 7) == 0) {
                q_scale[vi >> 3] = ST(s);
            }
        }
    }
}

// INT8 per-output-channel weight quantize: one 128-thread block per row, row kept in registers/re-read.
template<typename T>
__global__ void __launch_bounds__(256)
int8_weight_quant_kernel(float* w_scale, int8_t* qw, const T* w, const float* pre, size_t d_in)
{
    __shared__ float red[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t     row  = blockIdx.x;
    const T*         wrow = w + row * d_in;
    float            amax = 0.0f;
    for (size_t c = threadIdx.x; c < d_in; c += blockDim.x) {
        float v = to_f32(wrow[c]);
        if (pre != nullptr) {
            v = v / ld_f32(pre + c);
        }
        amax = fmaxf(amax, fabsf(v));
    }
    amax          = team_reduce<true>(amax, 256, red);
    const float s = (float)((double)amax / 127.0);
    if (threadIdx.x == 0) {
        w_scale[row] = s;
    }
    for (size_t c = threadIdx.x; c < d_in; c += blockDim.x) {
        float v = to_f32(wrow[c]);
        if (pre != nullptr) {
            v = v / ld_f32(pre + c);
        }
        qw[row * d_in + c] = (int8_t)f32_to_s8(v / s);
    }
}

static unsigned flat_grid(size_t nvec)
{
    size_t g = (nvec + 255) / 256;
    // enough blocks to fill 148 SMs eight times over; the kernels are grid-stride
    const size_t cap = 148 * 8;
    if (g > cap) {
        g = cap;
    }
    return g == 0 ? 1u : (unsigned)g;
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {

int lyraq_debug_set_row_vectors_per_thread(int max_vpt)
{
    if (max_vpt != 4 && max_vpt != 6) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    g_row_max_vpt = max_vpt;
    return LYRAQ_OK;
}

int lyraq_debug_set_special_row_kernels(int on)
{
    g_special_rows_on = on != 0;
    return LYRAQ_OK;
}

int lyraq_quant_int8(int8_t* dst, const void* src, int src_dtype, const float* pre_quant_scale, float* scale,
                     int scale_mode, size_t rows, size_t dim, void* stream)
{
    if (rows == 0 && scale_mode >= 0 && scale_mode <= 2) {
        return LYRAQ_OK;
    }
    if (dst == nullptr || src == nullptr || scale == nullptr || scale_mode < 0 || scale_mode > 2) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 7u) != 0 ||
        (pre_quant_scale != nullptr && !aligned16(pre_quant_scale))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (dim > 16384) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    RowParams p{};
    p.x          = src;
    p.pre        = pre_quant_scale;
    p.q8         = dst;
    p.q8_scale   = scale;
    p.scale_mode = scale_mode;
    p.rows       = rows;
    p.dim        = (int)dim;
    p.in_cols    = (int)dim;
    return dispatch_row<ROW_PLAIN>(src_dtype, p, (cudaStream_t)stream);
}

int lyraq_quant_fp8(uint8_t* dst, const void* src, int src_dtype, const float* scale, int invert_scale, size_t n,
                    void* stream)
{
    if (n == 0) {
        return LYRAQ_OK;
    }
    if (dst == nullptr || src == nullptr || scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 7u) != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (src_dtype != LYRAQ_F16 && src_dtype != LYRAQ_BF16) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    // One 32 KB chunk per block through the bulk-staged kernel; fewer than 8 elements fall through to the grid-stride
    // kernel's scalar tail.
    const size_t chunks = ((n & ~(size_t)7) + kBulkElems - 1) / kBulkElems;
    if (chunks >= 1 && chunks <= 0x7fffffffu) {
        unsigned int* status = status_word_ptr();
        if (status == nullptr) {
            return LYRAQ_ERR_CUDA;
        }
        if (src_dtype == LYRAQ_F16) {
            launch_kernel(fp8_cast_bulk_kernel<__half>, (unsigned)chunks, 256u, (size_t)kBulkSmem, (cudaStream_t)stream, 1u, dst,
                          (const __half*)src, scale, invert_scale, n, status);
        } else {
            launch_kernel(fp8_cast_bulk_kernel<__nv_bfloat16>, (unsigned)chunks, 256u, (size_t)kBulkSmem, (cudaStream_t)stream, 1u, dst,
                          (const __nv_bfloat16*)src, scale, invert_scale, n, status);
        }
        return launch_status();
    }
    const unsigned grid = flat_grid(n >> 3);
    if (src_dtype == LYRAQ_F16) {
        launch_kernel(fp8_cast_kernel<__half>, (unsigned)(grid), 256u, (size_t)0, (cudaStream_t)stream, 1u, dst, (const __half*)src, scale, invert_scale, n);
    } else {
        launch_kernel(fp8_cast_kernel<__nv_bfloat16>, (unsigned)(grid), 256u, (size_t)0, (cudaStream_t)stream, 1u, dst, (const __nv_bfloat16*)src, scale, invert_scale, n);
    }
    return launch_status();
}

int lyraq_fp8_amax_scale(float* scale, const void* w, int w_dtype, size_t n, void* stream)
{
    if (n == 0) {
        return LYRAQ_OK;
    }
    if (scale == nullptr || w == nullptr || !aligned16(w)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    const unsigned grid = flat_grid(n >> 3);
    if (w_dtype == LYRAQ_F16) {
        launch_kernel(fp8_amax_kernel<__half>, (unsigned)(grid), 256u, (size_t)0, (cudaStream_t)stream, 1u, scale, (const __half*)w, n);
    } else if (w_dtype == LYRAQ_BF16) {
        launch_kernel(fp8_amax_kernel<__nv_bfloat16>, (unsigned)(grid), 256u, (size_t)0, (cudaStream_t)stream, 1u, scale, (const __nv_bfloat16*)w, n);
    } else {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    return launch_status();
}

int lyraq_weight_quant_fp8(uint8_t* qw, float* scale, const void* w, int w_dtype, size_t n, void* stream)
{
    if (n == 0) {
        return LYRAQ_OK;
    }
    if (qw == nullptr || scale == nullptr || w == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    const cudaError_t e = cudaMemsetAsync(scale, 0, sizeof(float), (cudaStream_t)stream);
    if (e != cudaSuccess) {
        return cuda_status(e, "cudaMemsetAsync(weight scale)");
    }
    const int st = lyraq_fp8_amax_scale(scale, w, w_dtype, n, stream);
    if (st != LYRAQ_OK) {
        return st;
    }
    return lyraq_quant_fp8(qw, w, w_dtype, scale, 1, n, stream);
}

int lyraq_weight_quant_int8(float* w_scale, int8_t* qw, const void* w, int w_dtype, const float* pre_quant_scale,
                            size_t d_out, size_t d_in, void* stream)
{
    if (d_out == 0 || d_in == 0) {
        return LYRAQ_OK;
    }
    if (w_scale == nullptr || qw == nullptr || w == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (d_out > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (w_dtype == LYRAQ_F16) {
        launch_kernel(int8_weight_quant_kernel<__half>, (unsigned)((unsigned)d_out), 256u, (size_t)0, (cudaStream_t)stream, 1u, w_scale, qw, (const __half*)w, pre_quant_scale, d_in);
    } else if (w_dtype == LYRAQ_BF16) {
        launch_kernel(int8_weight_quant_kernel<__nv_bfloat16>, (unsigned)((unsigned)d_out), 256u, (size_t)0, (cudaStream_t)stream, 1u, 
            w_scale, qw, (const __nv_bfloat16*)w, pre_quant_scale, d_in);
    } else {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    return launch_status();
}

static int int4_g64_dispatch(uint8_t* q, void* q_scale, int scale_dtype, const void* x, int x_dtype, const float* smooth,
                             size_t rows, size_t k, cudaStream_t stream)
{
    if (rows == 0 && k != 0 && (k & 63) == 0) {
        return LYRAQ_OK;
    }
    if (q == nullptr || q_scale == nullptr || x == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 3u) != 0 || (smooth != nullptr && !aligned16(smooth))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (k == 0 || (k & 63) != 0 || k > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (rows == 0) {
        return LYRAQ_OK;
    }
    const unsigned grid = flat_grid(rows * (k >> 3));
    uint32_t*      qo   = reinterpret_cast<uint32_t*>(q);
    const char* where = "cudaLaunchKernelEx(int4_g64_kernel)";
    if (x_dtype == LYRAQ_BF16 && scale_dtype == LYRAQ_F32) {
        return cuda_status(launch_kernel(int4_g64_kernel<__nv_bfloat16, float>, grid, 256u, (size_t)0, stream, 1u, qo, (float*)q_scale,
                                         (const __nv_bfloat16*)x, smooth, rows, (int)k), where);
    }
    if (x_dtype == LYRAQ_F16 && scale_dtype == LYRAQ_F32) {
        return cuda_status(launch_kernel(int4_g64_kernel<__half, float>, grid, 256u, (size_t)0, stream, 1u, qo, (float*)q_scale,
                                         (const __half*)x, smooth, rows, (int)k), where);
    }
    if (x_dtype == LYRAQ_BF16 && scale_dtype == LYRAQ_F16) {
        return cuda_status(launch_kernel(int4_g64_kernel<__nv_bfloat16, __half>, grid, 256u, (size_t)0, stream, 1u, qo, (__half*)q_scale,
                                         (const __nv_bfloat16*)x, smooth, rows, (int)k), where);
    }
    if (x_dtype == LYRAQ_F16 && scale_dtype == LYRAQ_F16) {
        return cuda_status(launch_kernel(int4_g64_kernel<__half, __half>, grid, 256u, (size_t)0, stream, 1u, qo, (__half*)q_scale,
                                         (const __half*)x, smooth, rows, (int)k), where);
    }
    return LYRAQ_ERR_UNSUPPORTED;
}

int lyraq_quant_int4_g64(uint8_t* q, float* q_scale, float* lora_act, const void* x, int x_dtype, const float* smooth,
                         const void* lora_down, size_t m, size_t k, void* stream)
{
    if ((lora_act == nullptr) != (lora_down == nullptr)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (lora_act == nullptr || m == 0) {
        return int4_g64_dispatch(q, q_scale, LYRAQ_F32, x, x_dtype, smooth, m, k, (cudaStream_t)stream);
    }
    if (q == nullptr || q_scale == nullptr || x == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    // quantize and low-rank down projection in one launch over one read of x: the quantizer warps work on the tiles the
    // down projection's TMA ring has staged (lora_down.cu)
    return launch_quant_int4_lora_down(q, q_scale, lora_act, x, lora_down, smooth, x_dtype, m, k, (cudaStream_t)stream);
}

int lyraq_weight_quant_int4_g64(uint8_t* qw, void* w_scale, int scale_dtype, const void* w, int w_dtype, size_t n,
                                size_t k, void* stream)
{
    return int4_g64_dispatch(qw, w_scale, scale_dtype, w, w_dtype, nullptr, n, k, (cudaStream_t)stream);
}

int lyraq_adaln_quant(void* y, int8_t* q8, float* q8_scale, uint8_t* qf8, const float* f8_scale, const void* x,
                      const void* scale, const void* shift, int dtype, const float* pre_quant_scale, size_t B, size_t S,
                      size_t D, double eps, void* stream)
{
    if (B * S == 0) {
        return LYRAQ_OK;
    }
    if (x == nullptr || scale == nullptr || shift == nullptr || (q8 != nullptr && q8_scale == nullptr) ||
        (qf8 != nullptr && f8_scale == nullptr) || (y == nullptr && q8 == nullptr && qf8 == nullptr)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(x) || !aligned16(scale) || !aligned16(shift) || (y != nullptr && !aligned16(y)) ||
        (reinterpret_cast<uintptr_t>(q8) & 7u) != 0 || (reinterpret_cast<uintptr_t>(qf8) & 7u) != 0 ||
        (pre_quant_scale != nullptr && !aligned16(pre_quant_scale))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (D > 16384 || S > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    RowParams p{};
    p.x              = x;
    p.ada_scale      = scale;
    p.ada_shift      = shift;
    p.pre            = pre_quant_scale;
    p.y              = y;
    p.q8             = q8;
    p.q8_scale       = q8_scale;
    p.scale_mode     = LYRAQ_SCALE_PER_TOKEN_DYNAMIC;
    p.qf8            = qf8;
    p.f8_scale       = f8_scale;
    p.f8_invert      = 1;
    p.rows           = B * S;
    p.dim            = (int)D;
    p.in_cols        = (int)D;
    p.rows_per_batch = (int)S;
    p.eps            = (float)eps;
    return dispatch_row<ROW_ADALN>(dtype, p, (cudaStream_t)stream);
}

int lyraq_adaln_quant_fp8x2(void* y, uint8_t* qa, const float* scale_a, uint8_t* qb, const float* scale_b, const void* x,
                            const void* scale, const void* shift, int dtype, size_t B, size_t S, size_t D, double eps, void* stream)
{
    if (B * S == 0) {
        return LYRAQ_OK;
    }
    if (x == nullptr || scale == nullptr || shift == nullptr || qa == nullptr || qb == nullptr || scale_a == nullptr ||
        scale_b == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(x) || !aligned16(scale) || !aligned16(shift) || (y != nullptr && !aligned16(y)) ||
        (reinterpret_cast<uintptr_t>(qa) & 7u) != 0 || (reinterpret_cast<uintptr_t>(qb) & 7u) != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (D > 16384 || S > 0x7fffffffu) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    RowParams p{};
    p.x              = x;
    p.ada_scale      = scale;
    p.ada_shift      = shift;
    p.y              = y;
    p.qf8            = qa;
    p.f8_scale       = scale_a;
    p.f8_invert      = 1;
    p.qf8b           = qb;
    p.f8_scale_b     = scale_b;
    p.rows           = B * S;
    p.dim            = (int)D;
    p.in_cols        = (int)D;
    p.rows_per_batch = (int)S;
    p.eps            = (float)eps;
    return dispatch_row<ROW_ADALN>(dtype, p, (cudaStream_t)stream);
}

int lyraq_ln_quant_int8(int8_t* dst, void* sum_out, const void* x, const void* residual, const void* bias,
                        const void* gamma, const void* beta, int dtype, const float* pre_quant_scale,
                        const float* input_quant_scale, size_t rows, size_t dim, double eps, void* stream)
{
    if (rows == 0) {
        return LYRAQ_OK;
    }
    if (dst == nullptr || x == nullptr || gamma == nullptr || beta == nullptr || input_quant_scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(beta) || (residual != nullptr && !aligned16(residual)) ||
        (bias != nullptr && !aligned16(bias)) || (sum_out != nullptr && !aligned16(sum_out)) ||
        (reinterpret_cast<uintptr_t>(dst) & 7u) != 0 || (pre_quant_scale != nullptr && !aligned16(pre_quant_scale))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (dim > 16384) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    RowParams p{};
    p.x          = x;
    p.residual   = residual;
    p.bias       = bias;
    p.gamma      = gamma;
    p.beta       = beta;
    p.pre        = pre_quant_scale;
    p.sum_out    = sum_out;
    p.q8         = dst;
    p.q8_scale   = const_cast<float*>(input_quant_scale);
    p.scale_mode = LYRAQ_SCALE_PER_TENSOR;
    p.rows       = rows;
    p.dim        = (int)dim;
    p.in_cols    = (int)dim;
    p.eps        = (float)eps;
    return dispatch_row<ROW_LN>(dtype, p, (cudaStream_t)stream);
}

int lyraq_geglu_quant_int8(int8_t* dst, const void* h, const void* bias, int dtype, const float* pre_quant_scale,
                           const float* input_quant_scale, size_t rows, size_t dim, void* stream)
{
    if (rows == 0) {
        return LYRAQ_OK;
    }
    if (dst == nullptr || h == nullptr || input_quant_scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(h) || (bias != nullptr && !aligned16(bias)) || (reinterpret_cast<uintptr_t>(dst) & 7u) != 0 ||
        (pre_quant_scale != nullptr && !aligned16(pre_quant_scale))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (dim > 16384) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    RowParams p{};
    p.x          = h;
    p.bias       = bias;
    p.pre        = pre_quant_scale;
    p.q8         = dst;
    p.q8_scale   = const_cast<float*>(input_quant_scale);
    p.scale_mode = LYRAQ_SCALE_PER_TENSOR;
    p.rows       = rows;
    p.dim        = (int)dim;
    p.in_cols    = (int)(2 * dim);
    return dispatch_row<ROW_GEGLU>(dtype, p, (cudaStream_t)stream);
}

}  // extern "C"
