// Shared helpers of the lyraq kernels: dtype dispatch, 16-byte vector access, conversions with the
// reference's rounding, the device status word, and argument checks used by every C entry point.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lyraq.h"

namespace lyraq {

// ---------------------------------------------------------------------------------------------
// Device status word.  Kernels with bounded waits record the first wait that gave up in a small
// per-device array (word 0: code, 0 = ok; word 1: detail); the host reads it through
// lyraq_last_status().  The array lives in the library's own device memory (api.cu); kernels get
// its device address as a parameter.
unsigned int* status_word_ptr();  // device address for the current device, NULL on failure

__device__ __forceinline__ void report_timeout(unsigned int* status, unsigned int detail)
{
    if (atomicCAS(&status[0], 0u, (unsigned int)LYRAQ_ERR_DEVICE_TIMEOUT) == 0u) {
        status[1] = detail;
    }
}

// ---------------------------------------------------------------------------------------------
template<typename T> struct TypeTag;
template<> struct TypeTag<__half> { static constexpr int value = LYRAQ_F16; };
template<> struct TypeTag<__nv_bfloat16> { static constexpr int value = LYRAQ_BF16; };
template<> struct TypeTag<float> { static constexpr int value = LYRAQ_F32; };

__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }

template<typename T> __device__ __forceinline__ T from_f32(float v);
template<> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template<> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template<> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// One arithmetic step "in T": the fp32 result of an operation on T operands, rounded to T.
// For 16-bit T an fp32 add or multiply of two T values followed by this rounding equals the
// native single-rounding T operation (products are exact in fp32; a sum that is inexact in fp32
// is far from any T rounding boundary).
template<typename T> __device__ __forceinline__ float round_t(float v) { return to_f32(from_f32<T>(v)); }

// q = sat_s8(rne(v)): cvt.rni.sat.s8.f32, NaN -> 0 (reference: kernels/quant_kernels/int8_utils.cuh:23-28).
__device__ __forceinline__ int f32_to_s8(float v)
{
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d)
{
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
}

// Two floats -> two e4m3 codes (RNE, saturate to +-448), low byte = first.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t)r;
}

__device__ __forceinline__ float tanh_approx(float x)
{
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// tanh-GELU in fp32 (reference: kernels/activation_kernels.h:56-68).
__device__ __forceinline__ float gelu_tanh_f32(float v)
{
    const float cdf = 0.5f * (1.0f + tanh_approx(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return v * cdf;
}

// ---------------------------------------------------------------------------------------------
// Packed fp32 pairs (sm_100: one instruction, two IEEE-rounded results; lane-wise identical to the scalar op).
__device__ __forceinline__ float2 mul_f32x2(float2 a, float2 b)
{
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b)
{
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
    return d;
}
__device__ __forceinline__ float2 fma_f32x2(float2 a, float2 b, float2 c)
{
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
          "l"(reinterpret_cast<const unsigned long long&>(c)));
    return d;
}

// tanh-GELU of two values at once: the same formula as gelu_tanh_f32 with the polynomial on packed pairs,
// 0.5 v (1 + tanh(0.79788 v (1 + 0.044715 v^2))); the two forms agree to an fp32 ulp or two.
__device__ __forceinline__ float2 gelu_tanh_f32x2(float2 v)
{
    const float2 v2  = mul_f32x2(v, v);
    const float2 p   = fma_f32x2(v2, make_float2(0.044715f, 0.044715f), make_float2(1.0f, 1.0f));
    const float2 a   = mul_f32x2(mul_f32x2(v, make_float2(0.7978845608028654f, 0.7978845608028654f)), p);
    const float2 th  = make_float2(tanh_approx(a.x), tanh_approx(a.y));
    const float2 h   = mul_f32x2(v, make_float2(0.5f, 0.5f));
    return fma_f32x2(h, th, h);
}

// ---------------------------------------------------------------------------------------------
// 16-byte vectors of 8 sixteen-bit values or 4 floats.
struct alignas(16) Vec16 {
    uint32_t w[4];
};

__device__ __forceinline__ Vec16 ld_nc_16(const void* p)
{
    Vec16 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}

// Same, for vectors that every row re-reads (modulation scale / shift, gamma / beta, bias): kept in L1.
// A 16-byte load that stays where it is written (the compiler may not sink it towards its first use), for loads that
// are issued ahead of time on purpose; and a prefetch of one 128-byte line into L2.
__device__ __forceinline__ Vec16 ld_nc_16_here(const void* p)
{
    Vec16 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ Vec16 ld_nc_16_keep(const void* p)
{
    Vec16 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
                 : "l"(p));
    return v;
}

// Loads that stay where they are written.  Every kernel here may start before its predecessor in the stream has finished
// (programmatic dependent launch) and reads global memory only after griddepcontrol.wait.  __ldg() is an invariant load
// to the compiler, which may move it above that wait (an e4m3 cast then read its scale before the amax kernel in front
// of it had written it); a volatile asm load is never moved across another volatile asm statement.  Use these for
// anything a previous kernel may have produced: scales, per-token scale vectors, smoothing vectors, low-rank activations.
__device__ __forceinline__ float ld_f32(const float* p)
{
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_f32x4(const float4* p)
{
    float4 v;
    asm volatile("ld.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_u32x4(const uint4* p)
{
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_16(void* p, const Vec16& v)
{
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3])
                 : "memory");
}

__device__ __forceinline__ void st_8(void* p, uint32_t a, uint32_t b)
{
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Unpack 8 sixteen-bit values held in a Vec16 to fp32.
template<typename T> __device__ __forceinline__ void unpack8(const Vec16& v, float* out);
template<> __device__ __forceinline__ void unpack8<__half>(const Vec16& v, float* out)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&v.w[i]);
        float2  f = __half22float2(h);
        out[2 * i]     = f.x;
        out[2 * i + 1] = f.y;
    }
}
template<> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const Vec16& v, float* out)
{
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i]     = __uint_as_float(v.w[i] << 16);
        out[2 * i + 1] = __uint_as_float(v.w[i] & 0xffff0000u);
    }
}

template<typename T> __device__ __forceinline__ Vec16 pack8(const float* in);
template<> __device__ __forceinline__ Vec16 pack8<__half>(const float* in)
{
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
        v.w[i]    = *reinterpret_cast<uint32_t*>(&h);
    }
    return v;
}
template<> __device__ __forceinline__ Vec16 pack8<__nv_bfloat16>(const float* in)
{
    Vec16 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
        v.w[i]           = *reinterpret_cast<uint32_t*>(&h);
    }
    return v;
}

// ---------------------------------------------------------------------------------------------
// Arithmetic "in T" on packed pairs (two 16-bit values in one 32-bit register), using the native
// single-rounding add / multiply of the type.  `_rn` intrinsics are never contracted into an fma,
// so each step is rounded to T exactly as the reference's T-typed expressions are.
template<typename T> struct Pair;
template<> struct Pair<__half> {
    static __device__ __forceinline__ float2 to_f32(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
    static __device__ __forceinline__ uint32_t from_f32(float a, float b)
    {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b)
    {
        __half2 r = __hadd2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)
    {
        __half2 r = __hmul2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t one() { return 0x3C003C00u; }
};
template<> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 to_f32(uint32_t w)
    {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t from_f32(float a, float b)
    {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b)
    {
        __nv_bfloat162 r = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)
    {
        __nv_bfloat162 r = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t one() { return 0x3F803F80u; }
};

// Eight quotients v[j] / s quantized exactly as the reference does, q = sat_s8(rne(fl32(v / s))), without a
// division or a conversion per element.  r = fl32(1 / s) is computed once per row by the caller.
//   t  = fma(v, r, 1.5 * 2^23)   one rounding: v*r to the nearest integer, ties to even (one ulp is 1 up there)
//   tc = clamp(t, magic - 128, magic + 127); the low byte of tc's bit pattern is the two's-complement int8
//   d  = fma(v, r, -(tc - magic)) the distance of v*r from that integer
// v*r and fl32(v/s) both lie within |q| * 2^-24 <= 7.7e-6 of the true quotient, so they round to the same
// integer unless the quotient is within 1.6e-5 of a half-integer.  If any of the eight is within 6.1e-5 of one
// (or is NaN: 0/0, NaN input), the whole vector is redone with the IEEE divide and cvt.rni.sat.s8.f32, which
// also gives NaN -> 0.  That happens for about one vector in a thousand.
// Variant for scales computed from the row itself (s = amax / 127): the quotient cannot exceed 127 * (1 + 2^-23)
// in magnitude, so no clamp is needed, d always lies in [-0.5, 0.5], and the near-tie test reduces to one maximum.
__device__ __forceinline__ void quant8_s8_inrange(const float2* v, float s, float r, uint32_t& w0, uint32_t& w1)
{
    const float2 mg = make_float2(12582912.0f, 12582912.0f);
    const float2 r2 = make_float2(r, r);
    const float2 m1 = make_float2(-1.0f, -1.0f);
    uint32_t     b[8];
    float        dmax = 0.0f;
    float2       bad  = make_float2(0.0f, 0.0f);  // becomes NaN if any d is NaN or infinite (fmaxf would drop a NaN)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = fma_f32x2(v[j], r2, mg);
        const float2 d = fma_f32x2(v[j], r2, fma_f32x2(t, m1, mg));  // v * r - (t - magic), the second term exact
        dmax           = fmaxf(dmax, fmaxf(fabsf(d.x), fabsf(d.y)));
        bad            = fma_f32x2(d, make_float2(0.0f, 0.0f), bad);
        b[2 * j]       = __float_as_uint(t.x);
        b[2 * j + 1]   = __float_as_uint(t.y);
    }
    // NaN input, or a scale so small that r = 1 / s is infinite (inf * 0 = NaN): the IEEE divide and cvt give the
    // reference's bytes (NaN -> 0, saturation) where the integer trick would leave NaN bits in the byte
    if (dmax > 0.5f - 6.1e-5f || !(bad.x + bad.y == 0.0f)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            b[2 * j]     = (uint32_t)f32_to_s8(v[j].x / s);
            b[2 * j + 1] = (uint32_t)f32_to_s8(v[j].y / s);
        }
    }
    w0 = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
    w1 = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
}

__device__ __forceinline__ void quant8_s8(const float2* v, float s, float r, uint32_t& w0, uint32_t& w1)
{
    const float  magic = 12582912.0f;
    const float2 mg    = make_float2(magic, magic);
    const float2 r2    = make_float2(r, r);
    const float2 m1    = make_float2(-1.0f, -1.0f);
    uint32_t     b[8];
    bool         redo = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t  = fma_f32x2(v[j], r2, mg);
        const float2 tc = make_float2(fminf(fmaxf(t.x, magic - 128.0f), magic + 127.0f),
                                      fminf(fmaxf(t.y, magic - 128.0f), magic + 127.0f));
        const float2 d  = fma_f32x2(v[j], r2, fma_f32x2(tc, m1, mg));
        redo |= !(fabsf(fabsf(d.x) - 0.5f) >= 6.1e-5f);
        redo |= !(fabsf(fabsf(d.y) - 0.5f) >= 6.1e-5f);
        b[2 * j]     = __float_as_uint(tc.x);
        b[2 * j + 1] = __float_as_uint(tc.y);
    }
    if (redo) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            b[2 * j]     = (uint32_t)f32_to_s8(v[j].x / s);
            b[2 * j + 1] = (uint32_t)f32_to_s8(v[j].y / s);
        }
    }
    w0 = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
    w1 = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
}

// INT4 group-of-64 quantize, the part 8 consecutive lanes do together: each lane holds 8 consecutive values v of the group
// (already divided by the smoothing vector), the group maximum is formed with xor-shuffles over the 8 lanes, s = amax / 7,
// q = sat_s4(rne(fl(v / s))).  Returns the lane's 8 nibbles (element j at bits 4 j) and s.  All 32 lanes of the warp call it.
__device__ __forceinline__ uint32_t int4_g64_quantize8(const float (&v)[8], float& s_out)
{
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        amax = fmaxf(amax, fabsf(v[j]));
    }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
    }
    const float s = amax / 7.0f;
    uint32_t    w = 0;
    if (s > 0.0f && s <= 3.0e38f) {
        // q = rne(fl(v / s)) without a division or a conversion per element: |v / s| <= 7 (1 + 2^-23), so the exact
        // int8 form applies (reciprocal multiply, magic-number rounding, tie check with the IEEE divide as its
        // fallback); the nibbles are the low halves of its eight bytes
        const float2 vp[4] = {make_float2(v[0], v[1]), make_float2(v[2], v[3]), make_float2(v[4], v[5]), make_float2(v[6], v[7])};
        uint32_t     w0, w1;
        quant8_s8_inrange(vp, s, 1.0f / s, w0, w1);
        w0 &= 0x0F0F0F0Fu;
        w1 &= 0x0F0F0F0Fu;
        w = __byte_perm(w0 | (w0 >> 4), w1 | (w1 >> 4), 0x6420);
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int qi;
            // v/s with s == 0 is NaN (or inf); cvt.rni.s32.f32 maps NaN to 0 exactly as the reference's does.
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(qi) : "f"(v[j] / s));
            qi = max(-8, min(7, qi));
            w |= (uint32_t)(qi & 0xf) << (4 * j);
        }
    }
    s_out = s;
    return w;
}

// ---------------------------------------------------------------------------------------------
// Host-side checks.
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The last CUDA error any entry point saw (process-wide), readable through lyraq_last_cuda_error().
void record_cuda_error(cudaError_t e, const char* where);

inline int cuda_status(cudaError_t e, const char* where = "cuda call")
{
    if (e == cudaSuccess) {
        return LYRAQ_OK;
    }
    record_cuda_error(e, where);
    return LYRAQ_ERR_CUDA;
}

inline int launch_status() { return cuda_status(cudaGetLastError(), "kernel launch"); }

// Raises a kernel's dynamic shared-memory limit the first time its call site launches it on the current device: the
// attribute stays with the function on that device, so launches after the first skip the driver call.  `done` is the call
// site's own per-device record.
template<typename Kern> inline int raise_dynamic_smem_once(Kern kern, int bytes, bool (&done)[64], const char* what)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return LYRAQ_ERR_CUDA;
    }
    if (!done[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) {
            return cuda_status(e, what);
        }
        done[dev] = true;
    }
    return LYRAQ_OK;
}

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the library tells the scheduler at its start that the next kernel
// of the stream may begin launching (grid_launch_dependents), and waits for the kernels before it to have completed,
// with their writes visible, before its first access to global memory (grid_dependency_wait).  A kernel's set-up
// (barrier initialisation, tensor-memory allocation, descriptor prefetch) and its launch latency then overlap the
// tail of its predecessor instead of following it.  Both instructions do nothing when the launch carries no such
// dependency.  lyraq_debug_set_dependent_launch(0) turns the launch attribute off.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool dependent_launch_enabled();  // api.cu

template<typename Kernel, typename... Args>
inline cudaError_t launch_kernel(Kernel kernel, unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                                 unsigned cluster_x, Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3(grid, 1, 1);
    cfg.blockDim         = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[2];
    unsigned            n = 0;
    if (cluster_x > 1) {
        attr[n].id               = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    if (dependent_launch_enabled()) {
        attr[n].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs    = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace lyraq
