// Low-rank down projection of the W4A4 linear: act[m, 32] = x[m, k] * lora_down[32, k]^T, 16-bit inputs, fp32 out.
//
// The reference computes this inside its int4 quantize kernel with one mma.sync tile per 64 columns and a
// floating-point atomic add per tile (src/lyradiff/kernels/w4a4_gemm/w4a4_gemm.cu:769-954), so the order of the 48
// partial sums changes from run to run.  Here one CTA owns 32 rows of x for the whole of K and accumulates in tensor
// memory in a fixed order, so the result is reproducible and no output has to be zeroed first.
//
// The product is formed transposed, D[r, j] = sum_k lora_down[r, k] * x[row0 + j, k]: tcgen05.mma needs M >= 64, and
// with the 32 rows of x on the N side 4608 tokens give 144 CTAs (one per SM) instead of 36.  The M side is the 32 rows
// of lora_down followed by 96 rows that lie outside the tensor, which TMA fills with zeros without reading memory.
//
//   warp 0   lane 0: TMA producer (x tile 32 x 128 B, lora_down tile 128 x 128 B, ring of 8 stages);
//            afterwards the whole warp reads accumulator lanes 0..31 and stores act
//   warp 1   lane 0: MMA issuer; the warp owns the tensor-memory allocation
//   warps 2-17 (fused form only): the int4 quantize of the same x tiles.  One stage holds, for each of the CTA's 32 rows,
//            exactly one group of 64 values (a 128-byte row of the swizzled tile), so x is read from memory once for
//            both results, as in the reference's fused kernel.  Eight lanes share a group (the arithmetic of
//            int4_g64_kernel, bit for bit), so a warp takes 4 rows and eight warps one stage; the two sets of eight warps
//            alternate over the stages, which keeps enough independent divides in flight to hide their latency.  A stage
//            goes back to the producer when the MMAs that read it and its eight quantizer warps are done.
// All waits are bounded; a timeout sets the status word and the block leaves.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

using namespace sm100;

int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t row_stride_bytes,
                       uint32_t box_rows, uint32_t box_bytes, bool swizzle128);  // gemm_dense.cu

namespace lora {

constexpr int kRank      = 32;
constexpr int kRows      = 32;                    // rows of x per CTA (the MMA's N)
constexpr int kBlockKB   = 128;                   // bytes of K per stage = 64 elements
constexpr int kStages    = 8;
constexpr int kDownTile  = 128 * kBlockKB;        // 16 KB, of which 4 KB come from memory
constexpr int kXTile     = kRows * kBlockKB;      // 4 KB
constexpr int kStage     = kDownTile + kXTile;
constexpr int kBarOffset = kStages * kStage;
constexpr int kSmemTotal = kBarOffset + 256 + 1024;
constexpr int kThreads   = 64;                    // down projection alone
constexpr int kQuantWarps = 16;               // two sets of eight: a set covers the 32 rows of one stage
constexpr int kThreadsFused = kThreads + 32 * kQuantWarps;

struct Params {
    float*        act;   // [m, 32]
    int           m, k;
    int           is_bf16;
    unsigned int* status;
    // fused int4 quantize (all null / 0 for the down projection alone)
    uint32_t*     q;        // [m, k / 8]: eight nibbles per word
    float*        q_scale;  // [m, k / 64]
    const float*  smooth;   // [k] or null
};

template<bool FUSED>
__global__ void __launch_bounds__(FUSED ? kThreadsFused : kThreads, 1)
lora_down_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_down, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t*       gen_base  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars      = smem_base + kBarOffset;
    auto full_bar  = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (kStages + s); };
    const uint32_t done_bar   = bars + 8u * (2 * kStages);
    uint32_t*      tmem_slot  = reinterpret_cast<uint32_t*>(gen_base + kBarOffset + 8 * (2 * kStages + 1));
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), FUSED ? 9 : 1);   // the MMAs' commit, and the stage's eight quantizer warps
        }
        mbar_init(done_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_down);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 32);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();

    const int num_kb = (p.k * 2 + kBlockKB - 1) / kBlockKB;
    const int row0   = blockIdx.x * kRows;

    if (warp == 0) {
        if (lane == 0) {
            int      stage = 0, issued = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    report_timeout(p.status, 0x2100u | (unsigned)stage);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t dst = smem_base + stage * kStage;
                mbar_arrive_expect_tx(full_bar(stage), (uint32_t)kStage);
                tma_load_2d(dst, &tmap_down, full_bar(stage), kb * kBlockKB, 0);
                tma_load_2d(dst + kDownTile, &tmap_x, full_bar(stage), kb * kBlockKB, row0);
                ++issued;
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            // no load may still be in flight when the block leaves: walk back over the last slots that were filled
            int      s  = stage;
            uint32_t ph = phase;
            for (int i = 0; i < kStages && i < issued; ++i) {
                if (s == 0) {
                    s = kStages;
                    ph ^= 1u;
                }
                --s;
                const uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(full_bar(s), ph)) {
                    if (global_timer_ns() - t0 > kWaitLimitNs) {
                        report_timeout(p.status, 0x2400u | (unsigned)s);
                        break;
                    }
                }
            }
        }
        __syncwarp();
        // every load has landed once the last MMA, which waited for it, has completed
        if (__all_sync(0xffffffffu, mbar_wait(done_bar, 0u, abort_flag))) {
            tc_fence_after_sync();
            uint32_t d[32];
            tmem_ld_32x32(tmem_base, d);  // lane r of the warp = rank r; column j = row row0 + j
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < kRows; ++j) {
                if (row0 + j < p.m) {
                    p.act[(size_t)(row0 + j) * kRank + lane] = __uint_as_float(d[j]);
                }
            }
        } else if (lane == 0) {
            report_timeout(p.status, 0x2300u);
        }
    } else if (FUSED && warp >= 2) {
        // ------------------------------------------------------------------ int4 quantize of the staged x tiles
        const int part = lane & 7;                  // which 8 values of the group of 64
        const int sub  = lane >> 3;                 // which of the pass's 4 rows
        bool      ok   = true;
        const int qw  = warp - 2;
        const int r   = (qw & 7) * 4 + sub;      // this lane's row of the tile
        for (int kb = qw >> 3; kb < num_kb && ok; kb += 2) {
            const int      stage = kb % kStages;
            const uint32_t phase = (uint32_t)((kb / kStages) & 1);
            if (!__all_sync(0xffffffffu, mbar_wait(full_bar(stage), phase, abort_flag))) {
                if (lane == 0) {
                    report_timeout(p.status, 0x2500u | (unsigned)stage);
                    *abort_flag = 1;
                }
                ok = false;
                break;
            }
            const uint8_t* xt  = gen_base + stage * kStage + kDownTile;   // 32 rows x 128 B, 128-byte swizzle
            const Vec16    raw = *reinterpret_cast<const Vec16*>(xt + r * 128 + ((part ^ (r & 7)) << 4));
            float          v[8];
            if (p.is_bf16) {
                unpack8<__nv_bfloat16>(raw, v);
            } else {
                unpack8<__half>(raw, v);
            }
            if (p.smooth != nullptr) {
                const float4 s0 = ld_f32x4(reinterpret_cast<const float4*>(p.smooth + kb * 64 + part * 8));
                const float4 s1 = ld_f32x4(reinterpret_cast<const float4*>(p.smooth + kb * 64 + part * 8 + 4));
                v[0] /= s0.x; v[1] /= s0.y; v[2] /= s0.z; v[3] /= s0.w;
                v[4] /= s1.x; v[5] /= s1.y; v[6] /= s1.z; v[7] /= s1.w;
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty_bar(stage));      // the tile is in registers: this warp's share of the stage's release
            }
            float          sc;
            const uint32_t w = int4_g64_quantize8(v, sc);
            if (row0 + r < p.m) {
                p.q[(size_t)(row0 + r) * (size_t)(p.k >> 3) + (size_t)(kb * 8 + part)] = w;
                if (part == 0) {
                    p.q_scale[(size_t)(row0 + r) * (size_t)(p.k >> 6) + (size_t)kb] = sc;
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        int      stage = 0;
        uint32_t phase = 0;
        bool     ok    = true;
        const uint32_t idesc = umma_idesc(1u, p.is_bf16 ? 1u : 0u, 128, kRows);
        for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                report_timeout(p.status, 0x2200u | (unsigned)stage);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after_sync();
            const uint64_t adesc = umma_desc_k_sw128(smem_base + stage * kStage);
            const uint64_t bdesc = umma_desc_k_sw128(smem_base + stage * kStage + kDownTile);
#pragma unroll
            for (int ks = 0; ks < kBlockKB / 32; ++ks) {
                mma_f16(tmem_base, adesc + (uint64_t)(2 * ks), bdesc + (uint64_t)(2 * ks), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
            }
            tc_commit(empty_bar(stage));
            if (++stage == kStages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        if (ok) {
            tc_commit(done_bar);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 32);
    }
}

}  // namespace lora

// act[m, 32] (fp32) = x[m, k] * down[32, k]^T; x and down of the same 16-bit type; k a multiple of 8.  With q != null the
// same launch also writes the int4 group-64 quantization of x / smooth (packed nibbles q [m, k / 2 bytes], fp32 scales
// q_scale [m, k / 64]); k then has to be a multiple of 64.
static int launch_lora_down_impl(float* act, const void* x, const void* down, int dtype, size_t m, size_t k, uint8_t* q, float* q_scale,
                                 const float* smooth, cudaStream_t stream)
{
    if (act == nullptr || x == nullptr || down == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (dtype != LYRAQ_BF16 && dtype != LYRAQ_F16) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (!aligned16(x) || !aligned16(down) || (reinterpret_cast<uintptr_t>(act) & 3u) != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    const bool fused = q != nullptr;
    if (fused && (q_scale == nullptr || (reinterpret_cast<uintptr_t>(q) & 3u) != 0 || (smooth != nullptr && !aligned16(smooth)))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((k & 7) != 0 || k == 0 || k > 0x3fffffffu || m > 0x7fffffffu || (fused && (k & 63) != 0)) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    lora::Params p{};
    p.act     = act;
    p.m       = (int)m;
    p.k       = (int)k;
    p.is_bf16 = (dtype == LYRAQ_BF16) ? 1 : 0;
    p.q       = reinterpret_cast<uint32_t*>(q);
    p.q_scale = q_scale;
    p.smooth  = smooth;
    p.status  = status_word_ptr();
    if (p.status == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    CUtensorMap tx, td;
    int st = make_tmap_bytes_2d(&tx, x, (uint64_t)m, (uint64_t)k * 2, (uint64_t)k * 2, lora::kRows, lora::kBlockKB, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    st = make_tmap_bytes_2d(&td, down, (uint64_t)lora::kRank, (uint64_t)k * 2, (uint64_t)k * 2, 128, lora::kBlockKB, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    const unsigned grid = (unsigned)((m + lora::kRows - 1) / lora::kRows);
    if (fused) {
        static bool smem_raised_fused[64] = {};
        st = raise_dynamic_smem_once(lora::lora_down_kernel<true>, (int)lora::kSmemTotal, smem_raised_fused,
                                     "cudaFuncSetAttribute(lora_down_kernel<fused>, dynamic shared memory)");
        if (st != LYRAQ_OK) {
            return st;
        }
        return cuda_status(launch_kernel(lora::lora_down_kernel<true>, grid, (unsigned)lora::kThreadsFused, (size_t)lora::kSmemTotal,
                                         stream, 1u, tx, td, p),
                           "cudaLaunchKernelEx(lora_down_kernel<fused>)");
    }
    static bool smem_raised[64] = {};
    st = raise_dynamic_smem_once(lora::lora_down_kernel<false>, (int)lora::kSmemTotal, smem_raised,
                                 "cudaFuncSetAttribute(lora_down_kernel, dynamic shared memory)");
    if (st != LYRAQ_OK) {
        return st;
    }
    return cuda_status(launch_kernel(lora::lora_down_kernel<false>, grid, (unsigned)lora::kThreads, (size_t)lora::kSmemTotal, stream, 1u,
                                     tx, td, p),
                       "cudaLaunchKernelEx(lora_down_kernel)");
}

int launch_lora_down(float* act, const void* x, const void* down, int dtype, size_t m, size_t k, cudaStream_t stream)
{
    return launch_lora_down_impl(act, x, down, dtype, m, k, nullptr, nullptr, nullptr, stream);
}

// The reference's fused_quantized_and_lora_down_simple (w4a4_gemm.cu:769-954) as ONE launch over one read of x.
int launch_quant_int4_lora_down(uint8_t* q, float* q_scale, float* act, const void* x, const void* down, const float* smooth, int dtype,
                                size_t m, size_t k, cudaStream_t stream)
{
    if (q == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    return launch_lora_down_impl(act, x, down, dtype, m, k, q, q_scale, smooth, stream);
}

}  // namespace lyraq
