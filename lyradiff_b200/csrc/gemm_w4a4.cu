// W4A4 GEMM, groups of 64 along K, for sm_100a.
//
//   D[m,n] = T( epi( sum_g (float(sum_{k in g} a[m,k]*b[n,k]) * sa[m,g]) * sb[n,g] + bias[n] ) + R[m,n] )
//
// Blackwell's tensor cores have no 4-bit integer MMA, so the packed nibbles are expanded to signed
// bytes in shared memory and multiplied with tcgen05.mma kind::i8.  The expansion keeps each nibble in
// the HIGH four bits of its byte (value * 16): that needs one AND (odd elements) or one shift + AND
// (even elements) per four values and no sign fix-up; the factor 16 * 16 = 256 on every integer dot
// product is an exact power of two and is folded into the activation scale (sa / 256), so the fp32
// result is bit-identical.  Even and odd elements of a 32-nibble chunk land in two separate 16-byte
// pieces; A and B use the same permutation, so dot products are unchanged and a group of 64 still
// occupies exactly 64 consecutive bytes (two K = 32 MMA steps).
//
// Each group's int32 partial must be rescaled in fp32 before the next group is added, so the
// accumulator leaves tensor memory once per group: four partial buffers (128 columns each) form two
// pairs, the two groups of a K block go into one pair behind one commit while the drain works on the
// other, and eight drain warps convert / scale / accumulate in registers.  That CUDA-core work and the
// hand-offs around it, not the tensor pipe, bound this kernel.
//
// 512 threads per CTA (sixteen warps, four per scheduler, hence at most 128 registers per thread), one persistent
// CTA per SM:
//   warp 0       TMA producer: packed A (128 x 64 B) and packed B (128 x 64 B) tiles, ring of 4 stages
//   warp 1       MMA issuer: both groups of a K block, one commit (warp 15 has no role)
//   warp 2       scale loader: every four K blocks (8 groups) it transposes sa[m, g] and sb[n, g] of the tile into
//                shared memory as [g][row] (ring of 3 slots), running ahead of the drain; also owns tensor memory
//   warps 3, 12-14  expand nibbles -> swizzled int8 operand tiles (ring of 4 stages)
//   warps 4-11   drain: warp w reads TMEM lanes 32*(w%4).., columns 64*((w-4)/4)..; final epilogue
// The optional low-rank branch (D += T(act)[m, 32] * up[n, 32]^T, the reference's lora_up_gemm, w4a4_gemm.cu:515-663,
// with the fp32 -> T conversion of act that W4A4Gemm.cc:143 runs as a separate kernel folded in) rides the same
// pipeline as one more K block per tile: the expansion warps convert / copy the two 32-wide operands into an operand
// stage, the MMA warp issues two kind::f16 steps into the next partial buffer, and the drain warps add that fp32
// partial to their accumulators after the last group, as the reference does.
// All waits are bounded (see sm100_ptx.cuh); a timeout sets the status word and every role exits.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

using namespace sm100;

// defined in gemm_dense.cu
int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t row_stride_bytes,
                       uint32_t box_rows, uint32_t box_bytes, bool swizzle128);
int device_sm_count();

namespace w4 {


constexpr int kBM          = 128;
constexpr int kBN          = 128;
constexpr int kKBlock      = 128;            // K elements per block = 2 groups
constexpr int kPackedRowB  = kKBlock / 2;    // 64 bytes
constexpr int kThreads     = 512;
constexpr int kExpandWarps = 4;
constexpr int kPStages     = 4;
constexpr int kUStages     = 4;
constexpr int kPBufs       = 4;              // partial accumulator buffers in tensor memory
constexpr int kSSlots      = 3;              // scale ring
constexpr int kSlotGroups  = 8;              // groups per scale slot = 4 K blocks
constexpr int kPackedTile  = kBM * kPackedRowB;   // 8 KB (A) ; B the same with kBN rows
constexpr int kPackedStage = 2 * kPackedTile;     // 16 KB
constexpr int kOperandTile = kBM * kKBlock;       // 16 KB
constexpr int kUStage      = 2 * kOperandTile;    // 32 KB
constexpr int kScaleSlot   = kSlotGroups * (kBM + kBN) * 4;  // 8 KB: sas[8][128] then sbs[8][128], fp32
constexpr int kScaleOffset = kPStages * kPackedStage + kUStages * kUStage;
constexpr int kBarOffset   = kScaleOffset + kSSlots * kScaleSlot;
constexpr int kSmemTotal   = kBarOffset + 512 + 1024;

struct Params {
    int           M, N, K, G;  // G = K / 64
    int           m_tiles, n_tiles;
    const float*  sa;
    const void*   sb;
    int           sb_is_f16;
    int           scale_vec_ok;  // G % 4 == 0 and 16-byte aligned scale arrays: 16-byte scale loads are legal
    void*         D;
    int           c_dtype;
    const void*   bias;
    const void*   residual;
    int           gelu;
    int           round_each;    // round to D's type after every epilogue step (the reference's separate 16-bit kernels)
    const void*   lora_act;      // [M, 32], fp32 or already of D's 16-bit type, or null
    int           lora_act_is_f32;
    const void*   lora_up;       // [N, 32] of D's 16-bit type or null
    unsigned int* status;
};

constexpr int kLoraRank = 32;

template<typename T>
__device__ __forceinline__ void final_store32(const Params& p, const float* acc, int row, int col0, int valid, bool vec_ok)
{
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = acc[i];
    }
    const bool each = p.round_each != 0 && sizeof(T) == 2;
    auto round_all = [&]() {
        if (each) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = to_f32(from_f32<T>(v[i]));
            }
        }
    };
    round_all();
    if (p.bias != nullptr) {
        const T* b = reinterpret_cast<const T*>(p.bias) + col0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < valid) {
                v[i] += to_f32(b[i]);
            }
        }
        round_all();
    }
    if (p.gelu) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            v[i] = gelu_tanh_f32(v[i]);
        }
        round_all();
    }
    T* drow = reinterpret_cast<T*>(p.D) + (size_t)row * p.N + col0;
    if (p.residual != nullptr) {
        const T* r = reinterpret_cast<const T*>(p.residual) + (size_t)row * p.N + col0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < valid) {
                v[i] += to_f32(r[i]);
            }
        }
    }
    if (vec_ok && valid >= 32) {
        if (sizeof(T) == 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float tmp[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    tmp[j] = v[8 * i + j];
                }
                Vec16 w;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    T lo = from_f32<T>(tmp[2 * j]);
                    T hi = from_f32<T>(tmp[2 * j + 1]);
                    w.w[j] = (uint32_t)(*reinterpret_cast<uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&hi)) << 16);
                }
                st_16(drow + 8 * i, w);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                Vec16 w;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    w.w[j] = __float_as_uint(v[4 * i + j]);
                }
                st_16(drow + 4 * i, w);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < valid) {
                drow[i] = from_f32<T>(v[i]);
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_w4a4_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const Params p)
{
    constexpr uint32_t kTmemCols = kPBufs * kBN;  // 512
    constexpr uint32_t kIdesc    = umma_idesc(2u, 1u, kBM, kBN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t*       gen_base  = smem_raw + (smem_base - smem_u32(smem_raw));
    // [packed ring][operand ring: A int8 | B int8][scale ring][barriers]
    const uint32_t packed0 = smem_base;
    const uint32_t ustage0 = smem_base + kPStages * kPackedStage;
    const uint32_t bars    = smem_base + kBarOffset;
    auto full_p     = [&](int s) { return bars + 8u * s; };
    auto empty_p    = [&](int s) { return bars + 8u * (kPStages + s); };
    auto full_u     = [&](int s) { return bars + 8u * (2 * kPStages + s); };
    auto empty_u    = [&](int s) { return bars + 8u * (2 * kPStages + kUStages + s); };
    auto part_full  = [&](int b) { return bars + 8u * (2 * kPStages + 2 * kUStages + b); };
    auto part_empty = [&](int b) { return bars + 8u * (2 * kPStages + 2 * kUStages + kPBufs + b); };
    auto sc_full    = [&](int s) { return bars + 8u * (2 * kPStages + 2 * kUStages + 2 * kPBufs + s); };
    auto sc_empty   = [&](int s) { return bars + 8u * (2 * kPStages + 2 * kUStages + 2 * kPBufs + kSSlots + s); };
    constexpr int kNumBars   = 2 * kPStages + 2 * kUStages + 2 * kPBufs + 2 * kSSlots;
    uint32_t*     tmem_slot  = reinterpret_cast<uint32_t*>(gen_base + kBarOffset + 8 * kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(full_p(s), 1);
            mbar_init(empty_p(s), kExpandWarps);
        }
        for (int s = 0; s < kUStages; ++s) {
            mbar_init(full_u(s), kExpandWarps);
            mbar_init(empty_u(s), 1);   // the issuer's commit
        }
        for (int b = 0; b < kPBufs; ++b) {
            mbar_init(part_full(b), 1);
            mbar_init(part_empty(b), 8);
        }
        for (int s = 0; s < kSSlots; ++s) {
            mbar_init(sc_full(s), 1);
            mbar_init(sc_empty(s), 8);  // eight drain warps
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();

    const int num_tiles = p.m_tiles * p.n_tiles;
    const int num_kb    = (p.K + kKBlock - 1) / kKBlock;
    const int num_slots = (num_kb + 3) / 4;  // scale slots per tile

    if (warp == 0) {
        if (lane == 0) {
            // -------------------------------------------------------------- TMA producer
            int      stage = 0, issued = 0;
            uint32_t phase = 0;
            bool     ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int m_blk = tile % p.m_tiles;
                const int n_blk = tile / p.m_tiles;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty_p(stage), phase ^ 1u, abort_flag)) {
                        report_timeout(p.status, 0x1100u | (unsigned)stage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t dst = packed0 + stage * kPackedStage;
                    {
                        mbar_arrive_expect_tx(full_p(stage), (uint32_t)kPackedStage);
                        tma_load_2d(dst, &tmap_a, full_p(stage), kb * kPackedRowB, m_blk * kBM);
                        tma_load_2d(dst + kPackedTile, &tmap_b, full_p(stage), kb * kPackedRowB, n_blk * kBN);
                    }
                    ++issued;
                    if (++stage == kPStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            int      s  = stage;
            uint32_t ph = phase;
            for (int i = 0; i < kPStages && i < issued; ++i) {
                if (s == 0) {
                    s = kPStages;
                    ph ^= 1u;
                }
                --s;
                const uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(full_p(s), ph)) {
                    if (global_timer_ns() - t0 > kWaitLimitNs) {
                        report_timeout(p.status, 0x1500u | (unsigned)s);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // -------------------------------------------------------------- MMA issuer
            // One hand-off per K block, not per group: both groups of a block go into the two partial buffers of a pair
            // (pairs alternate between blocks) behind one commit, and the drain warps wait once for both.  A hand-off through
            // an mbarrier costs each side a couple of hundred cycles, a group is 128 cycles of tensor work.
            int       ustage = 0;
            uint32_t  uphase = 0;
            uint32_t  n      = 0;  // K-block steps issued
            bool      ok     = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int steps = num_kb + (p.lora_act != nullptr ? 1 : 0);  // the low-rank product is one more step
                for (int kb = 0; ok && kb < steps; ++kb) {
                    if (!mbar_wait(full_u(ustage), uphase, abort_flag)) {
                        report_timeout(p.status, 0x1200u | (unsigned)ustage);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const int q = (int)(n & 1u);
                    if (!mbar_wait(part_empty(q), ((n >> 1) & 1u) ^ 1u, abort_flag)) {
                        report_timeout(p.status, 0x1300u | (unsigned)q);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const bool     lora_step = (kb == num_kb);
                    const int      groups    = lora_step ? 1 : min(2, p.G - 2 * kb);
                    const uint32_t a_addr    = ustage0 + ustage * kUStage;
                    const uint64_t adesc     = umma_desc_k_sw128(a_addr);
                    const uint64_t bdesc     = umma_desc_k_sw128(a_addr + kOperandTile);
                    if (lora_step) {
                        // two K = 16 MMAs on 16-bit operands: the fp32 low-rank product
                        const uint32_t idesc = umma_idesc(1u, p.c_dtype == LYRAQ_BF16 ? 1u : 0u, kBM, kBN);
#pragma unroll
                        for (int k = 0; k < kLoraRank / 16; ++k) {
                            mma_f16(tmem_base + (uint32_t)(2 * q * kBN), adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (uint32_t)k);
                        }
                    } else {
                        for (int g = 0; g < groups; ++g) {
                            const uint32_t d_tmem = tmem_base + (uint32_t)((2 * q + g) * kBN);
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const uint64_t koff = (uint64_t)((g * 2 + k) * 2);  // 32-byte K steps, in 16-byte units
                                mma_i8(d_tmem, adesc + koff, bdesc + koff, kIdesc, (uint32_t)k);
                            }
                        }
                    }
                    tc_commit(part_full(q));
                    ++n;
                    tc_commit(empty_u(ustage));
                    if (++ustage == kUStages) {
                        ustage = 0;
                        uphase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ scale loader
        int      slot = 0;
        uint32_t sphase = 0;
        bool     ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int m_blk = tile % p.m_tiles;
            const int n_blk = tile / p.m_tiles;
            for (int sl = 0; sl < num_slots; ++sl) {
                if (!__all_sync(0xffffffffu, mbar_wait(sc_empty(slot), sphase ^ 1u, abort_flag))) {
                    if (lane == 0) {
                        report_timeout(p.status, 0x1800u | (unsigned)slot);
                    }
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                float*     sas  = reinterpret_cast<float*>(gen_base + kScaleOffset + slot * kScaleSlot);
                float*     sbs  = sas + kSlotGroups * kBM;
                const int  g0   = sl * kSlotGroups;
                const bool full = p.scale_vec_ok && (g0 + kSlotGroups <= p.G);
                float      va[4][8], vb[4][8];
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {
                    const int    r    = lane + 32 * rr;
                    const int    grow = m_blk * kBM + r;
                    const int    gcol = n_blk * kBN + r;
                    const float* pa   = p.sa + (size_t)grow * p.G + g0;
                    if (full && grow < p.M) {
                        const float4 x0 = ld_f32x4(reinterpret_cast<const float4*>(pa));
                        const float4 x1 = ld_f32x4(reinterpret_cast<const float4*>(pa) + 1);
                        va[rr][0] = x0.x; va[rr][1] = x0.y; va[rr][2] = x0.z; va[rr][3] = x0.w;
                        va[rr][4] = x1.x; va[rr][5] = x1.y; va[rr][6] = x1.z; va[rr][7] = x1.w;
                    } else {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            va[rr][g] = (grow < p.M && g0 + g < p.G) ? ld_f32(pa + g) : 0.0f;
                        }
                    }
                    if (p.sb_is_f16) {
                        const __half* pb = reinterpret_cast<const __half*>(p.sb) + (size_t)gcol * p.G + g0;
                        if (full && gcol < p.N) {
                            float tmp[8];
                            unpack8<__half>(ld_nc_16(pb), tmp);
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                vb[rr][g] = tmp[g];
                            }
                        } else {
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                vb[rr][g] = (gcol < p.N && g0 + g < p.G) ? __half2float(pb[g]) : 0.0f;
                            }
                        }
                    } else {
                        const float* pb = reinterpret_cast<const float*>(p.sb) + (size_t)gcol * p.G + g0;
                        if (full && gcol < p.N) {
                            const float4 x0 = ld_f32x4(reinterpret_cast<const float4*>(pb));
                            const float4 x1 = ld_f32x4(reinterpret_cast<const float4*>(pb) + 1);
                            vb[rr][0] = x0.x; vb[rr][1] = x0.y; vb[rr][2] = x0.z; vb[rr][3] = x0.w;
                            vb[rr][4] = x1.x; vb[rr][5] = x1.y; vb[rr][6] = x1.z; vb[rr][7] = x1.w;
                        } else {
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                vb[rr][g] = (gcol < p.N && g0 + g < p.G) ? ld_f32(pb + g) : 0.0f;
                            }
                        }
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; ++rr) {
                    const int r = lane + 32 * rr;
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        sas[g * kBM + r] = va[rr][g] * (1.0f / 256.0f);  // the 16 * 16 of the nibble expansion, exactly
                        sbs[g * kBN + r] = vb[rr][g];
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sc_full(slot));
                }
                if (++slot == kSSlots) {
                    slot = 0;
                    sphase ^= 1u;
                }
            }
        }
    } else if (warp == 3 || (warp >= 12 && warp <= 14)) {
        // ------------------------------------------------------------------ nibble expansion
        // 2 tiles x 128 rows x 4 packed 16-byte chunks = 1024 tasks over 128 threads; thread tu owns chunk (tu & 3) of
        // rows (tu >> 2) + 32 * it, it = 0..7 (it < 4: A, it >= 4: B), so every address is a base plus it * constant.
        const int tu     = (warp == 3 ? 0 : (warp - 11) * 32) + lane;  // 0..127
        const int c      = tu & 3;
        const int r0     = tu >> 2;       // 0..31
        const int sw     = r0 & 7;        // (r0 + 32 * it) & 7 == r0 & 7
        const int src_o  = r0 * kPackedRowB + c * 16;
        const int dst_ev = (r0 >> 3) * 1024 + (r0 & 7) * 128 + (((2 * c) ^ sw) << 4);
        const int dst_od = (r0 >> 3) * 1024 + (r0 & 7) * 128 + (((2 * c + 1) ^ sw) << 4);
        int       pstage = 0, ustage = 0;
        uint32_t  pphase = 0, uphase = 0;
        bool      ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            for (int kb = 0; kb < num_kb; ++kb) {
                bool w = mbar_wait(full_p(pstage), pphase, abort_flag);
                w      = w && mbar_wait(empty_u(ustage), uphase ^ 1u, abort_flag);
                if (!__all_sync(0xffffffffu, w)) {
                    if (lane == 0) {
                        report_timeout(p.status, 0x1400u | (unsigned)(pstage * 16 + ustage));
                    }
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint8_t* src = gen_base + (packed0 - smem_base) + pstage * kPackedStage + src_o;
                uint8_t*       dst = gen_base + (ustage0 - smem_base) + ustage * kUStage;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    // 32 rows further per step: 32 * 64 B in the packed tile, 4 * 1024 B in the operand tile;
                    // it >= 4 switches to the B tile (its packed and operand tiles follow A's contiguously)
                    const uint4 w4 = *reinterpret_cast<const uint4*>(src + it * 32 * kPackedRowB);
                    uint4       ev, od;
                    ev.x = (w4.x << 4) & 0xF0F0F0F0u; od.x = w4.x & 0xF0F0F0F0u;
                    ev.y = (w4.y << 4) & 0xF0F0F0F0u; od.y = w4.y & 0xF0F0F0F0u;
                    ev.z = (w4.z << 4) & 0xF0F0F0F0u; od.z = w4.z & 0xF0F0F0F0u;
                    ev.w = (w4.w << 4) & 0xF0F0F0F0u; od.w = w4.w & 0xF0F0F0F0u;
                    *reinterpret_cast<uint4*>(dst + it * 4096 + dst_ev) = ev;
                    *reinterpret_cast<uint4*>(dst + it * 4096 + dst_od) = od;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_u(ustage));
                    mbar_arrive(empty_p(pstage));
                }
                if (++pstage == kPStages) {
                    pstage = 0;
                    pphase ^= 1u;
                }
                if (++ustage == kUStages) {
                    ustage = 0;
                    uphase ^= 1u;
                }
            }
            if (ok && p.lora_act != nullptr) {
                // low-rank operands: row tu of T(act) and of up, 64 bytes each, into the first four (swizzled) 16-byte
                // pieces of the row's 128-byte line; the other four pieces are never read by the two K = 16 steps
                if (!__all_sync(0xffffffffu, mbar_wait(empty_u(ustage), uphase ^ 1u, abort_flag))) {
                    if (lane == 0) {
                        report_timeout(p.status, 0x1a00u | (unsigned)ustage);
                    }
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const int m_blk = tile % p.m_tiles;
                const int n_blk = tile / p.m_tiles;
                uint8_t*  dst   = gen_base + (ustage0 - smem_base) + ustage * kUStage + (tu >> 3) * 1024 + (tu & 7) * 128;
                const int arow  = m_blk * kBM + tu;
                const int brow  = n_blk * kBN + tu;
                const int swz   = tu & 7;
                const float4* asrc = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.lora_act) + (size_t)arow * kLoraRank);
                const uint4*  a16  = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.lora_act) + (size_t)arow * kLoraRank);
                const uint4*  bsrc = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.lora_up) + (size_t)brow * kLoraRank);
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx) {
                    uint4 av = make_uint4(0u, 0u, 0u, 0u), bv = make_uint4(0u, 0u, 0u, 0u);
                    if (arow < p.M && !p.lora_act_is_f32) {
                        av = ld_u32x4(a16 + cidx);
                    } else if (arow < p.M) {
                        const float4 f0 = ld_f32x4(asrc + 2 * cidx), f1 = ld_f32x4(asrc + 2 * cidx + 1);
                        if (p.c_dtype == LYRAQ_BF16) {
                            av.x = Pair<__nv_bfloat16>::from_f32(f0.x, f0.y); av.y = Pair<__nv_bfloat16>::from_f32(f0.z, f0.w);
                            av.z = Pair<__nv_bfloat16>::from_f32(f1.x, f1.y); av.w = Pair<__nv_bfloat16>::from_f32(f1.z, f1.w);
                        } else {
                            av.x = Pair<__half>::from_f32(f0.x, f0.y); av.y = Pair<__half>::from_f32(f0.z, f0.w);
                            av.z = Pair<__half>::from_f32(f1.x, f1.y); av.w = Pair<__half>::from_f32(f1.z, f1.w);
                        }
                    }
                    if (brow < p.N) {
                        bv = ld_u32x4(bsrc + cidx);
                    }
                    *reinterpret_cast<uint4*>(dst + ((cidx ^ swz) << 4))                = av;
                    *reinterpret_cast<uint4*>(dst + kOperandTile + ((cidx ^ swz) << 4)) = bv;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(full_u(ustage));
                }
                if (++ustage == kUStages) {
                    ustage = 0;
                    uphase ^= 1u;
                }
            }
        }
    } else if (warp >= 4 && warp <= 11) {
        // ------------------------------------------------------------------ drain + epilogue (warps 4..11)
        const int      quad      = warp & 3;
        const int      half      = (warp - 4) >> 2;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const int      trow      = quad * 32 + lane;
        const bool     vec_ok    = (p.c_dtype == LYRAQ_F32) ? ((p.N & 3) == 0) : ((p.N & 7) == 0);
        int            slot = 0;
        uint32_t       sphase = 0;
        uint32_t       n = 0;  // K-block steps drained (step s uses the partial buffers 2 (s & 1) and 2 (s & 1) + 1)
        bool           ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int m_blk = tile % p.m_tiles;
            const int n_blk = tile / p.m_tiles;
            float2    acc[32];  // 64 columns of this thread's row, as packed pairs
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                acc[i] = make_float2(0.0f, 0.0f);
            }
            for (int kb = 0; ok && kb < num_kb; ++kb) {
                if ((kb & 3) == 0) {
                    const bool got_s = mbar_wait(sc_full(slot), sphase, abort_flag);
                    if (!__all_sync(0xffffffffu, got_s)) {
                        if (lane == 0) {
                            report_timeout(p.status, 0x1600u | (unsigned)slot);
                        }
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                }
                const float* sas    = reinterpret_cast<const float*>(gen_base + kScaleOffset + slot * kScaleSlot);
                const float* sbs    = sas + kSlotGroups * kBM;
                const int    groups = min(2, p.G - 2 * kb);
                const int    q      = (int)(n & 1u);
                const bool   got_p  = mbar_wait(part_full(q), (n >> 1) & 1u, abort_flag);
                ++n;
                if (!__all_sync(0xffffffffu, got_p)) {
                    if (lane == 0) {
                        report_timeout(p.status, 0x1700u | (unsigned)q);
                    }
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
#pragma unroll 1
                for (int g = 0; g < groups; ++g) {
                    const int pb = 2 * q + g;
                    const int gs = (kb & 3) * 2 + g;  // group index inside the scale slot
                    const float  sa_s = sas[gs * kBM + trow];
                    const float2 sa_v = make_float2(sa_s, sa_s);
                    const uint32_t t_addr = tmem_base + lane_addr + (uint32_t)(pb * kBN + half * 64);
                    // the load of chunk c + 1 is in flight while chunk c is rescaled
                    uint32_t pcs[2][16];
                    tmem_ld_32x16(t_addr, pcs[0]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld_wait();
                        if (c + 1 < 4) {
                            tmem_ld_32x16(t_addr + (uint32_t)((c + 1) * 16), pcs[(c + 1) & 1]);
                        }
                        const uint32_t* pc  = pcs[c & 1];
                        const float4*   sb4 = reinterpret_cast<const float4*>(sbs + gs * kBN + half * 64 + c * 16);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 s = sb4[j];
                            // acc = fma(float(p) * sa, sb, acc): the contraction the reference's compiler makes of
                            // `acc += float(p) * sa * sb` (w4a4_gemm.cu:504-507); two columns per instruction
                            const float2 p0 = make_float2((float)(int)pc[4 * j], (float)(int)pc[4 * j + 1]);
                            const float2 p1 = make_float2((float)(int)pc[4 * j + 2], (float)(int)pc[4 * j + 3]);
                            acc[c * 8 + 2 * j]     = fma_f32x2(mul_f32x2(p0, sa_v), make_float2(s.x, s.y), acc[c * 8 + 2 * j]);
                            acc[c * 8 + 2 * j + 1] = fma_f32x2(mul_f32x2(p1, sa_v), make_float2(s.z, s.w), acc[c * 8 + 2 * j + 1]);
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(part_empty(q));
                }
                if (ok && ((kb & 3) == 3 || kb == num_kb - 1)) {
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(sc_empty(slot));
                    }
                    if (++slot == kSSlots) {
                        slot = 0;
                        sphase ^= 1u;
                    }
                }
            }
            if (ok && p.lora_act != nullptr) {
                const int q  = (int)(n & 1u);
                const int pb = 2 * q;
                if (!__all_sync(0xffffffffu, mbar_wait(part_full(q), (n >> 1) & 1u, abort_flag))) {
                    if (lane == 0) {
                        report_timeout(p.status, 0x1b00u | (unsigned)pb);
                    }
                    *abort_flag = 1;
                    ok = false;
                } else {
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t part[16];
                        tmem_ld_32x16(tmem_base + lane_addr + (uint32_t)(pb * kBN + half * 64 + c * 16), part);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            acc[c * 8 + j] = add_f32x2(acc[c * 8 + j], make_float2(__uint_as_float(part[2 * j]), __uint_as_float(part[2 * j + 1])));
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(part_empty(q));
                    }
                    ++n;
                }
            }
            if (!ok) {
                break;
            }
            const int row = m_blk * kBM + trow;
            if (row < p.M) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int col0  = n_blk * kBN + half * 64 + c * 32;
                    const int valid = p.N - col0;
                    if (valid > 0) {
                        if (p.c_dtype == LYRAQ_BF16) {
                            final_store32<__nv_bfloat16>(p, reinterpret_cast<const float*>(acc) + c * 32, row, col0, valid, vec_ok);
                        } else if (p.c_dtype == LYRAQ_F16) {
                            final_store32<__half>(p, reinterpret_cast<const float*>(acc) + c * 32, row, col0, valid, vec_ok);
                        } else {
                            final_store32<float>(p, reinterpret_cast<const float*>(acc) + c * 32, row, col0, valid, vec_ok);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace w4
}  // namespace lyraq

using namespace lyraq;


extern "C" int lyraq_gemm_w4a4(const uint8_t* A, const uint8_t* B, const float* sa, const void* sb, int sb_dtype, void* D,
                               int c_dtype, const void* lora_act, int lora_act_dtype, const void* lora_up, const void* bias,
                               const void* residual, int epilogue, int m, int n, int k, void* workspace,
                               size_t workspace_bytes, void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if (m == 0 || n == 0) {
        return LYRAQ_OK;
    }
    if (A == nullptr || B == nullptr || sa == nullptr || sb == nullptr || D == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (c_dtype < LYRAQ_F16 || c_dtype > LYRAQ_F32 || (sb_dtype != LYRAQ_F32 && sb_dtype != LYRAQ_F16) ||
        (epilogue & ~(LYRAQ_EPI_GELU_TANH | LYRAQ_EPI_ROUND_EACH)) != 0 || m < 0 || n < 0 || k < 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((lora_act == nullptr) != (lora_up == nullptr)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (lora_act != nullptr) {
        if (c_dtype == LYRAQ_F32) {
            return LYRAQ_ERR_UNSUPPORTED;  // lora_up has D's type, which must be a 16-bit one
        }
        if (lora_act_dtype != LYRAQ_F32 && lora_act_dtype != c_dtype) {
            return LYRAQ_ERR_INVALID_ARG;
        }
        if (!aligned16(lora_act) || !aligned16(lora_up)) {
            return LYRAQ_ERR_INVALID_ARG;
        }
    }
    if (k == 0 || (k & 63) != 0) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (!aligned16(A) || !aligned16(B) || !aligned16(D) || (residual != nullptr && !aligned16(residual))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    w4::Params p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.G = k / 64;
    p.m_tiles   = (m + w4::kBM - 1) / w4::kBM;
    p.n_tiles   = (n + w4::kBN - 1) / w4::kBN;
    p.sa        = sa;
    p.sb        = sb;
    p.sb_is_f16 = (sb_dtype == LYRAQ_F16) ? 1 : 0;
    p.scale_vec_ok = ((p.G & 7) == 0 || ((p.G & 3) == 0 && sb_dtype == LYRAQ_F32)) && aligned16(sa) && aligned16(sb) ? 1 : 0;
    p.D         = D;
    p.c_dtype   = c_dtype;
    p.bias      = bias;
    p.residual  = residual;
    p.gelu      = (epilogue & LYRAQ_EPI_GELU_TANH) ? 1 : 0;
    p.round_each = (epilogue & LYRAQ_EPI_ROUND_EACH) ? 1 : 0;
    p.lora_act  = lora_act;
    p.lora_act_is_f32 = (lora_act_dtype == LYRAQ_F32) ? 1 : 0;
    p.lora_up   = lora_up;
    p.status    = status_word_ptr();
    if (p.status == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    const int sms = device_sm_count();
    if (sms <= 0) {
        return LYRAQ_ERR_CUDA;
    }
    CUtensorMap ta, tb;
    int st = make_tmap_bytes_2d(&ta, A, (uint64_t)m, (uint64_t)k / 2, (uint64_t)k / 2, w4::kBM, w4::kPackedRowB, false);
    if (st != LYRAQ_OK) {
        return st;
    }
    st = make_tmap_bytes_2d(&tb, B, (uint64_t)n, (uint64_t)k / 2, (uint64_t)k / 2, w4::kBN, w4::kPackedRowB, false);
    if (st != LYRAQ_OK) {
        return st;
    }
    const long tiles = (long)p.m_tiles * p.n_tiles;
    const int  grid  = (int)(tiles < sms ? tiles : sms);
    static bool smem_raised[64] = {};
    st = raise_dynamic_smem_once(w4::gemm_w4a4_kernel, (int)w4::kSmemTotal, smem_raised,
                                 "cudaFuncSetAttribute(gemm_w4a4_kernel, dynamic shared memory)");
    if (st != LYRAQ_OK) {
        return st;
    }
    return cuda_status(launch_kernel(w4::gemm_w4a4_kernel, (unsigned)grid, (unsigned)w4::kThreads, (size_t)w4::kSmemTotal,
                                     (cudaStream_t)stream, 1u, ta, tb, p),
                       "cudaLaunchKernelEx(gemm_w4a4_kernel)");
}
