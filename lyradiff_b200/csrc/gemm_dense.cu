// INT8 (kind::i8, s32 accumulators) and FP8 e4m3 (kind::f8f6f4, f32 accumulators) GEMMs for sm_100a.
//
//   Y[M,N] = epilogue( sum_k A[M,k] * B[N,k] ),  A and B both K-contiguous 8-bit.
//
// One persistent CTA per SM, 256 threads, warp-specialised:
//   warp 0   : TMA producer   - streams 128x128-byte A tiles and BLOCK_N x128-byte B tiles into a ring of
//                               shared-memory stages (128-byte swizzle), one mbarrier per stage.
//   warp 1   : MMA issuer     - one thread issues four tcgen05.mma (K = 32 bytes each) per stage into one of
//                               two accumulator buffers in tensor memory, and commits to free the stage.
//   warp 2   : allocates / frees tensor memory.
//   warps 4-7: epilogue       - tcgen05.ld the finished accumulator (warp w reads TMEM lanes 32(w-4)..),
//                               apply dequant scales / bias / GELU / residual in registers, store.
// The two accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on a timeout the role records it in the status word, raises the
// block's abort flag and all roles fall through to the common exit, where tensor memory is freed.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

using namespace sm100;

constexpr int kBlockM     = 128;
constexpr int kBlockK     = 128;  // bytes == elements for 8-bit operands
constexpr int kUmmaK      = 32;
constexpr int kThreads    = 256;
constexpr int kEpiWarp0   = 4;
constexpr int kSmemBudget = 227 * 1024;

enum GemmKind { KIND_I8 = 0, KIND_F8 = 1 };

struct EpilogueParams {
    void*        C;
    int          c_dtype;
    int          ldc;
    // int8: y = T(float(acc) * (col_scale[n] * row_scale)), then T(y + bias)
    const float* col_scale;
    const float* row_scale;
    int          row_scale_per_token;
    // fp8: y = T(epi(acc * (alpha * s_a * s_b) + beta * R + bias))
    const float* s_a;
    const float* s_b;
    float        alpha;
    float        beta;
    const void*  bias;
    const void*  residual;
    int          gelu;
};

struct GemmParams {
    int            M, N, K;
    int            m_tiles, n_tiles;
    unsigned int*  status;
    EpilogueParams epi;
};

template<int BLOCK_N> struct GemmSmem {
    static constexpr int kABytes     = kBlockM * kBlockK;
    static constexpr int kBBytes     = BLOCK_N * kBlockK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages     = (kSmemBudget - 2048) / kStageBytes;  // 4 for BLOCK_N=256, 6 for 128
    static constexpr int kBarBytes   = 256;
    static constexpr int kTotal      = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

// Load 32 values of a T row (or a scalar-predicated tail) to fp32.
template<typename T>
__device__ __forceinline__ void load_row32(const T* p, int valid, bool vec_ok, float* out)
{
    if (vec_ok && valid >= 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unpack8<T>(ld_nc_16(p + 8 * i), out + 8 * i);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            out[i] = (i < valid) ? to_f32(p[i]) : 0.0f;
        }
    }
}
template<>
__device__ __forceinline__ void load_row32<float>(const float* p, int valid, bool vec_ok, float* out)
{
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        out[i] = (i < valid) ? p[i] : 0.0f;
    }
}

template<typename T> __device__ __forceinline__ void store_row32(T* p, int valid, bool vec_ok, const float* v)
{
    if (vec_ok && valid >= 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            st_16(p + 8 * i, pack8<T>(v + 8 * i));
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < valid) {
                p[i] = from_f32<T>(v[i]);
            }
        }
    }
}
template<> __device__ __forceinline__ void store_row32<float>(float* p, int valid, bool vec_ok, const float* v)
{
    if (vec_ok && valid >= 32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            Vec16 w;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w.w[j] = __float_as_uint(v[4 * i + j]);
            }
            st_16(p + 4 * i, w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < valid) {
                p[i] = v[i];
            }
        }
    }
}

// Epilogue for one 32-column chunk of one row.  acc holds raw accumulator bits (s32 or f32).
template<int KIND, typename T>
__device__ __forceinline__ void epilogue_chunk(const EpilogueParams& e, const uint32_t* acc, int row, int col0, int valid,
                                               float row_scale, float fp8_scale, bool vec_ok)
{
    float v[32];
    T*    crow = reinterpret_cast<T*>(e.C) + (size_t)row * e.ldc + col0;
    if (KIND == KIND_I8) {
        float cs[32];
        if (valid >= 32) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 f = __ldg(reinterpret_cast<const float4*>(e.col_scale + col0) + i);
                cs[4 * i] = f.x; cs[4 * i + 1] = f.y; cs[4 * i + 2] = f.z; cs[4 * i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                cs[i] = (i < valid) ? __ldg(e.col_scale + col0 + i) : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            v[i] = round_t<T>((float)(int)acc[i] * (cs[i] * row_scale));
        }
        if (e.bias != nullptr) {
            float b[32];
            load_row32<T>(reinterpret_cast<const T*>(e.bias) + col0, valid, vec_ok, b);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = v[i] + b[i];  // rounded to T by the store: T(T(acc*scale) + bias)
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            v[i] = __uint_as_float(acc[i]) * fp8_scale;
        }
        if (e.residual != nullptr) {
            float r[32];
            load_row32<T>(reinterpret_cast<const T*>(e.residual) + (size_t)row * e.ldc + col0, valid, vec_ok, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = fmaf(e.beta, r[i], v[i]);
            }
        }
        if (e.bias != nullptr) {
            float b[32];
            load_row32<T>(reinterpret_cast<const T*>(e.bias) + col0, valid, vec_ok, b);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] += b[i];
            }
        }
        if (e.gelu) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                v[i] = gelu_tanh_f32(v[i]);
            }
        }
    }
    store_row32<T>(crow, valid, vec_ok, v);
}

template<int KIND, int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p)
{
    using S = GemmSmem<BLOCK_N>;
    constexpr int      kStages   = S::kStages;
    constexpr uint32_t kTmemCols = 2 * BLOCK_N;  // two accumulator buffers (power of two: 256 or 512)
    constexpr uint32_t kIdesc    = (KIND == KIND_I8) ? umma_idesc(2u, 1u, kBlockM, BLOCK_N) : umma_idesc(1u, 0u, kBlockM, BLOCK_N);

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is what the 128-byte swizzle pattern of TMA and UMMA is anchored to.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t smem_a    = smem_base;
    const uint32_t smem_b    = smem_base + kStages * S::kABytes;
    const uint32_t bars      = smem_base + kStages * S::kStageBytes;
    // barrier slots (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    auto full_bar       = [&](int s) { return bars + 8u * s; };
    auto empty_bar      = [&](int s) { return bars + 8u * (kStages + s); };
    auto tmem_full_bar  = [&](int b) { return bars + 8u * (2 * kStages + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * kStages + 2 + b); };
    uint8_t*       gen_base   = smem_raw + (smem_base - smem_u32(smem_raw));
    uint32_t*      tmem_slot  = reinterpret_cast<uint32_t*>(gen_base + kStages * S::kStageBytes + 8 * (2 * kStages + 4));
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 128);
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

    const int num_tiles = p.m_tiles * p.n_tiles;
    const int num_kb    = (p.K + kBlockK - 1) / kBlockK;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ TMA producer
        int      stage = 0;
        uint32_t phase = 0;
        int      issued = 0;
        bool     ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int m_blk = tile % p.m_tiles;
            const int n_blk = tile / p.m_tiles;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    report_timeout(p.status, 0x100u | (unsigned)stage);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(full_bar(stage), (uint32_t)S::kStageBytes);
                tma_load_2d(smem_a + stage * S::kABytes, &tmap_a, full_bar(stage), kb * kBlockK, m_blk * kBlockM);
                tma_load_2d(smem_b + stage * S::kBBytes, &tmap_b, full_bar(stage), kb * kBlockK, n_blk * BLOCK_N);
                ++issued;
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        // Drain: every load this thread issued must have landed before the block may exit.
        // (stage, phase) now name the next slot to fill; walk back over the last min(issued, kStages) slots.
        int      s  = stage;
        uint32_t ph = phase;
        for (int i = 0; i < kStages && i < issued; ++i) {
            if (s == 0) {
                s = kStages;
                ph ^= 1u;
            }
            --s;
            uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(full_bar(s), ph)) {
                if (global_timer_ns() - t0 > kWaitLimitNs) {
                    report_timeout(p.status, 0x500u | (unsigned)s);
                    break;
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------------ MMA issuer
        int      stage = 0;
        uint32_t phase = 0;
        int      local = 0;
        bool     ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local) {
            const int      buf       = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(tmem_empty_bar(buf), acc_phase ^ 1u, abort_flag)) {
                report_timeout(p.status, 0x200u | (unsigned)buf);
                *abort_flag = 1;
                break;
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BLOCK_N);
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    report_timeout(p.status, 0x300u | (unsigned)stage);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint64_t adesc = umma_desc_k_sw128(smem_a + stage * S::kABytes);
                const uint64_t bdesc = umma_desc_k_sw128(smem_b + stage * S::kBBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                    // advancing K by 32 bytes inside the swizzled 128-byte row: +2 in 16-byte units
                    const uint64_t koff = (uint64_t)(k * (kUmmaK >> 4));
                    const uint32_t acc  = (kb > 0 || k > 0) ? 1u : 0u;
                    if (KIND == KIND_I8) {
                        mma_i8(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                    } else {
                        mma_f8f6f4(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                    }
                }
                tc_commit(empty_bar(stage));  // the stage is free once these MMAs have read it
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok) {
                tc_commit(tmem_full_bar(buf));  // accumulator complete
            }
        }
    } else if (warp >= kEpiWarp0) {
        // ------------------------------------------------------------------ epilogue
        const int      quad      = warp - kEpiWarp0;  // == warp % 4: the TMEM lane quadrant this warp may read
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const EpilogueParams& e  = p.epi;
        float fp8_scale = 0.0f;
        if (KIND == KIND_F8) {
            fp8_scale = e.alpha * __ldg(e.s_a) * __ldg(e.s_b);
        }
        const bool vec_ok = (e.c_dtype == LYRAQ_F32 || e.c_dtype == LYRAQ_S32) ? ((e.ldc & 3) == 0) : ((e.ldc & 7) == 0);
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int      buf       = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            const int      m_blk     = tile % p.m_tiles;
            const int      n_blk     = tile / p.m_tiles;
            // the verdict is made warp-uniform: the tensor-memory loads below need the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_phase, abort_flag))) {
                if (lane == 0) {
                    report_timeout(p.status, 0x400u | (unsigned)buf);
                }
                *abort_flag = 1;
                break;
            }
            tc_fence_after_sync();
            const int row = m_blk * kBlockM + quad * 32 + lane;
            float     row_scale = 1.0f;
            if (KIND == KIND_I8 && e.c_dtype != LYRAQ_S32) {
                row_scale = e.row_scale_per_token ? ((row < p.M) ? __ldg(e.row_scale + row) : 0.0f) : __ldg(e.row_scale);
            }
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / 32; ++c) {
                uint32_t acc[32];
                tmem_ld_32x32(tmem_base + lane_addr + (uint32_t)(buf * BLOCK_N + c * 32), acc);
                tmem_ld_wait();
                const int col0  = n_blk * BLOCK_N + c * 32;
                const int valid = p.N - col0;
                if (row < p.M && valid > 0) {
                    if (e.c_dtype == LYRAQ_BF16) {
                        epilogue_chunk<KIND, __nv_bfloat16>(e, acc, row, col0, valid, row_scale, fp8_scale, vec_ok);
                    } else if (e.c_dtype == LYRAQ_F16) {
                        epilogue_chunk<KIND, __half>(e, acc, row, col0, valid, row_scale, fp8_scale, vec_ok);
                    } else if (e.c_dtype == LYRAQ_F32) {
                        epilogue_chunk<KIND, float>(e, acc, row, col0, valid, row_scale, fp8_scale, vec_ok);
                    } else {
                        // raw s32 accumulators
                        int32_t* crow = reinterpret_cast<int32_t*>(e.C) + (size_t)row * e.ldc + col0;
                        if (vec_ok && valid >= 32) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                Vec16 w;
                                w.w[0] = acc[4 * i]; w.w[1] = acc[4 * i + 1]; w.w[2] = acc[4 * i + 2]; w.w[3] = acc[4 * i + 3];
                                st_16(crow + 4 * i, w);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (i < valid) {
                                    crow[i] = (int32_t)acc[i];
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(tmem_empty_bar(buf));
        }
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side.

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void*                           p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

// Tensor map of a row-major [rows, k_bytes] byte matrix, tiles of box_rows x 128 bytes, 128-byte swizzle,
// out-of-range elements read as zero.
int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t row_stride_bytes,
                       uint32_t box_rows, uint32_t box_bytes, bool swizzle128)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    const cuuint64_t dims[2]    = {k_bytes, rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2]     = {box_bytes, box_rows};
    const cuuint32_t estr[2]    = {1, 1};
    const CUresult   r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LYRAQ_OK : LYRAQ_ERR_CUDA;
}

int device_sm_count()
{
    static int cached[64];
    int        dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return 0;
    }
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            return 0;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

// Cost model for the N tile: waves of (tiles / SMs) times the tile's width.
static int pick_block_n(int m, int n, int sms)
{
    const long m_tiles = (m + kBlockM - 1) / kBlockM;
    const long t256    = m_tiles * ((n + 255) / 256);
    const long t128    = m_tiles * ((n + 127) / 128);
    const long c256    = ((t256 + sms - 1) / sms) * 256;
    const long c128    = ((t128 + sms - 1) / sms) * 128;
    return (c128 < c256) ? 128 : 256;
}

template<int KIND, int BLOCK_N>
static int launch_gemm(const void* A, const void* B, GemmParams p, int sms, cudaStream_t stream)
{
    using S = GemmSmem<BLOCK_N>;
    CUtensorMap ta, tb;
    int         st = make_tmap_bytes_2d(&ta, A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.K, kBlockM, kBlockK, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    st = make_tmap_bytes_2d(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, BLOCK_N, kBlockK, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    p.m_tiles = (p.M + kBlockM - 1) / kBlockM;
    p.n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
    const long tiles = (long)p.m_tiles * p.n_tiles;
    const int  grid  = (int)(tiles < sms ? tiles : sms);
    auto       kern  = gemm_tcgen05_kernel<KIND, BLOCK_N>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess) {
        return LYRAQ_ERR_CUDA;
    }
    kern<<<grid, kThreads, S::kTotal, stream>>>(ta, tb, p);
    return launch_status();
}

template<int KIND> static int run_gemm(const void* A, const void* B, GemmParams p, cudaStream_t stream)
{
    if (p.M < 0 || p.N < 0 || p.K < 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (p.M == 0 || p.N == 0) {
        return LYRAQ_OK;
    }
    if (A == nullptr || B == nullptr || p.epi.C == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (p.K == 0 || (p.K & 15) != 0) {
        return LYRAQ_ERR_UNSUPPORTED;  // TMA needs 16-byte row pitch
    }
    if (!aligned16(A) || !aligned16(B) || !aligned16(p.epi.C) || (p.epi.bias != nullptr && !aligned16(p.epi.bias)) ||
        (p.epi.residual != nullptr && !aligned16(p.epi.residual)) || (p.epi.col_scale != nullptr && !aligned16(p.epi.col_scale))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    p.status = status_word_ptr();
    if (p.status == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    const int sms = device_sm_count();
    if (sms <= 0) {
        return LYRAQ_ERR_CUDA;
    }
    p.epi.ldc = p.N;
    if (pick_block_n(p.M, p.N, sms) == 128) {
        return launch_gemm<KIND, 128>(A, B, p, sms, stream);
    }
    return launch_gemm<KIND, 256>(A, B, p, sms, stream);
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {

int lyraq_gemm_int8(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row, int row_scale_mode,
                    void* C, int c_dtype, const void* bias, int m, int n, int k, void* workspace, size_t workspace_bytes,
                    void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if (c_dtype < LYRAQ_F16 || c_dtype > LYRAQ_S32) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (c_dtype != LYRAQ_S32 && (alpha_col == nullptr || alpha_row == nullptr)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (row_scale_mode != LYRAQ_SCALE_PER_TENSOR && row_scale_mode != LYRAQ_SCALE_PER_TOKEN) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    GemmParams p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.epi.C                   = C;
    p.epi.c_dtype             = c_dtype;
    p.epi.col_scale           = alpha_col;
    p.epi.row_scale           = alpha_row;
    p.epi.row_scale_per_token = (row_scale_mode == LYRAQ_SCALE_PER_TOKEN) ? 1 : 0;
    p.epi.bias                = (c_dtype == LYRAQ_S32) ? nullptr : bias;
    return run_gemm<KIND_I8>(A, B, p, (cudaStream_t)stream);
}

int lyraq_gemm_fp8(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, int c_dtype,
                   const void* bias, const void* residual, float alpha, float beta, int epilogue, int m, int n, int k,
                   void* workspace, size_t workspace_bytes, void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if (c_dtype < LYRAQ_F16 || c_dtype > LYRAQ_F32 || s_x == nullptr || s_w == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((epilogue & ~LYRAQ_EPI_GELU_TANH) != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    GemmParams p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.epi.C        = Y;
    p.epi.c_dtype  = c_dtype;
    p.epi.s_a      = s_x;
    p.epi.s_b      = s_w;
    p.epi.alpha    = alpha;
    p.epi.beta     = (residual == nullptr) ? 0.0f : beta;
    p.epi.bias     = bias;
    p.epi.residual = residual;
    p.epi.gelu     = (epilogue & LYRAQ_EPI_GELU_TANH) ? 1 : 0;
    return run_gemm<KIND_F8>(X, W, p, (cudaStream_t)stream);
}

}  // extern "C"
