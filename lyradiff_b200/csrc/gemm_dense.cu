// INT8 (kind::i8, s32 accumulators) and FP8 e4m3 (kind::f8f6f4, f32 accumulators) GEMMs for sm_100a.
//
//   Y[M,N] = epilogue( sum_k A[M,k] * B[N,k] ),  A and B both K-contiguous 8-bit.
//
// One persistent CTA per SM, 384 threads, warp-specialised.  Large problems run as CTA PAIRS (a cluster of two):
// tcgen05.mma.cta_group::2 computes a 256 x 256 tile across the two SMs, each CTA loading only its half of the A
// rows and its half of the B rows, which cuts the operand traffic from L2 per flop by a third against a single
// CTA's 128 x 256 tile.  Roles per CTA:
//   warp 0    : TMA producer  - streams 128 x 128-byte A tiles and B tiles into a ring of shared-memory stages
//                               (128-byte swizzle), one mbarrier per stage.
//   warp 1    : MMA issuer    - one thread issues the stage's tcgen05.mma (K = 32 bytes each; four per K block, and a
//                               stage of a pair or of the 128-wide tile holds two K blocks) into one of two accumulator
//                               buffers in tensor memory, and commits to free the stage.
//   warp 2    : allocates / frees tensor memory.
//   warps 4-11: epilogue      - warp w reads TMEM lanes 32 (w % 4).. and the column half (w - 4) / 4.  Per tile the
//                               each warp first stages its half-tile's column scales and bias in its own piece of
//                               shared memory (no barrier across warps), then streams 32-column chunks: tcgen05.ld of chunk
//                               c+1 is in flight while chunk c gets its scales / bias / GELU / residual in registers;
//                               16-bit results go through a 64-byte-swizzled shared-memory box and leave with one TMA
//                               store per chunk (full 64-byte row segments, rows and columns clipped by the hardware);
//                               with one CTA per 256-wide tile (short-K problems, where the epilogue sets the pace) two
//                               chunks share a 128-byte-swizzled box and one store.
// The two accumulator buffers let the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded; on a timeout the role records it in the status word, raises the
// block's abort flag and all roles fall through to the common exit, where tensor memory is freed.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

using namespace sm100;

constexpr int kBlockM      = 128;
constexpr int kBlockK      = 128;  // bytes == elements for 8-bit operands
constexpr int kUmmaK       = 32;
constexpr int kThreads     = 384;
constexpr int kEpiWarp0    = 4;
constexpr int kEpiWarps    = 8;
constexpr int kSmemBudget  = 227 * 1024;
constexpr int kStoreBox    = 32 * 64;                       // one warp's staging box: 32 rows x 64 bytes
// per epilogue warp: one store box, then the (column scale, bias as fp32) pairs and the bias as stored (16-bit) of
// the 128 columns the warp covers
constexpr int kColParams   = 128 * 8 + 128 * 2;
constexpr int kStoreBoxWide = 32 * 128;                     // 32 rows x 128 bytes: two chunks of a 16-bit output behind one TMA store
constexpr int kBarBytes    = 256;

enum GemmKind { KIND_I8 = 0, KIND_F8 = 1 };


struct EpilogueParams {
    void*        C;
    int          c_dtype;
    int          ldc;
    int          tma_store;  // 16-bit output whose row pitch allows TMA stores
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
    // optional fused output quantize: C receives e4m3 codes of T(result) / out_q_scale[0] instead of T values
    const float* out_q_scale;
    // optional gate (fp8, 16-bit outputs): y = T(T(T(acc * scale + bias) * gate[batch, n]) + R), gate of type T [batches, N]
    const void*  gate;
    int          rows_per_batch;
    // optional QK RMSNorm + rotary embedding on a packed QKV projection (fp8, 16-bit outputs, 256-wide tiles, N = 3 * heads * 128):
    // the heads of q and k (columns below 2 * qk_heads * 128) leave normalised and rotated, the v heads as they are
    const void*  qk_norm;     // T [2][128]: RMSNorm weights of q, then of k
    const void*  rope;        // T [M][64][2][2]: the rotation of every row (token)
    int          qk_heads;
    float        qk_eps;
};

struct GemmParams {
    int            M, N, K;
    int            m_tiles, n_tiles;
    unsigned int*  status;
    EpilogueParams epi;
};

// QK RMSNorm + rotary embedding inside the epilogue of the QKV projection.  Arithmetic and order are those of
// rmsnorm_rope_kernel (block_kernels.cu; reference fuseRmsNormAndRope, src/lyradiff/kernels/rope/flux_apply_rope.cu:8-76),
// so the fused epilogue leaves the bits the GEMM followed by that kernel leaves: there sixteen lanes own eight elements of a
// head each, sum their squares with an fma chain and combine the sixteen partial sums with xor shuffles over 8, 4, 2, 1;
// here one thread owns the head's row and adds the same sixteen partial sums in the same tree.
template<typename T>
__device__ __forceinline__ void qk_sumsq_chunk(const uint32_t* o, float* part)
{
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = Pair<T>::to_f32(o[4 * g + j]);
            ss             = fmaf(f.x, f.x, ss);
            ss             = fmaf(f.y, f.y, ss);
        }
        part[g] = ss;
    }
}

__device__ __forceinline__ float qk_sumsq_tree(const float* part)
{
    float a[8], b[4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = part[i] + part[i + 8];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        b[i] = a[i] + a[i + 4];
    }
    return (b[0] + b[2]) + (b[1] + b[3]);
}

// o: the 32 values of chunk c of this row's head, as 16 words of two T values; norm: the head's 128 weights; rope_row: the row's
// 64 x 2 x 2 rotation values
template<typename T>
__device__ __forceinline__ void qk_norm_rope_chunk(uint32_t* o, int c, float inv, const T* norm, const T* rope_row)
{
    using P2 = Pair<T>;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int   part = c * 4 + g;                       // which 8 elements of the head
        const Vec16 sc   = ld_nc_16_keep(norm + part * 8);
        const Vec16 r0   = ld_nc_16_keep(rope_row + part * 16);
        const Vec16 r1   = ld_nc_16_keep(rope_row + part * 16 + 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = P2::to_f32(o[4 * g + j]);
            uint32_t     t = P2::from_f32(f.x * inv, f.y * inv);
            t              = P2::mul(t, sc.w[j]);
            const uint32_t ra = (j < 2) ? r0.w[2 * j] : r1.w[2 * (j - 2)];
            const uint32_t rb = (j < 2) ? r0.w[2 * j + 1] : r1.w[2 * (j - 2) + 1];
            const float2   pa = P2::to_f32(P2::mul(t, ra));
            const float2   pb = P2::to_f32(P2::mul(t, rb));
            o[4 * g + j]      = P2::from_f32(pa.x + pa.y, pb.x + pb.y);
        }
    }
}

// BLOCK_N is the width of the output tile; CTAS = 1: one CTA computes 128 x BLOCK_N; CTAS = 2: a pair of CTAs
// computes 256 x BLOCK_N with cta_group::2 MMAs, each CTA staging 128 A rows and BLOCK_N / 2 B rows per K block.
template<int BLOCK_N, int CTAS> struct GemmSmem {
    // A stage of a CTA pair, or of the 128-wide tile, holds two K blocks: issuing a tcgen05 instruction costs the single
    // MMA thread about 50 cycles and a stage adds a barrier wait and one or two commits, so with stages of four MMAs the
    // issue loop, not the tensor pipe, set the pace (86 % of the MMA rate for pairs); eight MMAs per stage hide it.
    static constexpr int kSub        = (CTAS == 2 || BLOCK_N == 128) ? 2 : 1;
    static constexpr int kASub       = kBlockM * kBlockK;
    static constexpr int kBSub       = (BLOCK_N / CTAS) * kBlockK;
    static constexpr int kABytes     = kASub * kSub;
    static constexpr int kBBytes     = kBSub * kSub;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // One CTA with the 256-wide tile is what short-K problems get (the pair needs K >= 2048), and there the epilogue, not the
    // main loop, sets the pace: its warps get boxes of two chunks (one TMA store per 64 columns) and the ring one stage less.
    static constexpr int kBox        = (CTAS == 1 && BLOCK_N == 256) ? kStoreBoxWide : kStoreBox;
    static constexpr int kEpiSmem    = kEpiWarps * (kBox + kColParams);
    static constexpr int kStages     = (kSmemBudget - 1024 - kBarBytes - kEpiSmem) / kStageBytes;  // 3 (1 x 256), 6 (1 x 128) or 3 double stages (pair)
    static constexpr int kEpiOffset  = kStages * kStageBytes;           // 1024-aligned: stage sizes are multiples of 16 KB
    static constexpr int kBarOffset  = kEpiOffset + kEpiSmem;
    static constexpr int kTotal      = kBarOffset + kBarBytes + 1024;   // + alignment slack
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t smem_src, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's committed stores have finished READING shared memory (the box may be overwritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// 32 values of one output row -> global memory, directly (fp32 / int32 outputs, or rows whose pitch rules out TMA).
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

// 64 bytes of a residual row (32 values of a 16-bit type), or a predicated tail.
template<typename T> __device__ __forceinline__ void load_res32(const T* p, int valid, bool vec_ok, float* out)
{
    if (sizeof(T) == 2 && vec_ok && valid >= 32) {
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
template<> __device__ __forceinline__ void load_res32<float>(const float* p, int valid, bool vec_ok, float* out)
{
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        out[i] = (i < valid) ? p[i] : 0.0f;
    }
}

// Tile order.  Tiles are numbered so that the tiles running at the same time (consecutive numbers) form bands of
// kGroupM tile rows swept along N: a wave then touches about as many A rows as B rows, and both operands of a
// deep-K problem stay in L2 between waves instead of one of them being re-read from HBM every wave.
constexpr int kGroupM = 8;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& m_blk, int& n_blk)
{
    const int per_group = kGroupM * n_tiles;
    const int group     = tile / per_group;
    const int first_m   = group * kGroupM;
    const int rows      = min(kGroupM, m_tiles - first_m);
    const int in_group  = tile - group * per_group;
    m_blk               = first_m + in_group % rows;
    n_blk               = in_group / rows;
}

// The arithmetic of one 32-column chunk of one row: raw accumulator bits -> fp32 results (not yet rounded to T,
// except where the reference's sequence rounds in between).  colp holds (column scale, bias) pairs of the chunk.
template<int KIND, typename T>
__device__ __forceinline__ void epilogue_math(const EpilogueParams& e, const uint32_t* acc, const float2* colp, float row_scale,
                                              float fp8_scale, bool has_res, const float* res, float* v)
{
    if (KIND == KIND_I8) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float2 cp = colp[i];  // same address in every lane: a shared-memory broadcast
            // T(T(acc * (s_w * s_a)) + bias): the first rounding here, the second when the value is stored as T
            // (explicitly rounded multiply: for T = float nothing sits between it and the add, and it must not fuse)
            float t = round_t<T>(__fmul_rn((float)(int)acc[i], cp.x * row_scale));
            if (has_res) {
                t = round_t<T>(t + res[i]);  // T(T(acc * scale) + R) before the bias, as fusedBiasResidualAdd orders it
            }
            v[i] = t + cp.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            float t = __uint_as_float(acc[i]) * fp8_scale;
            if (has_res) {
                t = fmaf(e.beta, res[i], t);
            }
            t += colp[i].y;
            v[i] = e.gelu ? gelu_tanh_f32(t) : t;
        }
    }
}

// The same chunk for 16-bit outputs, in packed arithmetic throughout: two columns per instruction (fp32 pairs with
// IEEE rounding per lane, then the output type's native paired add), result as 16 words of two T values.
// bias2: the chunk's bias as stored (pairs of T); res: the chunk's residual row segment (four 16-byte vectors).
template<int KIND, typename T, bool RES>
__device__ __forceinline__ void epilogue_math16(const EpilogueParams& e, const uint32_t* acc, const float2* colp, const uint32_t* bias2,
                                                float row_scale, float fp8_scale, bool has_res, const Vec16* res, uint32_t* o)
{
    using P2 = Pair<T>;
    if (KIND == KIND_I8) {
        const float2 rs2 = make_float2(row_scale, row_scale);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float4 c   = *reinterpret_cast<const float4*>(colp + 2 * i);  // (s_w, bias, s_w, bias) of two columns
            const float2 sc2 = mul_f32x2(make_float2(c.x, c.z), rs2);          // s_w * s_a first, as the reference does
            const float2 y2  = mul_f32x2(make_float2((float)(int)acc[2 * i], (float)(int)acc[2 * i + 1]), sc2);
            uint32_t     h   = P2::from_f32(y2.x, y2.y);                       // T(acc * scale)
            if (RES && has_res) {
                h = P2::add(h, res[i >> 2].w[i & 3]);                          // T(T(acc * scale) + R)
            }
            if (e.bias != nullptr) {
                h = P2::add(h, bias2[i]);                                      // T(T(acc * scale) + bias)
            }
            o[i] = h;
        }
    } else {
        const float2 fs2 = make_float2(fp8_scale, fp8_scale);
        const float2 be2 = make_float2(e.beta, e.beta);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float4 c = *reinterpret_cast<const float4*>(colp + 2 * i);
            float2       t = mul_f32x2(make_float2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1])), fs2);
            if (RES && e.gate != nullptr) {
                // the linear's own 16-bit result, then the gate and the residual in T arithmetic, as the reference's
                // separate kernel applies them: T(T(y * gate) + R); c.x / c.z hold the gate of the two columns
                const uint32_t y = P2::from_f32(t.x + c.y, t.y + c.w);
                const float2   g = mul_f32x2(P2::to_f32(y), make_float2(c.x, c.z));  // exact product of two T values
                uint32_t       h = P2::from_f32(g.x, g.y);
                if (has_res) {
                    h = P2::add(h, res[i >> 2].w[i & 3]);
                }
                o[i] = h;
                continue;
            }
            if (RES && has_res) {
                t = fma_f32x2(be2, P2::to_f32(res[i >> 2].w[i & 3]), t);
            }
            t = add_f32x2(t, make_float2(c.y, c.w));
            if (e.gelu) {
                t = gelu_tanh_f32x2(t);
            }
            o[i] = P2::from_f32(t.x, t.y);
        }
    }
}

// RES: the instance carries the residual / gate code of the epilogue.  Problems without a residual run an instance
// without it: the extra registers and branches cost the GELU + quantize epilogue of the MLP linear 15-20 %.
template<int KIND, int BLOCK_N, int CTAS, bool RES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const GemmParams p)
{
    using S = GemmSmem<BLOCK_N, CTAS>;
    constexpr int      kStages   = S::kStages;
    constexpr int      kTileM    = kBlockM * CTAS;
    constexpr int      kHalfN    = BLOCK_N / 2;            // columns per epilogue warp
    constexpr int      kChunks   = kHalfN / 32;            // 4 or 2, always even
    constexpr uint32_t kTmemCols = 2 * BLOCK_N;  // two accumulator buffers (power of two: 256 or 512)
    constexpr uint32_t kIdesc    = (KIND == KIND_I8) ? umma_idesc(2u, 1u, kTileM, BLOCK_N) : umma_idesc(1u, 0u, kTileM, BLOCK_N);

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is what the 128-byte swizzle pattern of TMA and UMMA is anchored to.  The dynamic shared
    // window starts at the same offset in every CTA of the kernel, so both CTAs of a pair get the same layout.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t*       gen_base  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t smem_a    = smem_base;
    const uint32_t smem_b    = smem_base + kStages * S::kABytes;
    const uint32_t bars      = smem_base + S::kBarOffset;
    // barrier slots (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    auto full_bar       = [&](int s) { return bars + 8u * s; };
    auto empty_bar      = [&](int s) { return bars + 8u * (kStages + s); };
    auto tmem_full_bar  = [&](int b) { return bars + 8u * (2 * kStages + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * kStages + 2 + b); };
    uint32_t*      tmem_slot  = reinterpret_cast<uint32_t*>(gen_base + S::kBarOffset + 8 * (2 * kStages + 4));
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int      warp    = threadIdx.x >> 5;
    const int      lane    = threadIdx.x & 31;
    const uint32_t rank    = (CTAS == 2) ? cluster_ctarank() : 0u;  // position in the pair; 0 = leader
    const bool     leader  = (rank == 0);
    const int      unit    = (CTAS == 2) ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;  // CTA or CTA pair
    const int      n_units = (CTAS == 2) ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), kEpiWarps * CTAS);  // one arrival per epilogue warp of every CTA of the unit
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_a);
        prefetch_tensormap(&tmap_b);
        prefetch_tensormap(&tmap_c);
    }
    if (warp == 2) {
        if (CTAS == 2) {
            tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    if (CTAS == 2) {
        cluster_sync_all();  // the peer's barriers are initialised before anything is signalled across the pair
    } else {
        __syncthreads();
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();  // everything above overlapped the previous kernel's tail; global memory is touched from here on

    const int num_tiles = p.m_tiles * p.n_tiles;
    const int num_kb    = (p.K + kBlockK - 1) / kBlockK;

    if (warp == 0 && lane == 0) {
        // ------------------------------------------------------------------ TMA producer (every CTA loads its own halves)
        int      stage = 0;
        uint32_t phase = 0;
        int      issued = 0;
        bool     ok = true;
        // Every other tile of a CTA walks K from the far end: the K slices a wave touched last are the ones the next wave
        // asks for first, so for a deep K they are still in L2 instead of being fetched from HBM once per wave.
        const int kb_far = ((num_kb - 1) / S::kSub) * S::kSub;
        bool      flip   = false;
        for (int tile = unit; ok && tile < num_tiles; tile += n_units, flip = !flip) {
            int m_blk, n_blk;
            tile_coords(tile, p.m_tiles, p.n_tiles, m_blk, n_blk);
            const int a_row = m_blk * kTileM + (int)rank * kBlockM;
            const int b_row = n_blk * BLOCK_N + (int)rank * (BLOCK_N / CTAS);
            for (int step = 0; step < num_kb; step += S::kSub) {
                const int kb = flip ? kb_far - step : step;
                if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                    report_timeout(p.status, 0x100u | (unsigned)stage);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                if (CTAS == 2) {
                    // both CTAs' bytes are counted on the leader's barrier, which the leader arms for the pair
                    const uint32_t lbar = map_to_cta(full_bar(stage), 0u);
                    if (leader) {
                        mbar_arrive_expect_tx(full_bar(stage), 2u * (uint32_t)S::kStageBytes);
                    }
#pragma unroll
                    for (int sub = 0; sub < S::kSub; ++sub) {
                        // a K block past the end of K is all zero fill (and still counts its bytes on the barrier)
                        tma_load_2d_pair(smem_a + stage * S::kABytes + sub * S::kASub, &tmap_a, lbar, (kb + sub) * kBlockK, a_row);
                        tma_load_2d_pair(smem_b + stage * S::kBBytes + sub * S::kBSub, &tmap_b, lbar, (kb + sub) * kBlockK, b_row);
                    }
                } else {
                    mbar_arrive_expect_tx(full_bar(stage), (uint32_t)S::kStageBytes);
#pragma unroll
                    for (int sub = 0; sub < S::kSub; ++sub) {
                        tma_load_2d(smem_a + stage * S::kABytes + sub * S::kASub, &tmap_a, full_bar(stage), (kb + sub) * kBlockK, a_row);
                        tma_load_2d(smem_b + stage * S::kBBytes + sub * S::kBSub, &tmap_b, full_bar(stage), (kb + sub) * kBlockK, b_row);
                    }
                }
                ++issued;
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        if (CTAS == 1 || leader) {
            // Drain: every load counted on this CTA's barriers must have landed before the block may exit.
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
        }
    } else if (warp == 1 && lane == 0 && leader) {
        // ------------------------------------------------------------------ MMA issuer (the leader CTA only)
        int      stage = 0;
        uint32_t phase = 0;
        int      local = 0;
        bool     ok = true;
        // cluster addresses of the peer's barriers (same offsets): its producer and epilogue wait on those
        const uint32_t peer = (CTAS == 2) ? 1u : 0u;
        for (int tile = unit; ok && tile < num_tiles; tile += n_units, ++local) {
            const int      buf       = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(tmem_empty_bar(buf), acc_phase ^ 1u, abort_flag)) {
                report_timeout(p.status, 0x200u | (unsigned)buf);
                *abort_flag = 1;
                break;
            }
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BLOCK_N);
            for (int kb = 0; kb < num_kb; kb += S::kSub) {
                if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                    report_timeout(p.status, 0x300u | (unsigned)stage);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int sk = 0; sk < S::kSub * (kBlockK / kUmmaK); ++sk) {
                    const int      sub   = sk / (kBlockK / kUmmaK);
                    const int      k     = sk % (kBlockK / kUmmaK);
                    const uint64_t adesc = umma_desc_k_sw128(smem_a + stage * S::kABytes + sub * S::kASub);
                    const uint64_t bdesc = umma_desc_k_sw128(smem_b + stage * S::kBBytes + sub * S::kBSub);
                    // advancing K by 32 bytes inside the swizzled 128-byte row: +2 in 16-byte units
                    const uint64_t koff = (uint64_t)(k * (kUmmaK >> 4));
                    const uint32_t acc  = (kb > 0 || sk > 0) ? 1u : 0u;
                    if (CTAS == 2) {
                        if (KIND == KIND_I8) {
                            mma_i8_pair(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                        } else {
                            mma_f8f6f4_pair(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                        }
                    } else {
                        if (KIND == KIND_I8) {
                            mma_i8(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                        } else {
                            mma_f8f6f4(d_tmem, adesc + koff, bdesc + koff, kIdesc, acc);
                        }
                    }
                }
                // the stage is free, in both CTAs, once these MMAs have read it
                if (CTAS == 2) {
                    tc_commit_pair(empty_bar(stage));
                    tc_commit_pair(map_to_cta(empty_bar(stage), peer));
                } else {
                    tc_commit(empty_bar(stage));
                }
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok) {
                // accumulator complete: each CTA's epilogue reads its own half of the rows
                if (CTAS == 2) {
                    tc_commit_pair(tmem_full_bar(buf));
                    tc_commit_pair(map_to_cta(tmem_full_bar(buf), peer));
                } else {
                    tc_commit(tmem_full_bar(buf));
                }
            }
        }
    } else if (warp >= kEpiWarp0) {
        // ------------------------------------------------------------------ epilogue (warps 4..11)
        const int      quad      = warp & 3;                 // the TMEM lane quadrant this warp may read
        const int      half      = (warp - kEpiWarp0) >> 2;  // which half of the tile's columns
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const EpilogueParams& e  = p.epi;
        // this warp's private column parameters: no other warp reads or writes them, so __syncwarp is all they need
        float2*        cp_tile   = reinterpret_cast<float2*>(gen_base + S::kEpiOffset + kEpiWarps * S::kBox +
                                                             (warp - kEpiWarp0) * kColParams);  // [128]
        uint16_t*      b16       = reinterpret_cast<uint16_t*>(cp_tile + 128);                  // [128]
        uint8_t*       box       = gen_base + S::kEpiOffset + (warp - kEpiWarp0) * S::kBox;
        const uint32_t box_addr  = smem_base + S::kEpiOffset + (warp - kEpiWarp0) * S::kBox;
        float fp8_scale = 0.0f;
        if (KIND == KIND_F8) {
            fp8_scale = e.alpha * ld_f32(e.s_a) * ld_f32(e.s_b);
        }
        const bool vec_ok = (e.c_dtype == LYRAQ_F32 || e.c_dtype == LYRAQ_S32) ? ((e.ldc & 3) == 0) : ((e.ldc & 7) == 0);
        int local = 0;
        for (int tile = unit; tile < num_tiles; tile += n_units, ++local) {
            const int      buf       = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            int m_blk, n_blk;
            tile_coords(tile, p.m_tiles, p.n_tiles, m_blk, n_blk);
            // column parameters of this warp's half of the tile, staged while the main loop of the tile may still run
            __syncwarp();
            {
                // All of a lane's loads are issued before any of them is used: the loop below is not hidden behind the main
                // loop when K is small, and one load after the other costs a round trip to L2 per column.
                constexpr int kPer = kHalfN / 32;   // columns per lane: 4 or 2
                float    cs[kPer];
                uint16_t braw[kPer], graw[kPer];
                float    b32[kPer];
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    const int col = n_blk * BLOCK_N + half * kHalfN + lane + 32 * i;
                    cs[i]   = 0.0f;
                    braw[i] = 0;
                    graw[i] = 0;
                    b32[i]  = 0.0f;
                    if (col < p.N) {
                        if (KIND == KIND_I8 && e.col_scale != nullptr) {
                            cs[i] = ld_f32(e.col_scale + col);
                        }
                        if (RES && KIND == KIND_F8 && e.gate != nullptr) {
                            // all rows of a tile belong to one batch entry (checked on the host)
                            const size_t gi = (size_t)((m_blk * kTileM) / e.rows_per_batch) * (size_t)p.N + (size_t)col;
                            graw[i] = reinterpret_cast<const uint16_t*>(e.gate)[gi];
                        }
                        if (e.bias != nullptr) {
                            if (e.c_dtype == LYRAQ_F32) {
                                b32[i] = reinterpret_cast<const float*>(e.bias)[col];
                            } else {
                                braw[i] = reinterpret_cast<const uint16_t*>(e.bias)[col];
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    const int cc  = lane + 32 * i;
                    const int col = n_blk * BLOCK_N + half * kHalfN + cc;
                    float2    v   = make_float2(0.0f, 0.0f);
                    if (col < p.N) {
                        v.x = cs[i];
                        if (RES && KIND == KIND_F8 && e.gate != nullptr) {
                            v.x = (e.c_dtype == LYRAQ_BF16) ? __uint_as_float((uint32_t)graw[i] << 16) : __half2float(__ushort_as_half(graw[i]));
                        }
                        if (e.bias != nullptr) {
                            v.y = (e.c_dtype == LYRAQ_F32)    ? b32[i]
                                  : (e.c_dtype == LYRAQ_BF16) ? __uint_as_float((uint32_t)braw[i] << 16)
                                                              : __half2float(__ushort_as_half(braw[i]));
                        }
                    }
                    cp_tile[cc] = v;
                    b16[cc]     = (col < p.N && e.bias != nullptr && e.c_dtype != LYRAQ_F32) ? braw[i] : (uint16_t)0;
                }
            }
            __syncwarp();
            // 16-bit residual: this thread's row segment of the tile is asked into L2 now, while the main loop of the tile
            // still runs, and chunk c + 1's 64 bytes are fetched into registers while chunk c is computed, so that the
            // epilogue does not stand on a DRAM round trip in front of every chunk
            const int  row_r    = m_blk * kTileM + (int)rank * kBlockM + quad * 32 + lane;
            const bool res16    = RES && e.residual != nullptr && e.c_dtype != LYRAQ_F32 && e.c_dtype != LYRAQ_S32;
            const bool vec_ok_r = (e.ldc & 7) == 0;
            Vec16      resb[RES ? 2 : 1][RES ? 4 : 1];
            auto load_res16 = [&](int c, Vec16* dst) {
                const int col0r  = n_blk * BLOCK_N + half * kHalfN + c * 32;
                const int validr = p.N - col0r;
                if (!res16 || row_r >= p.M || validr <= 0) {
                    return;
                }
                const uint16_t* rrow = reinterpret_cast<const uint16_t*>(e.residual) + (size_t)row_r * e.ldc + col0r;
                if (vec_ok_r && validr >= 32) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        dst[q] = ld_nc_16_here(rrow + 8 * q);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int      i0 = 8 * q + 2 * j;
                            const uint32_t lo = (i0 < validr) ? rrow[i0] : 0u;
                            const uint32_t hi = (i0 + 1 < validr) ? rrow[i0 + 1] : 0u;
                            dst[q].w[j]       = lo | (hi << 16);
                        }
                    }
                }
            };
            if (res16 && row_r < p.M) {
                const int      col_h = n_blk * BLOCK_N + half * kHalfN;
                const uint8_t* seg   = reinterpret_cast<const uint8_t*>(e.residual) + ((size_t)row_r * e.ldc + col_h) * 2;
#pragma unroll
                for (int b = 0; b < kHalfN * 2; b += 128) {
                    if (col_h + b / 2 < p.N) {
                        prefetch_l2(seg + b);
                    }
                }
            }
            if (!RES && KIND == KIND_F8 && BLOCK_N == 256 && e.rope != nullptr && row_r < p.M) {
                // the row's rotation values (512 bytes) are asked into L2 / L1 now, while the main loop of the tile still runs
                const uint8_t* rr = reinterpret_cast<const uint8_t*>(e.rope) + (size_t)row_r * 512;
#pragma unroll
                for (int b = 0; b < 512; b += 128) {
                    prefetch_l2(rr + b);
                }
            }
            if (RES) {
                load_res16(0, resb[0]);
            }
            // the verdict is made warp-uniform: the tensor-memory loads below need the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_phase, abort_flag))) {
                if (lane == 0) {
                    report_timeout(p.status, 0x400u | (unsigned)buf);
                }
                *abort_flag = 1;
                break;
            }
            tc_fence_after_sync();
            const int row0 = m_blk * kTileM + (int)rank * kBlockM + quad * 32;  // first row of this warp
            const int row  = row0 + lane;
            float     row_scale = 1.0f;
            if (KIND == KIND_I8 && e.c_dtype != LYRAQ_S32) {
                row_scale = e.row_scale_per_token ? ((row < p.M) ? ld_f32(e.row_scale + row) : 0.0f) : ld_f32(e.row_scale);
            }
            const uint32_t t_addr = tmem_base + lane_addr + (uint32_t)(buf * BLOCK_N + half * kHalfN);

            // QK RMSNorm + RoPE: this warp's 128 columns are one head.  A first pass over the accumulator gives the row's sum
            // of squares of the values as they would be stored; the ordinary pass below then normalises and rotates them.
            bool  qk_rope = false;
            float qk_inv  = 0.0f;
            int   qk_head = 0;
            if (!RES && KIND == KIND_F8 && BLOCK_N == 256 && e.rope != nullptr) {
                qk_head = (n_blk * BLOCK_N + half * kHalfN) >> 7;
                if (qk_head < 2 * e.qk_heads) {
                    qk_rope = true;
                    float part[16];
#pragma unroll
                    for (int c = 0; c < kChunks; ++c) {
                        uint32_t a1[32], o1[16];
                        tmem_ld_32x32(t_addr + (uint32_t)(c * 32), a1);
                        tmem_ld_wait();
                        const uint32_t* bias1 = reinterpret_cast<const uint32_t*>(b16 + c * 32);
                        if (e.c_dtype == LYRAQ_BF16) {
                            epilogue_math16<KIND, __nv_bfloat16, RES>(e, a1, cp_tile + c * 32, bias1, row_scale, fp8_scale, false, resb[0], o1);
                            qk_sumsq_chunk<__nv_bfloat16>(o1, part + (c & 3) * 4);
                        } else {
                            epilogue_math16<KIND, __half, RES>(e, a1, cp_tile + c * 32, bias1, row_scale, fp8_scale, false, resb[0], o1);
                            qk_sumsq_chunk<__half>(o1, part + (c & 3) * 4);
                        }
                    }
                    qk_inv = rsqrtf(qk_sumsq_tree(part) / 128.0f + e.qk_eps);
                }
            }
            if (CTAS == 1 && BLOCK_N == 256 && !RES && e.tma_store == 2) {
                // Short-K problems, 16-bit output: 64 columns per step and ONE TMA store for them (the store box holds 32 rows x
                // 128 bytes in the 128-byte swizzle).  A store costs its warp ~450 cycles (waiting for the box, two re-convergences,
                // the proxy fence, the instruction itself) whatever its size, and with K this short the epilogue sets the pace.
#pragma unroll 1
                for (int c2 = 0; c2 < kHalfN / 64; ++c2) {
                    uint32_t a64[64];
                    tmem_ld_32x32(t_addr + (uint32_t)(c2 * 64), a64);
                    tmem_ld_32x32(t_addr + (uint32_t)(c2 * 64 + 32), a64 + 32);
                    tmem_ld_wait();
                    const int col0  = n_blk * BLOCK_N + half * kHalfN + c2 * 64;
                    const int valid = p.N - col0;
                    uint32_t  o64[32];
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const uint32_t* bias2 = reinterpret_cast<const uint32_t*>(b16 + c2 * 64 + h2 * 32);
                        if (e.c_dtype == LYRAQ_BF16) {
                            epilogue_math16<KIND, __nv_bfloat16, RES>(e, a64 + h2 * 32, cp_tile + c2 * 64 + h2 * 32, bias2, row_scale, fp8_scale, false, resb[0],
                                                                      o64 + h2 * 16);
                        } else {
                            epilogue_math16<KIND, __half, RES>(e, a64 + h2 * 32, cp_tile + c2 * 64 + h2 * 32, bias2, row_scale, fp8_scale, false, resb[0],
                                                               o64 + h2 * 16);
                        }
                    }
                    if (lane == 0) {
                        tma_store_wait_read();  // the previous store has drained the box
                    }
                    __syncwarp();
                    uint8_t*  brow = box + lane * 128;
                    const int sw   = lane & 7;   // 128-byte swizzle: 16-byte piece q of row r lies at piece q ^ (r & 7)
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        Vec16 w;
                        w.w[0] = o64[4 * q]; w.w[1] = o64[4 * q + 1]; w.w[2] = o64[4 * q + 2]; w.w[3] = o64[4 * q + 3];
                        *reinterpret_cast<Vec16*>(brow + ((q ^ sw) << 4)) = w;
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < p.M && valid > 0) {
                        tma_store_2d(&tmap_c, box_addr, col0, row0);
                        tma_store_commit();
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(tmem_empty_bar(buf));
                }
                continue;
            }
            uint32_t acc[2][32];
            tmem_ld_32x32(t_addr, acc[0]);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) {
                tmem_ld_wait();
                if (c + 1 < kChunks) {
                    tmem_ld_32x32(t_addr + (uint32_t)((c + 1) * 32), acc[(c + 1) & 1]);
                }
                const uint32_t* a     = acc[c & 1];
                const int       ccol  = half * kHalfN + c * 32;        // column of the chunk inside the tile
                const int       col0  = n_blk * BLOCK_N + ccol;
                const int       valid = p.N - col0;
                if (e.c_dtype == LYRAQ_S32) {
                    if (row < p.M && valid > 0) {
                        int32_t* crow = reinterpret_cast<int32_t*>(e.C) + (size_t)row * e.ldc + col0;
                        if (vec_ok && valid >= 32) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                Vec16 w;
                                w.w[0] = a[4 * i]; w.w[1] = a[4 * i + 1]; w.w[2] = a[4 * i + 2]; w.w[3] = a[4 * i + 3];
                                st_16(crow + 4 * i, w);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (i < valid) {
                                    crow[i] = (int32_t)a[i];
                                }
                            }
                        }
                    }
                    continue;
                }
                const bool has_res  = RES && e.residual != nullptr;
                const bool in_range = row < p.M && valid > 0;
                if (e.c_dtype == LYRAQ_F32) {
                    float v[32];
                    float res[32];
                    if (has_res && in_range) {
                        load_res32<float>(reinterpret_cast<const float*>(e.residual) + (size_t)row * e.ldc + col0, valid, vec_ok, res);
                    }
                    epilogue_math<KIND, float>(e, a, cp_tile + c * 32, row_scale, fp8_scale, has_res && in_range, res, v);
                    if (in_range) {
                        store_row32<float>(reinterpret_cast<float*>(e.C) + (size_t)row * e.ldc + col0, valid, vec_ok, v);
                    }
                    continue;
                }
                // 16-bit outputs: packed arithmetic, 16 words of two values each
                uint32_t     o[16];
                const Vec16* res = resb[RES ? (c & 1) : 0];
                if (RES && c + 1 < kChunks) {
                    load_res16(c + 1, resb[RES ? ((c + 1) & 1) : 0]);
                }
                const uint32_t* bias2 = reinterpret_cast<const uint32_t*>(b16 + c * 32);
                if (e.c_dtype == LYRAQ_BF16) {
                    epilogue_math16<KIND, __nv_bfloat16, RES>(e, a, cp_tile + c * 32, bias2, row_scale, fp8_scale, has_res && in_range, res, o);
                } else {
                    epilogue_math16<KIND, __half, RES>(e, a, cp_tile + c * 32, bias2, row_scale, fp8_scale, has_res && in_range, res, o);
                }
                if (qk_rope && row < p.M) {
                    const size_t noff = (qk_head >= e.qk_heads) ? 128 : 0;
                    if (e.c_dtype == LYRAQ_BF16) {
                        qk_norm_rope_chunk<__nv_bfloat16>(o, c & 3, qk_inv, reinterpret_cast<const __nv_bfloat16*>(e.qk_norm) + noff,
                                                          reinterpret_cast<const __nv_bfloat16*>(e.rope) + (size_t)row * 256);
                    } else {
                        qk_norm_rope_chunk<__half>(o, c & 3, qk_inv, reinterpret_cast<const __half*>(e.qk_norm) + noff,
                                                   reinterpret_cast<const __half*>(e.rope) + (size_t)row * 256);
                    }
                }
                if (e.out_q_scale != nullptr) {
                    // fused activation quantize for the next FP8 linear: the T-rounded result times 1/s, e4m3 RNE satfinite
                    if (in_range) {
                        const float r  = 1.0f / ld_f32(e.out_q_scale);
                        uint32_t    w[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 f0 = (e.c_dtype == LYRAQ_BF16) ? Pair<__nv_bfloat16>::to_f32(o[2 * i]) : Pair<__half>::to_f32(o[2 * i]);
                            const float2 f1 = (e.c_dtype == LYRAQ_BF16) ? Pair<__nv_bfloat16>::to_f32(o[2 * i + 1]) : Pair<__half>::to_f32(o[2 * i + 1]);
                            w[i] = f32x2_to_e4m3x2(f0.x * r, f0.y * r) | (f32x2_to_e4m3x2(f1.x * r, f1.y * r) << 16);
                        }
                        uint8_t* qrow = reinterpret_cast<uint8_t*>(e.C) + (size_t)row * e.ldc + col0;
                        if (e.tma_store) {
                            // handled below, by the whole warp
                        } else if ((e.ldc & 15) == 0 && valid >= 32) {
                            Vec16 a0, a1;
                            a0.w[0] = w[0]; a0.w[1] = w[1]; a0.w[2] = w[2]; a0.w[3] = w[3];
                            a1.w[0] = w[4]; a1.w[1] = w[5]; a1.w[2] = w[6]; a1.w[3] = w[7];
                            st_16(qrow, a0);
                            st_16(qrow + 16, a1);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (i < valid) {
                                    qrow[i] = (uint8_t)((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
                                }
                            }
                        }
                        if (e.tma_store) {
                            // stash for the warp-wide store below (rows out of range never get here, TMA clips them)
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                o[i] = w[i];
                            }
                        }
                    }
                    if (e.tma_store) {
                        // 32 rows x 32 bytes through this warp's box; the two 16-byte halves of a row swap places in rows
                        // 4-7 of every eight, which is the 32-byte TMA swizzle (and keeps the shared stores conflict-free)
                        if (lane == 0) {
                            tma_store_wait_read();
                        }
                        __syncwarp();
                        uint8_t*  brow = box + lane * 32;
                        const int sw   = (lane >> 2) & 1;
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            Vec16 v16;
                            v16.w[0] = o[4 * q]; v16.w[1] = o[4 * q + 1]; v16.w[2] = o[4 * q + 2]; v16.w[3] = o[4 * q + 3];
                            *reinterpret_cast<Vec16*>(brow + ((q ^ sw) << 4)) = v16;
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && row0 < p.M && valid > 0) {
                            tma_store_2d(&tmap_c, box_addr, col0, row0);
                            tma_store_commit();
                        }
                    }
                    continue;
                }
                if (e.tma_store) {
                    // 32 rows x 64 bytes through this warp's box, 16-byte pieces XOR-swizzled by (row >> 1) & 3 as the
                    // 64-byte TMA swizzle expects (conflict-free for the 16-byte shared stores of a quarter warp)
                    if (lane == 0) {
                        tma_store_wait_read();  // the previous chunk's store has drained the box
                    }
                    __syncwarp();
                    uint8_t*  brow = box + lane * 64;
                    const int sw   = (lane >> 1) & 3;
                    {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            Vec16 w;
                            w.w[0] = o[4 * q]; w.w[1] = o[4 * q + 1]; w.w[2] = o[4 * q + 2]; w.w[3] = o[4 * q + 3];
                            *reinterpret_cast<Vec16*>(brow + ((q ^ sw) << 4)) = w;
                        }
                        fence_proxy_async_smem();
                    }
                    __syncwarp();
                    if (lane == 0 && row0 < p.M && valid > 0) {
                        tma_store_2d(&tmap_c, box_addr, col0, row0);
                        tma_store_commit();
                    }
                } else if (in_range) {
                    uint16_t* crow = reinterpret_cast<uint16_t*>(e.C) + (size_t)row * e.ldc + col0;
                    if (vec_ok && valid >= 32) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            Vec16 w;
                            w.w[0] = o[4 * q]; w.w[1] = o[4 * q + 1]; w.w[2] = o[4 * q + 2]; w.w[3] = o[4 * q + 3];
                            st_16(crow + 8 * q, w);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (2 * i < valid) {
                                crow[2 * i] = (uint16_t)(o[i] & 0xffffu);
                            }
                            if (2 * i + 1 < valid) {
                                crow[2 * i + 1] = (uint16_t)(o[i] >> 16);
                            }
                        }
                    }
                }
            }
            // this warp is done with the accumulator buffer: tell the MMA issuer (in the leader CTA)
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2 && !leader) {
                    mbar_arrive_cluster(map_to_cta(tmem_empty_bar(buf), 0u));
                } else {
                    mbar_arrive(tmem_empty_bar(buf));
                }
            }
        }
        if (lane == 0) {
            tma_store_wait_read();  // shared memory must outlive the last store's read of it
        }
    }

    // ---------------------------------------------------------------------- common exit
    tc_fence_before_sync();
    if (CTAS == 2) {
        cluster_sync_all();  // neither CTA may leave while its peer can still touch its shared or tensor memory
    } else {
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after_sync();
        if (CTAS == 2) {
            tmem_dealloc_pair(tmem_base, kTmemCols);
        } else {
            tmem_dealloc(tmem_base, kTmemCols);
        }
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

// Encoding a tensor map is a pure function of its arguments and costs a driver call of a microsecond or two; a forward
// re-uses the same few (pointer, shape) combinations launch after launch (weights always, activations whenever the
// caller's allocator hands the same block out again), so each host thread keeps the last maps it built.
struct TmapKey {
    const void* base;
    uint64_t    d0, d1, stride;
    uint32_t    b0, b1;
    int         kind;  // data type and swizzle of the encode call
    bool operator==(const TmapKey& o) const
    {
        return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1 && kind == o.kind;
    }
};
struct TmapCache {
    static constexpr int kEntries = 64;
    TmapKey     key[kEntries];
    CUtensorMap map[kEntries];
    bool        used[kEntries] = {};
    static unsigned slot(const TmapKey& k)
    {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (k.d0 * 31 + k.d1) * 0xC2B2AE3D27D4EB4Full + k.stride + ((uint64_t)k.b0 << 40) + ((uint64_t)k.b1 << 20) + (uint64_t)k.kind;
        return (unsigned)((h >> 32) % kEntries);
    }
    bool find(const TmapKey& k, CUtensorMap* out) const
    {
        const unsigned s = slot(k);
        if (used[s] && key[s] == k) {
            *out = map[s];
            return true;
        }
        return false;
    }
    void put(const TmapKey& k, const CUtensorMap& m)
    {
        const unsigned s = slot(k);
        key[s]  = k;
        map[s]  = m;
        used[s] = true;
    }
};
static TmapCache& tmap_cache()
{
    static thread_local TmapCache cache;
    return cache;
}

// Tensor map of a row-major [rows, k_bytes] byte matrix, tiles of box_rows x 128 bytes, 128-byte swizzle,
// out-of-range elements read as zero.
int make_tmap_bytes_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k_bytes, uint64_t row_stride_bytes,
                       uint32_t box_rows, uint32_t box_bytes, bool swizzle128)
{
    const TmapKey key{base, k_bytes, rows, row_stride_bytes, box_bytes, box_rows, swizzle128 ? 1 : 0};
    if (tmap_cache().find(key, map)) {
        return LYRAQ_OK;
    }
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
    if (r != CUDA_SUCCESS) {
        record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled refused the tensor map");
        return LYRAQ_ERR_CUDA;
    }
    tmap_cache().put(key, *map);
    return LYRAQ_OK;
}

// Tensor map of a row-major [rows, cols] matrix of 1- or 2-byte elements for TMA stores of 32 x 32 boxes whose
// shared-memory image uses the swizzle that matches the box's row size (32 or 64 bytes).
int make_tmap_store(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, int elem_bytes, bool wide = false)
{
    const TmapKey key{base, cols, rows, ld * (uint64_t)elem_bytes, wide ? 64u : 32u, 32, 16 + elem_bytes + (wide ? 8 : 0)};
    if (tmap_cache().find(key, map)) {
        return LYRAQ_OK;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    const cuuint64_t dims[2]    = {cols, rows};
    const cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};  // row pitch: cols, or more when the output is a column window
    // 32 rows x 32 columns (64 or 32 bytes a row), or, wide (16-bit only), 32 rows x 64 columns = 128 bytes a row
    const cuuint32_t box[2]     = {wide ? 64u : 32u, 32};
    const cuuint32_t estr[2]    = {1, 1};
    const CUresult   r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            wide ? CU_TENSOR_MAP_SWIZZLE_128B : elem_bytes == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled refused the output tensor map");
        return LYRAQ_ERR_CUDA;
    }
    tmap_cache().put(key, *map);
    return LYRAQ_OK;
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

// Tile choice.  Cost of a configuration = waves (tiles / units that run at once) x work per tile.  A CTA pair with a
// 256 x 256 tile moves a third less operand traffic per flop than a single CTA with 128 x 256, so it is preferred
// (10 % bonus) whenever its wave quantisation is not worse; small or narrow problems fall back to one CTA.
struct TileChoice {
    int block_n;
    int ctas;
};

static TileChoice pick_tile(int m, int n, int k, int sms)
{
    const long m128 = (m + 127) / 128, m256 = (m + 255) / 256;
    const long n128 = (n + 127) / 128, n256 = (n + 255) / 256;
    const long pairs = sms / 2;
    const double c1_256 = (double)((m128 * n256 + sms - 1) / sms) * 256.0;
    const double c1_128 = (double)((m128 * n128 + sms - 1) / sms) * 128.0;
    // with a shallow K the epilogue, not operand traffic, bounds the kernel, and a single CTA's smaller tile wins
    const double c2_256 = (pairs > 0 && k >= 2048) ? (double)((m256 * n256 + pairs - 1) / pairs) * 256.0 * 0.9 : 1e30;
    TileChoice best{256, 1};
    double     cost = c1_256;
    if (c1_128 < cost) {
        best = TileChoice{128, 1};
        cost = c1_128;
    }
    if (c2_256 <= cost) {
        best = TileChoice{256, 2};
    }
    return best;
}

template<int KIND, int BLOCK_N, int CTAS, bool RES>
static int launch_gemm(const void* A, const void* B, GemmParams p, int sms, cudaStream_t stream)
{
    using S = GemmSmem<BLOCK_N, CTAS>;
    CUtensorMap ta, tb;
    int         st = make_tmap_bytes_2d(&ta, A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.K, kBlockM, kBlockK, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    st = make_tmap_bytes_2d(&tb, B, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.K, BLOCK_N / CTAS, kBlockK, true);
    if (st != LYRAQ_OK) {
        return st;
    }
    // output map for TMA stores: 16-bit elements, boxes of 32 rows x 32 columns (64 bytes), 64-byte swizzle.
    // When the output does not qualify (fp32 / int32, or a row pitch that is not a multiple of 16 bytes) the kernel
    // stores directly and this map is a never-used copy of A's.
    CUtensorMap tc = ta;
    p.epi.tma_store = 0;
    if (p.epi.out_q_scale != nullptr) {
        if ((p.N & 15) == 0 && (p.epi.ldc & 15) == 0) {
            st = make_tmap_store(&tc, p.epi.C, (uint64_t)p.M, (uint64_t)p.N, (uint64_t)p.epi.ldc, 1);
            if (st != LYRAQ_OK) {
                return st;
            }
            p.epi.tma_store = 1;
        }
    } else if ((p.epi.c_dtype == LYRAQ_BF16 || p.epi.c_dtype == LYRAQ_F16) && (p.N & 7) == 0) {
        // one CTA, 256-wide tile, no residual, no rope: the epilogue stores 64 columns at a time (tma_store == 2)
        const bool wide = CTAS == 1 && BLOCK_N == 256 && !RES && p.epi.rope == nullptr;
        st = make_tmap_store(&tc, p.epi.C, (uint64_t)p.M, (uint64_t)p.N, (uint64_t)p.epi.ldc, 2, wide);
        if (st != LYRAQ_OK) {
            return st;
        }
        p.epi.tma_store = wide ? 2 : 1;
    }
    p.m_tiles = (p.M + kBlockM * CTAS - 1) / (kBlockM * CTAS);
    p.n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
    const long tiles = (long)p.m_tiles * p.n_tiles;
    const long units = sms / CTAS;
    const int  grid  = (int)(tiles < units ? tiles : units) * CTAS;
    auto       kern  = gemm_tcgen05_kernel<KIND, BLOCK_N, CTAS, RES>;
    // the dynamic shared-memory limit of this instance is raised once per device, not per launch
    static bool smem_raised[64] = {};
    const int   attr_st = raise_dynamic_smem_once(kern, (int)S::kTotal, smem_raised,
                                                  "cudaFuncSetAttribute(gemm_tcgen05_kernel, dynamic shared memory)");
    if (attr_st != LYRAQ_OK) {
        return attr_st;
    }
    return cuda_status(launch_kernel(kern, (unsigned)grid, (unsigned)kThreads, (size_t)S::kTotal, stream, (unsigned)CTAS, ta, tb, tc, p),
                       "cudaLaunchKernelEx(gemm_tcgen05_kernel)");
}

// forced tile configuration for tests and sweeps: 0 = automatic, else block_n * 10 + ctas (2561, 1281, 2562)
static int g_forced_tile = 0;

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
    if (p.epi.ldc == 0) {
        p.epi.ldc = p.N;
    }
    TileChoice t = pick_tile(p.M, p.N, p.K, sms);
    if (g_forced_tile != 0) {
        t = TileChoice{g_forced_tile / 10, g_forced_tile % 10};
    }
    if (p.epi.rope != nullptr && t.block_n != 256) {
        t = TileChoice{256, 1};   // the fused QK norm needs a whole head (128 columns) per epilogue warp
    }
    const bool res = p.epi.residual != nullptr || p.epi.gate != nullptr;
    if (t.ctas == 2) {
        return res ? launch_gemm<KIND, 256, 2, true>(A, B, p, sms, stream) : launch_gemm<KIND, 256, 2, false>(A, B, p, sms, stream);
    }
    if (t.block_n == 128) {
        return res ? launch_gemm<KIND, 128, 1, true>(A, B, p, sms, stream) : launch_gemm<KIND, 128, 1, false>(A, B, p, sms, stream);
    }
    return res ? launch_gemm<KIND, 256, 1, true>(A, B, p, sms, stream) : launch_gemm<KIND, 256, 1, false>(A, B, p, sms, stream);
}

}  // namespace lyraq

using namespace lyraq;

extern "C" {


int lyraq_debug_force_gemm_tile(int code)
{
    if (code != 0 && code != 2561 && code != 1281 && code != 2562) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    g_forced_tile = code;
    return LYRAQ_OK;
}

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

int lyraq_gemm_int8_residual(const int8_t* A, const int8_t* B, const float* alpha_col, const float* alpha_row,
                             int row_scale_mode, void* C, int c_dtype, const void* bias, const void* residual, int m, int n,
                             int k, void* workspace, size_t workspace_bytes, void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if (c_dtype < LYRAQ_F16 || c_dtype > LYRAQ_F32 || alpha_col == nullptr || alpha_row == nullptr) {
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
    p.epi.bias                = bias;
    p.epi.residual            = residual;
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

int lyraq_gemm_fp8_qk_rope(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, size_t ldy, int c_dtype,
                           const void* bias, const void* qk_norm, const void* rope, int heads, int head_dim, double eps, int m, int n, int k,
                           void* stream)
{
    if ((c_dtype != LYRAQ_F16 && c_dtype != LYRAQ_BF16) || s_x == nullptr || s_w == nullptr || qk_norm == nullptr || rope == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (head_dim != 128 || heads <= 0 || (long long)n != 3ll * heads * head_dim) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (!aligned16(qk_norm) || !aligned16(rope) || ldy < (size_t)n || (ldy & 7) != 0 || ldy > 0x7fffffffu) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    GemmParams p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.epi.C        = Y;
    p.epi.c_dtype  = c_dtype;
    p.epi.ldc      = (int)ldy;
    p.epi.s_a      = s_x;
    p.epi.s_b      = s_w;
    p.epi.alpha    = 1.0f;
    p.epi.beta     = 0.0f;
    p.epi.bias     = bias;
    p.epi.qk_norm  = qk_norm;
    p.epi.rope     = rope;
    p.epi.qk_heads = heads;
    p.epi.qk_eps   = (float)eps;
    return run_gemm<KIND_F8>(X, W, p, (cudaStream_t)stream);
}

int lyraq_gemm_fp8_gate(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, void* Y, int c_dtype,
                        const void* bias, const void* gate, const void* residual, int rows_per_batch, int m, int n, int k,
                        void* workspace, size_t workspace_bytes, void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if ((c_dtype != LYRAQ_F16 && c_dtype != LYRAQ_BF16) || s_x == nullptr || s_w == nullptr || gate == nullptr ||
        rows_per_batch <= 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (!aligned16(gate)) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    // a tile (up to 256 rows) must not straddle two batch entries, whose gates differ
    if (m > rows_per_batch && (rows_per_batch % 256) != 0) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    GemmParams p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.epi.C              = Y;
    p.epi.c_dtype        = c_dtype;
    p.epi.s_a            = s_x;
    p.epi.s_b            = s_w;
    p.epi.alpha          = 1.0f;
    p.epi.beta           = (residual == nullptr) ? 0.0f : 1.0f;
    p.epi.bias           = bias;
    p.epi.residual       = residual;
    p.epi.gate           = gate;
    p.epi.rows_per_batch = rows_per_batch;
    return run_gemm<KIND_F8>(X, W, p, (cudaStream_t)stream);
}

int lyraq_gemm_fp8_quant(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, uint8_t* Yq, const float* y_scale,
                         int dtype, const void* bias, const void* residual, float alpha, float beta, int epilogue, int m, int n, int k,
                         void* workspace, size_t workspace_bytes, void* stream)
{
    return lyraq_gemm_fp8_quant_ld(X, s_x, W, s_w, Yq, (size_t)n, y_scale, dtype, bias, residual, alpha, beta, epilogue, m, n, k,
                                   workspace, workspace_bytes, stream);
}

int lyraq_gemm_fp8_quant_ld(const uint8_t* X, const float* s_x, const uint8_t* W, const float* s_w, uint8_t* Yq, size_t ldy,
                            const float* y_scale, int dtype, const void* bias, const void* residual, float alpha, float beta,
                            int epilogue, int m, int n, int k, void* workspace, size_t workspace_bytes, void* stream)
{
    (void)workspace;
    (void)workspace_bytes;
    if ((dtype != LYRAQ_F16 && dtype != LYRAQ_BF16) || s_x == nullptr || s_w == nullptr || y_scale == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (ldy < (size_t)(n > 0 ? n : 0) || ldy > 0x7fffffffu) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if (ldy != (size_t)n && residual != nullptr) {
        return LYRAQ_ERR_UNSUPPORTED;  // the residual is read with the output's row pitch
    }
    if ((epilogue & ~LYRAQ_EPI_GELU_TANH) != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    GemmParams p{};
    p.M = m;
    p.N = n;
    p.K = k;
    p.epi.C           = Yq;
    p.epi.c_dtype     = dtype;
    p.epi.s_a         = s_x;
    p.epi.s_b         = s_w;
    p.epi.alpha       = alpha;
    p.epi.beta        = (residual == nullptr) ? 0.0f : beta;
    p.epi.bias        = bias;
    p.epi.residual    = residual;
    p.epi.gelu        = (epilogue & LYRAQ_EPI_GELU_TANH) ? 1 : 0;
    p.epi.out_q_scale = y_scale;
    p.epi.ldc         = (int)ldy;
    return run_gemm<KIND_F8>(X, W, p, (cudaStream_t)stream);
}

}  // extern "C"
