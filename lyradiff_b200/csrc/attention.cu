// Attention forward for the FLUX blocks: out[b, s, h, :] = softmax(q k^T * scale) v over the packed projection
// qkv [batch, seq, 3, heads, 128] (16-bit), no mask, no dropout.  Replaces the reference's FlashAttention-2 layer
// (src/lyradiff/layers/flash_attn2/flash_attn2.cu:59-118, kernels flash_fwd_kernel.h) on the path between the QKV
// linear and the output linear, and writes its result either in the 16-bit type or already quantized to e4m3 for the
// FP8 linear that follows (the reference runs cudaD2DScaleCpyConvert over the attention output as a separate pass,
// FluxSingleTransformerFP8Block.cc:254, FluxAttnPostFP8Processor.cc:135,168).
//
// One CTA owns 256 query rows of one head (two tiles of 128) and walks the keys in steps of 64:
//   warp 8      lane 0: TMA producer.  Q once (2 x 32 KB), then K_0, V_0, K_1, V_1, ... (tiles of 128 keys, two steps each)
//               through a ring of five 32 KB slots.  Every tile is two SWIZZLE_128B boxes of 128 rows x 64 columns, so q
//               and k tiles are K-major operands and the v tile is an MN-major operand as it lies in memory.
//   warps 9, 10 lane 0: MMA issuer of query tile 0 / 1.  Tensor memory (512 columns, owned by warp 9) per query tile:
//               S_a | S_b (64 fp32 columns each) | O (128 columns).  Step i: S[i & 1] = Q K_i^T (8 x tcgen05.mma kind::f16,
//               M 128, N 64, K 16); O += P_i V_i (4 MMAs, K 16) with P_i read from tensor memory, where the softmax warps
//               wrote it over the first half of S[i & 1].  The scores of step i + 1 are issued BEFORE the softmax of step i
//               has finished (they go to the other S buffer), so the softmax warps never wait for the tensor pipe and the
//               tensor pipe always has the next scores and the previous P V to work on.
//   warps 0-3   softmax of query tile 0, warps 4-7 of tile 1: a thread owns one query row (its tensor-memory lane), so
//               row maxima and sums need no shuffles.  exp2 with the scale folded in; the running maximum is only raised
//               when it grew by more than 2^8 (the accumulator and the row sum then share the stale reference, which
//               cancels in O / l), so O is rescaled in tensor memory rarely, by these same warps, between two of their
//               tile's P V products.  After the last step the warps normalise and store their rows.
// Every wait is bounded; on a timeout the role records it in the status word, raises the block's abort flag and all
// roles leave; tensor memory is freed at the common exit.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace lyraq {

using namespace sm100;

typedef CUresult (*EncodeTiledFnAttn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

namespace attn {

constexpr int kHeadDim   = 128;
constexpr int kTile      = 128;                       // rows of a q tile and of a k / v tile in shared memory
constexpr int kStep      = 64;                        // keys per softmax step
constexpr int kQTiles    = 2;
constexpr int kTileBytes = kTile * kHeadDim * 2;      // 32 KB: two boxes of 128 rows x 128 bytes
constexpr int kBoxBytes  = kTileBytes / 2;
constexpr int kSlots     = 5;
constexpr int kQOffset   = 0;
constexpr int kRingOffset = kQTiles * kTileBytes;
constexpr int kBarOffset = kRingOffset + kSlots * kTileBytes;
constexpr int kSmemUsed  = kBarOffset + 192;
constexpr int kSmemTotal = 232448;                    // all a block may have; the tiles need 1024-byte alignment, which leaves
static_assert(kSmemTotal - kSmemUsed >= 768, "");     // room for a base that is only 256-byte aligned
constexpr int kThreads   = 352;                       // 8 softmax warps, the TMA producer (warp 8), two MMA issuers (warps 9, 10)
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp   = 9;                         // + query tile
constexpr int kTmemCols  = 512;
constexpr int kTileCols  = 256;                       // tensor-memory columns per query tile: S_a 64 | S_b 64 | O 128
constexpr float kRescaleThreshold = 8.0f;             // in log2 units

struct Params {
    void*         out[2];        // rows [0, split) of every batch go to out[0], the rest to out[1] (row index - split)
    long long     out_ld[2];     // row pitch in elements of the output type
    long long     out_batch[2];  // batch pitch in elements
    const float*  out_scale[2];  // e4m3 output: per-tensor scale of each part (1 / scale applied); unused otherwise
    int           out_e4m3;
    int           split;
    int           batch, seq, heads;
    int           q_blocks;      // ceil(seq / 256)
    float         scale_log2;    // softmax scale * log2(e)
    unsigned int* status;
    unsigned long long wait_limit_ns;  // longest a single wait may last (2 s; a test hook shortens it)
    int           skip_loads;          // test hook: the producer issues no copy, so every consumer's wait runs out
};

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_dst), "l"(m), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

template<typename T>
__global__ void __launch_bounds__(kThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const Params p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t*       gen_base  = smem_raw + (smem_base - smem_u32(smem_raw));
    if (smem_base - smem_u32(smem_raw) + (uint32_t)kSmemUsed > (uint32_t)kSmemTotal) {
        if (threadIdx.x == 0) {
            report_timeout(p.status, 0x3001u);  // the aligned layout does not fit: nothing is touched
        }
        return;
    }
    const uint32_t bars = smem_base + kBarOffset;
    // barriers: q_full | slot_full[5] | slot_empty[5] | s_full[tile][buffer] | p_ready[tile][buffer] | pv_done[tile] | o_done[tile]
    const uint32_t q_full = bars;
    auto slot_full  = [&](int s) { return bars + 8u * (1 + s); };
    auto slot_empty = [&](int s) { return bars + 8u * (1 + kSlots + s); };
    auto s_full     = [&](int t, int b) { return bars + 8u * (1 + 2 * kSlots + 2 * t + b); };
    auto p_ready    = [&](int t, int b) { return bars + 8u * (5 + 2 * kSlots + 2 * t + b); };
    auto pv_done    = [&](int t) { return bars + 8u * (9 + 2 * kSlots + t); };
    auto o_done     = [&](int t) { return bars + 8u * (11 + 2 * kSlots + t); };
    uint32_t*     tmem_slot  = reinterpret_cast<uint32_t*>(gen_base + kBarOffset + 8 * (13 + 2 * kSlots));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    grid_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(slot_full(s), 1);
            mbar_init(slot_empty(s), kQTiles);           // both tiles' issuers release a slot
        }
        for (int t = 0; t < kQTiles; ++t) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(s_full(t, b), 1);
                mbar_init(p_ready(t, b), 128);
            }
            mbar_init(pv_done(t), 1);
            mbar_init(o_done(t), 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&tmap_qkv);
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dependency_wait();

    // work item: consecutive blocks share a head, so the CTAs in flight together read the same k / v through L2
    const int qb = blockIdx.x % p.q_blocks;
    const int h  = (blockIdx.x / p.q_blocks) % p.heads;
    const int b  = blockIdx.x / (p.q_blocks * p.heads);
    const int q0 = qb * (kQTiles * kTile);
    const int n_steps = (p.seq + kStep - 1) / kStep;    // softmax steps of 64 keys
    const int n_kv    = (n_steps + 1) / 2;              // k / v tiles of 128 keys
    const int col_q = h * kHeadDim, col_k = (p.heads + h) * kHeadDim, col_v = (2 * p.heads + h) * kHeadDim;

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && p.skip_loads == 0) {
            mbar_arrive_expect_tx(q_full, (uint32_t)(kQTiles * kTileBytes));
            for (int t = 0; t < kQTiles; ++t) {
                for (int half = 0; half < 2; ++half) {
                    tma_load_3d(smem_base + kQOffset + t * kTileBytes + half * kBoxBytes, &tmap_qkv, q_full, col_q + 64 * half,
                                q0 + t * kTile, b);
                }
            }
            int      slot = 0, issued = 0;
            uint32_t phase = 0;
            for (int i = 0; i < 2 * n_kv; ++i) {
                if (!mbar_wait(slot_empty(slot), phase ^ 1u, abort_flag, p.wait_limit_ns)) {
                    report_timeout(p.status, 0x3100u | (unsigned)slot);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t dst = smem_base + kRingOffset + slot * kTileBytes;
                const int      col = (i & 1) ? col_v : col_k;
                mbar_arrive_expect_tx(slot_full(slot), (uint32_t)kTileBytes);
                tma_load_3d(dst, &tmap_qkv, slot_full(slot), col, (i >> 1) * kTile, b);
                tma_load_3d(dst + kBoxBytes, &tmap_qkv, slot_full(slot), col + 64, (i >> 1) * kTile, b);
                ++issued;
                if (++slot == kSlots) {
                    slot = 0;
                    phase ^= 1u;
                }
            }
            // no copy may be in flight when the block leaves: wait (bounded) for the slots filled last, and for q
            int      s  = slot;
            uint32_t ph = phase;
            for (int i = 0; i < kSlots && i < issued; ++i) {
                if (s == 0) {
                    s = kSlots;
                    ph ^= 1u;
                }
                --s;
                const uint64_t t0 = global_timer_ns();
                while (!mbar_try_wait(slot_full(s), ph)) {
                    if (global_timer_ns() - t0 > p.wait_limit_ns) {
                        report_timeout(p.status, 0x3400u | (unsigned)s);
                        break;
                    }
                }
            }
            const uint64_t t0 = global_timer_ns();
            while (!mbar_try_wait(q_full, 0u)) {
                if (global_timer_ns() - t0 > p.wait_limit_ns) {
                    report_timeout(p.status, 0x3401u);
                    break;
                }
            }
        }
    } else if (warp >= kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer of query tile t
        if (lane == 0) {
            const int      t      = warp - kMmaWarp;
            const uint32_t tcol   = tmem_base + (uint32_t)(t * kTileCols);
            constexpr uint32_t kAb = TypeTag<T>::value == LYRAQ_BF16 ? 1u : 0u;
            const uint32_t idesc_qk = umma_idesc(1u, kAb, 128, kStep);
            const uint32_t idesc_pv = umma_idesc(1u, kAb, 128, 128) | kIdescBMajorMN;
            bool ok = true;
            auto wait_or_fail = [&](uint32_t bar, uint32_t parity, unsigned code) {
                if (ok && !mbar_wait(bar, parity, abort_flag, p.wait_limit_ns)) {
                    report_timeout(p.status, code);
                    *abort_flag = 1;
                    ok = false;
                }
                return ok;
            };
            auto slot_of  = [](int item) { return item % kSlots; };
            auto phase_of = [](int item) { return (uint32_t)((item / kSlots) & 1); };
            // the last step that reads a k / v tile gives the tile's slot back (this issuer's share of it)
            auto last_use = [&](int i) { return (i & 1) == 1 || i == n_steps - 1; };
            // S[i & 1] = Q_t K_i^T, 64 keys: rows (i & 1) * 64 .. + 63 of k tile i / 2
            auto issue_qk = [&](int i) {
                const int      kslot = slot_of(2 * (i >> 1));
                const uint32_t kbase = smem_base + kRingOffset + kslot * kTileBytes + (uint32_t)((i & 1) * kStep * 128);
                const uint32_t qbase = smem_base + kQOffset + t * kTileBytes;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (uint32_t)((ks >> 2) * kBoxBytes + (ks & 3) * 32);
                    mma_f16(tcol + (uint32_t)((i & 1) * kStep), umma_desc_k_sw128(qbase + off), umma_desc_k_sw128(kbase + off), idesc_qk,
                            ks > 0 ? 1u : 0u);
                }
                tc_commit(s_full(t, i & 1));
                if (last_use(i)) {
                    tc_commit(slot_empty(kslot));
                }
            };
            // O_t (+)= P_i V_i: P in tensor memory over the first 32 columns of S[i & 1], v rows (i & 1) * 64 .. + 63
            auto issue_pv = [&](int i) {
                const int      vslot = slot_of(2 * (i >> 1) + 1);
                const uint32_t vbase = smem_base + kRingOffset + vslot * kTileBytes + (uint32_t)((i & 1) * kStep * 128);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    mma_f16_ts(tcol + 128u, tcol + (uint32_t)((i & 1) * kStep + k4 * 8),
                               umma_desc_mn_sw128(vbase + (uint32_t)(k4 * 2048), (uint32_t)kBoxBytes), idesc_pv, (i > 0 || k4 > 0) ? 1u : 0u);
                }
                tc_commit(pv_done(t));
                if (last_use(i)) {
                    tc_commit(slot_empty(vslot));
                }
                if (i == n_steps - 1) {
                    tc_commit(o_done(t));   // the accumulator is final
                }
            };
            if (wait_or_fail(q_full, 0u, 0x3200u) && wait_or_fail(slot_full(slot_of(0)), phase_of(0), 0x3201u)) {
                tc_fence_after_sync();
                issue_qk(0);
                if (n_steps > 1) {
                    issue_qk(1);
                }
            }
            for (int i = 0; i < n_steps && ok; ++i) {
                if (!wait_or_fail(p_ready(t, i & 1), (uint32_t)((i >> 1) & 1), 0x3210u | (unsigned)t)) {
                    break;
                }
                if ((i & 1) == 0 && !wait_or_fail(slot_full(slot_of(i + 1)), phase_of(i + 1), 0x3220u | (unsigned)t)) {  // v tile i / 2
                    break;
                }
                tc_fence_after_sync();
                issue_pv(i);
                if (i + 2 < n_steps) {
                    if ((i & 1) == 0 && !wait_or_fail(slot_full(slot_of(i + 2)), phase_of(i + 2), 0x3230u | (unsigned)t)) {  // k tile i / 2 + 1
                        break;
                    }
                    tc_fence_after_sync();
                    issue_qk(i + 2);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + epilogue, one thread per query row
        const int      t        = warp >> 2;                                   // query tile
        const int      quadrant = warp & 3;                                    // tensor-memory lane quadrant of this warp
        const uint32_t tcol     = tmem_base + ((uint32_t)(quadrant * 32) << 16) + (uint32_t)(t * kTileCols);
        const uint32_t o_addr   = tcol + 128u;
        const float    c        = p.scale_log2;
        float          m        = -INFINITY;                                   // reference maximum of this row (raw scores)
        float          l        = 0.0f;                                        // sum of exp2((s - m) c)
        bool           ok       = true;

        for (int i = 0; i < n_steps && ok; ++i) {
            const uint32_t s_addr = tcol + (uint32_t)((i & 1) * kStep);
            if (!__all_sync(0xffffffffu, mbar_wait(s_full(t, i & 1), (uint32_t)((i >> 1) & 1), abort_flag, p.wait_limit_ns))) {
                report_timeout(p.status, 0x3300u | (unsigned)t);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after_sync();
            uint32_t s[64];
            tmem_ld_32x32(s_addr, s);
            tmem_ld_32x32(s_addr + 32, s + 32);
            tmem_ld_wait();
            const int valid = p.seq - i * kStep;                               // keys of this step inside the sequence
            if (valid < kStep) {
#pragma unroll
                for (int k = 0; k < 64; ++k) {
                    if (k >= valid) {
                        s[k] = 0xff800000u;                                    // -inf: zero-filled keys take no weight
                    }
                }
            }
            float mx0 = max3(__uint_as_float(s[0]), __uint_as_float(s[1]), __uint_as_float(s[2]));
            float mx1 = max3(__uint_as_float(s[3]), __uint_as_float(s[4]), __uint_as_float(s[5]));
            float mx2 = max3(__uint_as_float(s[6]), __uint_as_float(s[7]), __uint_as_float(s[8]));
            float mx3 = max3(__uint_as_float(s[9]), __uint_as_float(s[10]), __uint_as_float(s[11]));
#pragma unroll
            for (int k = 12; k < 60; k += 8) {
                mx0 = max3(mx0, __uint_as_float(s[k]), __uint_as_float(s[k + 1]));
                mx1 = max3(mx1, __uint_as_float(s[k + 2]), __uint_as_float(s[k + 3]));
                mx2 = max3(mx2, __uint_as_float(s[k + 4]), __uint_as_float(s[k + 5]));
                mx3 = max3(mx3, __uint_as_float(s[k + 6]), __uint_as_float(s[k + 7]));
            }
            mx0 = max3(mx0, __uint_as_float(s[60]), __uint_as_float(s[61]));
            mx1 = max3(mx1, __uint_as_float(s[62]), __uint_as_float(s[63]));
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
            if (i == 0) {
                m = mx;
            } else {
                const bool raise = (mx - m) * c > kRescaleThreshold;
                if (__any_sync(0xffffffffu, raise)) {
                    // the accumulator may only be touched between this tile's P V products: the previous one has to be complete
                    // (the next one is not issued before this step's P is ready).  S_i exists, so P V of step i - 2 is
                    // complete: pv_done has finished i - 1 or i phases, which the parity of phase i - 1 tells apart
                    if (!__all_sync(0xffffffffu, mbar_wait(pv_done(t), (uint32_t)((i - 1) & 1), abort_flag, p.wait_limit_ns))) {
                        report_timeout(p.status, 0x3310u | (unsigned)t);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const float f = raise ? ex2_approx((m - mx) * c) : 1.0f;
                    if (raise) {
                        m = mx;
                        l *= f;
                    }
#pragma unroll
                    for (int cc = 0; cc < 8; ++cc) {                             // rare path: small pieces keep the registers free
                        uint32_t o[16];
                        tmem_ld_32x16(o_addr + cc * 16, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int k = 0; k < 16; ++k) {
                            o[k] = __float_as_uint(__uint_as_float(o[k]) * f);
                        }
                        tmem_st_32x16(o_addr + cc * 16, o);
                    }
                    tmem_st_wait();
                }
            }
            const float2 c2   = make_float2(c, c);
            const float  nmc  = -m * c;
            const float2 nmc2 = make_float2(nmc, nmc);
            float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t w[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float2 x = fma_f32x2(make_float2(__uint_as_float(s[cc * 16 + 2 * k]), __uint_as_float(s[cc * 16 + 2 * k + 1])), c2, nmc2);
                    const float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                    if (k & 1) {
                        sum_b = add_f32x2(sum_b, e);
                    } else {
                        sum_a = add_f32x2(sum_a, e);
                    }
                    w[k] = Pair<T>::from_f32(e.x, e.y);
                }
                // P over the start of this S buffer: columns [8 cc, 8 cc + 8) hold keys [16 cc, 16 cc + 16), all in registers by now
                asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             ::"r"(s_addr + (uint32_t)(cc * 8)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
                               "r"(w[6]), "r"(w[7])
                             : "memory");
            }
            const float2 sum = add_f32x2(sum_a, sum_b);
            l += sum.x + sum.y;
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(p_ready(t, i & 1));
        }

        // ---- epilogue: O / l, rounded to T, stored as T or as e4m3 of that value.  The softmax runs up to two P V products
        // ahead of the tensor pipe here, which a parity wait on pv_done cannot tell apart (its phase may be one OR two
        // behind): the last product signals a barrier of its own.
        if (ok && !__all_sync(0xffffffffu, mbar_wait(o_done(t), 0u, abort_flag, p.wait_limit_ns))) {
            report_timeout(p.status, 0x3320u | (unsigned)t);
            *abort_flag = 1;
            ok = false;
        }
        if (ok) {
            tc_fence_after_sync();
            const int row = q0 + t * kTile + quadrant * 32 + lane;            // row inside the sequence
            const int part = row >= p.split ? 1 : 0;
            const long long r_out = part ? row - p.split : row;
            const float inv_l = 1.0f / l;
            // rows past the end of the sequence belong to no part (out_scale[1] may be NULL): they load nothing and store nothing
            const float qs = (p.out_e4m3 && row < p.seq) ? 1.0f / ld_f32(p.out_scale[part]) : 1.0f;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t o[32];
                tmem_ld_32x32(o_addr + cc * 32, o);
                tmem_ld_wait();
                if (row < p.seq) {
                    uint32_t w[16];
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        w[k] = Pair<T>::from_f32(__uint_as_float(o[2 * k]) * inv_l, __uint_as_float(o[2 * k + 1]) * inv_l);
                    }
                    const long long col = (long long)h * kHeadDim + cc * 32;
                    if (p.out_e4m3) {
                        uint8_t* dst = static_cast<uint8_t*>(p.out[part]) + (long long)b * p.out_batch[part] + r_out * p.out_ld[part] + col;
                        uint32_t q8[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const float2 a = Pair<T>::to_f32(w[2 * k]), bb = Pair<T>::to_f32(w[2 * k + 1]);
                            q8[k] = f32x2_to_e4m3x2(a.x * qs, a.y * qs) | (f32x2_to_e4m3x2(bb.x * qs, bb.y * qs) << 16);
                        }
                        *reinterpret_cast<uint4*>(dst)      = make_uint4(q8[0], q8[1], q8[2], q8[3]);
                        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(q8[4], q8[5], q8[6], q8[7]);
                    } else {
                        T* dst = static_cast<T*>(p.out[part]) + (long long)b * p.out_batch[part] + r_out * p.out_ld[part] + col;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            reinterpret_cast<uint4*>(dst)[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace attn

// Test hook (lyraq_debug_attention_wait_test): a producer that never signals and a short wait limit, so that the path a
// timed-out wait takes -- status word, abort flag, every role leaving, tensor memory freed -- can be run without a fault.
static int                g_attn_skip_loads    = 0;
static unsigned long long g_attn_wait_limit_ns = kWaitLimitNs;

int launch_attention(void* out, int out_dtype, size_t out_ld, const float* out_scale, void* out2, size_t out2_ld,
                     const float* out2_scale, size_t split, const void* qkv, int dtype, size_t batch, size_t seq, int heads,
                     int head_dim, float softmax_scale, cudaStream_t stream)
{
    if (out == nullptr || qkv == nullptr) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    if ((dtype != LYRAQ_BF16 && dtype != LYRAQ_F16) || head_dim != attn::kHeadDim || heads <= 0 ||
        (out_dtype != dtype && out_dtype != LYRAQ_E4M3)) {
        return LYRAQ_ERR_UNSUPPORTED;
    }
    if (batch == 0 || seq == 0) {
        return LYRAQ_OK;
    }
    if (out2 == nullptr) {
        split = seq;
    }
    const bool   e4m3 = out_dtype == LYRAQ_E4M3;
    const size_t esz  = e4m3 ? 1 : 2;
    if (split > seq || seq > 0x3fffffffu || batch > 0xffffu || (e4m3 && (out_scale == nullptr || (out2 != nullptr && out2_scale == nullptr)))) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    const size_t width = (size_t)heads * attn::kHeadDim;
    if (out_ld < width || (out2 != nullptr && out2_ld < width) || !aligned16(out) || !aligned16(out2) || !aligned16(qkv) ||
        (out_ld * esz) % 16 != 0 || (out2_ld * esz) % 16 != 0) {
        return LYRAQ_ERR_INVALID_ARG;
    }
    static EncodeTiledFnAttn encode = nullptr;
    if (encode == nullptr) {
        void*                           fp = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            return LYRAQ_ERR_CUDA;
        }
        encode = reinterpret_cast<EncodeTiledFnAttn>(fp);
    }
    CUtensorMap      tm;
    const cuuint64_t dims[3]    = {(cuuint64_t)(3 * width), (cuuint64_t)seq, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)(3 * width * 2), (cuuint64_t)(3 * width * 2) * seq};
    const cuuint32_t box[3]     = {64, (cuuint32_t)attn::kTile, 1};
    const cuuint32_t estr[3]    = {1, 1, 1};
    if (encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(qkv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled refused the qkv tensor map");
        return LYRAQ_ERR_CUDA;
    }
    attn::Params p{};
    p.out[0]       = out;
    p.out[1]       = out2;
    p.out_ld[0]    = (long long)out_ld;
    p.out_ld[1]    = (long long)out2_ld;
    p.out_batch[0] = (long long)(split * out_ld);
    p.out_batch[1] = (long long)((seq - split) * out2_ld);
    p.out_scale[0] = out_scale;
    p.out_scale[1] = out2_scale;
    p.out_e4m3     = e4m3 ? 1 : 0;
    p.split        = (int)split;
    p.batch        = (int)batch;
    p.seq          = (int)seq;
    p.heads        = heads;
    p.q_blocks     = (int)((seq + attn::kQTiles * attn::kTile - 1) / (attn::kQTiles * attn::kTile));
    p.scale_log2   = softmax_scale * 1.4426950408889634f;
    p.status       = status_word_ptr();
    p.wait_limit_ns = g_attn_wait_limit_ns;
    p.skip_loads    = g_attn_skip_loads;
    if (p.status == nullptr) {
        return LYRAQ_ERR_CUDA;
    }
    const unsigned grid = (unsigned)(batch * (size_t)heads * (size_t)p.q_blocks);
    if (dtype == LYRAQ_BF16) {
        static bool smem_raised[64] = {};
        const int   attr_st = raise_dynamic_smem_once(attn::attention_fwd_kernel<__nv_bfloat16>, (int)attn::kSmemTotal, smem_raised,
                                                      "cudaFuncSetAttribute(attention_fwd_kernel<bf16>)");
        if (attr_st != LYRAQ_OK) {
            return attr_st;
        }
        return cuda_status(launch_kernel(attn::attention_fwd_kernel<__nv_bfloat16>, grid, (unsigned)attn::kThreads, (size_t)attn::kSmemTotal,
                                         stream, 1u, tm, p),
                           "cudaLaunchKernelEx(attention_fwd_kernel<bf16>)");
    }
    static bool smem_raised_h[64] = {};
    const int   attr_st = raise_dynamic_smem_once(attn::attention_fwd_kernel<__half>, (int)attn::kSmemTotal, smem_raised_h,
                                                  "cudaFuncSetAttribute(attention_fwd_kernel<f16>)");
    if (attr_st != LYRAQ_OK) {
        return attr_st;
    }
    return cuda_status(launch_kernel(attn::attention_fwd_kernel<__half>, grid, (unsigned)attn::kThreads, (size_t)attn::kSmemTotal, stream,
                                     1u, tm, p),
                       "cudaLaunchKernelEx(attention_fwd_kernel<f16>)");
}

}  // namespace lyraq

extern "C" int lyraq_debug_attention_wait_test(int skip_loads, unsigned int wait_limit_ms)
{
    lyraq::g_attn_skip_loads    = skip_loads ? 1 : 0;
    lyraq::g_attn_wait_limit_ns = wait_limit_ms == 0 ? lyraq::sm100::kWaitLimitNs : (unsigned long long)wait_limit_ms * 1000000ull;
    return LYRAQ_OK;
}

extern "C" int lyraq_attention(void* out, int out_dtype, size_t out_ld, const float* out_scale, void* out2, size_t out2_ld,
                               const float* out2_scale, size_t split, const void* qkv, int dtype, size_t batch, size_t seq_len,
                               int heads, int head_dim, float softmax_scale, void* stream)
{
    return lyraq::launch_attention(out, out_dtype, out_ld, out_scale, out2, out2_ld, out2_scale, split, qkv, dtype, batch, seq_len,
                                   heads, head_dim, softmax_scale, (cudaStream_t)stream);
}
