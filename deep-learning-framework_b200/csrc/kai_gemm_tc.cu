// Tensor-core GEMM of the matmul / Linear path for sm_100a (B200).
//
//   C[M,N] (+)= A'[M,K] . B'[N,K]^T          fp32 in, fp32 out, fp32-grade accuracy
//
// Both operands are consumed "K-major" (the reduction index is contiguous), which is what
// the three reference layouts reduce to once an operand is transposed:
//   VMath::matmul            Y  = X  . W^T   A' = X         B' = W          (vmath.cu:2961-2977)
//   VMath::matmul_backward_x dX = dY . W     A' = dY        B' = W^T        (vmath.cu:3007-3022)
//   VMath::matmul_backward_w dW = dY^T . X   A' = dY^T      B' = X^T        (vmath.cu:3051-3067)
//
// Accuracy scheme (3xTF32): every fp32 operand value a is split once into
//   hi = rna_tf32(a)           (11 significant bits, exactly representable as TF32)
//   lo = rna_tf32(a - hi)      (the next 11 bits; a - hi is exact in fp32)
// and the product is formed as  a.b ~= lo_a.hi_b + hi_a.lo_b + hi_a.hi_b  with three
// tcgen05.mma.kind::tf32 instructions per K-step that accumulate in fp32 in tensor memory.
// The dropped lo.lo term is ~2^-22 relative.
//
// The tensor core's fp32 accumulate truncates instead of rounding to nearest: measured on
// B200, a sum kept in tensor memory drifts towards zero by ~7e-9 (relative) per unit of K,
// i.e. 5.7e-5 at K = 8192 -- far outside the fp32 budget.  The accumulation is therefore
// chunked: tensor memory only ever holds the sum over `kc` K-blocks (16..128 values of K,
// chosen from K), and the epilogue warps add each finished chunk into fp32 registers with
// round-to-nearest adds (the second TMEM buffer takes the next chunk meanwhile).
//
// Pipeline per call:
//   1. split kernels write hi/lo planes of A' and B' (and do the transposes) into the
//      per-device workspace.  One HBM pass per operand: 4 B read + 8 B written per element.
//      (Prefetching the boxes of later K blocks into L2 from the producer thread, 2 to 16 blocks ahead, was
//      measured and dropped: 8192^3 went from 4.29 ms to 6.8 ms -- the extra requests compete with the loads.
//      So was hiding the split behind the GEMM: the call cut into 2 to 8 ranges of K, a side stream splitting
//      range c+1 while the kernel works on range c and later ranges accumulating into C.  The split blocks take
//      the SMs' thread slots ahead of the persistent CTAs and the short kernels pay their start-up each time:
//      8192^3 3.64 -> 4.6 ms with two ranges, 6.8 ms with four; the 8192 x 1024 x 8192 shard 0.63 -> 0.76 / 1.09 ms.)
//   2. the GEMM kernel: persistent, one CTA per SM, 10 warps
//        warp 0    TMA producer: cp.async.bulk.tensor 2-D boxes of the four planes into a
//                  swizzled shared-memory ring (mbarrier complete_tx)
//        warp 1    MMA issuer (one elected lane): tcgen05.mma, accumulators in TMEM,
//                  tcgen05.commit releases ring slots and publishes finished accumulators
//        warps 2-9 epilogue: tcgen05.ld each finished chunk of the 128 x BN accumulator
//                  (double buffered in TMEM so the next chunk's MMAs overlap) and add it into
//                  registers; after the last chunk: fused bias + activation (+ old C), stores
//   3. when the tile count does not fill the last round of the persistent grid, the K-blocks of
//      the last round's tiles are dealt out as equal ranges instead (stream-K style); a fix-up
//      kernel sums the pieces of those tiles in a fixed order (deterministic) and applies the
//      same epilogue.
//
// Every device-side wait is bounded: after ~2 s it records KAI_E_DEVICE_WAIT in the status
// word, raises a CTA-wide abort flag, lets copies in flight land, frees TMEM and returns.
#include <cuda.h>
#include <math.h>

#include <vector>

#include "kai_act.cuh"
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {
namespace {

constexpr int BM = 128;          // tile rows = TMEM lanes
constexpr int UMMA_K = 8;        // K per tcgen05.mma.kind::tf32 (32 bytes)
constexpr int kEpiWarps = 8;     // two warps per TMEM lane quarter, each half of the columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kSmemBudget = 196608 + 2048;  // ring + barriers/alignment slack
constexpr int64_t kCrossMinK = 2048;        // shortest reduction that takes the mixed scheme by itself

template <int BN, int BK>
struct Cfg {
    static constexpr int A_BYTES = BM * BK * 4;  // one plane (hi or lo) of one stage
    static constexpr int B_BYTES = BN * BK * 4;
    static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
    static constexpr int STAGES = 196608 / STAGE_BYTES;
    static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;  // two accumulator buffers; allocations are powers of two
    static_assert(BK == 16 || BK == 32, "BK must give 64- or 128-byte rows");
    static_assert(STAGES >= 2, "ring too shallow");
    static_assert(2 * BN <= 512, "TMEM overflow");
};

// ---------------------------------------------------------------------------------------
// Kernel parameters
// ---------------------------------------------------------------------------------------
struct TcParams {
    int64_t M, N, K;
    int64_t ldc;
    float* c;
    const float* bias;
    const float* leaky_alpha;
    int act;
    int accumulate;
    int tiles_m, tiles_n;
    int kb_total;      // K blocks of BK in the whole reduction
    int kc_blocks;     // K blocks accumulated in tensor memory before promotion to registers
    int group_m;       // rasterisation: tiles walk group_m rows of tiles before the next column
    // Work decomposition (see WorkIter): tiles [0, full_tiles) are computed whole, one per CTA per
    // round; the K-blocks of the remaining sk_tiles tiles form one sequence that is cut into
    // sk_ranges contiguous ranges of sk_per blocks, so that the last round is shared evenly.
    int full_tiles;
    int sk_tiles;
    int sk_per;
    int sk_ranges;
    float* partial;    // slots of BM x BN floats for the pieces of range-split tiles
    int* status;       // device view of the status word
    // Tap-row form of the B operand (KH > 0, the convolution's kernel gradient): a B tile is KH boxes of xb rows,
    // one per kernel row, from 3-D planes [column shift][channel][position]; tile n_blk = (column shift, channel block).
    int xb = 0;        // channels per box
    int xblocks = 1;   // channel blocks per column shift
    int mixed = 0;     // second planes hold bf16 cross-term operands: one TF32 and one BF16 MMA per K step
};

// The tensor maps of the tap-row form: per kernel row one hi and one lo map whose base is that row's offset.
struct TapMaps {
    CUtensorMap hi[4];
    CUtensorMap lo[4];
};

struct WorkItem {
    int m_blk, n_blk, kb_begin, kb_end;
    int slot;  // >= 0: this piece of a tile goes to partial slot `slot`; -1: final output
};

__device__ __forceinline__ void tile_coords(const TcParams& p, int tile, int& m_blk, int& n_blk) {
    const int group_size = p.group_m * p.tiles_n;
    const int g = tile / group_size;
    const int first_m = g * p.group_m;
    const int gm = min(p.group_m, p.tiles_m - first_m);
    const int local = tile - g * group_size;
    m_blk = first_m + local % gm;
    n_blk = local / gm;
}

// The sequence of work items of one CTA.  All three roles walk it identically.
//   1. whole tiles blockIdx.x, blockIdx.x + gridDim.x, ... below full_tiles;
//   2. ranges r = blockIdx.x, blockIdx.x + gridDim.x, ... below sk_ranges of the remainder's
//      K-block sequence; a range can cross tile boundaries, each crossing starts a new item.
//      Range r's piece of remainder tile j is stored in slot r + j (unique and increasing).
struct WorkIter {
    int w, range, pos, end;
    __device__ __forceinline__ explicit WorkIter(const TcParams& p) {
        w = blockIdx.x;
        range = blockIdx.x;
        pos = end = 0;
        load_range(p);
    }
    __device__ __forceinline__ void load_range(const TcParams& p) {
        if (range < p.sk_ranges) {
            pos = range * p.sk_per;
            end = min(pos + p.sk_per, p.sk_tiles * p.kb_total);
        } else {
            pos = end = 0;
        }
    }
    __device__ __forceinline__ bool next(const TcParams& p, WorkItem& it) {
        if (w < p.full_tiles) {
            tile_coords(p, w, it.m_blk, it.n_blk);
            it.kb_begin = 0;
            it.kb_end = p.kb_total;
            it.slot = -1;
            w += gridDim.x;
            return true;
        }
        while (range < p.sk_ranges) {
            if (pos < end) {
                const int j = pos / p.kb_total;
                tile_coords(p, p.full_tiles + j, it.m_blk, it.n_blk);
                it.kb_begin = pos - j * p.kb_total;
                it.kb_end = min(p.kb_total, it.kb_begin + (end - pos));
                it.slot = range + j;
                pos += it.kb_end - it.kb_begin;
                return true;
            }
            range += gridDim.x;
            load_range(p);
        }
        return false;
    }
};

// ---------------------------------------------------------------------------------------
// Epilogue store of 32 consecutive columns of one row
// ---------------------------------------------------------------------------------------
template <int BN>
__device__ __forceinline__ void store_chunk(const TcParams& p, const WorkItem& it, int row_in_tile,
                                            int col_in_tile, const float* r, bool vec_ok, float alpha) {
    if (it.slot >= 0) {
        // Piece of a range-split tile: raw sums, tile-local layout, always 16-byte aligned.
        float* out = p.partial + (static_cast<int64_t>(it.slot) * BM + row_in_tile) * BN + col_in_tile;
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(out + 4 * j) = make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        return;
    }
    const int64_t row = static_cast<int64_t>(it.m_blk) * BM + row_in_tile;
    const int64_t n0 = static_cast<int64_t>(it.n_blk) * BN + col_in_tile;
    if (row >= p.M || n0 >= p.N) return;
    float* out = p.c + row * p.ldc + n0;
    const bool plain = !p.bias && !p.accumulate && p.act == KAI_ACT_NONE;
    const int64_t ncols = (p.N - n0 < 32) ? (p.N - n0) : 32;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = r[4 * j + i];
        const bool full = (4 * j + 3) < ncols;
        if (!plain) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (4 * j + i < ncols) {
                    float t = v[i];
                    if (p.accumulate) t = out[4 * j + i] + t;
                    if (p.bias) t = t + __ldg(p.bias + n0 + 4 * j + i);
                    v[i] = act_forward(p.act, t, alpha);
                }
            }
        }
        if (full && vec_ok) {
            *reinterpret_cast<float4*>(out + 4 * j) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (4 * j + i < ncols) out[4 * j + i] = v[i];
        }
    }
}

// ---------------------------------------------------------------------------------------
// The GEMM kernel
// ---------------------------------------------------------------------------------------
template <int BN, int BK, int KH>
__device__ __forceinline__ void
gemm_3xtf32_body(const CUtensorMap& map_a_hi, const CUtensorMap& map_a_lo, const CUtensorMap& map_b_hi,
                 const CUtensorMap& map_b_lo, const TapMaps* taps, const TcParams& p) {
    using C = Cfg<BN, BK>;
    extern __shared__ uint8_t smem_raw[];
    // Swizzled tiles need their base on a 1024-byte boundary.
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + C::STAGES;          // [STAGES]  MMA -> TMA
    uint64_t* tmem_full_bar = bars + 2 * C::STAGES;  // [2]       MMA -> epilogue
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]       epilogue -> MMA
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), kEpiWarps);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a_hi);
            tma_prefetch_desc(&map_a_lo);
            if (KH == 0) {
                tma_prefetch_desc(&map_b_hi);
                tma_prefetch_desc(&map_b_lo);
            } else {
#pragma unroll
                for (int kr = 0; kr < (KH > 0 ? KH : 1); ++kr) {
                    tma_prefetch_desc(&taps->hi[kr]);
                    tma_prefetch_desc(&taps->lo[kr]);
                }
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            WorkIter iter(p);
            WorkItem it;
            while (ok && iter.next(p, it)) {
                const int row_a = it.m_blk * BM;
                const int row_b = it.n_blk * BN;
                const int shift = (KH > 0) ? it.n_blk / p.xblocks : 0;                 // column shift = plane index
                const int chan0 = (KH > 0) ? (it.n_blk - shift * p.xblocks) * p.xb : 0;
                for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 1);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&full_bar[stage]);
                    uint8_t* base = smem + stage * C::STAGE_BYTES;
                    mbar_expect_tx(full, C::STAGE_BYTES);
                    const int k0 = kb * BK;
                    tma_load_2d(smem_u32(base), &map_a_hi, full, k0, row_a);
                    tma_load_2d(smem_u32(base + C::A_BYTES), &map_a_lo, full, k0, row_a);
                    if (KH == 0) {
                        tma_load_2d(smem_u32(base + 2 * C::A_BYTES), &map_b_hi, full, k0, row_b);
                        tma_load_2d(smem_u32(base + 2 * C::A_BYTES + C::B_BYTES), &map_b_lo, full, k0, row_b);
                    } else {
                        // KH boxes of BN / KH channel rows each: rows of the tile are ordered (kernel row, channel)
                        constexpr int SUB = (BN / (KH > 0 ? KH : 1)) * BK * 4;
#pragma unroll
                        for (int kr = 0; kr < (KH > 0 ? KH : 1); ++kr) {
                            tma_load_3d(smem_u32(base + 2 * C::A_BYTES + kr * SUB), &taps->hi[kr], full, k0, chan0, shift);
                            tma_load_3d(smem_u32(base + 2 * C::A_BYTES + C::B_BYTES + kr * SUB), &taps->lo[kr], full, k0,
                                        chan0, shift);
                        }
                    }
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(BM, BN);
            const uint32_t idesc16 = instr_desc_bf16(BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc_buf = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            WorkIter iter(p);
            WorkItem it;
            while (ok && iter.next(p, it)) {
                // One accumulator buffer per chunk of kc_blocks K-blocks.
                for (int kb0 = it.kb_begin; ok && kb0 < it.kb_end; kb0 += p.kc_blocks) {
                    const int kb1 = min(it.kb_end, kb0 + p.kc_blocks);
                    ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_buf]), acc_phase ^ 1u, abort_flag,
                                   p.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc_buf * BN);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 3);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t base = smem_u32(smem + stage * C::STAGE_BYTES);
                        const uint64_t a_hi = smem_desc_kmajor<BK>(base);
                        const uint64_t a_lo = smem_desc_kmajor<BK>(base + C::A_BYTES);
                        const uint64_t b_hi = smem_desc_kmajor<BK>(base + 2 * C::A_BYTES);
                        const uint64_t b_lo = smem_desc_kmajor<BK>(base + 2 * C::A_BYTES + C::B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // Advancing inside the swizzle span: +32 bytes = +2 in the (addr >> 4) field.
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            const uint32_t first = (kb == kb0 && k == 0) ? 0u : 1u;
                            // Small cross terms first, the dominant hi.hi term last.
                            if (KH == 0 && p.mixed) {
                                umma_bf16(d_tmem, a_lo + adv, b_lo + adv, idesc16, first);
                            } else {
                                umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, first);
                                umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                            }
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                        umma_commit(smem_u32(&empty_bar[stage]));  // slot reusable once these MMAs retire
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    umma_commit(smem_u32(&tmem_full_bar[acc_buf]));  // chunk complete
                    acc_buf ^= 1;
                    if (acc_buf == 0) acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        // A warp may only read the TMEM lane quarter (warp index % 4); the two warps of a quarter
        // take one half of the columns each.
        constexpr int HALF = BN / 2;
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const float alpha = (p.leaky_alpha != nullptr) ? __ldg(p.leaky_alpha) : 0.0f;
        const bool vec_ok = (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        WorkIter iter(p);
        WorkItem it;
        while (ok && iter.next(p, it)) {
            float acc[HALF];
            bool first_chunk = true;
            for (int kb0 = it.kb_begin; kb0 < it.kb_end; kb0 += p.kc_blocks) {
                ok = mbar_wait(smem_u32(&tmem_full_bar[acc_buf]), acc_phase, abort_flag, p.status, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * BN + half * HALF);
#pragma unroll
                for (int cc = 0; cc < HALF / 32; ++cc) {
                    uint32_t r[32];
                    tmem_ld32(taddr + static_cast<uint32_t>(cc * 32), r);
                    tmem_ld_wait(r);
                    if (first_chunk) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] = __uint_as_float(r[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] += __uint_as_float(r[i]);
                    }
                }
                first_chunk = false;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_buf]));
                acc_buf ^= 1;
                if (acc_buf == 0) acc_phase ^= 1u;
            }
            if (!ok) break;
#pragma unroll
            for (int cc = 0; cc < HALF / 32; ++cc)
                store_chunk<BN>(p, it, quarter * 32 + lane, half * HALF + cc * 32, &acc[cc * 32], vec_ok, alpha);
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // Something gave up: give bulk copies and MMAs still in flight time to land in this
        // CTA's shared/tensor memory before it is released.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <int BN, int BK>
__global__ void __launch_bounds__(kThreads, 1)
gemm_3xtf32_kernel(const __grid_constant__ CUtensorMap map_a_hi,
                   const __grid_constant__ CUtensorMap map_a_lo,
                   const __grid_constant__ CUtensorMap map_b_hi,
                   const __grid_constant__ CUtensorMap map_b_lo, const TcParams p) {
    gemm_3xtf32_body<BN, BK, 0>(map_a_hi, map_a_lo, map_b_hi, map_b_lo, nullptr, p);
}

// The same kernel with the B operand in tap-row form (see TcParams): the kernel gradient of a convolution read
// straight from padded, column-shifted planes of the input instead of an unfolded matrix.
template <int BN, int KH>
__global__ void __launch_bounds__(kThreads, 1)
gemm_3xtf32_taps_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                        const __grid_constant__ TapMaps taps, const TcParams p) {
    gemm_3xtf32_body<BN, 16, KH>(map_a_hi, map_a_lo, map_a_hi, map_a_lo, &taps, p);
}

// ---------------------------------------------------------------------------------------
// The CTA-pair form (whole 256 x 256 tiles only).  With one CTA per tile the kernel above is bound by shared-memory
// bandwidth, not by the tensor pipe: per 16-wide K block a 128 x 256 tile writes 48 KB of operand planes into shared
// memory and its six MMAs read 72 KB back, 156 bytes per clock of the 768 clocks the MMAs need, against the 128 bytes
// per clock an SM's shared memory delivers (measured: a 128 x 256 x 8 TF32 MMA takes 128 clocks, and so does the
// 256 x 256 x 8 MMA of a pair on each of its two SMs).  A pair of CTAs on the two SMs of one TPC computes a 256 x 256
// tile with cta_group::2 MMAs: each CTA loads its own 128 rows of A and only half of the B tile (128 rows), the tensor
// cores exchange the B halves, and every CTA ends up with its 128 x 256 rows of the accumulator in its own tensor
// memory.  Per SM that is 32 KB written and 48 KB read per K block, 104 bytes per clock.
//   * both CTAs run the same roles; only the leader's (cluster rank 0) MMA thread issues;
//   * "full" barriers live in the leader: both producers announce their bytes there and their (non-multicast)
//     bulk-tensor copies credit it;
//   * "empty" and "accumulator full" barriers exist in both CTAs: the leader commits to each of the two addresses;
//   * "accumulator empty" lives in the leader and counts the epilogue warps of both CTAs.
// The remote arrivals use the plain (CTA-scope release) form of mbarrier.arrive: with `.release.cluster` on the
// producers' expect_tx the producer threads spent ~2000 clocks per stage in that one instruction and the MMA thread
// waited for data 27-43 % of the time (8192^3: 4.5 ms; 3.5 ms with the plain form).  K blocks of 32 (three 64 KB
// stages) measured faster than 16 (six 32 KB stages): 3.5 vs 4.1 ms.
// Range-splitting an uneven last round (128 tiles on 74 pairs: the K blocks of the last 54 tiles cut into 74 equal
// ranges, pieces in per-CTA partial slots, the fix-up kernel adding them) was built for this kernel too and measured
// on the per-rank shapes of the column partition: 8192 x 1024 x 8192 0.62 ms against 0.53 ms without, 8192 x 2048 x
// 8192 0.97 against 1.00 ms -- the partial tiles and the extra kernel cost what the balance gains; not kept.
// Every wait is bounded as above; the CTAs of a pair meet at a cluster barrier before tensor memory is released.
// ---------------------------------------------------------------------------------------
template <int BK>
struct PairCfg {
    static constexpr int BNP = 256;                     // columns of the pair's tile
    static constexpr int T_BYTES = BM * BK * 4;         // one plane of 128 operand rows
    static constexpr int STAGE_BYTES = 4 * T_BYTES;     // A hi, A lo, B-half hi, B-half lo
    static constexpr int STAGES = 196608 / STAGE_BYTES;
    static constexpr int TMEM_COLS = 512;               // two accumulator buffers of 256 columns
};

template <int BK>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_3xtf32_pair_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                        const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                        const TcParams p) {
    using C = PairCfg<BK>;
    constexpr int BN = C::BNP;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
    uint64_t* full_bar = bars;                       // [STAGES]  both producers -> leader's MMA thread
    uint64_t* empty_bar = bars + C::STAGES;          // [STAGES]  leader's MMA thread -> each CTA's producer
    uint64_t* tmem_full_bar = bars + 2 * C::STAGES;  // [2]       leader's MMA thread -> each CTA's epilogue
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;    // [2]       both epilogues -> leader's MMA thread
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    // byte distance from a local shared-memory address to the same variable in the leader / in the peer
    const uint32_t bars_local = smem_u32(bars);
    const uint32_t to_leader = mapa_u32(bars_local, 0) - bars_local;
    const uint32_t to_peer = mapa_u32(bars_local, rank ^ 1u) - bars_local;
    const uint32_t to_self = mapa_u32(bars_local, rank) - bars_local;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 2);                 // one announcement per producer
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 2 * kEpiWarps);   // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_base_slot), C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a_hi);
            tma_prefetch_desc(&map_a_lo);
            tma_prefetch_desc(&map_b_hi);
            tma_prefetch_desc(&map_b_lo);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.full_tiles; t += pairs) {
                int pm, n_blk;
                tile_coords(p, t, pm, n_blk);
                const int row_a = (2 * pm + static_cast<int>(rank)) * BM;
                const int row_b = n_blk * BN + static_cast<int>(rank) * (BN / 2);
                for (int kb = 0; kb < p.kb_total; ++kb) {
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 5);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&full_bar[stage]) + to_leader;
                    const uint32_t base = smem_u32(smem + stage * C::STAGE_BYTES);
                    mbar_expect_tx_cluster(full, C::STAGE_BYTES);
                    const int k0 = kb * BK;
                    tma_load_2d_pair(base, &map_a_hi, full, k0, row_a);
                    tma_load_2d_pair(base + C::T_BYTES, &map_a_lo, full, k0, row_a);
                    tma_load_2d_pair(base + 2 * C::T_BYTES, &map_b_hi, full, k0, row_b);
                    tma_load_2d_pair(base + 3 * C::T_BYTES, &map_b_lo, full, k0, row_b);
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader only) ------------------------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc_tf32(2 * BM, BN);
            const uint32_t idesc16 = instr_desc_bf16(2 * BM, BN);
            int stage = 0;
            uint32_t phase = 0;
            int acc_buf = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = pair; ok && t < p.full_tiles; t += pairs) {
                for (int kb0 = 0; ok && kb0 < p.kb_total; kb0 += p.kc_blocks) {
                    const int kb1 = min(p.kb_total, kb0 + p.kc_blocks);
                    ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 6);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc_buf * BN);
                    for (int kb = kb0; kb < kb1; ++kb) {
                        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 7);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t base = smem_u32(smem + stage * C::STAGE_BYTES);
                        const uint64_t a_hi = smem_desc_kmajor<BK>(base);
                        const uint64_t a_lo = smem_desc_kmajor<BK>(base + C::T_BYTES);
                        const uint64_t b_hi = smem_desc_kmajor<BK>(base + 2 * C::T_BYTES);
                        const uint64_t b_lo = smem_desc_kmajor<BK>(base + 3 * C::T_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            const uint32_t first = (kb == kb0 && k == 0) ? 0u : 1u;
                            if (p.mixed) {
                                umma_bf16_pair(d_tmem, a_lo + adv, b_lo + adv, idesc16, first);
                            } else {
                                umma_tf32_pair(d_tmem, a_lo + adv, b_hi + adv, idesc, first);
                                umma_tf32_pair(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                            }
                            umma_tf32_pair(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                        const uint32_t e = smem_u32(&empty_bar[stage]);
                        umma_commit_pair(e + to_self);      // both producers may refill the slot
                        umma_commit_pair(e + to_peer);
                        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    const uint32_t f = smem_u32(&tmem_full_bar[acc_buf]);
                    umma_commit_pair(f + to_self);          // chunk complete in both CTAs' tensor memory
                    umma_commit_pair(f + to_peer);
                    acc_buf ^= 1;
                    if (acc_buf == 0) acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs, own 128 rows) --------------------
        constexpr int HALF = BN / 2;
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const float alpha = (p.leaky_alpha != nullptr) ? __ldg(p.leaky_alpha) : 0.0f;
        const bool vec_ok = (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = pair; ok && t < p.full_tiles; t += pairs) {
            WorkItem it;
            int pm;
            tile_coords(p, t, pm, it.n_blk);
            it.m_blk = 2 * pm + static_cast<int>(rank);
            it.kb_begin = 0; it.kb_end = p.kb_total; it.slot = -1;
            float acc[HALF];
            bool first_chunk = true;
            for (int kb0 = 0; kb0 < p.kb_total; kb0 += p.kc_blocks) {
                ok = mbar_wait(smem_u32(&tmem_full_bar[acc_buf]), acc_phase, abort_flag, p.status, 8);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * BN + half * HALF);
#pragma unroll
                for (int cc = 0; cc < HALF / 32; ++cc) {
                    uint32_t r[32];
                    tmem_ld32(taddr + static_cast<uint32_t>(cc * 32), r);
                    tmem_ld_wait(r);
                    if (first_chunk) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] = __uint_as_float(r[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[cc * 32 + i] += __uint_as_float(r[i]);
                    }
                }
                first_chunk = false;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(smem_u32(&tmem_empty_bar[acc_buf]) + to_leader);
                acc_buf ^= 1;
                if (acc_buf == 0) acc_phase ^= 1u;
            }
            if (!ok) break;
#pragma unroll
            for (int cc = 0; cc < HALF / 32; ++cc)
                store_chunk<BN>(p, it, quarter * 32 + lane, half * HALF + cc * 32, &acc[cc * 32], vec_ok, alpha);
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();          // neither CTA's shared or tensor memory goes away while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// Operand split kernels: fp32 -> (hi, lo) TF32 planes, optionally transposed
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void split_tf32(float a, float& hi, float& lo) {
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(a));
    hi = __uint_as_float(h);
    if (isinf(hi) && !isinf(a)) hi = __uint_as_float(__float_as_uint(a) & 0xFFFFE000u);  // no overflow by rounding
    const float rest = isfinite(hi) ? (a - hi) : 0.0f;  // exact; inf/nan carry no low part
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    lo = __uint_as_float(l);
}

// The cross-term plane of the mixed scheme.  For a product with a long reduction the two cross terms hi_a.lo_b and
// lo_a.hi_b are formed by ONE BF16 MMA instead of two TF32 MMAs: an 8-wide K step of the plane holds 16 bf16 values
// (32 bytes, the same as 8 floats, so plane geometry, tensor maps and shared-memory tiles do not change),
//   left operand  (xside 1): [bf16(hi) of the 8 values | bf16(lo) of the 8 values]
//   right operand (xside 2): [bf16(lo)                 | bf16(hi)                 ]
// so that the instruction's 16-long dot product is sum hi_a.lo_b + lo_a.hi_b over the 8 values of K.  The cross
// terms are 2^-12 of the product, so their bf16 rounding (2^-9) leaves 2^-21 of the product: measured 5.6e-7
// relative (Frobenius) against fp64, independent of K, next to ~1.8e-8 sqrt(K) of a sequential fp32 sum.
// `v` are the values at k .. k+3 of one row (k % 4 == 0), `h` their high parts as the tensor core sees them.
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));   // low half = a
    return r;
}
__device__ __forceinline__ void store_cross4(float* row, int64_t k, const float v[4], const float h[4], int xside) {
    float l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) l[j] = isfinite(h[j]) ? (v[j] - h[j]) : 0.0f;
    const uint2 H = make_uint2(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]));
    const uint2 L = make_uint2(pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]));
    uint8_t* g = reinterpret_cast<uint8_t*>(row) + (k >> 3) * 32 + ((k >> 2) & 1) * 8;
    *reinterpret_cast<uint2*>(g) = (xside == 1) ? H : L;
    *reinterpret_cast<uint2*>(g + 16) = (xside == 1) ? L : H;
}

// dst planes are [rows][kp] with kp % 4 == 0; src is [rows][cols] with row stride ld.
// Columns cols..kp-1 are written as zeros.
//
// With hi == nullptr only the lo plane is written, against the TRUNCATED high part
// (a & 0xffffe000): the GEMM then reads the caller's fp32 matrix itself as the hi plane, the
// tensor core ignoring the low 13 mantissa bits of a TF32 operand.
__global__ void split_rows_kernel(const float* __restrict__ src, int64_t rows, int64_t cols,
                                  int64_t ld, float* __restrict__ hi, float* __restrict__ lo,
                                  int64_t kp, int vec_src, int xside) {
    const int64_t quads_per_row = kp >> 2;
    const int64_t total = rows * quads_per_row;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / quads_per_row;
        const int64_t k = (i - r * quads_per_row) << 2;
        float v[4];
        const float* s = src + r * ld + k;
        if (vec_src && k + 3 < cols) {
            const float4 t = *reinterpret_cast<const float4*>(s);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = (k + j < cols) ? s[j] : 0.0f;
        }
        float h[4], l[4];
        if (hi != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) split_tf32(v[j], h[j], l[j]);
            *reinterpret_cast<float4*>(hi + r * kp + k) = make_float4(h[0], h[1], h[2], h[3]);
            if (xside) { store_cross4(lo + r * kp, k, v, h, xside); continue; }
        } else {
            if (xside) {
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __uint_as_float(__float_as_uint(v[j]) & 0xFFFFE000u);
                store_cross4(lo + r * kp, k, v, h, xside);
                continue;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float t = __uint_as_float(__float_as_uint(v[j]) & 0xFFFFE000u);
                const float rest = isfinite(v[j]) ? (v[j] - t) : 0.0f;
                uint32_t lw;
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(rest));
                l[j] = __uint_as_float(lw);
            }
        }
        *reinterpret_cast<float4*>(lo + r * kp + k) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// Lo planes of two dense, 16-byte aligned tensors of `n` float4 each in one launch (blockIdx.y picks
// the tensor), against the truncated high part as above.  Four independent 16-byte loads per thread.
__global__ void __launch_bounds__(256)
split_lo_flat_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ lo_a,
                     float4* __restrict__ lo_b, int64_t n, int xside) {
    const float4* src = blockIdx.y ? b : a;
    float4* dst = blockIdx.y ? lo_b : lo_a;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * 1024 + threadIdx.x;
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int64_t i = base + 256 * u;
        v[u] = (i < n) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int64_t i = base + 256 * u;
        if (i >= n) continue;
        const float in[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        float l[4];
        if (xside) {
            // dense rows whose length is a multiple of 8: the group of a value depends on its flat index alone
            float h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) h[j] = __uint_as_float(__float_as_uint(in[j]) & 0xFFFFE000u);
            store_cross4(reinterpret_cast<float*>(dst), i * 4, in, h, xside);
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float t = __uint_as_float(__float_as_uint(in[j]) & 0xFFFFE000u);
            const float rest = isfinite(in[j]) ? (in[j] - t) : 0.0f;
            uint32_t lw;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(rest));
            l[j] = __uint_as_float(lw);
        }
        dst[i] = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// Transposing variant: src is [src_rows][src_cols] (row stride ld); dst planes are
// [src_cols][kp] with the reduction index = src row.  64 x 64 tiles through shared memory,
// 16-byte loads when the source allows them and 16-byte stores always (kp % 4 == 0).
__global__ void __launch_bounds__(256)
split_transpose_kernel(const float* __restrict__ src, int64_t src_rows, int64_t src_cols, int64_t ld,
                       float* __restrict__ hi, float* __restrict__ lo, int64_t kp, int vec_src,
                       int64_t src_batch_stride, int64_t dst_batch_stride, int xside) {
    __shared__ float tile[64][65];
    src += blockIdx.z * src_batch_stride;   // batched form: one matrix per blockIdx.z
    hi += blockIdx.z * dst_batch_stride;
    lo += blockIdx.z * dst_batch_stride;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 64;  // source rows  = k of dst
    const int64_t c0 = static_cast<int64_t>(blockIdx.x) * 64;  // source cols  = rows of dst
    const int q = threadIdx.x & 15;   // which group of 4 consecutive elements
    const int l = threadIdx.x >> 4;   // 0..15
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int i = l + 16 * pass;
        const int64_t r = r0 + i, c = c0 + 4 * q;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < src_rows) {
            if (vec_src && c + 3 < src_cols) {
                const float4 t = *reinterpret_cast<const float4*>(src + r * ld + c);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c + e < src_cols) v[e] = src[r * ld + c + e];
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) tile[i][4 * q + e] = v[e];
    }
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int i = l + 16 * pass;        // dst row inside the tile (= source column)
        const int64_t dr = c0 + i;
        const int64_t dk = r0 + 4 * q;      // dst k (= source row), 4 at a time
        if (dr < src_cols && dk < kp) {
            float h[4], lw[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_tf32(tile[4 * q + e][i], h[e], lw[e]);  // zero beyond src_rows
            *reinterpret_cast<float4*>(hi + dr * kp + dk) = make_float4(h[0], h[1], h[2], h[3]);
            if (xside) {
                const float v[4] = {tile[4 * q][i], tile[4 * q + 1][i], tile[4 * q + 2][i], tile[4 * q + 3][i]};
                store_cross4(lo + dr * kp, dk, v, h, xside);
            } else {
                *reinterpret_cast<float4*>(lo + dr * kp + dk) = make_float4(lw[0], lw[1], lw[2], lw[3]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Fix-up of range-split tiles: sums the pieces of every remainder tile in range order (fixed,
// hence deterministic) and applies the fused epilogue.  FIXUP_PARTS blocks per tile, each a slice of the tile's
// elements (every element's pieces are still added in range order by one thread).
// ---------------------------------------------------------------------------------------
constexpr int FIXUP_PARTS = 32;
template <int BN>
__global__ void __launch_bounds__(256)
fixup_kernel(const TcParams p) {
    const int j = blockIdx.x;  // remainder tile
    int m_blk, n_blk;
    tile_coords(p, p.full_tiles + j, m_blk, n_blk);
    const int r_first = (j * p.kb_total) / p.sk_per;
    const int r_last = ((j + 1) * p.kb_total - 1) / p.sk_per;
    const float alpha = (p.leaky_alpha != nullptr) ? __ldg(p.leaky_alpha) : 0.0f;
    const bool vec_ok = (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15) == 0;
    const bool plain = !p.bias && !p.accumulate && p.act == KAI_ACT_NONE;
    constexpr int QUADS = BM * BN / 4, PER_BLOCK = QUADS / FIXUP_PARTS;
    static_assert(QUADS % FIXUP_PARTS == 0, "tile elements divide among the blocks");
    const int q_end = (blockIdx.y + 1) * PER_BLOCK;
    for (int q = blockIdx.y * PER_BLOCK + threadIdx.x; q < q_end; q += 256) {
        const int row_in = q / (BN / 4), col_in = (q % (BN / 4)) * 4;
        const int64_t row = static_cast<int64_t>(m_blk) * BM + row_in;
        const int64_t n0 = static_cast<int64_t>(n_blk) * BN + col_in;
        if (row >= p.M || n0 >= p.N) continue;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        // eight pieces are fetched before any is added (the loads are independent, the adds keep range order)
        for (int r = r_first; r <= r_last; r += 8) {
            float4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                t[u] = (r + u <= r_last) ? __ldcs(reinterpret_cast<const float4*>(
                                               p.partial + (static_cast<int64_t>(r + u + j) * BM + row_in) * BN + col_in))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (r + u <= r_last) { sum.x += t[u].x; sum.y += t[u].y; sum.z += t[u].z; sum.w += t[u].w; }
            }
        }
        float v[4] = {sum.x, sum.y, sum.z, sum.w};
        float* out = p.c + row * p.ldc + n0;
        const int64_t ncols = (p.N - n0 < 4) ? (p.N - n0) : 4;
        if (!plain) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < ncols) {
                    float t = v[i];
                    if (p.accumulate) t = out[i] + t;
                    if (p.bias) t = t + __ldg(p.bias + n0 + i);
                    v[i] = act_forward(p.act, t, alpha);
                }
            }
        }
        if (ncols == 4 && vec_ok) {
            *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < ncols) out[i] = v[i];
        }
    }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
// Writes the K-major hi/lo planes of one operand.
//   transpose == false: src is [rows][k]   (row stride ld)
//   transpose == true : src is [k][rows]   (row stride ld)
// xside != 0: the second plane is written in the cross-term form (see store_cross4; k % 8 == 0 then).
int split_flat(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, int xside, cudaStream_t s);
int launch_split(const float* src, int64_t rows, int64_t k, int64_t ld, bool transpose, float* hi,
                 float* lo, int64_t kp, int sm_count, cudaStream_t s, int xside = 0) {
    if (!transpose) {
        // lo plane only, of a dense 16-byte aligned matrix: the flat kernel with four loads in flight per thread
        if (hi == nullptr && ld == k && kp == k && (reinterpret_cast<uintptr_t>(src) & 15) == 0)
            return split_flat(src, nullptr, rows * k, lo, nullptr, xside, s);
        const int vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (ld & 3) == 0) ? 1 : 0;
        const int64_t total = rows * (kp >> 2);
        int64_t blocks = (total + 255) / 256;
        const int64_t cap = static_cast<int64_t>(sm_count) * 16;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        split_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, rows, k, ld, hi, lo, kp, vec, xside);
        count_launch();
        return check_launch("split_rows_kernel");
    }
    dim3 grid(static_cast<unsigned>((rows + 63) / 64), static_cast<unsigned>((kp + 63) / 64));
    const int vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (ld & 3) == 0) ? 1 : 0;
    split_transpose_kernel<<<grid, 256, 0, s>>>(src, k, rows, ld, hi, lo, kp, vec, 0, 0, xside);
    count_launch();
    return check_launch("split_transpose_kernel");
}

template <int BN, int BK>
int launch_gemm(const CUtensorMap maps[4], const TcParams& p, int grid, cudaStream_t s) {
    using C = Cfg<BN, BK>;
    constexpr int smem = C::STAGES * C::STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static_assert(smem <= kSmemBudget + 30000, "shared memory budget");
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(gemm_3xtf32_kernel<BN, BK>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    gemm_3xtf32_kernel<BN, BK><<<grid, kThreads, smem, s>>>(maps[0], maps[1], maps[2], maps[3], p);
    count_launch();
    count_tc_launch();
    return check_launch("gemm_3xtf32_kernel");
}

template <int BK>
int launch_gemm_pair(const CUtensorMap maps[4], const TcParams& p, int grid, cudaStream_t s) {
    using C = PairCfg<BK>;
    constexpr int smem = C::STAGES * C::STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(gemm_3xtf32_pair_kernel<BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    gemm_3xtf32_pair_kernel<BK><<<grid, kThreads, smem, s>>>(maps[0], maps[1], maps[2], maps[3], p);
    count_launch();
    count_tc_launch();
    count_tc_pair_launch();
    return check_launch("gemm_3xtf32_pair_kernel");
}

// ---- optional timing of the kernels of one call (CUDA events on the launching stream) --------
struct Profiler {
    std::mutex mu;
    bool on = false;
    struct Span { cudaEvent_t e0, e1; int kind; };
    std::vector<Span> spans;
};
Profiler g_prof;

struct ProfSpan {
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t s;
    int kind;
    bool active;
    ProfSpan(int kind_, cudaStream_t s_) : s(s_), kind(kind_), active(g_prof.on && !capturing()) {
        if (!active) return;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) { active = false; return; }
        cudaEventRecord(e0, s);
    }
    ~ProfSpan() {
        if (!active) return;
        cudaEventRecord(e1, s);
        std::lock_guard<std::mutex> lock(g_prof.mu);
        g_prof.spans.push_back({e0, e1, kind});
    }
};

}  // namespace

// Operand-split entry for the other tensor-core kernels of the library: K-major hi/lo planes of a
// row-major [rows][cols] fp32 matrix (row pitch of the planes = round_up(cols, 4)).
int split_planes(const float* src, int64_t rows, int64_t cols, float* hi, float* lo, int sm_count, cudaStream_t s) {
    return launch_split(src, rows, cols, cols, false, hi, lo, round_up(cols, 4), sm_count, s);
}

// Lo planes of two dense tensors of `count` floats each (count % 4 == 0, all four pointers 16-byte
// aligned); the caller feeds the tensors themselves to the tensor core as the hi operands.
int split_lo_pair(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, cudaStream_t s) {
    return split_flat(a, b, count, lo_a, lo_b, 0, s);
}
namespace {
int split_flat(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, int xside, cudaStream_t s) {
    const int64_t n = count >> 2;
    dim3 grid(static_cast<unsigned>((n + 1023) / 1024), (b == nullptr) ? 1 : 2);   // b == nullptr: one tensor only
    split_lo_flat_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const float4*>(a), reinterpret_cast<const float4*>(b),
                                              reinterpret_cast<float4*>(lo_a), reinterpret_cast<float4*>(lo_b), n, xside);
    count_launch();
    return check_launch("split_lo_flat_kernel");
}
}  // namespace

// Batched transposing split: `batch` row-major [k][rows] matrices (consecutive in memory) become
// K-major planes [batch][rows][kp], kp = round_up(k, 4).
int split_planes_transposed(const float* src, int64_t batch, int64_t k, int64_t rows, float* hi, float* lo,
                            cudaStream_t s) {
    const int64_t kp = round_up(k, 4);
    if (batch > 65535) return fail(KAI_E_TOO_LARGE, "split_planes_transposed: batch > 65535");
    dim3 grid(static_cast<unsigned>((rows + 63) / 64), static_cast<unsigned>((kp + 63) / 64),
              static_cast<unsigned>(batch));
    const int vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (rows & 3) == 0) ? 1 : 0;
    split_transpose_kernel<<<grid, 256, 0, s>>>(src, k, rows, rows, hi, lo, kp, vec, k * rows, rows * kp, 0);
    count_launch();
    return check_launch("split_transpose_kernel");
}

void profile_enable(bool on) {
    std::lock_guard<std::mutex> lock(g_prof.mu);
    g_prof.on = on;
}

// Sums and clears the recorded spans: kind 0 = GEMM kernel, 1 = operand split kernels, 2 = fix-up of range-split tiles.
int profile_read(double ms[3], int64_t launches[3]) {
    std::lock_guard<std::mutex> lock(g_prof.mu);
    for (int i = 0; i < 3; ++i) { ms[i] = 0.0; launches[i] = 0; }
    for (auto& sp : g_prof.spans) {
        KAI_CUDA(cudaEventSynchronize(sp.e1));
        float t = 0.f;
        KAI_CUDA(cudaEventElapsedTime(&t, sp.e0, sp.e1));
        ms[sp.kind] += t;
        launches[sp.kind] += 1;
        cudaEventDestroy(sp.e0);
        cudaEventDestroy(sp.e1);
    }
    g_prof.spans.clear();
    return KAI_OK;
}

// ---------------------------------------------------------------------------------------
// Plan of one tensor-core GEMM: tile shape, work decomposition, promotion interval.
// ---------------------------------------------------------------------------------------
struct TcPlan {
    bool pair;           // CTA-pair kernel: tiles_m counts 256-row tiles, whole tiles only
    int bn, bk;
    int tiles_m, tiles_n, kb_total;
    int full_tiles, sk_tiles, sk_per, sk_ranges;
    int64_t slots;       // partial tiles of BM x bn floats the range split needs
    int kc_blocks, group_m, grid;
};

// Partial slots a range split of `tiles` tiles can need on `sms` SMs: at most one range per CTA plus
// one piece per remainder tile, or -- with a forced split_k = s -- s pieces per tile plus one.
static int64_t max_slots(int64_t tiles, int sms, int forced) {
    if (forced > 1) return tiles * (forced + 1);
    const int64_t rem = (tiles * 2 <= sms) ? tiles : (tiles % sms);
    return rem > 0 ? rem + sms : 0;
}

static int plan_tc(const DeviceState* st, int64_t M, int64_t N, int64_t K, TcPlan* out, int force_bn = 0) {
    if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31))
        return fail(KAI_E_TOO_LARGE, "gemm_tc: a dimension exceeds 2^31-1");
    Options& opt = options();
    TcPlan pl;
    pl.pair = false;
    pl.bk = (opt.tc_bk.load() == 32) ? 32 : 16;
    pl.bn = (opt.tc_bn.load() == 128) ? 128 : 256;
    if (N <= 128) pl.bn = 128;
    if (force_bn > 0) { pl.bn = force_bn; pl.bk = 16; }
    pl.tiles_m = static_cast<int>((M + BM - 1) / BM);
    pl.tiles_n = static_cast<int>((N + pl.bn - 1) / pl.bn);
    pl.kb_total = static_cast<int>((K + pl.bk - 1) / pl.bk);
    const int64_t tiles = static_cast<int64_t>(pl.tiles_m) * pl.tiles_n;
    if (tiles >= (int64_t(1) << 26)) return fail(KAI_E_TOO_LARGE, "gemm_tc: too many tiles");

    // CTAs of the persistent grid: one per SM, or fewer when the caller keeps SMs free for work that
    // has to run beside this kernel ("tc_max_ctas": a collective's kernels cannot start on an SM whose
    // shared memory a GEMM CTA holds, and the tile schedule is static, so a collective enqueued beside
    // a full grid runs between the GEMM kernels instead of under them).
    int sms = st->sm_count;
    const int64_t cap = opt.tc_max_ctas.load();
    if (cap > 0 && cap < sms) sms = static_cast<int>(cap);

    // Work decomposition.  When there are fewer tiles than half the SMs and the reduction is long,
    // the K-blocks of all tiles form one sequence that is cut into equal ranges, one per CTA
    // (stream-K style: pieces land in partial slots, a fix-up kernel adds them in a fixed order).
    // The same mechanism could even out the last round of a grid whose tile count is not a multiple
    // of the SM count (256 tiles on 148 SMs), but measured on B200 it does not pay there: the kernel
    // runs at the board's power limit, where idle SMs in the last round let the busy ones clock
    // higher, and the extra partial traffic costs more than the balance gains (0.78 ms without,
    // 0.86 ms with, for 8192 x 1024 x 8192).  "split_k" = 1 switches range splitting off, s > 1
    // cuts every tile into ranges of ceil(K-blocks / s).
    const int forced = static_cast<int>(opt.split_k.load());
    pl.full_tiles = static_cast<int>(tiles); pl.sk_tiles = 0; pl.sk_per = pl.kb_total; pl.sk_ranges = 0;

    // The CTA-pair kernel takes the call when the 256 x 256 tiles fill at least half a round of the pairs and the
    // second half of the last tile row is not mostly padding.
    if (opt.tc_pair.load() != 0 && pl.bn == 256 && force_bn == 0 && forced <= 0 && sms >= 2 &&
        (pl.tiles_m % 2 == 0 || pl.tiles_m >= 9)) {
        const int tiles_mp = (pl.tiles_m + 1) / 2;
        const int64_t tiles_p = static_cast<int64_t>(tiles_mp) * pl.tiles_n;
        const int pairs = sms / 2;
        if (tiles_p * 2 >= pairs) {      // from half a round on: the same share of SMs is busy as with 128-row tiles
            pl.pair = true;
            pl.bk = (opt.tc_pair_bk.load() == 16) ? 16 : 32;
            pl.kb_total = static_cast<int>((K + pl.bk - 1) / pl.bk);
            pl.tiles_m = tiles_mp;
            pl.full_tiles = static_cast<int>(tiles_p);
        }
    }
    const int min_per = (128 / pl.bk) < 1 ? 1 : (128 / pl.bk);  // at least 128 values of K per range
    if (pl.pair) {
        // whole tiles only
    } else if (forced > 1) {
        pl.full_tiles = 0;
        pl.sk_tiles = static_cast<int>(tiles);
        pl.sk_per = (pl.kb_total + forced - 1) / forced;
    } else if (forced <= 0) {
        const int64_t rounds = (tiles + sms - 1) / sms;
        const int64_t rem_last = tiles % sms;
        const bool starved = tiles * 2 <= sms;
        const bool uneven = opt.tc_balance.load() != 0 && rem_last != 0 && rounds <= 4 &&
                            static_cast<double>(tiles) / static_cast<double>(rounds * sms) < 0.93;
        if ((starved || uneven) && pl.kb_total >= 2 * min_per) {
            const int64_t rem = starved ? tiles : rem_last;
            pl.full_tiles = static_cast<int>(tiles - rem);
            pl.sk_tiles = static_cast<int>(rem);
            const int64_t seq = rem * pl.kb_total;
            pl.sk_per = static_cast<int>((seq + sms - 1) / sms);
            if (pl.sk_per < min_per) pl.sk_per = min_per;
            if (pl.sk_per >= pl.kb_total) { pl.full_tiles = static_cast<int>(tiles); pl.sk_tiles = 0; pl.sk_per = pl.kb_total; }
        }
    }
    if (pl.sk_tiles > 0) {
        const int64_t seq = static_cast<int64_t>(pl.sk_tiles) * pl.kb_total;
        pl.sk_ranges = static_cast<int>((seq + pl.sk_per - 1) / pl.sk_per);
    }
    pl.slots = (pl.sk_tiles > 0) ? static_cast<int64_t>(pl.sk_ranges) + pl.sk_tiles : 0;

    // Promotion interval: the truncation drift is ~7e-9 * (K held in tensor memory); keep it at
    // about half of the reference's own error (~1.8e-8 * sqrt(K)): K_chunk <= 2.5 * sqrt(K).
    int64_t kc = opt.tc_kc.load();
    if (kc <= 0) {
        kc = 16;
        while (kc * 2 <= 128 && static_cast<double>(kc * 2) <= 2.5 * sqrt(static_cast<double>(K))) kc *= 2;
    }
    pl.kc_blocks = static_cast<int>(kc / pl.bk < 1 ? 1 : kc / pl.bk);
    int gm = static_cast<int>(opt.tc_group_m.load());
    if (pl.pair) gm = (gm + 1) / 2;      // the option counts 128-row tiles; a pair's tile is two of them tall
    pl.group_m = gm < 1 ? 1 : gm;
    // Enough CTAs for one round of whole tiles or for all ranges, at most one per (usable) SM.
    const int64_t work = pl.full_tiles > pl.sk_ranges ? pl.full_tiles : pl.sk_ranges;
    pl.grid = static_cast<int>(work < sms ? work : sms);
    if (pl.pair) pl.grid = 2 * static_cast<int>(pl.full_tiles < sms / 2 ? pl.full_tiles : sms / 2);
    *out = pl;
    return KAI_OK;
}

// Launches the GEMM kernel (and the fix-up of range-split tiles) on ready-made K-major planes
// [rows][kp]; `partial` holds pl.slots tiles of BM x bn floats.
static int run_tc(DeviceState* st, const TcPlan& pl, float* c, const float* a_hi, const float* a_lo,
                  const float* b_hi, const float* b_lo, int64_t M, int64_t N, int64_t K, int64_t kp, int64_t ldc,
                  const Epilogue& ep, float* partial, int* status_dev, cudaStream_t s, bool mixed = false) {
    CUtensorMap maps[4];
    KAI_TRY(make_map(&maps[0], a_hi, M, K, kp, BM, pl.bk));
    KAI_TRY(make_map(&maps[1], a_lo, M, K, kp, BM, pl.bk));
    KAI_TRY(make_map(&maps[2], b_hi, N, K, kp, pl.pair ? pl.bn / 2 : pl.bn, pl.bk));
    KAI_TRY(make_map(&maps[3], b_lo, N, K, kp, pl.pair ? pl.bn / 2 : pl.bn, pl.bk));

    TcParams p;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.c = c;
    p.bias = ep.bias; p.leaky_alpha = ep.leaky_alpha; p.act = ep.act; p.accumulate = ep.accumulate;
    p.tiles_m = pl.tiles_m; p.tiles_n = pl.tiles_n;
    p.kb_total = pl.kb_total;
    p.full_tiles = pl.full_tiles; p.sk_tiles = pl.sk_tiles; p.sk_per = pl.sk_per; p.sk_ranges = pl.sk_ranges;
    p.kc_blocks = pl.kc_blocks;
    p.group_m = pl.group_m;
    p.partial = partial;
    p.status = status_dev;
    p.mixed = mixed ? 1 : 0;

    int rc;
    {
        ProfSpan span(0, s);
        if (pl.pair) rc = (pl.bk == 16) ? launch_gemm_pair<16>(maps, p, pl.grid, s) : launch_gemm_pair<32>(maps, p, pl.grid, s);
        else if (pl.bn == 256 && pl.bk == 16) rc = launch_gemm<256, 16>(maps, p, pl.grid, s);
        else if (pl.bn == 256 && pl.bk == 32) rc = launch_gemm<256, 32>(maps, p, pl.grid, s);
        else if (pl.bn == 128 && pl.bk == 16) rc = launch_gemm<128, 16>(maps, p, pl.grid, s);
        else rc = launch_gemm<128, 32>(maps, p, pl.grid, s);
    }
    KAI_TRY(rc);

    if (pl.sk_tiles > 0) {
        ProfSpan span(2, s);
        const dim3 fgrid(static_cast<unsigned>(pl.sk_tiles), FIXUP_PARTS);
        if (pl.bn == 256) fixup_kernel<256><<<fgrid, 256, 0, s>>>(p);
        else if (pl.bn == 192) fixup_kernel<192><<<fgrid, 256, 0, s>>>(p);
        else fixup_kernel<128><<<fgrid, 256, 0, s>>>(p);
        count_launch();
        KAI_TRY(check_launch("fixup_kernel"));
    }
    (void)st;
    return KAI_OK;
}

template <int BN, int KH>
static int launch_gemm_taps(const CUtensorMap& a_hi, const CUtensorMap& a_lo, const TapMaps& taps, const TcParams& p, int grid,
                            cudaStream_t s) {
    using C = Cfg<BN, 16>;
    constexpr int smem = C::STAGES * C::STAGE_BYTES + 1024 + 256;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(gemm_3xtf32_taps_kernel<BN, KH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    gemm_3xtf32_taps_kernel<BN, KH><<<grid, kThreads, smem, s>>>(a_hi, a_lo, taps, p);
    count_launch();
    count_tc_launch();
    return check_launch("gemm_3xtf32_taps_kernel");
}

// Columns of a tile of the tap-row form: kh kernel rows x xb channels, xb = 64 for kh = 3 (192 columns) and
// 256 / kh for kh = 1, 2, 4.
int taps_tile_channels(int64_t kh) { return kh == 3 ? 64 : (kh == 1 || kh == 2 || kh == 4) ? static_cast<int>(256 / kh) : 0; }

// C[M][ncols] = A'[M][K] . B^T with B in tap-row form: column ((shift * xblocks + xblk) * kh + kr) * xb + xi of C is
//   sum_k A'[m][k] * plane[shift][xblk * xb + xi][k + kr * row_step]
// a_hi / a_lo: K-major planes [M][K] (K % 4 == 0); b_hi / b_lo: planes [shifts][chan][chan_pitch] (floats;
// chan_pitch >= K + (kh - 1) * row_step, chan_pitch and row_step multiples of 4).  ncols = shifts * xblocks * kh * xb.
int gemm_tc_taps(DeviceState* st, int device, float* c, const float* a_hi, const float* a_lo, int64_t M, int64_t K,
                 const float* b_hi, const float* b_lo, int64_t chan, int64_t chan_pitch, int64_t shifts, int64_t kh,
                 int64_t row_step, cudaStream_t s) {
    const int xb = taps_tile_channels(kh);
    if (xb == 0 || shifts < 1 || shifts > 64 || (K & 3) != 0 || (chan_pitch & 3) != 0 || (row_step & 3) != 0)
        return fail(KAI_E_INVALID_ARG, "gemm_tc_taps: shape outside the tap-row form");
    const int bn = static_cast<int>(kh) * xb;
    const int64_t xblocks = (chan + xb - 1) / xb;
    const int64_t ncols = shifts * xblocks * bn;
    TcPlan pl;
    KAI_TRY(plan_tc(st, M, ncols, K, &pl, bn));
    const int64_t part_bytes = pl.slots * BM * pl.bn * 4;
    const int64_t front = round_up(st->ws_front, 256);
    if (front + part_bytes > st->ws_bytes)
        return fail(KAI_E_ALLOC, "gemm_tc_taps: the workspace reserved by the caller is too small (%lld bytes needed)",
                    (long long)(front + part_bytes));
    float* partial = (pl.slots > 0) ? reinterpret_cast<float*>(static_cast<uint8_t*>(st->ws) + front) : nullptr;
    (void)device;

    CUtensorMap ma_hi, ma_lo;
    KAI_TRY(make_map(&ma_hi, a_hi, M, K, K, BM, 16));
    KAI_TRY(make_map(&ma_lo, a_lo, M, K, K, BM, 16));
    TapMaps taps;
    for (int kr = 0; kr < kh; ++kr) {
        KAI_TRY(make_map_3d(&taps.hi[kr], b_hi + kr * row_step, K, chan, shifts, chan_pitch, chan * chan_pitch, 16, xb, 1, 64));
        KAI_TRY(make_map_3d(&taps.lo[kr], b_lo + kr * row_step, K, chan, shifts, chan_pitch, chan * chan_pitch, 16, xb, 1, 64));
    }
    for (int kr = static_cast<int>(kh); kr < 4; ++kr) { taps.hi[kr] = taps.hi[0]; taps.lo[kr] = taps.lo[0]; }

    TcParams p;
    p.M = M; p.N = ncols; p.K = K; p.ldc = ncols; p.c = c;
    p.bias = nullptr; p.leaky_alpha = nullptr; p.act = KAI_ACT_NONE; p.accumulate = 0;
    p.tiles_m = pl.tiles_m; p.tiles_n = pl.tiles_n; p.kb_total = pl.kb_total;
    p.full_tiles = pl.full_tiles; p.sk_tiles = pl.sk_tiles; p.sk_per = pl.sk_per; p.sk_ranges = pl.sk_ranges;
    p.kc_blocks = pl.kc_blocks; p.group_m = pl.group_m;
    p.partial = partial; p.status = st->status_dev;
    p.xb = xb; p.xblocks = static_cast<int>(xblocks);
    int rc;
    {
        ProfSpan span(0, s);
        if (kh == 3) rc = launch_gemm_taps<192, 3>(ma_hi, ma_lo, taps, p, pl.grid, s);
        else if (kh == 1) rc = launch_gemm_taps<256, 1>(ma_hi, ma_lo, taps, p, pl.grid, s);
        else if (kh == 2) rc = launch_gemm_taps<256, 2>(ma_hi, ma_lo, taps, p, pl.grid, s);
        else rc = launch_gemm_taps<256, 4>(ma_hi, ma_lo, taps, p, pl.grid, s);
    }
    KAI_TRY(rc);
    if (pl.sk_tiles > 0) {
        ProfSpan span(2, s);
        const dim3 fgrid(static_cast<unsigned>(pl.sk_tiles), FIXUP_PARTS);
        if (pl.bn == 256) fixup_kernel<256><<<fgrid, 256, 0, s>>>(p);
        else fixup_kernel<192><<<fgrid, 256, 0, s>>>(p);
        count_launch();
        KAI_TRY(check_launch("fixup_kernel"));
    }
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

// Partial-tile bytes gemm_tc_taps may need behind the caller's front of the workspace.
int64_t gemm_tc_taps_scratch(int64_t M, int64_t chan, int64_t shifts, int64_t kh) {
    const int xb = taps_tile_channels(kh);
    if (xb == 0) return 0;
    const int64_t bn = kh * xb, tiles = ((M + BM - 1) / BM) * shifts * ((chan + xb - 1) / xb);
    return max_slots(tiles, 148, static_cast<int>(options().split_k.load())) * BM * bn * 4 + 256;
}

// Upper bound of the scratch gemm_tc takes for an M x N x K problem: operand planes plus the partial
// tiles of a range split, for every value of the "split_k" / "tc_balance" options.
int64_t gemm_tc_scratch_bound(int64_t M, int64_t N, int64_t K) {
    const int64_t kp = round_up(K, 4);
    const int64_t bn = (N <= 128 || options().tc_bn.load() == 128) ? 128 : 256;
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const int64_t slots = max_slots(tiles, 148, static_cast<int>(options().split_k.load()));
    return 2 * round_up(M * kp * 4, 256) + 2 * round_up(N * kp * 4, 256) + slots * BM * bn * 4;
}

// `b_lo_given` (NT layout only): the caller has already written the lo plane of B against the truncated
// high part ([N][K] floats, K % 4 == 0, 16-byte aligned like b); B itself then serves as the hi operand and
// no split pass runs over it.
// `a_prep` / `b_prep`: ready-made K-major hi/lo planes of that operand (kai_operand_prepare); the matching
// pointer argument is then ignored, as is `layout` for that operand, and no split pass runs over it.
int gemm_tc(DeviceState* st, int device, int layout, float* c, const float* a, const float* b,
            int64_t M, int64_t N, int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s,
            const float* b_lo_given, const PlanePair* a_prep, const PlanePair* b_prep) {
    TcPlan pl;
    KAI_TRY(plan_tc(st, M, N, K, &pl));
    Options& opt = options();
    const int64_t kp = round_up(K, 4);
    if ((a_prep && a_prep->kp != kp) || (b_prep && b_prep->kp != kp))
        return fail(KAI_E_INVALID_ARG, "gemm_tc: a prepared operand has another reduction length");

    // Workspace: hi/lo planes of the operands that are not prepared (+ split-K partial planes).
    const int64_t a_plane = a_prep ? 0 : round_up(M * kp * 4, 256);
    const int64_t b_plane = b_prep ? 0 : round_up(N * kp * 4, 256);
    const int64_t part_bytes = pl.slots * BM * pl.bn * 4;
    const int64_t front = round_up(st->ws_front, 256);
    const int64_t need = front + 2 * a_plane + 2 * b_plane + part_bytes;
    // A caller that keeps data at the front of the workspace has sized it for this call already; growing it
    // here would move that data.
    if (front > 0 && need > st->ws_bytes)
        return fail(KAI_E_ALLOC, "gemm_tc: the workspace reserved by the caller is too small for this GEMM (%lld bytes needed)",
                    (long long)need);
    if (need > 0) KAI_TRY(ensure_workspace(st, device, need));
    uint8_t* ws = static_cast<uint8_t*>(st->ws) + front;
    float* a_hi = reinterpret_cast<float*>(ws);
    float* a_lo = reinterpret_cast<float*>(ws + a_plane);
    float* b_hi = reinterpret_cast<float*>(ws + 2 * a_plane);
    float* b_lo = reinterpret_cast<float*>(ws + 2 * a_plane + b_plane);
    float* partial = (pl.slots > 0) ? reinterpret_cast<float*>(ws + 2 * a_plane + 2 * b_plane) : nullptr;

    // An operand that already is K-major with a TMA-legal pitch can serve as its own hi plane: the
    // tensor core ignores the low 13 mantissa bits of a TF32 operand, so only the lo plane (against
    // the truncated hi) has to be written -- a third less split traffic for that operand.  Measured:
    // it pays when the operand's split is a visible share of the call (the other dimension is small,
    // e.g. the 1024-column shard of an 8-way split: 0.69 vs 0.72 ms), and costs a little on large
    // square problems, where raw mantissas make the power-bound MMA loop draw more.  (Deriving the lo
    // tile inside the GEMM kernel instead -- two extra warps converting each stage in shared memory,
    // no split pass over that operand at all -- was measured too: 0.71 ms for the same shard and 20 %
    // slower at 8192^3, because the main loop is already bound by shared-memory traffic.)
    // "tc_raw_hi": 0 = decide by shape, 1 = whenever possible, 2 = never.
    // Mixed scheme (cross terms as one BF16 MMA, see store_cross4): for long reductions, where its constant 5.6e-7
    // stays below the error of the reference's own sequential fp32 sum.  A prepared operand dictates the form.
    const int a_fmt = a_prep ? a_prep->xfmt : -1, b_fmt = b_prep ? b_prep->xfmt : -1;
    if (a_fmt == 2 || b_fmt == 1)
        return fail(KAI_E_INVALID_ARG, "gemm_tc: a prepared operand's cross-term plane was written for the other side of the product");
    if (a_fmt >= 0 && b_fmt >= 0 && (a_fmt != 0) != (b_fmt != 0))
        return fail(KAI_E_INVALID_ARG, "gemm_tc: one prepared operand has a cross-term plane, the other a TF32 lo plane");
    bool mixed = opt.tc_cross_bf16.load() != 0 && K >= kCrossMinK && (K & 7) == 0 && b_lo_given == nullptr;
    if (a_fmt >= 0) mixed = a_fmt != 0;
    if (b_fmt >= 0) mixed = b_fmt != 0;
    if (mixed && b_lo_given != nullptr)
        return fail(KAI_E_INVALID_ARG, "gemm_tc: a ready-made lo plane cannot be combined with a cross-term operand");
    const int64_t raw_mode = opt.tc_raw_hi.load();
    const bool raw_ok = raw_mode != 2 && (K & 3) == 0;
    // With bf16 cross terms the lo part against a truncated hi is twice as large, and so is its bf16 rounding error
    // (both operands raw, values whose low mantissa bits are all set, K = 2048: 1.8e-6 instead of 2.2e-7).  The mixed
    // scheme therefore reads at most A as its own hi plane, and only from K = 4096 on, where the reference's own
    // sequential sum is at 1.15e-6 and more (simulated split error then: 8.7e-7 on U[-1,1), 1.2e-6 on such values).
    const bool raw_a = !a_prep && raw_ok && layout != KAI_GEMM_TN && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                       (mixed ? (raw_mode != 2 && K >= 4096 && N <= 2048) : (raw_mode == 1 || N <= 2048));
    if (b_lo_given != nullptr && (b_prep || layout != KAI_GEMM_NT || (K & 3) != 0 ||
                                  ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(b_lo_given)) & 15) != 0))
        return fail(KAI_E_INVALID_ARG, "gemm_tc: a ready-made lo plane needs the NT layout, K %% 4 == 0 and 16-byte alignment");
    const bool raw_b = b_lo_given != nullptr ||
                       (!b_prep && raw_ok && !mixed && layout == KAI_GEMM_NT && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                        (raw_mode == 1 || M <= 2048));
    if (layout < KAI_GEMM_NT || layout > KAI_GEMM_TN) return fail(KAI_E_INVALID_ARG, "gemm_tc: unknown layout %d", layout);
    // Operand A' [M][K] and B' [N][K], by reference layout.
    {
        ProfSpan span(1, s);
        if (!a_prep) {
            if (layout == KAI_GEMM_TN)     // A = dY[K,M] -> transpose
                KAI_TRY(launch_split(a, M, K, M, true, a_hi, a_lo, kp, st->sm_count, s, mixed ? 1 : 0));
            else                           // A = X[M,K]
                KAI_TRY(launch_split(a, M, K, K, false, raw_a ? nullptr : a_hi, a_lo, kp, st->sm_count, s, mixed ? 1 : 0));
        }
        if (!b_prep && b_lo_given == nullptr) {
            if (layout == KAI_GEMM_NT)     // B = W[N,K]
                KAI_TRY(launch_split(b, N, K, K, false, raw_b ? nullptr : b_hi, b_lo, kp, st->sm_count, s, mixed ? 2 : 0));
            else                           // B = W[K,N] -> transpose
                KAI_TRY(launch_split(b, N, K, N, true, b_hi, b_lo, kp, st->sm_count, s, mixed ? 2 : 0));
        }
    }
    const float* pa_hi = a_prep ? a_prep->hi : (raw_a ? a : a_hi);
    const float* pa_lo = a_prep ? a_prep->lo : a_lo;
    const float* pb_hi = b_prep ? b_prep->hi : (raw_b ? b : b_hi);
    const float* pb_lo = b_prep ? b_prep->lo : (b_lo_given ? b_lo_given : b_lo);
    KAI_TRY(run_tc(st, pl, c, pa_hi, pa_lo, pb_hi, pb_lo, M, N, K, kp, ldc, ep, partial, st->status_dev, s, mixed));
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

// Writes the K-major hi/lo planes of one operand into caller-provided planes (kai_operand_prepare).
int split_operand(const float* src, int64_t rows, int64_t k, int64_t ld, bool transpose, float* hi, float* lo,
                  int sm_count, cudaStream_t s, int xside) {
    ProfSpan span(1, s);
    return launch_split(src, rows, k, ld, transpose, hi, lo, round_up(k, 4), sm_count, s, xside);
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded wait: one CTA waits, with the same routine every kernel of the library
// uses, on an mbarrier that nothing will ever arrive at.  After `limit_ns` the wait gives up, writes
// KAI_E_DEVICE_WAIT and the location code 99 to the status word and the kernel returns by itself;
// nothing faults or hangs, and the context stays usable.
// ---------------------------------------------------------------------------------------
namespace {
__global__ void bounded_wait_selftest_kernel(int* status, uint64_t limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // phase 0 never completes: no thread arrives
        if (!mbar_try_wait(smem_u32(&bar), 0u))
            mbar_wait_slow(smem_u32(&bar), 0u, &abort_flag, status, 99, limit_ns);
    }
    __syncthreads();
}
}  // namespace

int selftest_bounded_wait(DeviceState* st, int64_t limit_ns, cudaStream_t s) {
    bounded_wait_selftest_kernel<<<1, 32, 0, s>>>(st->status_dev, static_cast<uint64_t>(limit_ns));
    count_launch();
    return check_launch("bounded_wait_selftest_kernel");
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of the Linear forward GEMM
// ---------------------------------------------------------------------------------------
// Some callers of this library must not allocate device memory while they run: the engine's
// tracer replay re-issues a recorded list of math calls with fixed pointers and is built on the
// assumption that nothing is allocated or freed between the first run and the replays; a host
// application may also have handed every byte of HBM to its own pool, so that a cudaMalloc
// from inside a library simply fails.  The regular tensor-core path needs scratch (the hi/lo
// operand planes) and grows a cudaMalloc'ed workspace for it.  This variant keeps the scratch
// in a fixed array that is part of the library image instead: every GPU that loads the library
// holds these 32 MiB from load to exit, whether the entry point is
// used or not, and problems whose planes do not fit are refused.
namespace {

constexpr int64_t kStaticScratchBytes = int64_t(32) << 20;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Bounded-wait report of the kernels launched from here: one page of ordinary host memory per
// process, page-locked and mapped at set-up (cudaHostRegister registers existing memory; nothing is
// allocated), two ints per device.  Kernels write through the device view; the host reads its own
// copy without a synchronisation.
static __attribute__((aligned(4096))) int g_static_status_page[1024];
static std::mutex g_static_page_mu;
static bool g_static_page_registered = false;

struct StaticSetup {
    std::mutex mu;
    bool ready = false;
    unsigned char* scratch = nullptr;  // DEVICE address of g_static_scratch on this device
    int* status = nullptr;             // this device's view of its two status ints
    int* status_host = nullptr;        // the same two ints as the host sees them
    int sm_count = 0;
};
StaticSetup g_static[kMaxDevices];

// Once per device, with that device current.  In host code the name g_static_scratch is only a
// host-side handle of the device symbol: the address a kernel can use has to be asked for.
int static_setup(int device, StaticSetup** out) {
    StaticSetup* su = &g_static[device];
    std::lock_guard<std::mutex> lock(su->mu);
    if (!su->ready) {
        int major = 0, sms = 0;
        KAI_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return fail(KAI_E_INVALID_ARG, "device %d is not sm_100", device);
        KAI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        void* p = nullptr;
        KAI_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        su->scratch = static_cast<unsigned char*>(p);
        {
            std::lock_guard<std::mutex> page_lock(g_static_page_mu);
            if (!g_static_page_registered) {
                KAI_CUDA(cudaHostRegister(g_static_status_page, sizeof(g_static_status_page),
                                          cudaHostRegisterPortable | cudaHostRegisterMapped));
                g_static_page_registered = true;
            }
        }
        su->status_host = g_static_status_page + 2 * device;
        void* dp = nullptr;
        KAI_CUDA(cudaHostGetDevicePointer(&dp, su->status_host, 0));
        su->status = static_cast<int*>(dp);
        su->sm_count = sms;
        su->ready = true;
    }
    *out = su;
    return KAI_OK;
}

}  // namespace

// Status words of the allocation-free entry point on `device` (zeros when it was never used there).
void static_status_peek(int device, int out[2], bool clear) {
    out[0] = out[1] = 0;
    if (device < 0 || device >= kMaxDevices) return;
    StaticSetup* su = &g_static[device];
    std::lock_guard<std::mutex> lock(su->mu);
    if (!su->ready) return;
    volatile int* h = su->status_host;
    out[0] = h[0];
    out[1] = h[1];
    if (clear) { h[0] = 0; h[1] = 0; }
}

}  // namespace kai

extern "C" int kai_linear_forward_static(int device, float* py, const float* pw, const float* px, const float* pb,
                                         int64_t yvec, int64_t ndat, int64_t xvec, int64_t ldy, int act,
                                         const float* leaky_alpha, void* stream) {
    using namespace kai;
    if (device < 0) return fail(KAI_E_NO_HOST_PATH, "linear_forward_static: no CPU branch");
    if (device >= kMaxDevices) return fail(KAI_E_INVALID_ARG, "device %d out of range", device);
    const int64_t M = ndat, N = yvec, K = xvec;
    if (M < 0 || N < 0 || K < 1) return fail(KAI_E_INVALID_ARG, "linear_forward_static: bad dimension (xvec must be >= 1)");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "linear_forward_static: activation %d is not an elementwise epilogue", act);
    if (M == 0 || N == 0) return KAI_OK;
    if (!py || !pw || !px) return fail(KAI_E_INVALID_ARG, "linear_forward_static: null operand");
    if (ldy < N) return fail(KAI_E_INVALID_ARG, "linear_forward_static: ldy < yvec");
    // Size check in a form that cannot wrap: first a coarse bound on the row count (at most
    // 32 MiB / (8 bytes x kp) rows fit), after which the exact byte count is far below 2^63.
    if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31))
        return fail(KAI_E_TOO_LARGE, "linear_forward_static: a dimension exceeds 2^31-1");
    const int64_t kp = round_up(K, 4);
    const int64_t row_budget = kStaticScratchBytes / (8 * kp);
    const int64_t a_plane = (M <= row_budget) ? round_up(M * kp * 4, 256) : 0;
    const int64_t b_plane = (N <= row_budget) ? round_up(N * kp * 4, 256) : 0;
    if (M > row_budget || N > row_budget || 2 * a_plane + 2 * b_plane > kStaticScratchBytes)
        return fail(KAI_E_TOO_LARGE,
                    "linear_forward_static: (ndat + yvec) = %lld rows of %lld values need more than the %lld bytes of "
                    "built-in scratch (about %lld rows fit at this xvec; use kai_linear_forward for larger problems)",
                    (long long)(M + N), (long long)K, (long long)kStaticScratchBytes, (long long)row_budget);
    DeviceGuard guard;
    KAI_TRY(guard.enter(device));
    StaticSetup* su = nullptr;
    KAI_TRY(static_setup(device, &su));
    cudaStream_t s = as_stream(stream);

    // Report a bounded wait that gave up in an earlier call (the kernels write the word through
    // mapped host memory; reading it needs no synchronisation and is safe while a stream captures).
    {
        volatile int* h = su->status_host;
        if (h[0] != 0)
            return fail(KAI_E_DEVICE_WAIT, "linear_forward_static: a device-side wait ran out earlier (where=%d)", h[1]);
    }

    float* a_hi = reinterpret_cast<float*>(su->scratch);
    float* a_lo = reinterpret_cast<float*>(su->scratch + a_plane);
    float* b_hi = reinterpret_cast<float*>(su->scratch + 2 * a_plane);
    float* b_lo = reinterpret_cast<float*>(su->scratch + 2 * a_plane + b_plane);
    // Every byte of the planes that the tensor maps can reach is rewritten by the two split kernels
    // (pad columns included), so nothing of the previous call's contents has to be cleared.
    KAI_TRY(launch_split(px, M, K, K, false, a_hi, a_lo, kp, su->sm_count, s));
    KAI_TRY(launch_split(pw, N, K, K, false, b_hi, b_lo, kp, su->sm_count, s));

    const int bk = 16;
    const int bn = (N <= 128) ? 128 : 256;
    CUtensorMap maps[4];
    KAI_TRY(make_map(&maps[0], a_hi, M, K, kp, BM, bk));
    KAI_TRY(make_map(&maps[1], a_lo, M, K, kp, BM, bk));
    KAI_TRY(make_map(&maps[2], b_hi, N, K, kp, bn, bk));
    KAI_TRY(make_map(&maps[3], b_lo, N, K, kp, bn, bk));

    TcParams p;
    p.M = M; p.N = N; p.K = K; p.ldc = ldy; p.c = py;
    p.bias = pb; p.leaky_alpha = leaky_alpha; p.act = act; p.accumulate = 0;
    p.tiles_m = static_cast<int>((M + BM - 1) / BM);
    p.tiles_n = static_cast<int>((N + bn - 1) / bn);
    p.kb_total = static_cast<int>((K + bk - 1) / bk);
    // Whole tiles only: pieces of range-split tiles would need more scratch.
    p.full_tiles = p.tiles_m * p.tiles_n; p.sk_tiles = 0; p.sk_per = p.kb_total; p.sk_ranges = 0;
    int64_t kc = 16;
    while (kc * 2 <= 128 && static_cast<double>(kc * 2) <= 2.5 * sqrt(static_cast<double>(K))) kc *= 2;
    p.kc_blocks = static_cast<int>(kc / bk);
    p.group_m = 16;
    p.partial = nullptr;
    p.status = su->status;
    const int64_t work = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
    const int grid = static_cast<int>(work < su->sm_count ? work : su->sm_count);
    return (bn == 256) ? launch_gemm<256, 16>(maps, p, grid, s) : launch_gemm<128, 16>(maps, p, grid, s);
}
