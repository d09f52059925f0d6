// Implicit-GEMM convolution fed by TMA alone (sm_100a): conv2d and conv2d_backward_x of the reference
// (support/vmath.cu:3490-3655; NCHW, stride 1, zero padding, group 1; also the dilated family).
//
//   out[nd, n, r, c] = sum_{kr,kc,cn} src[nd, cn, r + dr(kr), c + dc(kc)] * w[n][(kr,kc,cn)]
//
// The source is first copied into a zero-padded channels-last tensor P[nd][row][col][channel] (channels padded to a
// multiple of 32), as two planes: the values themselves -- the tensor core ignores the low 13 mantissa bits, so they
// serve as the hi operand -- and the rounded remainders (lo operand).  With the reduction ordered (tap, channel),
// one 128-position x 32-channel operand tile of one tap is a 4-D box of P: 32 channels x `ow` columns x R rows of
// one image, shifted by the tap's offset, and TMA writes it into shared memory in exactly the 128-byte-swizzled
// K-major layout the MMA reads (a box position = one 128-byte row).  No thread touches the operands.  A tile is
// R = floor(128 / ow) whole output rows of one image; rows of the 128-row MMA tile past R*ow hold stale data, which
// only reaches accumulator rows that are never stored.  The weights are permuted to [n][(tap, channel)] and split
// into hi / lo planes by a small kernel.  Roles (one CTA per SM, persistent over tiles):
//   warps 0-1   TMA producers (warp 0: the two operand planes of a stage, warp 1: the two weight planes)
//   warps 2-5   MMA issuers (lo.hi + hi.lo + hi.hi per 8-wide k-step).  Accumulation chunk c belongs to issuer
//               c % 4: with 64 output channels an MMA occupies the tensor pipe for 48 clocks, less than one
//               thread needs to wait for a stage, build descriptors, issue and commit (measured: ~650 clocks of
//               such overhead per stage against 576 of MMA time), so a single issuer leaves the pipe idle more
//               than half the time.  Each chunk has its own accumulator buffer in tensor memory, so the
//               instruction streams never share one.
//   then 8 warps accumulate + store: tensor memory holds at most `chunk` stages of the sum (the truncating fp32
//               accumulate, as in the GEMM kernel); finished chunks are added into fp32 registers; NCHW stores.
// Every wait is bounded and reports through the device status word.
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {
namespace {

constexpr int IT_BM = 128;                 // rows of the MMA tile (TMEM lanes)
constexpr int IT_BK = 32;                  // channels per stage (128-byte rows)
constexpr int IT_A_TILE = IT_BM * IT_BK * 4;
constexpr int IT_ISSUERS = 4;               // MMA-issuing warps (<= accumulator buffers of the widest tile, 512 / 128)
constexpr int IT_FIRST_ACC = 2 + IT_ISSUERS;   // warps 0, 1: TMA producers; then the issuers; then 8 accumulate warps
constexpr int IT_THREADS = (IT_FIRST_ACC + 8) * 32;

struct ItParams {
    float* out;                 // [ndat][nout][oh*ow]
    int nout, oh, ow, pix;
    int rows_per_tile;          // R
    int tiles_per_image, m_tiles;
    int cblocks;                // padded channels / 32
    int kh, kw, ph, pw, gh, gw, flip, pt, pl;
    int k_stages, chunk_stages;
    int* status;
};

__device__ __forceinline__ float lo_part(float x) {
    const float rest = isfinite(x) ? (x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u)) : 0.0f;
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    return __uint_as_float(l);
}

// NCHW source -> zero-padded channels-last planes hi[nd][shP][swP][cp] (the values) and lo (their remainders).
// One block: PAD_ROWS padded rows, 32 columns, 32 channels, transposed through shared memory (all loads of the
// block in flight before the first store).
constexpr int PAD_ROWS = 4;
__global__ void __launch_bounds__(256)
pad_channels_last_kernel(float* __restrict__ hi, float* __restrict__ lo, const float* __restrict__ src, int cchn, int sh,
                         int sw, int shP, int swP, int pt, int pl, int cblocks) {
    __shared__ float tile[PAD_ROWS][32][33];
    const int nd = blockIdx.z / cblocks, cb = blockIdx.z - nd * cblocks;
    const int prow0 = blockIdx.y * PAD_ROWS;
    const int col0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int rr = 0; rr < PAD_ROWS; ++rr) {
        const int r = prow0 + rr - pt;
#pragma unroll
        for (int i = ty; i < 32; i += 8) {
            const int cn = cb * 32 + i, c = col0 + tx - pl;
            float v = 0.0f;
            if (cn < cchn && r >= 0 && r < sh && c >= 0 && c < sw)
                v = __ldg(src + ((static_cast<int64_t>(nd) * cchn + cn) * sh + r) * sw + c);
            tile[rr][i][tx] = v;
        }
    }
    __syncthreads();
    const int cp = cblocks * 32;
#pragma unroll
    for (int rr = 0; rr < PAD_ROWS; ++rr) {
        const int prow = prow0 + rr;
        if (prow >= shP) break;
#pragma unroll
        for (int i = ty; i < 32; i += 8) {
            const int col = col0 + i;
            if (col < swP) {
                const float v = tile[rr][tx][i];
                const int64_t o = ((static_cast<int64_t>(nd) * shP + prow) * swP + col) * cp + cb * 32 + tx;
                hi[o] = v;
                lo[o] = lo_part(v);
            }
        }
    }
}

// Weight planes [nout][(tap, channel)], channels padded with zeros to cp: w(n, cn, tap) = src[n*sn + cn*sc + tap].
__global__ void __launch_bounds__(256)
split_weights_taps_kernel(float* __restrict__ hi, float* __restrict__ lo, const float* __restrict__ src, int64_t sn,
                          int64_t sc, int nout, int cchn, int cp, int taps) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<int64_t>(nout) * taps * cp) return;
    const int cn = static_cast<int>(idx % cp);
    const int tap = static_cast<int>((idx / cp) % taps);
    const int64_t n = idx / (static_cast<int64_t>(cp) * taps);
    const float v = (cn < cchn) ? __ldg(src + n * sn + cn * sc + tap) : 0.0f;
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    float hv = __uint_as_float(h);
    if (isinf(hv) && !isinf(v)) hv = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    const float rest = isfinite(hv) ? (v - hv) : 0.0f;
    uint32_t l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
    hi[idx] = hv;
    lo[idx] = __uint_as_float(l);
}

template <int BN>
__global__ void __launch_bounds__(IT_THREADS, 1)
conv_igemm_tma_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                      const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                      const ItParams p) {
    constexpr int STAGES = (BN <= 64) ? 4 : 3;
    constexpr int IT_ACC_BUFS = 512 / BN;      // accumulator buffers: all of tensor memory, so that the issuers can run
                                               // ahead while the accumulate warps store a finished tile
    constexpr int B_TILE = BN * IT_BK * 4;
    constexpr int STAGE = 2 * IT_A_TILE + 2 * B_TILE;
    extern __shared__ uint8_t it_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(it_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    // An issuer waits only for its own stages, so it must not share "full" barriers with the others: a parity
    // wait on a barrier that is two phases behind passes at once.  Each issuer has its own ring of STAGES full
    // barriers, used in the order of its own stages; the shared-memory slot is still the global stage number.
    uint64_t* full_bar = bars;                                   // [issuers][stages] TMA -> MMA
    uint64_t* empty_bar = bars + IT_ISSUERS * STAGES;            // [stages] MMA -> TMA
    uint64_t* tmem_full = bars + (IT_ISSUERS + 1) * STAGES;      // [IT_ACC_BUFS]
    uint64_t* tmem_empty = tmem_full + IT_ACC_BUFS;  // [IT_ACC_BUFS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + IT_ACC_BUFS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < IT_ISSUERS * STAGES; ++s)
            mbar_init(smem_u32(&full_bar[s]), 2);     // one arrival (with its byte count) per producer warp
        for (int s = 0; s < STAGES; ++s) mbar_init(smem_u32(&empty_bar[s]), 1);
        for (int s = 0; s < IT_ACC_BUFS; ++s) {
            mbar_init(smem_u32(&tmem_full[s]), 1);
            mbar_init(smem_u32(&tmem_empty[s]), 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), IT_ACC_BUFS * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp <= 1) {
        // ------------------------------ TMA producers: warp 0 the operand boxes, warp 1 the weight tiles --------
        if (lane == 0) {
            if (warp == 0) { tma_prefetch_desc(&map_a_hi); tma_prefetch_desc(&map_a_lo); }
            else { tma_prefetch_desc(&map_w_hi); tma_prefetch_desc(&map_w_lo); }
            const uint32_t a_bytes = static_cast<uint32_t>(2 * p.rows_per_tile * p.ow * IT_BK * 4);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            uint32_t owner = 0;                      // issuer of the current chunk
            uint32_t given[IT_ISSUERS];              // stages handed to each issuer so far
#pragma unroll
            for (int i = 0; i < IT_ISSUERS; ++i) given[i] = 0;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                const int nd = t / p.tiles_per_image;
                const int r0 = (t - nd * p.tiles_per_image) * p.rows_per_tile;
                int ks = 0, in_chunk = 0;
                for (int kr = 0; ok && kr < p.kh; ++kr) {
                    const int row = r0 + p.pt + (p.flip ? (p.ph - kr) : (kr - p.ph)) * p.gh;
                    for (int kc = 0; ok && kc < p.kw; ++kc) {
                        const int col = p.pl + (p.flip ? (p.pw - kc) : (kc - p.pw)) * p.gw;
                        for (int cb = 0; cb < p.cblocks; ++cb, ++ks) {
                            ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 66);
                            if (!ok) break;
                            uint32_t mine = 0;
#pragma unroll
                            for (int i = 0; i < IT_ISSUERS; ++i)
                                if (static_cast<uint32_t>(i) == owner) { mine = given[i]; ++given[i]; }
                            const uint32_t full = smem_u32(&full_bar[owner * STAGES + mine % STAGES]);
                            if (++in_chunk == p.chunk_stages || ks == p.k_stages - 1) {
                                in_chunk = 0;
                                if (++owner == IT_ISSUERS) owner = 0;
                            }
                            const uint32_t base = smem_u32(smem + stage * STAGE);
                            if (warp == 0) {
                                mbar_expect_tx(full, a_bytes);
                                tma_load_4d(base, &map_a_hi, full, cb * IT_BK, col, row, nd);
                                tma_load_4d(base + IT_A_TILE, &map_a_lo, full, cb * IT_BK, col, row, nd);
                            } else {
                                mbar_expect_tx(full, 2 * B_TILE);
                                tma_load_2d(base + 2 * IT_A_TILE, &map_w_hi, full, ks * IT_BK, 0);
                                tma_load_2d(base + 2 * IT_A_TILE + B_TILE, &map_w_lo, full, ks * IT_BK, 0);
                            }
                            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                        }
                    }
                }
            }
        }
    } else if (warp < IT_FIRST_ACC) {
        // ------------------------------ MMA issuers: chunk c belongs to issuer c % IT_ISSUERS -----
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(IT_BM, BN);
            const uint32_t mine = static_cast<uint32_t>(warp - 2);
            uint32_t g = 0;          // stages before the current one (all tiles of this CTA)
            uint32_t c = 0;          // chunks before the current one
            uint32_t j = 0;          // this issuer's own stages before the current one
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                for (int ks0 = 0; ok && ks0 < p.k_stages; ks0 += p.chunk_stages, ++c) {
                    const int ks1 = min(p.k_stages, ks0 + p.chunk_stages);
                    if (c % IT_ISSUERS != mine) { g += static_cast<uint32_t>(ks1 - ks0); continue; }
                    const uint32_t acc_buf = c % IT_ACC_BUFS, acc_phase = (c / IT_ACC_BUFS) & 1u;
                    ok = mbar_wait(smem_u32(&tmem_empty[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 67);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc_buf * BN;
                    for (int ks = ks0; ks < ks1; ++ks, ++g, ++j) {
                        const uint32_t stage = g % STAGES;
                        ok = mbar_wait(smem_u32(&full_bar[mine * STAGES + j % STAGES]), (j / STAGES) & 1u, abort_flag,
                                       p.status, 68);
                        if (!ok) break;
                        const uint32_t base = smem_u32(smem + stage * STAGE);
                        const uint64_t a_hi = smem_desc_kmajor<IT_BK>(base), a_lo = smem_desc_kmajor<IT_BK>(base + IT_A_TILE);
                        const uint64_t b_hi = smem_desc_kmajor<IT_BK>(base + 2 * IT_A_TILE);
                        const uint64_t b_lo = smem_desc_kmajor<IT_BK>(base + 2 * IT_A_TILE + B_TILE);
#pragma unroll
                        for (int k = 0; k < IT_BK / 8; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            const uint32_t first = (ks == ks0 && k == 0) ? 0u : 1u;
                            umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, first);
                            umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                        umma_commit(smem_u32(&empty_bar[stage]));
                    }
                    if (!ok) break;
                    umma_commit(smem_u32(&tmem_full[acc_buf]));
                }
            }
        }
    } else {
        // ------------------------------ accumulate + store (8 warps) -------------------------------
        constexpr int COLS = BN / 2;                  // channels per thread
        const int quarter = warp & 3;                 // the TMEM lane quarter this warp may read
        const int chalf = (warp - IT_FIRST_ACC) >> 2; // which half of the channels
        const int row = quarter * 32 + lane;          // row of the MMA tile = position (row / ow, row % ow) of the box
        const int rr = row / p.ow, cc = row - rr * p.ow;
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const int n_chunks = (p.k_stages + p.chunk_stages - 1) / p.chunk_stages;
        for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
            float acc[COLS];
#pragma unroll
            for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
            for (int c = 0; c < n_chunks; ++c) {
                ok = mbar_wait(smem_u32(&tmem_full[acc_buf]), acc_phase, abort_flag, p.status, 69);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * BN + chalf * COLS);
                // all loads of the chunk in flight together, one wait
                uint32_t r[COLS / 16][16];
#pragma unroll
                for (int q = 0; q < COLS / 16; ++q) tmem_ld16(taddr + static_cast<uint32_t>(q * 16), r[q]);
                tmem_ld_wait_all();
#pragma unroll
                for (int q = 0; q < COLS / 16; ++q) {
                    pin_regs16(r[q]);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[q * 16 + i] += __uint_as_float(r[q][i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[acc_buf]));
                if (++acc_buf == IT_ACC_BUFS) { acc_buf = 0; acc_phase ^= 1u; }
            }
            if (!ok) break;
            const int nd = t / p.tiles_per_image;
            const int orow = (t - nd * p.tiles_per_image) * p.rows_per_tile + rr;
            if (rr < p.rows_per_tile && orow < p.oh) {
                float* out = p.out + (static_cast<int64_t>(nd) * p.nout + chalf * COLS) * p.pix + orow * p.ow + cc;
#pragma unroll
                for (int i = 0; i < COLS; ++i)
                    if (chalf * COLS + i < p.nout) out[static_cast<int64_t>(i) * p.pix] = acc[i];
            }
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: give copies and MMAs still in flight time to land before the CTA's memory is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, IT_ACC_BUFS * BN);
    }
}

// ---------------------------------------------------------------------------------------
// The same convolution with one operand box per kernel ROW.  The taps of one kernel row read the same image rows
// shifted by one (dilated: gw) column, so a box that is kw - 1 (x gw) columns wider than the output row holds the
// operand of all of them: tap kc is the box read from `shift(kc)` positions later, i.e. an MMA descriptor that starts
// shift(kc) * 128 bytes into the tile (measured on B200: a K-major SWIZZLE_128B descriptor may start at any 128-byte
// row of a tile, the swizzle follows the shared-memory address).  Rows of the MMA tile then run over the box's
// positions, (row, column) with W = ow + (kw - 1) gw columns, and the outputs at columns >= ow are not stored.  A tile
// is R = floor(128 / W) output rows.  Per tile the operand traffic from L2 drops from kh * kw boxes to kh (for 3 x 3:
// 516 KB -> 178 KB of the 811 KB a tile used to fetch).  One stage = (kernel row, channel block): the box (hi, lo)
// and the kw weight tiles (hi, lo) of that row; 64 output channels only (two 84 KB stages fit).  Issuer warp m issues
// tap m of every stage into an accumulator chunk of its own.
// Measured (32 x 64 x 56 x 56 -> 64 channels, 3 x 3, whole call with the padding and weight kernels): 88.6 us against
// 94.2 us with one box per tap; with a stage owned by ONE issuer (36 MMAs in a row) it was slower than per-tap boxes.
// Wait counters for one run: the issuers wait 14 % of the kernel and issue the rest of the time, 188 clocks per MMA
// each, i.e. one MMA per 63 clocks between the three of them -- the tensor pipe's floor for a 64-column MMA is 54
// (its math needs 32), so the kernel is bound by the number of MMAs, not by operand traffic.  Reading the weights' hi
// and lo tiles as one 128-row operand (a_hi x [w_hi; w_lo] = hi.hi | hi.lo in one 64-clock MMA, then a_lo x w_hi) cuts
// the MMA clocks by a quarter on paper; with 128-column accumulator chunks (four buffers instead of eight, two
// read-backs per chunk) the call measured 93.0 us: not kept.
// ---------------------------------------------------------------------------------------
constexpr int IW_BN = 64;
constexpr int IW_A_SLOT = (IT_BM + 16) * IT_BK * 4;      // the box plus the rows a shifted 128-row read can touch
constexpr int IW_B_TILE = IW_BN * IT_BK * 4;
constexpr int IW_MAX_KW = 3;
constexpr int IW_STAGE = 2 * IW_A_SLOT + 2 * IW_MAX_KW * IW_B_TILE;     // 84 KB
constexpr int IW_STAGES = 2;
constexpr int IW_ACC_BUFS = 512 / IW_BN;

struct IwParams {
    ItParams it;
    int box_w;            // W
    int col_base;         // first column of the box in the padded plane
    int shift[IW_MAX_KW]; // positions by which tap kc starts later
};

__global__ void __launch_bounds__(IT_THREADS, 1)
conv_igemm_wide_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                       const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                       const IwParams q) {
    const ItParams& p = q.it;
    extern __shared__ uint8_t it_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(it_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + IW_STAGES * IW_STAGE);
    // Every issuer works on every stage (issuer m on the stage's tap m), so they follow the stages' barriers in
    // lockstep and one ring of full barriers serves all of them.
    uint64_t* full_bar = bars;                                    // [stages]  TMA (2 producers) -> issuers
    uint64_t* empty_bar = bars + IW_STAGES;                       // [stages]  kw issuers -> TMA
    uint64_t* tmem_full = bars + 2 * IW_STAGES;                   // [IW_ACC_BUFS]
    uint64_t* tmem_empty = tmem_full + IW_ACC_BUFS;               // [IW_ACC_BUFS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + IW_ACC_BUFS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < IW_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 2);
            mbar_init(smem_u32(&empty_bar[s]), static_cast<uint32_t>(p.kw));
        }
        for (int s = 0; s < IW_ACC_BUFS; ++s) {
            mbar_init(smem_u32(&tmem_full[s]), 1);
            mbar_init(smem_u32(&tmem_empty[s]), 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // the rows behind a box are read by shifted descriptors (into accumulator rows that are never stored): give them
    // finite contents once
    for (int i = threadIdx.x; i < IW_STAGES * 2 * (IW_A_SLOT / 4); i += blockDim.x) {
        const int slot = i / (IW_A_SLOT / 4), w = i - slot * (IW_A_SLOT / 4);
        reinterpret_cast<float*>(smem + (slot >> 1) * IW_STAGE + (slot & 1) * IW_A_SLOT)[w] = 0.0f;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int stages_per_tile = p.kh * p.cblocks;          // wide stages: (kernel row, channel block)

    if (warp <= 1) {
        // ------------------------------ TMA producers: warp 0 the boxes, warp 1 the weight tiles --------
        if (lane == 0) {
            if (warp == 0) { tma_prefetch_desc(&map_a_hi); tma_prefetch_desc(&map_a_lo); }
            else { tma_prefetch_desc(&map_w_hi); tma_prefetch_desc(&map_w_lo); }
            const uint32_t a_bytes = static_cast<uint32_t>(2 * p.rows_per_tile * q.box_w * IT_BK * 4);
            int stage = 0;
            uint32_t phase = 0, g = 0;       // g: stages before the current one (all tiles of this CTA)
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                const int nd = t / p.tiles_per_image;
                const int r0 = (t - nd * p.tiles_per_image) * p.rows_per_tile;
                for (int kr = 0; ok && kr < p.kh; ++kr) {
                    const int row = r0 + p.pt + (p.flip ? (p.ph - kr) : (kr - p.ph)) * p.gh;
                    for (int cb = 0; cb < p.cblocks; ++cb, ++g) {
                        ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 76);
                        if (!ok) break;
                        const uint32_t full = smem_u32(&full_bar[stage]);
                        const uint32_t base = smem_u32(smem + stage * IW_STAGE);
                        if (warp == 0) {
                            mbar_expect_tx(full, a_bytes);
                            tma_load_4d(base, &map_a_hi, full, cb * IT_BK, q.col_base, row, nd);
                            tma_load_4d(base + IW_A_SLOT, &map_a_lo, full, cb * IT_BK, q.col_base, row, nd);
                        } else {
                            mbar_expect_tx(full, static_cast<uint32_t>(2 * p.kw * IW_B_TILE));
                            for (int kc = 0; kc < p.kw; ++kc) {
                                const int ks = (kr * p.kw + kc) * p.cblocks + cb;
                                tma_load_2d(base + 2 * IW_A_SLOT + kc * IW_B_TILE, &map_w_hi, full, ks * IT_BK, 0);
                                tma_load_2d(base + 2 * IW_A_SLOT + (IW_MAX_KW + kc) * IW_B_TILE, &map_w_lo, full, ks * IT_BK, 0);
                            }
                        }
                        if (++stage == IW_STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp < IT_FIRST_ACC) {
        // ------------------------------ MMA issuers: issuer m issues tap m of every stage -----
        const int kc = warp - 2;
        if (lane == 0 && kc < p.kw) {
            const uint32_t idesc = instr_desc_tf32(IT_BM, IW_BN);
            const uint32_t a_off = static_cast<uint32_t>(q.shift[kc] * IT_BK * 4);
            uint32_t g = 0;          // stages before the current one (all tiles of this CTA)
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                for (int st = 0; ok && st < stages_per_tile; ++st, ++g) {
                    const uint32_t stage = g % IW_STAGES;
                    const uint32_t c = g * static_cast<uint32_t>(p.kw) + static_cast<uint32_t>(kc);   // chunk number
                    const uint32_t acc_buf = c % IW_ACC_BUFS, acc_phase = (c / IW_ACC_BUFS) & 1u;
                    ok = mbar_wait(smem_u32(&tmem_empty[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 77) &&
                         mbar_wait(smem_u32(&full_bar[stage]), (g / IW_STAGES) & 1u, abort_flag, p.status, 78);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + stage * IW_STAGE);
                    const uint32_t d_tmem = tmem_base + acc_buf * IW_BN;
                    const uint64_t a_hi = smem_desc_kmajor<IT_BK>(base + a_off);
                    const uint64_t a_lo = smem_desc_kmajor<IT_BK>(base + IW_A_SLOT + a_off);
                    const uint64_t b_hi = smem_desc_kmajor<IT_BK>(base + 2 * IW_A_SLOT + kc * IW_B_TILE);
                    const uint64_t b_lo = smem_desc_kmajor<IT_BK>(base + 2 * IW_A_SLOT + (IW_MAX_KW + kc) * IW_B_TILE);
#pragma unroll
                    for (int k = 0; k < IT_BK / 8; ++k) {
                        const uint64_t adv = static_cast<uint64_t>(k * 2);
                        umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, k == 0 ? 0u : 1u);
                        umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                        umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                    }
                    umma_commit(smem_u32(&tmem_full[acc_buf]));
                    umma_commit(smem_u32(&empty_bar[stage]));
                }
            }
        }
    } else {
        // ------------------------------ accumulate + store (8 warps) -------------------------------
        constexpr int COLS = IW_BN / 2;
        const int quarter = warp & 3;
        const int chalf = (warp - IT_FIRST_ACC) >> 2;
        const int row = quarter * 32 + lane;          // position (row / W, row % W) of the box
        const int rr = row / q.box_w, cc = row - rr * q.box_w;
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const int n_chunks = stages_per_tile * p.kw;
        for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
            float acc[COLS];
#pragma unroll
            for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
            for (int c = 0; c < n_chunks; ++c) {
                ok = mbar_wait(smem_u32(&tmem_full[acc_buf]), acc_phase, abort_flag, p.status, 79);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * IW_BN + chalf * COLS);
                uint32_t r[COLS / 16][16];
#pragma unroll
                for (int u = 0; u < COLS / 16; ++u) tmem_ld16(taddr + static_cast<uint32_t>(u * 16), r[u]);
                tmem_ld_wait_all();
#pragma unroll
                for (int u = 0; u < COLS / 16; ++u) {
                    pin_regs16(r[u]);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[u * 16 + i] += __uint_as_float(r[u][i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[acc_buf]));
                if (++acc_buf == IW_ACC_BUFS) { acc_buf = 0; acc_phase ^= 1u; }
            }
            if (!ok) break;
            const int nd = t / p.tiles_per_image;
            const int orow = (t - nd * p.tiles_per_image) * p.rows_per_tile + rr;
            if (rr < p.rows_per_tile && cc < p.ow && orow < p.oh) {
                float* out = p.out + (static_cast<int64_t>(nd) * p.nout + chalf * COLS) * p.pix + orow * p.ow + cc;
#pragma unroll
                for (int i = 0; i < COLS; ++i)
                    if (chalf * COLS + i < p.nout) out[static_cast<int64_t>(i) * p.pix] = acc[i];
            }
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
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

int launch_igemm_wide(const CUtensorMap maps[4], const IwParams& q, int grid, cudaStream_t s) {
    constexpr int smem = IW_STAGES * IW_STAGE + 512 + 1024;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(conv_igemm_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    conv_igemm_wide_kernel<<<grid, IT_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], q);
    count_launch();
    count_tc_launch();
    return check_launch("conv_igemm_wide_kernel");
}

template <int BN>
int launch_igemm_tma(const CUtensorMap maps[4], const ItParams& p, int grid, cudaStream_t s) {
    constexpr int stages = (BN <= 64) ? 4 : 3;
    constexpr int smem = stages * (2 * IT_A_TILE + 2 * BN * IT_BK * 4) + 512 + 1024;   // barriers (<= 33) + alignment
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(conv_igemm_tma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    conv_igemm_tma_kernel<BN><<<grid, IT_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], p);
    count_launch();
    count_tc_launch();
    return check_launch("conv_igemm_tma_kernel");
}

inline int64_t al256(int64_t v) { return (v + 255) / 256 * 256; }

}  // namespace

// Shapes the TMA-fed kernel takes: whole output rows must fill most of a 128-row tile, and rounding the channels up
// to a multiple of 32 must not add more than a quarter.
bool conv_igemm_tma_fits(int64_t ndat, int64_t cchn, int64_t oh, int64_t ow, int64_t nout, int64_t kh, int64_t kw,
                         int64_t shP, int64_t swP) {
    if (nout < 16 || nout > 128 || ow < 1 || ow > IT_BM || cchn < 24) return false;
    const int64_t cp = round_up(cchn, 32), rows = IT_BM / ow;
    if ((cp - cchn) * 4 > cchn) return false;
    if (rows * ow * 4 < IT_BM * 3) return false;
    if (ndat * oh * ow < 4 * IT_BM || kh * kw * cp > (int64_t(1) << 20)) return false;
    if (shP > 65535 || ndat * (cp / 32) > 65535) return false;                  // grid of the padding kernel
    return ndat * shP * swP * cp < (int64_t(1) << 31) && ndat * nout * oh * ow < (int64_t(1) << 40);
}

// Scratch the call needs at `scratch` (256-byte aligned): two padded planes and two weight planes.
int64_t conv_igemm_tma_bytes(int64_t ndat, int64_t cchn, int64_t nout, int64_t kh, int64_t kw, int64_t shP, int64_t swP) {
    const int64_t cp = round_up(cchn, 32);
    return 2 * al256(ndat * shP * swP * cp * 4) + 2 * al256(nout * kh * kw * cp * 4);
}

// out[nd][n][pix] of the convolution of src[nd][cchn][sh][sw] with weights w(n, cn, tap) = wsrc[n*wsn + cn*wsc + tap].
int conv_igemm_tma(DeviceState* st, float* out, const float* src, const float* wsrc, int64_t wsn, int64_t wsc,
                   void* scratch, int64_t ndat, int64_t cchn, int64_t sh, int64_t sw, int64_t oh, int64_t ow,
                   int64_t nout, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t gh, int64_t gw, int flip,
                   int shP, int swP, int pt, int pl, cudaStream_t s) {
    const int64_t cp = round_up(cchn, 32), cblocks = cp / 32, taps = kh * kw, K = taps * cp;
    const int64_t plane_bytes = al256(ndat * shP * swP * cp * 4), w_bytes = al256(nout * K * 4);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    float* a_hi = reinterpret_cast<float*>(base);
    float* a_lo = reinterpret_cast<float*>(base + plane_bytes);
    float* w_hi = reinterpret_cast<float*>(base + 2 * plane_bytes);
    float* w_lo = reinterpret_cast<float*>(base + 2 * plane_bytes + w_bytes);

    // (the tensor maps are encoded before the first launch so that the three kernels follow each other closely)
    const int bn = (nout <= 64) ? 64 : 128;
    // one box per kernel row (see conv_igemm_wide_kernel) where the kernel has 2 or 3 columns, 64 output channels
    // suffice and the widened row still fills most of a 128-row tile
    const int64_t box_w = ow + (kw - 1) * gw;
    const int col_first = static_cast<int>(pl + (flip ? (pw - (kw - 1)) : (0 - pw)) * gw);
    const bool wide = options().conv_wide.load() != 0 && bn == 64 && kw >= 2 && kw <= IW_MAX_KW && (kw - 1) * gw <= 16 &&
                      box_w <= IT_BM && (IT_BM / box_w) * box_w * 4 >= IT_BM * 3 && col_first >= 0 &&
                      col_first + box_w <= swP;
    const int rows = static_cast<int>(IT_BM / (wide ? box_w : ow));
    CUtensorMap maps[4];
    KAI_TRY(make_map_4d_sw128(&maps[0], a_hi, cp, swP, shP, ndat, static_cast<int>(wide ? box_w : ow), rows));
    KAI_TRY(make_map_4d_sw128(&maps[1], a_lo, cp, swP, shP, ndat, static_cast<int>(wide ? box_w : ow), rows));
    KAI_TRY(make_map(&maps[2], w_hi, nout, K, K, bn, IT_BK));
    KAI_TRY(make_map(&maps[3], w_lo, nout, K, K, bn, IT_BK));

    dim3 pgrid(static_cast<unsigned>((swP + 31) / 32), static_cast<unsigned>((shP + PAD_ROWS - 1) / PAD_ROWS),
               static_cast<unsigned>(ndat * cblocks));
    pad_channels_last_kernel<<<pgrid, 256, 0, s>>>(a_hi, a_lo, src, static_cast<int>(cchn), static_cast<int>(sh),
                                                   static_cast<int>(sw), shP, swP, pt, pl, static_cast<int>(cblocks));
    count_launch();
    KAI_TRY(check_launch("pad_channels_last_kernel"));
    const int64_t wcount = nout * K;
    split_weights_taps_kernel<<<static_cast<unsigned>((wcount + 255) / 256), 256, 0, s>>>(
        w_hi, w_lo, wsrc, wsn, wsc, static_cast<int>(nout), static_cast<int>(cchn), static_cast<int>(cp),
        static_cast<int>(taps));
    count_launch();
    KAI_TRY(check_launch("split_weights_taps_kernel"));

    ItParams p;
    p.out = out;
    p.nout = static_cast<int>(nout); p.oh = static_cast<int>(oh); p.ow = static_cast<int>(ow);
    p.pix = static_cast<int>(oh * ow);
    p.rows_per_tile = rows;
    p.tiles_per_image = static_cast<int>((oh + rows - 1) / rows);
    p.m_tiles = static_cast<int>(ndat) * p.tiles_per_image;
    p.cblocks = static_cast<int>(cblocks);
    p.kh = static_cast<int>(kh); p.kw = static_cast<int>(kw); p.ph = static_cast<int>(ph); p.pw = static_cast<int>(pw);
    p.gh = static_cast<int>(gh); p.gw = static_cast<int>(gw); p.flip = flip; p.pt = pt; p.pl = pl;
    p.k_stages = static_cast<int>(taps * cblocks);
    // promotion interval as in the GEMM kernel: reduction held in tensor memory <= 2.5 * sqrt(K)
    int64_t kc = 32;
    while (kc * 2 <= 128 && static_cast<double>(kc * 2) <= 2.5 * sqrt(static_cast<double>(cchn * taps))) kc *= 2;
    p.chunk_stages = static_cast<int>(kc / IT_BK);
    p.status = st->status_dev;
    const int grid = p.m_tiles < st->sm_count ? p.m_tiles : st->sm_count;
    if (wide) {
        IwParams q;
        q.it = p;
        q.box_w = static_cast<int>(box_w);
        q.col_base = col_first;
        for (int t = 0; t < IW_MAX_KW; ++t)
            q.shift[t] = (t < kw) ? static_cast<int>((flip ? (kw - 1 - t) : t) * gw) : 0;
        KAI_TRY(launch_igemm_wide(maps, q, grid, s));
    } else {
        KAI_TRY(bn == 64 ? launch_igemm_tma<64>(maps, p, grid, s) : launch_igemm_tma<128>(maps, p, grid, s));
    }
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai
