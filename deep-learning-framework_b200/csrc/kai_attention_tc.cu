// mult_on_heads on the tcgen05 tensor cores (sm_100a) for the attention shape of the benchmark
// family: head width npiece = 64.
//
//   probs[b,q,k,h] = coef * sum_p K[b,k,h*64+p] * Q[b,q,h*64+p]      (support/vmath.cu:6729-6750)
//
// Q and K are [nbat*ntimes, nvec] row-major matrices whose column block h*64..h*64+63 is head h,
// so a (128 queries x 64) or (64 keys x 64) operand tile of one head is a plain 2-D TMA box.
// One work item = (batch b, 128 keys, 64 queries, up to 4 heads).  Keys sit on the 128 TMEM lanes
// (the "M" side of the MMA) because consecutive keys of one query are adjacent in probs: a warp
// of the epilogue, one key per lane, then writes a contiguous 1 KB stretch per query.
//   * split kernels first write hi/lo TF32 planes of Q and K (one HBM pass over 2 small tensors);
//   * warp 0 streams, per head, the four operand tiles (K hi/lo, Q hi/lo, 96 KB) into a 2-stage ring;
//   * warp 1 issues, per head, 16 cross-term MMAs (lo.hi, hi.lo) and then the 8 hi.hi MMAs of the
//     64-wide reduction into that head's own 64 TMEM columns (4 heads x 64 columns, double
//     buffered so the next item's MMAs overlap the read-back).  Cross terms go first so that the
//     truncating fp32 accumulate of the tensor core acts on a full-size sum only 8 times
//     (measured drift ~2e-8 per accumulate);
//   * warps 2-9 read the four accumulators back 16 queries at a time and store, for every (q,k),
//     the four head values as one 16-byte piece of the head-minor probs tensor.
// Wait counters compiled in for one run (benchmark shape, 217 k clocks per CTA): the epilogue warps are busy 66 % of the
// kernel -- 32 store instructions per thread and item, each a warp-wide write of 32 half-filled 32-byte sectors (four
// of the eight heads of a (q, k)), about 0.8 sectors per clock and SM -- the MMA thread issues for 64 % (104 clocks per
// 128 x 64 x 8 MMA) and waits for operands 35 %, the TMA thread waits for a free stage 56 %.  The stores of the
// head-minor layout bound the kernel; whole sectors need all eight heads in one thread, i.e. all 512 tensor-memory
// columns and no overlap of MMAs and read-back (built and measured: slower).  A second issuing warp (heads
// alternating between the two) was built and measured as well: 0.4687 against 0.4696 ms for the three calls.
// All waits are bounded (see kai_gemm_tc.cu).  Shapes outside this fast path return 1 and are
// served by the warp-MMA / CUDA-core kernels.
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {

int split_planes(const float* src, int64_t rows, int64_t cols, float* hi, float* lo, int sm_count, cudaStream_t s);
int split_lo_pair(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, cudaStream_t s);

namespace {

constexpr int AT_BM = 128;       // keys per tile (TMEM lanes)
constexpr int AT_BN = 64;        // queries per tile
constexpr int AT_P = 64;         // head width
constexpr int AT_HG = 4;         // heads per work item
constexpr int AT_THREADS = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int AT_KBOX = AT_BM * 32 * 4;   // one 128-key x 32 fp32 box   (16 KB)
constexpr int AT_QBOX = AT_BN * 32 * 4;   // one  64-query x 32 fp32 box ( 8 KB)
constexpr int AT_STAGE = 4 * AT_KBOX + 4 * AT_QBOX;   // K hi/lo + Q hi/lo, two boxes each = 96 KB
constexpr int AT_ACC_COLS = AT_HG * AT_BN;            // TMEM columns of one accumulator buffer
constexpr int AT_STAGES = 2;

struct AtParams {
    float* pp;
    const float* coef;
    int nbat, ntimes, nhead;
    int q_tiles, k_tiles, h_groups;
    int* status;
};

struct AtItem { int b, q0, k0, hg, nh; };

__device__ __forceinline__ bool at_item(const AtParams& p, int w, AtItem& it) {
    const int total = p.nbat * p.q_tiles * p.k_tiles * p.h_groups;
    if (w >= total) return false;
    const int hgi = w % p.h_groups; w /= p.h_groups;   // head groups of one (q,k) tile back to back
    const int qt = w % p.q_tiles; w /= p.q_tiles;
    const int kt = w % p.k_tiles;
    it.b = w / p.k_tiles;
    it.q0 = qt * AT_BN;
    it.k0 = kt * AT_BM;
    it.hg = hgi * AT_HG;
    it.nh = min(AT_HG, p.nhead - it.hg);
    return true;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
mult_on_heads_tc_kernel(const __grid_constant__ CUtensorMap map_q_hi, const __grid_constant__ CUtensorMap map_q_lo,
                        const __grid_constant__ CUtensorMap map_k_hi, const __grid_constant__ CUtensorMap map_k_lo,
                        const AtParams p) {
    extern __shared__ uint8_t at_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AT_STAGES * AT_STAGE);
    uint64_t* full_bar = bars;                    // [2] TMA -> MMA
    uint64_t* empty_bar = bars + AT_STAGES;       // [2] MMA -> TMA
    uint64_t* tmem_full_bar = bars + 2 * AT_STAGES;       // [2] MMA -> epilogue
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;         // [2] epilogue -> MMA
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_q_hi); tma_prefetch_desc(&map_q_lo);
            tma_prefetch_desc(&map_k_hi); tma_prefetch_desc(&map_k_lo);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            AtItem it;
            for (int w = blockIdx.x; ok && at_item(p, w, it); w += gridDim.x) {
                const int row_q = it.b * p.ntimes + it.q0;
                const int row_k = it.b * p.ntimes + it.k0;
                for (int h = 0; h < it.nh; ++h) {
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 11);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&full_bar[stage]);
                    uint8_t* base = smem + stage * AT_STAGE;
                    mbar_expect_tx(full, AT_STAGE);
                    const int col = (it.hg + h) * AT_P;
                    // A tile that straddles the end of a batch item reads rows of the next item (or
                    // zero fill past the tensor); those rows/keys are never stored.
#pragma unroll
                    for (int kb = 0; kb < 2; ++kb) {
                        tma_load_2d(smem_u32(base + kb * AT_KBOX), &map_k_hi, full, col + kb * 32, row_k);
                        tma_load_2d(smem_u32(base + (2 + kb) * AT_KBOX), &map_k_lo, full, col + kb * 32, row_k);
                        tma_load_2d(smem_u32(base + 4 * AT_KBOX + kb * AT_QBOX), &map_q_hi, full, col + kb * 32, row_q);
                        tma_load_2d(smem_u32(base + 4 * AT_KBOX + (2 + kb) * AT_QBOX), &map_q_lo, full, col + kb * 32,
                                    row_q);
                    }
                    if (++stage == AT_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(AT_BM, AT_BN);
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            int acc_buf = 0;
            bool ok = true;
            AtItem it;
            for (int w = blockIdx.x; ok && at_item(p, w, it); w += gridDim.x) {
                ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 12);
                if (!ok) break;
                tc_fence_after();
                for (int h = 0; h < it.nh; ++h) {
                    ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, 13);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t base = smem_u32(smem + stage * AT_STAGE);
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc_buf * AT_ACC_COLS + h * AT_BN);
                    uint32_t first = 0u;
                    // cross terms of the whole 64-wide reduction first ...
#pragma unroll
                    for (int kb = 0; kb < 2; ++kb) {
                        const uint64_t k_hi = smem_desc_kmajor<32>(base + kb * AT_KBOX);
                        const uint64_t k_lo = smem_desc_kmajor<32>(base + (2 + kb) * AT_KBOX);
                        const uint64_t q_hi = smem_desc_kmajor<32>(base + 4 * AT_KBOX + kb * AT_QBOX);
                        const uint64_t q_lo = smem_desc_kmajor<32>(base + 4 * AT_KBOX + (2 + kb) * AT_QBOX);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);   // +32 bytes inside the 128-byte span
                            umma_tf32(d_tmem, k_lo + adv, q_hi + adv, idesc, first);
                            first = 1u;
                            umma_tf32(d_tmem, k_hi + adv, q_lo + adv, idesc, 1u);
                        }
                    }
                    // ... then the dominant hi.hi chain
#pragma unroll
                    for (int kb = 0; kb < 2; ++kb) {
                        const uint64_t k_hi = smem_desc_kmajor<32>(base + kb * AT_KBOX);
                        const uint64_t q_hi = smem_desc_kmajor<32>(base + 4 * AT_KBOX + kb * AT_QBOX);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            umma_tf32(d_tmem, k_hi + adv, q_hi + adv, idesc, 1u);
                        }
                    }
                    umma_commit(smem_u32(&empty_bar[stage]));
                    if (++stage == AT_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&tmem_full_bar[acc_buf]));
                acc_buf ^= 1;
                if (acc_buf == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quarter = warp & 3;            // TMEM lane quarter this warp may read: 32 keys
        const int qhalf = (warp - 2) >> 2;       // which 32 queries of the tile
        const float coef = (p.coef != nullptr) ? __ldg(p.coef) : 0.0f;
        const bool vec_out = (p.nhead % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.pp) & 15) == 0);
        uint32_t acc_phase = 0;
        int acc_buf = 0;
        bool ok = true;
        AtItem it;
        for (int w = blockIdx.x; ok && at_item(p, w, it); w += gridDim.x) {
            ok = mbar_wait(smem_u32(&tmem_full_bar[acc_buf]), acc_phase, abort_flag, p.status, 14);
            if (!ok) break;
            tc_fence_after();
            const int k = it.k0 + quarter * 32 + lane;    // this lane's key
            float* key_out = p.pp + (static_cast<int64_t>(it.b) * p.ntimes * p.ntimes + k) * p.nhead + it.hg;
#pragma unroll 1
            for (int chunk = 0; chunk < 2; ++chunk) {
                const int qcol = qhalf * 32 + chunk * 16;
                uint32_t r[AT_HG][16];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * AT_ACC_COLS + qcol);
#pragma unroll
                for (int h = 0; h < AT_HG; ++h) tmem_ld16(taddr + h * AT_BN, r[h]);
                tmem_ld_wait_all();
#pragma unroll
                for (int h = 0; h < AT_HG; ++h) pin_regs16(r[h]);
                if (k < p.ntimes) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int q = it.q0 + qcol + j;
                        if (q < p.ntimes) {
                            float* out = key_out + static_cast<int64_t>(q) * p.ntimes * p.nhead;
                            if (vec_out && it.nh == AT_HG) {
                                *reinterpret_cast<float4*>(out) =
                                    make_float4(__uint_as_float(r[0][j]) * coef, __uint_as_float(r[1][j]) * coef,
                                                __uint_as_float(r[2][j]) * coef, __uint_as_float(r[3][j]) * coef);
                            } else {
#pragma unroll
                                for (int h = 0; h < AT_HG; ++h)
                                    if (h < it.nh) out[h] = __uint_as_float(r[h][j]) * coef;
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_buf]));
            acc_buf ^= 1;
            if (acc_buf == 0) acc_phase ^= 1u;
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

// Returns 1 when the shape is outside the fast path.
int attn_mult_on_heads_tc(DeviceState* st, int device, float* pp, const float* pK, const float* pQ, int64_t nbat,
                          int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, const float* coef,
                          cudaStream_t s) {
    const int64_t rows = nbat * ntimes;
    const bool ok = npiece == AT_P && nvec == nhead * npiece && ntimes >= 64 && rows < (int64_t(1) << 31) &&
                    nhead < (1 << 16) && nbat * ((ntimes + AT_BM - 1) / AT_BM) * ((ntimes + AT_BN - 1) / AT_BN) *
                                                 ((nhead + AT_HG - 1) / AT_HG) < (int64_t(1) << 30);
    if (!ok) return 1;
    const int64_t plane = round_up(rows * nvec * 4, 256);
    KAI_TRY(ensure_workspace(st, device, 4 * plane));
    uint8_t* ws = static_cast<uint8_t*>(st->ws);
    float* q_hi = reinterpret_cast<float*>(ws);
    float* q_lo = reinterpret_cast<float*>(ws + plane);
    float* k_hi = reinterpret_cast<float*>(ws + 2 * plane);
    float* k_lo = reinterpret_cast<float*>(ws + 3 * plane);
    // 16-byte aligned Q and K serve as their own hi operands (the tensor core ignores the low 13 mantissa
    // bits); then only the lo planes are written, by one launch.
    const bool raw_hi = ((reinterpret_cast<uintptr_t>(pQ) | reinterpret_cast<uintptr_t>(pK)) & 15) == 0;
    if (raw_hi) {
        KAI_TRY(split_lo_pair(pQ, pK, rows * nvec, q_lo, k_lo, s));
    } else {
        KAI_TRY(split_planes(pQ, rows, nvec, q_hi, q_lo, st->sm_count, s));
        KAI_TRY(split_planes(pK, rows, nvec, k_hi, k_lo, st->sm_count, s));
    }
    CUtensorMap maps[4];
    KAI_TRY(make_map(&maps[0], raw_hi ? pQ : q_hi, rows, nvec, nvec, AT_BN, 32));
    KAI_TRY(make_map(&maps[1], q_lo, rows, nvec, nvec, AT_BN, 32));
    KAI_TRY(make_map(&maps[2], raw_hi ? pK : k_hi, rows, nvec, nvec, AT_BM, 32));
    KAI_TRY(make_map(&maps[3], k_lo, rows, nvec, nvec, AT_BM, 32));
    AtParams p;
    p.pp = pp; p.coef = coef;
    p.nbat = static_cast<int>(nbat); p.ntimes = static_cast<int>(ntimes); p.nhead = static_cast<int>(nhead);
    p.q_tiles = static_cast<int>((ntimes + AT_BN - 1) / AT_BN);
    p.k_tiles = static_cast<int>((ntimes + AT_BM - 1) / AT_BM);
    p.h_groups = static_cast<int>((nhead + AT_HG - 1) / AT_HG);
    p.status = st->status_dev;
    const int64_t items = static_cast<int64_t>(p.nbat) * p.q_tiles * p.k_tiles * p.h_groups;
    const int grid = static_cast<int>(items < st->sm_count ? items : st->sm_count);
    constexpr int smem = AT_STAGES * AT_STAGE + 1024 + 256;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(mult_on_heads_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    mult_on_heads_tc_kernel<<<grid, AT_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], p);
    count_launch();
    count_tc_launch();
    KAI_TRY(check_launch("mult_on_heads_tc_kernel"));
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai

namespace kai {

// =======================================================================================
// mix_values on the tcgen05 tensor cores, head width 64:
//
//   out[b,q,h,p] = sum_k probs[b,q,k,h] * V[b,k,h*64+p]             (support/vmath.cu:6977-6997)
//
// Per head this is O_h[q,p] = P_h[q,k] . V_h[k,p] with the reduction over the keys.  P_h is not a
// matrix a 2-D bulk copy can fetch (in probs the key index is strided by nhead), so:
//   * one work item = (batch b, 128 queries, 2 heads); its accumulator is 128 x (2 x 64) fp32;
//   * warp 0 streams two things with TMA: the raw probs slab of the next 16 keys as a 3-D box
//     [128 q][16 k][4 heads] (a 16-byte piece per (q,k), the item's head pair is one half of it),
//     and the V_h^T tiles (64 x 16 keys, hi/lo) from planes written by a transposing split kernel.
//     (Measured for the benchmark shape: 244 us; 343 us when the converter threads fetch the pieces
//     with cp.async instead; 290 us with four heads per item.  In all variants the time follows the
//     number of MMAs: a 128 x 64 x 8 TF32 MMA costs ~160 clocks here, five times its tensor time.
//     Wait counters compiled in for one run say where the time goes: the TMA thread spends 62 % of the kernel
//     waiting for a free raw slot, the converter warps are busy 47 % and wait for raw data 23 %, the MMA thread
//     waits for converted tiles 38 %.  Eight converter warps instead of four halve the conversion time and change
//     nothing else: the slab's box has a 16-byte inner extent, 2048 pieces per stage, and the copy engine delivers
//     ~0.6 such pieces per clock per SM -- the raw slabs are the limiter.)
//   * warps 4-7 turn each raw slab into the A operand: per (q,k) they read the 16-byte piece from
//     shared memory, split the item's two values into hi/lo TF32 and store them into that head's
//     128 x 16 K-major tiles, in the 64-byte-swizzled layout the MMA descriptors expect;
//   * warp 1 issues 3 MMAs per head and 8-key step;
//   * tensor memory only ever holds 32 keys of the sum: warps 8-15 add each finished chunk into
//     fp32 registers (round to nearest) while the other TMEM buffer fills, as the GEMM does.
// =======================================================================================
int split_planes_transposed(const float* src, int64_t batch, int64_t k, int64_t rows, float* hi, float* lo,
                            cudaStream_t s);

namespace {

constexpr int MV_BM = 128;                  // queries per item
constexpr int MV_P = 64;                    // head width = N of one MMA
constexpr int MV_HP = 2;                    // heads per item
constexpr int MV_BOXH = 4;                  // heads per raw 16-byte piece
constexpr int MV_BK = 16;                   // keys per stage (64-byte rows)
constexpr int MV_A_TILE = MV_BM * MV_BK * 4;   // 8 KB
constexpr int MV_B_TILE = MV_P * MV_BK * 4;    // 4 KB
constexpr int MV_STAGE = MV_HP * 2 * (MV_A_TILE + MV_B_TILE);   // 48 KB
constexpr int MV_STAGES = 3;
constexpr int MV_RAW = MV_BM * MV_BK * MV_BOXH * 4;             // 32 KB raw slab
constexpr int MV_RAW_STAGES = 2;
constexpr int MV_ACC_COLS = 2 * MV_HP * MV_P;   // TMEM columns per buffer: [h0 main][h1 main][h0 cross][h1 cross]
constexpr int MV_CHUNK_STAGES = 2;          // 32 keys accumulate in tensor memory, then promote
constexpr int MV_THREADS = 512;             // warp 0 TMA, 1 MMA, 2-3 idle, 4-7 convert, 8-15 accumulate + store

struct MvParams {
    float* py;
    int nbat, ntimes, nhead;
    int q_tiles, h_pairs, k_stages;
    int* status;
};

struct MvItem { int b, q0, h0, nh; };

__device__ __forceinline__ bool mv_item(const MvParams& p, int w, MvItem& it) {
    const int total = p.nbat * p.q_tiles * p.h_pairs;
    if (w >= total) return false;
    const int hp = w % p.h_pairs; w /= p.h_pairs;   // the head pairs of one probs slab run back to back
    it.q0 = (w % p.q_tiles) * MV_BM;
    it.b = w / p.q_tiles;
    it.h0 = hp * MV_HP;
    it.nh = min(MV_HP, p.nhead - it.h0);
    return true;
}

// MMA stage layout: [head 0: A hi, A lo][head 1: A hi, A lo][head 0: B hi, B lo][head 1: B hi, B lo]
__device__ __forceinline__ int mv_a_off(int h, int lo) { return (2 * h + lo) * MV_A_TILE; }
__device__ __forceinline__ int mv_b_off(int h, int lo) { return MV_HP * 2 * MV_A_TILE + (2 * h + lo) * MV_B_TILE; }

// TR = true is the value gradient, out[b,k,h,p] = sum_q probs[b,q,k,h] * gy[b,q,h*P+p]: the output
// rows run along the SECOND time axis of probs and the sum along the first.  Only the raw slab's
// box ([16 q][128 k][4 heads] instead of [128 q][16 k][4 heads]) and the converter's indexing change.
template <bool TR>
__global__ void __launch_bounds__(MV_THREADS, 1)
mix_values_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_v_hi,
                     const __grid_constant__ CUtensorMap map_v_lo, const MvParams p) {
    extern __shared__ uint8_t mv_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mv_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint8_t* raw_base = smem + MV_STAGES * MV_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(raw_base + MV_RAW_STAGES * MV_RAW);
    uint64_t* full_b = bars;                          // [3] TMA (V tiles) -> MMA
    uint64_t* full_a = full_b + MV_STAGES;            // [3] converter warps (P tiles) -> MMA
    uint64_t* empty_bar = full_a + MV_STAGES;         // [3] MMA -> TMA + converters
    uint64_t* raw_full = empty_bar + MV_STAGES;       // [2] TMA (raw probs slab) -> converters
    uint64_t* raw_empty = raw_full + MV_RAW_STAGES;   // [2] converters -> TMA
    uint64_t* tmem_full_bar = raw_empty + MV_RAW_STAGES;   // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;          // [2]
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < MV_STAGES; ++s) {
            mbar_init(smem_u32(&full_b[s]), 1);
            mbar_init(smem_u32(&full_a[s]), 4);        // one arrival per converter warp
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < MV_RAW_STAGES; ++s) {
            mbar_init(smem_u32(&raw_full[s]), 1);
            mbar_init(smem_u32(&raw_empty[s]), 4);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full_bar[s]), 1);
            mbar_init(smem_u32(&tmem_empty_bar[s]), 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), 2 * MV_ACC_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int nvec = p.nhead * MV_P;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_p);
            tma_prefetch_desc(&map_v_hi);
            tma_prefetch_desc(&map_v_lo);
            int stage = 0, rstage = 0;
            uint32_t phase = 0, rphase = 0;
            bool ok = true;
            MvItem it;
            for (int w = blockIdx.x; ok && mv_item(p, w, it); w += gridDim.x) {
                const int row_v = it.b * nvec + it.h0 * MV_P;          // plane row of (head h0, p = 0)
                const int row_q = it.b * p.ntimes + it.q0;             // a tile past the end of a batch item
                const int box_h = (it.h0 / MV_BOXH) * MV_BOXH;         // reads rows that are never stored
                for (int ks = 0; ks < p.k_stages; ++ks) {
                    // raw probs slab [128 q][16 k][4 heads]
                    ok = mbar_wait(smem_u32(&raw_empty[rstage]), rphase ^ 1u, abort_flag, p.status, 20);
                    if (!ok) break;
                    const uint32_t rfull = smem_u32(&raw_full[rstage]);
                    mbar_expect_tx(rfull, MV_RAW);
                    if (TR) tma_load_3d(smem_u32(raw_base + rstage * MV_RAW), &map_p, rfull, box_h, it.q0,
                                        it.b * p.ntimes + ks * MV_BK);
                    else tma_load_3d(smem_u32(raw_base + rstage * MV_RAW), &map_p, rfull, box_h, ks * MV_BK, row_q);
                    if (++rstage == MV_RAW_STAGES) { rstage = 0; rphase ^= 1u; }
                    // V_h^T tiles
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 21);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&full_b[stage]);
                    uint8_t* base = smem + stage * MV_STAGE;
                    mbar_expect_tx(full, static_cast<uint32_t>(it.nh) * 2 * MV_B_TILE);
                    for (int h = 0; h < it.nh; ++h) {
                        tma_load_2d(smem_u32(base + mv_b_off(h, 0)), &map_v_hi, full, ks * MV_BK, row_v + h * MV_P);
                        tma_load_2d(smem_u32(base + mv_b_off(h, 1)), &map_v_lo, full, ks * MV_BK, row_v + h * MV_P);
                    }
                    if (++stage == MV_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(MV_BM, MV_P);
            int stage = 0, acc_buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            MvItem it;
            for (int w = blockIdx.x; ok && mv_item(p, w, it); w += gridDim.x) {
                for (int ks0 = 0; ok && ks0 < p.k_stages; ks0 += MV_CHUNK_STAGES) {
                    const int ks1 = min(p.k_stages, ks0 + MV_CHUNK_STAGES);
                    ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 22);
                    if (!ok) break;
                    tc_fence_after();
                    for (int ks = ks0; ks < ks1; ++ks) {
                        ok = mbar_wait(smem_u32(&full_b[stage]), phase, abort_flag, p.status, 23) &&
                             mbar_wait(smem_u32(&full_a[stage]), phase, abort_flag, p.status, 24);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t base = smem_u32(smem + stage * MV_STAGE);
                        // MMAs that accumulate into the same tensor-memory columns execute back to back
                        // with the full pipeline latency between them, and a 128 x 64 x 8 MMA is short.
                        // Four independent chains are therefore interleaved: per head one for the hi.hi
                        // terms and one for the two cross terms (the accumulate warps add them).
                        uint64_t a_hi[MV_HP], a_lo[MV_HP], b_hi[MV_HP], b_lo[MV_HP];
#pragma unroll
                        for (int h = 0; h < MV_HP; ++h) {
                            a_hi[h] = smem_desc_kmajor<MV_BK>(base + mv_a_off(h, 0));
                            a_lo[h] = smem_desc_kmajor<MV_BK>(base + mv_a_off(h, 1));
                            b_hi[h] = smem_desc_kmajor<MV_BK>(base + mv_b_off(h, 0));
                            b_lo[h] = smem_desc_kmajor<MV_BK>(base + mv_b_off(h, 1));
                        }
                        const uint32_t d_main = tmem_base + static_cast<uint32_t>(acc_buf * MV_ACC_COLS);
                        const uint32_t d_cross = d_main + MV_HP * MV_P;
#pragma unroll
                        for (int k = 0; k < MV_BK / 8; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            const uint32_t first = (ks == ks0 && k == 0) ? 0u : 1u;
#pragma unroll
                            for (int h = 0; h < MV_HP; ++h)
                                if (h < it.nh) umma_tf32(d_cross + h * MV_P, a_lo[h] + adv, b_hi[h] + adv, idesc, first);
#pragma unroll
                            for (int h = 0; h < MV_HP; ++h)
                                if (h < it.nh) umma_tf32(d_main + h * MV_P, a_hi[h] + adv, b_hi[h] + adv, idesc, first);
#pragma unroll
                            for (int h = 0; h < MV_HP; ++h)
                                if (h < it.nh) umma_tf32(d_cross + h * MV_P, a_hi[h] + adv, b_lo[h] + adv, idesc, 1u);
                        }
                        umma_commit(smem_u32(&empty_bar[stage]));
                        if (++stage == MV_STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    umma_commit(smem_u32(&tmem_full_bar[acc_buf]));
                    acc_buf ^= 1;
                    if (acc_buf == 0) acc_phase ^= 1u;
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------ converter warps (4..7) ------------------------------
        const int ct = threadIdx.x - 128;         // 0..127
        int stage = 0, rstage = 0;
        uint32_t phase = 0, rphase = 0;
        bool ok = true;
        MvItem it;
        for (int w = blockIdx.x; ok && mv_item(p, w, it); w += gridDim.x) {
            const int sel = it.h0 % MV_BOXH;      // which two of the piece's four heads: 0 or 2
            for (int ks = 0; ks < p.k_stages; ++ks) {
                ok = mbar_wait(smem_u32(&raw_full[rstage]), rphase, abort_flag, p.status, 27) &&
                     mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 25);
                if (!ok) break;
                const float4* slab = reinterpret_cast<const float4*>(raw_base + rstage * MV_RAW);
                uint8_t* base = smem + stage * MV_STAGE;
                // 128 q x 16 k pieces, 16 per thread; piece e = ct + 128 i -> k = e % 16, q = e / 16
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    int e, kk, qi;
                    if (!TR) {
                        e = ct + 128 * i;
                        kk = e & 15;
                        qi = e >> 4;
                    } else {
                        // slab = [16 sum rows][128 output rows]; a warp takes 8 output rows x 4 sum rows so
                        // that both its 16-byte reads and its swizzled 4-byte writes are free of bank conflicts
                        const int combo = (ct >> 5) * 16 + i;
                        qi = (combo & 15) * 8 + (lane & 7);
                        kk = (combo >> 4) * 4 + (lane >> 3);
                        e = kk * MV_BM + qi;
                    }
                    float4 v = slab[e];
                    // sum rows past the end of this batch item belong to the next one: they must not count
                    if (TR && ks * MV_BK + kk >= p.ntimes) v = make_float4(0.f, 0.f, 0.f, 0.f);
                    const float v0 = sel ? v.z : v.x, v1 = sel ? v.w : v.y;
                    // 64-byte rows, 16-byte pieces XOR-swizzled by bits 7..8 of the byte offset (SWIZZLE_64B)
                    const int off = qi * 64 + ((((kk >> 2) ^ (qi >> 1)) & 3) << 4) + ((kk & 3) << 2);
                    // hi = the value rounded to TF32 by integer arithmetic on its bits (a carry out of the mantissa
                    // ripples into the exponent: the correctly rounded result), lo = the exact remainder, whose bits
                    // below TF32 the tensor core drops.  The conversion instruction issues at a fraction of the rate
                    // of integer and add instructions, and there were four per piece.
                    uint32_t hi = (__float_as_uint(v0) + 0x1000u) & 0xFFFFE000u;
                    *reinterpret_cast<uint32_t*>(base + mv_a_off(0, 0) + off) = hi;
                    *reinterpret_cast<float*>(base + mv_a_off(0, 1) + off) = v0 - __uint_as_float(hi);
                    hi = (__float_as_uint(v1) + 0x1000u) & 0xFFFFE000u;
                    *reinterpret_cast<uint32_t*>(base + mv_a_off(1, 0) + off) = hi;
                    *reinterpret_cast<float*>(base + mv_a_off(1, 1) + off) = v1 - __uint_as_float(hi);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&full_a[stage]));
                    mbar_arrive(smem_u32(&raw_empty[rstage]));
                }
                if (++stage == MV_STAGES) { stage = 0; phase ^= 1u; }
                if (++rstage == MV_RAW_STAGES) { rstage = 0; rphase ^= 1u; }
            }
        }
    } else if (warp >= 8) {
        // ------------------------------ accumulate + store warps (8..15) ------------------------
        const int quarter = warp & 3;             // TMEM lane quarter
        const int hsel = (warp - 8) >> 2;         // which head of the pair (64 accumulator columns)
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        MvItem it;
        const int n_chunks = (p.k_stages + MV_CHUNK_STAGES - 1) / MV_CHUNK_STAGES;
        for (int w = blockIdx.x; ok && mv_item(p, w, it); w += gridDim.x) {
            float acc[MV_P];
            for (int c = 0; c < n_chunks; ++c) {
                ok = mbar_wait(smem_u32(&tmem_full_bar[acc_buf]), acc_phase, abort_flag, p.status, 26);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * MV_ACC_COLS + hsel * MV_P);
#pragma unroll
                for (int cc = 0; cc < MV_P / 16; ++cc) {
                    uint32_t rm[16], rx[16];   // hi.hi chain and cross-term chain of the same outputs
                    tmem_ld16(taddr + static_cast<uint32_t>(cc * 16), rm);
                    tmem_ld16(taddr + static_cast<uint32_t>(MV_HP * MV_P + cc * 16), rx);
                    tmem_ld_wait_all();
                    pin_regs16(rm);
                    pin_regs16(rx);
                    if (c == 0) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[cc * 16 + i] = __uint_as_float(rm[i]) + __uint_as_float(rx[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i)   // round-to-nearest promotion
                            acc[cc * 16 + i] += __uint_as_float(rm[i]) + __uint_as_float(rx[i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_buf]));
                acc_buf ^= 1;
                if (acc_buf == 0) acc_phase ^= 1u;
            }
            if (!ok) break;
            const int q = it.q0 + quarter * 32 + lane;
            if (q < p.ntimes && hsel < it.nh) {
                float* out = p.py + (static_cast<int64_t>(it.b) * p.ntimes + q) * nvec + (it.h0 + hsel) * MV_P;
#pragma unroll
                for (int j = 0; j < MV_P / 4; ++j)
                    *reinterpret_cast<float4*>(out + 4 * j) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * MV_ACC_COLS);
    }
}

}  // namespace

// Returns 1 when the shape is outside the fast path.
int attn_mix_values_tc(DeviceState* st, int device, float* py, const float* pp, const float* pV, int64_t nbat,
                       int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, cudaStream_t s, bool transposed) {
    const bool ok = npiece == MV_P && nvec == nhead * npiece && ntimes >= 64 && nbat <= 65535 && nhead % 4 == 0 &&
                    nbat * nvec < (int64_t(1) << 31) && nbat * ntimes < (int64_t(1) << 31) && nhead < (1 << 16) &&
                    ((reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pp)) & 15) == 0 &&
                    nbat * ((ntimes + MV_BM - 1) / MV_BM) * ((nhead + MV_HP - 1) / MV_HP) < (int64_t(1) << 30);
    if (!ok) return 1;
    const int64_t kp = round_up(ntimes, 4);
    const int64_t plane = round_up(nbat * nvec * kp * 4, 256);
    KAI_TRY(ensure_workspace(st, device, 2 * plane));
    uint8_t* ws = static_cast<uint8_t*>(st->ws);
    float* v_hi = reinterpret_cast<float*>(ws);
    float* v_lo = reinterpret_cast<float*>(ws + plane);
    // V[b] is [ntimes][nvec]; the planes are [b][nvec][kp]: row (b, h*64+p) holds V_h[:, p] along the keys.
    KAI_TRY(split_planes_transposed(pV, nbat, ntimes, nvec, v_hi, v_lo, s));
    CUtensorMap maps[3];
    // probs as [nbat*ntimes (q)][ntimes (k)][nhead]: box = 128 q x 16 k x 4 heads, unswizzled
    // (transposed: 16 q x 128 k x 4 heads)
    KAI_TRY(make_map_3d(&maps[0], pp, nhead, ntimes, nbat * ntimes, nhead, ntimes * nhead, MV_BOXH,
                        transposed ? MV_BM : MV_BK, transposed ? MV_BK : MV_BM));
    KAI_TRY(make_map(&maps[1], v_hi, nbat * nvec, ntimes, kp, MV_P, MV_BK));
    KAI_TRY(make_map(&maps[2], v_lo, nbat * nvec, ntimes, kp, MV_P, MV_BK));
    MvParams p;
    p.py = py;
    p.nbat = static_cast<int>(nbat); p.ntimes = static_cast<int>(ntimes); p.nhead = static_cast<int>(nhead);
    p.q_tiles = static_cast<int>((ntimes + MV_BM - 1) / MV_BM);
    p.h_pairs = static_cast<int>((nhead + MV_HP - 1) / MV_HP);
    p.k_stages = static_cast<int>((ntimes + MV_BK - 1) / MV_BK);
    p.status = st->status_dev;
    const int64_t items = static_cast<int64_t>(p.nbat) * p.q_tiles * p.h_pairs;
    const int grid = static_cast<int>(items < st->sm_count ? items : st->sm_count);
    constexpr int smem = MV_STAGES * MV_STAGE + MV_RAW_STAGES * MV_RAW + 1024 + 256;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(mix_values_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        KAI_CUDA(cudaFuncSetAttribute(mix_values_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    if (transposed) mix_values_tc_kernel<true><<<grid, MV_THREADS, smem, s>>>(maps[0], maps[1], maps[2], p);
    else mix_values_tc_kernel<false><<<grid, MV_THREADS, smem, s>>>(maps[0], maps[1], maps[2], p);
    count_launch();
    count_tc_launch();
    KAI_TRY(check_launch("mix_values_tc_kernel"));
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai
