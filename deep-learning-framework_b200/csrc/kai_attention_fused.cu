// Fused multi-head attention forward on the tcgen05 tensor cores (sm_100a), head width 64:
//
//   out[b,q,h,:] = sum_k softmax_k( coef * <Q[b,q,h,:], K[b,k,h,:]> ) * V[b,k,h,:]
//
// i.e. mix_values(softmax_direct_on_axis(mult_on_heads(K, Q))) of the reference
// (support/vmath.cu:6729-6750, 6864-6885, 6977-6997; call order api_objects/vtensor.cpp:3036-3044)
// without writing the [nbat, ntimes, ntimes, nhead] probs tensor to memory.  It serves callers that
// do not need probs afterwards (inference, no_grad).
//
// One work item = (batch b, head h, 128 queries).  Keys are visited in blocks of 64:
//   S_j  = Q . K_j^T          128 x 64, reduction over the 64 head columns   (tensor memory, 2 buffers)
//   P_j  = exp(coef * S_j - m) with the running row maximum m               (registers -> shared memory)
//   O_j  = P_j . V_j          128 x 64, reduction over the 64 keys           (tensor memory, 2 buffers)
//   O    = O * exp(m_old - m_new) + O_j                                      (fp32 registers)
// All products are 3xTF32 (hi.hi + lo.hi + hi.lo), so both contractions are fp32-accurate, and the
// running sum over key blocks is kept in fp32 registers with round-to-nearest adds (the tensor
// core's own fp32 accumulate truncates, so it only ever holds 64 keys).
//
// Roles (352 threads, one CTA per SM, persistent over items):
//   warp 0     TMA producer: the item's Q tile (hi/lo, 64 KB) and, through a 3-slot ring of 32 KB
//              stages, the K_j and V_j^T tiles in the order the MMA warp consumes them
//              (K0, K1, V0, K2, V1, ...).  The planes come from split kernels (V transposed so that the
//              keys are the contiguous "K" of the second product).
//   warp 1     issues the S_j = Q . K_j^T products, warp 10 the P_j . V_j products.  One thread needs longer
//              to wait for a stage, build descriptors, issue 24 small MMAs (N = 64: 48 clocks of pipe time
//              each) and commit than the pipe needs to run them, so two instruction streams keep it busier
//              than one; each issuer has its own "stage loaded" barriers (a thread that waited only for
//              every other phase of a shared barrier could see one that is two phases behind as complete).
//   warps 2-9  one query row per thread; the two warps that share a tensor-memory lane quarter split
//              the 64 keys / 64 output columns of a block in halves.  They read S_j, keep the running
//              maximum and sum, write P_j hi/lo as the swizzled K-major A operand, and accumulate O.
// Every wait is bounded; a wait that gives up sets the status word and the CTA drains and exits.
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {

int split_lo_pair(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, cudaStream_t s);
int split_planes_transposed(const float* src, int64_t batch, int64_t k, int64_t rows, float* hi, float* lo,
                            cudaStream_t s);

namespace {

constexpr int FA_BM = 128;                 // queries per item (TMEM lanes)
constexpr int FA_BN = 64;                  // keys per block
constexpr int FA_P = 64;                   // head width
constexpr int FA_THREADS = 352;            // TMA warp, S issuer, 8 row warps, P.V issuer
constexpr int FA_BOX_Q = FA_BM * 32 * 4;   // 128 rows x 32 fp32 = 16 KB
constexpr int FA_BOX_K = FA_BN * 32 * 4;   //  64 rows x 32 fp32 =  8 KB
constexpr int FA_Q_BYTES = 4 * FA_BOX_Q;   // hi/lo x two 32-column boxes = 64 KB
constexpr int FA_STAGE = 4 * FA_BOX_K;     // hi/lo x two boxes = 32 KB (a K block or a V^T block)
constexpr int FA_SLOTS = 3;
constexpr int FA_P_BYTES = 4 * FA_BOX_Q;   // P hi/lo, two 32-key boxes each = 64 KB
constexpr int FA_OFF_RING = FA_Q_BYTES;
constexpr int FA_OFF_P = FA_OFF_RING + FA_SLOTS * FA_STAGE;
constexpr int FA_OFF_MISC = FA_OFF_P + FA_P_BYTES;          // 224 KB
constexpr int FA_MISC_BYTES = 2048 + 32 * 8 + 16;           // pair exchange, barriers, tmem slot, abort flag
constexpr int FA_SMEM_REQUEST = 232448;                     // the 227 KB a CTA may have
constexpr int FA_TMEM_COLS = 256;                           // S0 S1 O0 O1, 64 columns each

struct FaParams {
    float* out;
    const float* coef;
    int nbat, ntimes, nhead, q_tiles, causal;
    int* status;
};

struct FaItem { int b, h, q0, nb; };

__device__ __forceinline__ bool fa_item(const FaParams& p, int w, FaItem& it) {
    const int total = p.nbat * p.nhead * p.q_tiles;
    if (w >= total) return false;
    const int qt = w % p.q_tiles; w /= p.q_tiles;     // the query tiles of one (b, h) run on neighbouring CTAs
    it.h = w % p.nhead;
    it.b = w / p.nhead;
    it.q0 = qt * FA_BM;
    int nb = (p.ntimes + FA_BN - 1) / FA_BN;
    if (p.causal) {                                    // keys beyond the tile's last query are all masked
        const int last_q = min(it.q0 + FA_BM, p.ntimes) - 1;
        nb = min(nb, last_q / FA_BN + 1);
    }
    it.nb = nb;
    return true;
}

// 8 k-steps of one 64-wide reduction: cross terms first, then the hi.hi chain (the truncating
// accumulate of the tensor core then acts on a full-size sum only 8 times).
// a_* / b_* point at the first of two consecutive SW128 boxes (32 reduction columns each).
__device__ __forceinline__ void fa_mma_block(uint32_t d_tmem, uint32_t a_hi, uint32_t a_lo, uint32_t a_box,
                                             uint32_t b_hi, uint32_t b_lo, uint32_t b_box, uint32_t idesc) {
    uint32_t first = 0u;
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        const uint64_t ah = smem_desc_kmajor<32>(a_hi + kb * a_box), al = smem_desc_kmajor<32>(a_lo + kb * a_box);
        const uint64_t bh = smem_desc_kmajor<32>(b_hi + kb * b_box), bl = smem_desc_kmajor<32>(b_lo + kb * b_box);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint64_t adv = static_cast<uint64_t>(k * 2);     // +32 bytes inside the 128-byte span
            umma_tf32(d_tmem, al + adv, bh + adv, idesc, first);
            first = 1u;
            umma_tf32(d_tmem, ah + adv, bl + adv, idesc, 1u);
        }
    }
#pragma unroll
    for (int kb = 0; kb < 2; ++kb) {
        const uint64_t ah = smem_desc_kmajor<32>(a_hi + kb * a_box);
        const uint64_t bh = smem_desc_kmajor<32>(b_hi + kb * b_box);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint64_t adv = static_cast<uint64_t>(k * 2);
            umma_tf32(d_tmem, ah + adv, bh + adv, idesc, 1u);
        }
    }
}

__global__ void __launch_bounds__(FA_THREADS, 1)
mh_attention_fused_kernel(const __grid_constant__ CUtensorMap map_q_hi, const __grid_constant__ CUtensorMap map_q_lo,
                          const __grid_constant__ CUtensorMap map_k_hi, const __grid_constant__ CUtensorMap map_k_lo,
                          const __grid_constant__ CUtensorMap map_v_hi, const __grid_constant__ CUtensorMap map_v_lo,
                          const FaParams p) {
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    if (smem + FA_OFF_MISC + FA_MISC_BYTES > fa_smem_raw + FA_SMEM_REQUEST) {
        // the shared-memory window is not 1 KB aligned: the tiles do not fit (reported, nothing computed)
        if (threadIdx.x == 0 && atomicCAS(p.status, 0, KAI_E_DEVICE_WAIT) == 0) p.status[1] = 39;
        return;
    }
    float* pair_x = reinterpret_cast<float*>(smem + FA_OFF_MISC);          // [2 parity][2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FA_OFF_MISC + 2048);
    uint64_t* q_full = bars;                 // TMA -> MMA
    uint64_t* q_empty = bars + 1;            // MMA -> TMA
    uint64_t* ring_full = bars + 2;          // [3] TMA -> S issuer (K stages, in the order of the K stages)
    uint64_t* ring_full_v = bars + 22;       // [3] TMA -> P.V issuer (V stages)
    uint64_t* ring_empty = bars + 5;         // [3] MMA -> TMA
    uint64_t* s_full = bars + 8;             // [2] MMA -> row warps
    uint64_t* s_empty = bars + 10;           // [2] row warps -> MMA
    uint64_t* p_full = bars + 12;            // row warps -> MMA
    uint64_t* p_empty = bars + 13;           // MMA -> row warps
    uint64_t* o_full = bars + 14;            // [2] MMA -> row warps
    uint64_t* o_empty = bars + 16;           // [2] row warps -> MMA
    uint64_t* pair_bar = bars + 18;          // [4] between the two warps of a lane quarter
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        mbar_init(smem_u32(q_empty), 1);
        for (int s = 0; s < FA_SLOTS; ++s) {
            mbar_init(smem_u32(&ring_full[s]), 1);
            mbar_init(smem_u32(&ring_full_v[s]), 1);
            mbar_init(smem_u32(&ring_empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), 8);
            mbar_init(smem_u32(&o_full[s]), 1);
            mbar_init(smem_u32(&o_empty[s]), 8);
        }
        mbar_init(smem_u32(p_full), 8);
        mbar_init(smem_u32(p_empty), 1);
        for (int s = 0; s < 4; ++s) mbar_init(smem_u32(&pair_bar[s]), 2);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_base_slot), FA_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_slot;
    const int nvec = p.nhead * FA_P;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_q_hi); tma_prefetch_desc(&map_q_lo);
            tma_prefetch_desc(&map_k_hi); tma_prefetch_desc(&map_k_lo);
            tma_prefetch_desc(&map_v_hi); tma_prefetch_desc(&map_v_lo);
            uint32_t n_item = 0, n_load = 0, n_k = 0, n_v = 0;
            bool ok = true;
            FaItem it;
            auto load_stage = [&](const CUtensorMap* hi, const CUtensorMap* lo, int c0, int c1, int dc0, bool is_v) -> bool {
                const int slot = static_cast<int>(n_load % FA_SLOTS);
                const uint32_t phase = (n_load / FA_SLOTS) & 1u;
                if (!mbar_wait(smem_u32(&ring_empty[slot]), phase ^ 1u, abort_flag, p.status, 31)) return false;
                const uint32_t full = is_v ? smem_u32(&ring_full_v[n_v % FA_SLOTS]) : smem_u32(&ring_full[n_k % FA_SLOTS]);
                if (is_v) ++n_v; else ++n_k;
                const uint32_t base = smem_u32(smem + FA_OFF_RING + slot * FA_STAGE);
                mbar_expect_tx(full, FA_STAGE);
                tma_load_2d(base, hi, full, c0, c1);
                tma_load_2d(base + FA_BOX_K, hi, full, c0 + dc0, c1);
                tma_load_2d(base + 2 * FA_BOX_K, lo, full, c0, c1);
                tma_load_2d(base + 3 * FA_BOX_K, lo, full, c0 + dc0, c1);
                ++n_load;
                return true;
            };
            for (int w = blockIdx.x; ok && fa_item(p, w, it); w += gridDim.x, ++n_item) {
                const int col = it.h * FA_P;
                const int row0 = it.b * p.ntimes;
                // Q tile (rows past the batch item read the next item or zero fill; they are never stored)
                ok = mbar_wait(smem_u32(q_empty), (n_item & 1u) ^ 1u, abort_flag, p.status, 30);
                if (!ok) break;
                const uint32_t qf = smem_u32(q_full), qb = smem_u32(smem);
                mbar_expect_tx(qf, FA_Q_BYTES);
                tma_load_2d(qb, &map_q_hi, qf, col, row0 + it.q0);
                tma_load_2d(qb + FA_BOX_Q, &map_q_hi, qf, col + 32, row0 + it.q0);
                tma_load_2d(qb + 2 * FA_BOX_Q, &map_q_lo, qf, col, row0 + it.q0);
                tma_load_2d(qb + 3 * FA_BOX_Q, &map_q_lo, qf, col + 32, row0 + it.q0);
                // K_0, then per block K_{j+1} before V_j: the MMA warp's order
                const int vrow = it.b * nvec + col;           // V^T planes: row (b, h*64 + p), keys along the row
                ok = load_stage(&map_k_hi, &map_k_lo, col, row0, 32, false);
                for (int j = 0; ok && j < it.nb; ++j) {
                    if (j + 1 < it.nb) ok = load_stage(&map_k_hi, &map_k_lo, col, row0 + (j + 1) * FA_BN, 32, false);
                    if (ok) ok = load_stage(&map_v_hi, &map_v_lo, j * FA_BN, vrow, 32, true);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ S issuer -----------------------------------
        // Ring positions of an item with nb blocks, counted from the item's first stage:
        //   K_0 -> 0, K_j -> 2j - 1 (j >= 1);  V_j -> 2j + 2 (j <= nb - 2), V_{nb-1} -> 2 nb - 1.
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(FA_BM, FA_BN);   // 128 x 64 for both products
            const uint32_t q_base = smem_u32(smem);
            uint32_t n_item = 0, base = 0, n_s = 0;
            bool ok = true;
            FaItem it;
            for (int w = blockIdx.x; ok && fa_item(p, w, it); w += gridDim.x, ++n_item) {
                ok = mbar_wait(smem_u32(q_full), n_item & 1u, abort_flag, p.status, 37);
                for (int j = 0; ok && j < it.nb; ++j, ++n_s) {
                    const uint32_t pos = base + (j == 0 ? 0u : static_cast<uint32_t>(2 * j - 1));
                    const int slot = static_cast<int>(pos % FA_SLOTS);
                    const int buf = static_cast<int>(n_s & 1u);
                    ok = mbar_wait(smem_u32(&ring_full[n_s % FA_SLOTS]), (n_s / FA_SLOTS) & 1u, abort_flag, p.status, 32) &&
                         mbar_wait(smem_u32(&s_empty[buf]), ((n_s >> 1) & 1u) ^ 1u, abort_flag, p.status, 33);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t kb = smem_u32(smem + FA_OFF_RING + slot * FA_STAGE);
                    fa_mma_block(tmem_base + static_cast<uint32_t>(buf * FA_BN), q_base, q_base + 2 * FA_BOX_Q, FA_BOX_Q, kb,
                                 kb + 2 * FA_BOX_K, FA_BOX_K, idesc);
                    umma_commit(smem_u32(&ring_empty[slot]));
                    umma_commit(smem_u32(&s_full[buf]));
                    if (j + 1 == it.nb) umma_commit(smem_u32(q_empty));
                }
                base += static_cast<uint32_t>(2 * it.nb);
            }
        }
    } else if (warp == 10) {
        // ------------------------------ P.V issuer ---------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(FA_BM, FA_BN);
            const uint32_t p_base = smem_u32(smem + FA_OFF_P);
            uint32_t base = 0, n_pv = 0;
            bool ok = true;
            FaItem it;
            for (int w = blockIdx.x; ok && fa_item(p, w, it); w += gridDim.x) {
                for (int j = 0; ok && j < it.nb; ++j, ++n_pv) {
                    const uint32_t pos = base + static_cast<uint32_t>(j + 1 < it.nb ? 2 * j + 2 : 2 * it.nb - 1);
                    const int slot = static_cast<int>(pos % FA_SLOTS);
                    const int buf = static_cast<int>(n_pv & 1u);
                    ok = mbar_wait(smem_u32(&ring_full_v[n_pv % FA_SLOTS]), (n_pv / FA_SLOTS) & 1u, abort_flag, p.status, 34) &&
                         mbar_wait(smem_u32(p_full), n_pv & 1u, abort_flag, p.status, 35) &&
                         mbar_wait(smem_u32(&o_empty[buf]), ((n_pv >> 1) & 1u) ^ 1u, abort_flag, p.status, 36);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t vb = smem_u32(smem + FA_OFF_RING + slot * FA_STAGE);
                    fa_mma_block(tmem_base + static_cast<uint32_t>(2 * FA_BN + buf * FA_P), p_base, p_base + 2 * FA_BOX_Q,
                                 FA_BOX_Q, vb, vb + 2 * FA_BOX_K, FA_BOX_K, idesc);
                    umma_commit(smem_u32(&ring_empty[slot]));
                    umma_commit(smem_u32(p_empty));
                    umma_commit(smem_u32(&o_full[buf]));
                }
                base += static_cast<uint32_t>(2 * it.nb);
            }
        }
    } else {
        // ------------------------------ row warps (2..9) --------------------------
        const int quarter = warp & 3;                 // tensor-memory lane quarter this warp may read
        const int half = (warp - 2) >> 2;             // which 32 keys of a block / 32 output columns
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        const float c2 = ((p.coef != nullptr) ? __ldg(p.coef) : 0.0f) * 1.4426950408889634f;   // coef * log2(e)
        uint8_t* p_hi = smem + FA_OFF_P + half * FA_BOX_Q;
        uint8_t* p_lo = p_hi + 2 * FA_BOX_Q;
        const uint32_t pair = smem_u32(&pair_bar[quarter]);
        uint32_t n_s = 0, n_p = 0, n_pv = 0, n_pair = 0;
        bool ok = true;
        FaItem it;
        for (int w = blockIdx.x; ok && fa_item(p, w, it); w += gridDim.x) {
            const int q = it.q0 + row;
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
            float m_run = -INFINITY, l_run = 0.0f, alpha_pending = 0.0f;
            for (int j = 0; j <= it.nb && ok; ++j) {
                float alpha = 0.0f;
                if (j < it.nb) {
                    // ---- scores of block j -> P_j ----
                    const int sbuf = static_cast<int>(n_s & 1u);
                    ok = mbar_wait(smem_u32(&s_full[sbuf]), (n_s >> 1) & 1u, abort_flag, p.status, 40);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r[32];
                    tmem_ld32(lane_addr + static_cast<uint32_t>(sbuf * FA_BN + half * 32), r);
                    tmem_ld_wait(r);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&s_empty[sbuf]));
                    ++n_s;
                    // t = log2(e) * coef * s, so that exp(coef * s - max) = 2^(t - max_t): one multiply, one
                    // add and one ex2 per score.
                    const int k0 = j * FA_BN + half * 32;
                    float t[32];
                    float mx = -INFINITY;
                    // only the last key block (keys past ntimes) and, with the causal mask, blocks that reach
                    // above the diagonal need the per-element test
                    const bool need_mask = (k0 + 32 > p.ntimes) || (p.causal && k0 + 31 > it.q0);
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int k = k0 + i;
                            float v = __uint_as_float(r[i]) * c2;
                            if (k >= p.ntimes || (p.causal && k > q)) v = -INFINITY;
                            t[i] = v;
                            mx = fmaxf(mx, v);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            t[i] = __uint_as_float(r[i]) * c2;
                            mx = fmaxf(mx, t[i]);
                        }
                    }
                    // block maximum of the whole row: exchange with the warp that holds the other 32 keys
                    float* slot_x = pair_x + (n_pair & 1u) * 256;
                    slot_x[half * 128 + row] = mx;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(pair);
                    ok = mbar_wait(pair, n_pair & 1u, abort_flag, p.status, 41);
                    if (!ok) break;
                    mx = fmaxf(mx, slot_x[(half ^ 1) * 128 + row]);
                    ++n_pair;
                    const float m_new = fmaxf(m_run, mx);
                    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
                    alpha = exp2f(m_run - m_use);            // 0 for the first block (m_run = -inf)
                    m_run = m_new;
                    float sum = 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float e;
                        const float x = t[i] - m_use;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
                        t[i] = e;
                        sum += e;
                    }
                    l_run = fmaf(l_run, alpha, sum);
                    // P buffer is free once the product that read the previous P has completed
                    ok = mbar_wait(smem_u32(p_empty), (n_p & 1u) ^ 1u, abort_flag, p.status, 42);
                    if (!ok) break;
                    // row `row` of the 128 x 32 box: eight 16-byte pieces, piece c at (c ^ (row & 7))
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // hi = v rounded to TF32 by integer arithmetic on its bits, lo = the exact remainder (the
                            // tensor core drops its bits below TF32): the conversion instruction issues at a fraction
                            // of the ALU rate, and these warps bound the loop
                            const float v = t[4 * c + e];
                            hi[e] = (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u;
                            lo[e] = __float_as_uint(v - __uint_as_float(hi[e]));
                        }
                        const int off = row * 128 + ((c ^ (row & 7)) << 4);
                        *reinterpret_cast<uint4*>(p_hi + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        *reinterpret_cast<uint4*>(p_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(p_full));
                    ++n_p;
                }
                if (j > 0) {
                    // ---- O_{j-1}: rescale the running output and add ----
                    const int obuf = static_cast<int>(n_pv & 1u);
                    ok = mbar_wait(smem_u32(&o_full[obuf]), (n_pv >> 1) & 1u, abort_flag, p.status, 43);
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t o[32];
                    tmem_ld32(lane_addr + static_cast<uint32_t>(2 * FA_BN + obuf * FA_P + half * 32), o);
                    tmem_ld_wait(o);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&o_empty[obuf]));
                    ++n_pv;
                    if (__all_sync(0xffffffffu, alpha_pending == 1.0f)) {       // the running maxima did not move
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(o[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha_pending, __uint_as_float(o[i]));
                    }
                }
                alpha_pending = alpha;
            }
            if (!ok) break;
            // ---- normalise: the row sum is the sum of both halves' partial sums ----
            float* slot_x = pair_x + (n_pair & 1u) * 256;
            slot_x[half * 128 + row] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(pair);
            ok = mbar_wait(pair, n_pair & 1u, abort_flag, p.status, 44);
            if (!ok) break;
            const float l_all = l_run + slot_x[(half ^ 1) * 128 + row];
            ++n_pair;
            if (q < p.ntimes) {
                const float inv = 1.0f / l_all;
                float* out = p.out + (static_cast<int64_t>(it.b) * p.ntimes + q) * nvec + it.h * FA_P + half * 32;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<float4*>(out + 4 * c) =
                        make_float4(acc[4 * c] * inv, acc[4 * c + 1] * inv, acc[4 * c + 2] * inv, acc[4 * c + 3] * inv);
            }
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);   // copies in flight land before the CTA exits
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, FA_TMEM_COLS);
    }
}

}  // namespace

// Returns 1 when the shape is outside the fused path.
int attn_fused_forward_tc(DeviceState* st, int device, float* py, const float* pK, const float* pQ, const float* pV,
                          int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, const float* coef,
                          int causal, cudaStream_t s) {
    const int64_t rows = nbat * ntimes;
    const int64_t q_tiles = (ntimes + FA_BM - 1) / FA_BM;
    const bool ok = npiece == FA_P && nvec == nhead * npiece && ntimes >= FA_BN && rows < (int64_t(1) << 31) &&
                    nbat * nvec < (int64_t(1) << 31) && nbat * nhead * q_tiles < (int64_t(1) << 30) &&
                    ((reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pQ) | reinterpret_cast<uintptr_t>(pK)) & 15) == 0 &&
                    rows * nvec < (int64_t(1) << 40);
    if (!ok) return 1;
    const int64_t plane = round_up(rows * nvec * 4, 256);
    const int64_t kp = round_up(ntimes, 4);
    const int64_t vplane = round_up(nbat * nvec * kp * 4, 256);
    KAI_TRY(ensure_workspace(st, device, 2 * plane + 2 * vplane));
    uint8_t* ws = static_cast<uint8_t*>(st->ws);
    float* q_lo = reinterpret_cast<float*>(ws);
    float* k_lo = reinterpret_cast<float*>(ws + plane);
    float* v_hi = reinterpret_cast<float*>(ws + 2 * plane);
    float* v_lo = reinterpret_cast<float*>(ws + 2 * plane + vplane);
    // Q and K themselves are the hi operands (the tensor core ignores the low 13 mantissa bits of a TF32
    // operand); only their lo planes are written.  V needs the transposed copy either way.
    KAI_TRY(split_lo_pair(pQ, pK, rows * nvec, q_lo, k_lo, s));
    KAI_TRY(split_planes_transposed(pV, nbat, ntimes, nvec, v_hi, v_lo, s));
    CUtensorMap maps[6];
    KAI_TRY(make_map(&maps[0], pQ, rows, nvec, nvec, FA_BM, 32));
    KAI_TRY(make_map(&maps[1], q_lo, rows, nvec, nvec, FA_BM, 32));
    KAI_TRY(make_map(&maps[2], pK, rows, nvec, nvec, FA_BN, 32));
    KAI_TRY(make_map(&maps[3], k_lo, rows, nvec, nvec, FA_BN, 32));
    KAI_TRY(make_map(&maps[4], v_hi, nbat * nvec, ntimes, kp, FA_P, 32));
    KAI_TRY(make_map(&maps[5], v_lo, nbat * nvec, ntimes, kp, FA_P, 32));
    FaParams p;
    p.out = py; p.coef = coef;
    p.nbat = static_cast<int>(nbat); p.ntimes = static_cast<int>(ntimes); p.nhead = static_cast<int>(nhead);
    p.q_tiles = static_cast<int>(q_tiles);
    p.causal = causal ? 1 : 0;
    p.status = st->status_dev;
    const int64_t items = nbat * nhead * q_tiles;
    const int grid = static_cast<int>(items < st->sm_count ? items : st->sm_count);
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(mh_attention_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      FA_SMEM_REQUEST));
        configured[dev] = true;
    }
    mh_attention_fused_kernel<<<grid, FA_THREADS, FA_SMEM_REQUEST, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4],
                                                                         maps[5], p);
    count_launch();
    count_tc_launch();
    KAI_TRY(check_launch("mh_attention_fused_kernel"));
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai
