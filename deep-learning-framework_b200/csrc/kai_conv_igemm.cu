// Implicit-GEMM convolution on the tcgen05 tensor cores (sm_100a): conv2d and conv2d_backward_x of the
// reference (support/vmath.cu:3490-3655; NCHW, stride 1, zero padding, group 1; also the dilated family).
//
//   out[nd, n, r, c] = sum_{cn,kr,kc} src[nd, cn, r + dr(kr), c + dc(kc)] * wmat[n][(cn,kr,kc)]
//
// is a GEMM D[m][n] = A[m][k] . B[n][k]^T with m = (nd, r, c), k = (cn, kr, kc), whose A operand -- the unfolded
// image -- is never written to memory: converter warps build every 128 x 32 tile of it in shared memory straight
// from a zero-padded copy of the image (one table read for the tap's offset, one coalesced load: consecutive
// lanes hold consecutive pixels), store the value itself as the hi operand (the tensor core ignores the low 13
// mantissa bits) and its rounded remainder as the lo operand, in the 128-byte-swizzled K-major layout.  The weight
// matrix [n][k] comes from hi/lo planes through TMA.  Roles (576 threads, one CTA per SM, persistent over tiles
// of 128 output positions x all output channels):
//   warp 0      TMA producer (weight tiles)          warp 1       MMA issuer (3 MMAs per 8-wide k-step)
//   warps 2-9   converters: two groups of four warps take alternate 32-wide k stages (one output position per
//               thread, the loads of the group's next stage in flight while it converts the current one)
//   warps 10-17 accumulate + store: tensor memory holds at most `chunk` stages of the sum (the truncating
//               fp32 accumulate, as in the GEMM kernel); finished chunks are added into fp32 registers; the
//               result is written in NCHW order, a warp covering 32 consecutive pixels of one channel.
// Every wait is bounded and reports through the device status word.
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {

int split_planes(const float* src, int64_t rows, int64_t cols, float* hi, float* lo, int sm_count, cudaStream_t s);

namespace {

constexpr int IG_BM = 128;                 // output positions per tile (TMEM lanes)
constexpr int IG_BK = 32;                  // k per stage (128-byte rows)
constexpr int IG_A_TILE = IG_BM * IG_BK * 4;   // 16 KB
constexpr int IG_THREADS = 576;            // TMA, MMA, 2 x 4 converter warps, 8 accumulate warps
constexpr int IG_MAXK = 4096;

struct IgParams {
    float* out;                 // [ndat][nout][oh*ow]
    const float* srcp;          // zero-padded source [ndat*cchn][shP][swP]
    int M, K, kp, nout, pix;    // pix = oh*ow
    int ow, cchn, plane, swP, pt, pl;   // plane = shP*swP
    int kh, kw, ph, pw, gh, gw, flip;
    int m_tiles, k_stages, chunk_stages;
    int* status;
};

template <int BN>
__global__ void __launch_bounds__(IG_THREADS, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                  const IgParams p) {
    constexpr int IG_STAGES = (BN <= 64) ? 4 : 3;
    constexpr int B_TILE = BN * IG_BK * 4;
    constexpr int STAGE = 2 * IG_A_TILE + 2 * B_TILE;
    extern __shared__ uint8_t ig_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ig_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    int* tap_lin = reinterpret_cast<int*>(smem + IG_STAGES * STAGE);                 // [k_stages * 32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + IG_STAGES * STAGE + IG_MAXK * 4);
    uint64_t* full_b = bars;                         // [stages] TMA -> MMA
    uint64_t* full_a = bars + IG_STAGES;             // [stages] converters -> MMA
    uint64_t* empty_bar = bars + 2 * IG_STAGES;      // [stages] MMA -> TMA + converters
    uint64_t* tmem_full = bars + 3 * IG_STAGES;      // [2]
    uint64_t* tmem_empty = tmem_full + 2;            // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < IG_STAGES; ++s) {
            mbar_init(smem_u32(&full_b[s]), 1);
            mbar_init(smem_u32(&full_a[s]), 4);      // the four warps of the group that owns the stage
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&tmem_full[s]), 1);
            mbar_init(smem_u32(&tmem_empty[s]), 8);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // tap table: offset of tap k from an output's own position in the padded tensor (k >= K: first tap, the
    // weight planes are zero there)
    for (int k = threadIdx.x; k < p.k_stages * IG_BK; k += IG_THREADS) {
        int off = 0;
        if (k < p.K) {
            const int kc = k % p.kw, kr = (k / p.kw) % p.kh, cn = k / (p.kw * p.kh);
            const int dr = (p.flip ? (p.ph - kr) : (kr - p.ph)) * p.gh;
            const int dc = (p.flip ? (p.pw - kc) : (kc - p.pw)) * p.gw;
            off = cn * p.plane + dr * p.swP + dc;
        }
        tap_lin[k] = off;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer: weight tiles ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_w_hi);
            tma_prefetch_desc(&map_w_lo);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                for (int ks = 0; ks < p.k_stages; ++ks) {
                    ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 60);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&full_b[stage]);
                    uint8_t* base = smem + stage * STAGE + 2 * IG_A_TILE;
                    mbar_expect_tx(full, 2 * B_TILE);
                    tma_load_2d(smem_u32(base), &map_w_hi, full, ks * IG_BK, 0);
                    tma_load_2d(smem_u32(base + B_TILE), &map_w_lo, full, ks * IG_BK, 0);
                    if (++stage == IG_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ----------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_tf32(IG_BM, BN);
            int stage = 0, acc_buf = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
                for (int ks0 = 0; ok && ks0 < p.k_stages; ks0 += p.chunk_stages) {
                    const int ks1 = min(p.k_stages, ks0 + p.chunk_stages);
                    ok = mbar_wait(smem_u32(&tmem_empty[acc_buf]), acc_phase ^ 1u, abort_flag, p.status, 61);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc_buf * BN);
                    for (int ks = ks0; ks < ks1; ++ks) {
                        ok = mbar_wait(smem_u32(&full_b[stage]), phase, abort_flag, p.status, 62) &&
                             mbar_wait(smem_u32(&full_a[stage]), phase, abort_flag, p.status, 63);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t base = smem_u32(smem + stage * STAGE);
                        const uint64_t a_hi = smem_desc_kmajor<IG_BK>(base), a_lo = smem_desc_kmajor<IG_BK>(base + IG_A_TILE);
                        const uint64_t b_hi = smem_desc_kmajor<IG_BK>(base + 2 * IG_A_TILE);
                        const uint64_t b_lo = smem_desc_kmajor<IG_BK>(base + 2 * IG_A_TILE + B_TILE);
#pragma unroll
                        for (int k = 0; k < IG_BK / 8; ++k) {
                            const uint64_t adv = static_cast<uint64_t>(k * 2);
                            const uint32_t first = (ks == ks0 && k == 0) ? 0u : 1u;
                            umma_tf32(d_tmem, a_lo + adv, b_hi + adv, idesc, first);
                            umma_tf32(d_tmem, a_hi + adv, b_lo + adv, idesc, 1u);
                            umma_tf32(d_tmem, a_hi + adv, b_hi + adv, idesc, 1u);
                        }
                        umma_commit(smem_u32(&empty_bar[stage]));
                        if (++stage == IG_STAGES) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    umma_commit(smem_u32(&tmem_full[acc_buf]));
                    acc_buf ^= 1;
                    if (acc_buf == 0) acc_phase ^= 1u;
                }
            }
        }
    } else if (warp < 10) {
        // ------------------------------ converters (warps 2..9) ---------------------------------
        // Two groups of four warps take alternate stages; inside a group one output position per thread.
        const int group = (warp - 2) >> 2;
        const int row = threadIdx.x - 64 - group * 128;   // 0..127
        bool ok = true;
        uint32_t n_base = 0;                              // stages issued before this tile (all tiles of this CTA)
        for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x, n_base += static_cast<uint32_t>(p.k_stages)) {
            const int m = t * IG_BM + row;
            int pos = -1;
            if (m < p.M) {
                const int nd = m / p.pix, px = m - nd * p.pix;
                pos = nd * p.cchn * p.plane + (px / p.ow + p.pt) * p.swP + (px % p.ow + p.pl);
            }
            float va[IG_BK], vb[IG_BK];
            auto load = [&](float (&v)[IG_BK], int ks) {
                if (ks < p.k_stages && pos >= 0) {
#pragma unroll
                    for (int kk = 0; kk < IG_BK; ++kk)      // k past the end of the reduction contributes nothing
                        v[kk] = (ks * IG_BK + kk < p.K) ? __ldg(p.srcp + pos + tap_lin[ks * IG_BK + kk]) : 0.0f;
                } else {
#pragma unroll
                    for (int kk = 0; kk < IG_BK; ++kk) v[kk] = 0.0f;
                }
            };
            auto convert = [&](const float (&v)[IG_BK], int ks) -> bool {
                const uint32_t n = n_base + static_cast<uint32_t>(ks);
                const int stage = static_cast<int>(n % IG_STAGES);
                const uint32_t phase = (n / IG_STAGES) & 1u;
                if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, 64)) return false;
                uint8_t* base = smem + stage * STAGE;
#pragma unroll
                for (int c = 0; c < IG_BK / 4; ++c) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float x = v[4 * c + e];
                        hi[e] = __float_as_uint(x);
                        const float rest = isfinite(x) ? (x - __uint_as_float(hi[e] & 0xFFFFE000u)) : 0.0f;
                        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo[e]) : "f"(rest));
                    }
                    // 128-byte rows, 16-byte pieces XOR-swizzled by the row's low three bits (SWIZZLE_128B)
                    const int off = row * 128 + ((c ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(base + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4*>(base + IG_A_TILE + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&full_a[stage]));
                return true;
            };
            // this group's stages of the tile: those with (n_base + ks) % 2 == group
            int ks = static_cast<int>((group + 2u - (n_base & 1u)) & 1u);
            load(va, ks);
            for (; ok && ks < p.k_stages; ks += 4) {
                load(vb, ks + 2);
                ok = convert(va, ks);
                if (!ok || ks + 2 >= p.k_stages) break;
                load(va, ks + 4);
                ok = convert(vb, ks + 2);
            }
        }
    } else {
        // ------------------------------ accumulate + store (warps 10..17) -------------------------
        constexpr int COLS = BN / 2;                  // columns per thread
        const int quarter = warp & 3;                 // TMEM lane quarter
        const int chalf = (warp - 10) >> 2;           // which half of the channels
        const int row = quarter * 32 + lane;
        int acc_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        const int n_chunks = (p.k_stages + p.chunk_stages - 1) / p.chunk_stages;
        for (int t = blockIdx.x; ok && t < p.m_tiles; t += gridDim.x) {
            float acc[COLS];
#pragma unroll
            for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
            for (int c = 0; c < n_chunks; ++c) {
                ok = mbar_wait(smem_u32(&tmem_full[acc_buf]), acc_phase, abort_flag, p.status, 65);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(acc_buf * BN + chalf * COLS);
#pragma unroll
                for (int cc = 0; cc < COLS / 16; ++cc) {
                    uint32_t r[16];
                    tmem_ld16(taddr + static_cast<uint32_t>(cc * 16), r);
                    tmem_ld_wait16(r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[cc * 16 + i] += __uint_as_float(r[i]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[acc_buf]));
                acc_buf ^= 1;
                if (acc_buf == 0) acc_phase ^= 1u;
            }
            if (!ok) break;
            const int m = t * IG_BM + row;
            if (m < p.M) {
                const int nd = m / p.pix, px = m - nd * p.pix;
                float* out = p.out + (static_cast<int64_t>(nd) * p.nout + chalf * COLS) * p.pix + px;
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
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

template <int BN>
int launch_igemm(const CUtensorMap maps[2], const IgParams& p, int grid, cudaStream_t s) {
    constexpr int stages = (BN <= 64) ? 4 : 3;
    constexpr int smem = stages * (2 * IG_A_TILE + 2 * BN * IG_BK * 4) + IG_MAXK * 4 + 256 + 1024;
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(conv_igemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    conv_igemm_kernel<BN><<<grid, IG_THREADS, smem, s>>>(maps[0], maps[1], p);
    count_launch();
    count_tc_launch();
    return check_launch("conv_igemm_kernel");
}

}  // namespace

// Shapes the implicit-GEMM kernel takes (the caller has checked the padded tensor's size).
bool conv_igemm_fits(int64_t M, int64_t K, int64_t nout) {
    return nout >= 16 && nout <= 128 && K >= 32 && K <= IG_MAXK && M >= 4 * IG_BM && M < (int64_t(1) << 31) - IG_BM;
}

// out[nd][n][pix] = sum_k unfolded(srcp)[m][k] * wmat[n][k].  `w_hi`, `w_lo`: scratch for the weight planes
// ([nout][kp] floats each, kp = round_up(K, 4)).
int conv_igemm(DeviceState* st, float* out, const float* srcp, const float* wmat, float* w_hi, float* w_lo, int64_t ndat,
               int64_t cchn, int64_t oh, int64_t ow, int64_t nout, int64_t kh, int64_t kw, int64_t ph, int64_t pw,
               int64_t gh, int64_t gw, int flip, int shP, int swP, int pt, int pl, cudaStream_t s) {
    const int64_t M = ndat * oh * ow, K = cchn * kh * kw, kp = round_up(K, 4);
    KAI_TRY(split_planes(wmat, nout, K, w_hi, w_lo, st->sm_count, s));
    const int bn = (nout <= 64) ? 64 : 128;
    CUtensorMap maps[2];
    KAI_TRY(make_map(&maps[0], w_hi, nout, K, kp, bn, IG_BK));
    KAI_TRY(make_map(&maps[1], w_lo, nout, K, kp, bn, IG_BK));
    IgParams p;
    p.out = out; p.srcp = srcp;
    p.M = static_cast<int>(M); p.K = static_cast<int>(K); p.kp = static_cast<int>(kp); p.nout = static_cast<int>(nout);
    p.pix = static_cast<int>(oh * ow); p.ow = static_cast<int>(ow); p.cchn = static_cast<int>(cchn);
    p.plane = shP * swP; p.swP = swP; p.pt = pt; p.pl = pl;
    p.kh = static_cast<int>(kh); p.kw = static_cast<int>(kw); p.ph = static_cast<int>(ph); p.pw = static_cast<int>(pw);
    p.gh = static_cast<int>(gh); p.gw = static_cast<int>(gw); p.flip = flip;
    p.m_tiles = static_cast<int>((M + IG_BM - 1) / IG_BM);
    p.k_stages = static_cast<int>((K + IG_BK - 1) / IG_BK);
    // promotion interval as in the GEMM kernel: K held in tensor memory <= 2.5 * sqrt(K)
    int64_t kc = 32;
    while (kc * 2 <= 128 && static_cast<double>(kc * 2) <= 2.5 * sqrt(static_cast<double>(K))) kc *= 2;
    p.chunk_stages = static_cast<int>(kc / IG_BK);
    p.status = st->status_dev;
    const int grid = p.m_tiles < st->sm_count ? p.m_tiles : st->sm_count;
    KAI_TRY(bn == 64 ? launch_igemm<64>(maps, p, grid, s) : launch_igemm<128>(maps, p, grid, s));
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai
