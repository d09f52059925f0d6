// Tensor-core GEMM for the latency regime (a few hundred MFLOP: 512^3, the layers of a 128-row MLP, the
// per-timestep products of a recurrent layer): ONE launch, no scratch in global memory, no tensor maps.
//
//   C[m,n] (+)= sum_k A(m,k) B(n,k),   A(m,k) = a[m*sam + k*sak],  B(n,k) = b[n*sbn + k*sbk]
// (the three reference layouts of support/vmath.cu:2961-3093 are stride choices).
//
// A CTA owns a 128 x 64 output tile and one slice of the reduction; the slices of a tile belong to the
// CTAs of a thread-block cluster (up to 8), which add their partial tiles through distributed shared
// memory in rank order (deterministic), as the CUDA-core small-GEMM kernel does.  Inside a CTA:
//   * all 256 threads fetch the next 32-wide K-block of both operands from global memory into registers
//     while the tensor core works on the current one;
//   * they split each value into hi/lo TF32 (round to nearest) and store the four tiles in shared memory
//     in the 128-byte-swizzled K-major layout the tcgen05 descriptors expect (two buffers);
//   * one thread issues the 12 MMAs of the block (cross terms first) into a 64-column accumulator in
//     tensor memory and commits to the buffer's mbarrier;
//   * every `kc` values of K (the promotion interval of the large kernel) the accumulator is read back
//     and added into fp32 registers with round-to-nearest adds, because the tensor core's own fp32
//     accumulate truncates.
// Every wait is bounded and reports through the device status word.
//
// Measured on B200: correct on every shape of the GEMM tests, but slower than the CUDA-core cluster kernel
// at the sizes it was written for (512^3: 33 us against 12 us of kernel time; 64 x 2048 x 512: 30 us
// against 11 us).  With two to four 32-wide K-blocks per CTA the fixed costs -- tensor-memory allocation,
// two cluster barriers, the convert-and-store passes and one CTA of 182 registers per SM -- outweigh the
// faster multiply.  The automatic dispatch therefore does not pick it (option "small_tc" = 0); it stays
// selectable with KAI_PATH_SMALL_TC.
#include <cooperative_groups.h>

#include "kai_act.cuh"
#include "kai_common.cuh"
#include "kai_tcgen05.cuh"

namespace kai {
namespace {

namespace cg = cooperative_groups;

constexpr int ST_BM = 128;
constexpr int ST_BN = 64;
constexpr int ST_BK = 32;
constexpr int ST_THREADS = 256;
constexpr int ST_A_TILE = ST_BM * ST_BK * 4;                 // 16 KB
constexpr int ST_B_TILE = ST_BN * ST_BK * 4;                 //  8 KB
constexpr int ST_STAGE = 2 * ST_A_TILE + 2 * ST_B_TILE;      // hi/lo of both: 48 KB
constexpr int ST_PART_LD = ST_BN + 1;
constexpr int ST_SMEM = 2 * ST_STAGE + 1024 + 128;           // two buffers + alignment + barriers

struct StParams {
    const float* a; const float* b; float* c;
    int64_t M, N, K, sam, sak, sbn, sbk, ldc;
    const float* bias; const float* leaky_alpha;
    int act, accumulate;
    int64_t k_per_rank;
    int chunk_blocks;          // K-blocks accumulated in tensor memory between promotions
    int vec_a, vec_b;          // K-major operand whose rows allow 16-byte loads
    int* status;
};

// byte offset of element (row, k) in a [rows][32 fp32] tile with the 128-byte swizzle
__device__ __forceinline__ int st_swz(int row, int k) { return row * 128 + ((((k >> 2) ^ (row & 7)) & 7) << 4) + ((k & 3) << 2); }

template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(ST_THREADS, 1)
gemm_small_tc_kernel(const StParams p) {
    extern __shared__ uint8_t st_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(st_smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * ST_STAGE);   // [0..1] buffer free, [2] chunk done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = static_cast<int>(blockIdx.z), nrank = static_cast<int>(gridDim.z);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * ST_BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * ST_BN;
    const int64_t k_begin = rank * p.k_per_rank;
    const int64_t k_end = (k_begin + p.k_per_rank < p.K) ? k_begin + p.k_per_rank : p.K;
    const int nblocks = (k_end > k_begin) ? static_cast<int>((k_end - k_begin + ST_BK - 1) / ST_BK) : 0;

    if (tid == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        mbar_init(smem_u32(&bars[2]), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), 64);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // ---- register prefetch of one K-block: 16 values of A and 8 of B per thread ----
    float ra[16], rb[8];
    auto fetch = [&](int64_t k0) {
        if (A_KMAJOR && p.vec_a) {          // 16-byte loads: 8 pieces per row
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = tid + ST_THREADS * u;
                const int k4 = e & 7, mm = e >> 3;
                const int64_t m = m0 + mm, k = k0 + 4 * k4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m < p.M && k + 3 < k_end) v = __ldg(reinterpret_cast<const float4*>(p.a + m * p.sam + k));
                else if (m < p.M) {
                    if (k < k_end) v.x = __ldg(p.a + m * p.sam + k);
                    if (k + 1 < k_end) v.y = __ldg(p.a + m * p.sam + k + 1);
                    if (k + 2 < k_end) v.z = __ldg(p.a + m * p.sam + k + 2);
                }
                ra[4 * u] = v.x; ra[4 * u + 1] = v.y; ra[4 * u + 2] = v.z; ra[4 * u + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int e = tid + ST_THREADS * u;
                int kk, mm;
                if (A_KMAJOR) { kk = e & 31; mm = e >> 5; } else { mm = e & 127; kk = e >> 7; }
                const int64_t m = m0 + mm, k = k0 + kk;
                ra[u] = (m < p.M && k < k_end) ? __ldg(p.a + m * p.sam + k * p.sak) : 0.0f;
            }
        }
        if (B_KMAJOR && p.vec_b) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int e = tid + ST_THREADS * u;
                const int k4 = e & 7, nn = e >> 3;
                const int64_t n = n0 + nn, k = k0 + 4 * k4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (n < p.N && k + 3 < k_end) v = __ldg(reinterpret_cast<const float4*>(p.b + n * p.sbn + k));
                else if (n < p.N) {
                    if (k < k_end) v.x = __ldg(p.b + n * p.sbn + k);
                    if (k + 1 < k_end) v.y = __ldg(p.b + n * p.sbn + k + 1);
                    if (k + 2 < k_end) v.z = __ldg(p.b + n * p.sbn + k + 2);
                }
                rb[4 * u] = v.x; rb[4 * u + 1] = v.y; rb[4 * u + 2] = v.z; rb[4 * u + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = tid + ST_THREADS * u;
                int kk, nn;
                if (B_KMAJOR) { kk = e & 31; nn = e >> 5; } else { nn = e & 63; kk = e >> 6; }
                const int64_t n = n0 + nn, k = k0 + kk;
                rb[u] = (n < p.N && k < k_end) ? __ldg(p.b + n * p.sbn + k * p.sbk) : 0.0f;
            }
        }
    };
    auto split4 = [&](uint8_t* hi, uint8_t* lo, int off, const float* v) {   // four consecutive k: one 16-byte piece
        uint32_t h[4], l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h[j]) : "f"(v[j]));
            if (!isfinite(__uint_as_float(h[j])) && isfinite(v[j])) h[j] = __float_as_uint(v[j]) & 0xFFFFE000u;
            const float rest = isfinite(v[j]) ? (v[j] - __uint_as_float(h[j])) : 0.0f;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l[j]) : "f"(rest));
        }
        *reinterpret_cast<uint4*>(hi + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(lo + off) = make_uint4(l[0], l[1], l[2], l[3]);
    };
    auto split_store = [&](uint8_t* hi, uint8_t* lo, int off, float v) {
        uint32_t h, l;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
        // overflow by rounding or a non-finite input: keep the (truncated) value, no low part
        const bool fin = isfinite(__uint_as_float(h));
        if (!fin && isfinite(v)) h = __float_as_uint(v) & 0xFFFFE000u;
        const float rest = isfinite(v) ? (v - __uint_as_float(h)) : 0.0f;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(rest));
        *reinterpret_cast<uint32_t*>(hi + off) = h;
        *reinterpret_cast<uint32_t*>(lo + off) = l;
    };

    // this thread's part of the output tile: TMEM lane quarter (warp % 4), 32 of the 64 columns
    const int quarter = warp & 3, chalf = warp >> 2;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.0f;

    bool ok = true;
    uint32_t use[2] = {0, 0};        // completed uses of each buffer
    uint32_t chunks_done = 0;
    const uint32_t idesc = instr_desc_tf32(ST_BM, ST_BN);
    if (nblocks > 0) fetch(k_begin);
    int in_chunk = 0;
    for (int blk = 0; blk < nblocks && ok; ++blk) {
        const int buf = blk & 1;
        // The MMAs that read this buffer two blocks ago must be done.  One thread waits and the outcome is
        // shared through the barrier, so that all 256 threads leave the loop together if the wait gives up.
        int w = 1;
        if (tid == 0 && use[buf] > 0)
            w = mbar_wait(smem_u32(&bars[buf]), (use[buf] - 1) & 1u, abort_flag, p.status, 50) ? 1 : 0;
        if (!__syncthreads_and(w)) { ok = false; break; }
        uint8_t* base = smem + buf * ST_STAGE;
        uint8_t* a_hi = base, *a_lo = base + ST_A_TILE, *b_hi = base + 2 * ST_A_TILE, *b_lo = b_hi + ST_B_TILE;
        if (A_KMAJOR && p.vec_a) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = tid + ST_THREADS * u;
                split4(a_hi, a_lo, st_swz(e >> 3, 4 * (e & 7)), &ra[4 * u]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int e = tid + ST_THREADS * u;
                int kk, mm;
                if (A_KMAJOR) { kk = e & 31; mm = e >> 5; } else { mm = e & 127; kk = e >> 7; }
                split_store(a_hi, a_lo, st_swz(mm, kk), ra[u]);
            }
        }
        if (B_KMAJOR && p.vec_b) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int e = tid + ST_THREADS * u;
                split4(b_hi, b_lo, st_swz(e >> 3, 4 * (e & 7)), &rb[4 * u]);
            }
        } else {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int e = tid + ST_THREADS * u;
                int kk, nn;
                if (B_KMAJOR) { kk = e & 31; nn = e >> 5; } else { nn = e & 63; kk = e >> 6; }
                split_store(b_hi, b_lo, st_swz(nn, kk), rb[u]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // generic writes -> tensor-core reads
        __syncthreads();
        const bool last_of_chunk = (in_chunk + 1 == p.chunk_blocks) || (blk + 1 == nblocks);
        if (tid == 0) {
            tc_fence_after();
            const uint32_t ab = smem_u32(base);
            const uint64_t ah = smem_desc_kmajor<32>(ab), al = smem_desc_kmajor<32>(ab + ST_A_TILE);
            const uint64_t bh = smem_desc_kmajor<32>(ab + 2 * ST_A_TILE), bl = smem_desc_kmajor<32>(ab + 2 * ST_A_TILE + ST_B_TILE);
            uint32_t accum = (in_chunk == 0) ? 0u : 1u;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t adv = static_cast<uint64_t>(k * 2);
                umma_tf32(tmem_base, al + adv, bh + adv, idesc, accum);
                accum = 1u;
                umma_tf32(tmem_base, ah + adv, bl + adv, idesc, 1u);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t adv = static_cast<uint64_t>(k * 2);
                umma_tf32(tmem_base, ah + adv, bh + adv, idesc, 1u);
            }
            umma_commit(smem_u32(&bars[buf]));
            if (last_of_chunk) umma_commit(smem_u32(&bars[2]));
        }
        ++use[buf];
        if (blk + 1 < nblocks) fetch(k_begin + static_cast<int64_t>(blk + 1) * ST_BK);   // in flight during the MMAs
        if (last_of_chunk) {
            // promotion: add the finished chunk into the fp32 registers
            int w2 = 1;
            if (tid == 0) w2 = mbar_wait(smem_u32(&bars[2]), chunks_done & 1u, abort_flag, p.status, 51) ? 1 : 0;
            if (!__syncthreads_and(w2)) { ok = false; break; }
            ++chunks_done;
            tc_fence_after();
            uint32_t r[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(chalf * 32), r);
            tmem_ld_wait(r);
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] += __uint_as_float(r[i]);
            tc_fence_before();
            __syncthreads();           // every warp has read the accumulator before the next chunk overwrites it
            in_chunk = 0;
        } else {
            ++in_chunk;
        }
    }

    // ---- cluster reduction of the partial tiles (shared memory of the stage buffers is free now) ----
    // On an aborted wait the partial sums are meaningless, but every CTA still takes part in the cluster
    // barriers so that none is left waiting.
    // (After a normal loop every MMA has completed: the last chunk's barrier was waited for.)
    (void)ok;
    __syncthreads();
    float* part = reinterpret_cast<float*>(smem);
    {
        const int row = quarter * 32 + lane;
#pragma unroll
        for (int i = 0; i < 32; ++i) part[row * ST_PART_LD + chalf * 32 + i] = acc[i];
    }
    cluster.sync();
    const float alpha = (p.leaky_alpha != nullptr) ? __ldg(p.leaky_alpha) : 0.0f;
    const int rows = ST_BM / nrank;
    for (int e = tid; e < rows * ST_BN; e += ST_THREADS) {
        const int row = rank * rows + e / ST_BN, col = e % ST_BN;
        float t = 0.0f;
        for (int z = 0; z < nrank; ++z) t += cluster.map_shared_rank(part, z)[row * ST_PART_LD + col];
        const int64_t m = m0 + row, n = n0 + col;
        if (m < p.M && n < p.N) {
            float* out = p.c + m * p.ldc + n;
            if (p.accumulate) t = *out + t;
            if (p.bias) t = t + __ldg(p.bias + n);
            *out = act_forward(p.act, t, alpha);
        }
    }
    cluster.sync();   // nobody leaves while a neighbour may still read its partial tile

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 64);
    }
}

template <bool A_KMAJOR, bool B_KMAJOR>
int launch_small_tc(dim3 grid, int ranks, const StParams& p, cudaStream_t s) {
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(gemm_small_tc_kernel<A_KMAJOR, B_KMAJOR>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(ST_THREADS);
    cfg.dynamicSmemBytes = ST_SMEM;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = static_cast<unsigned>(ranks);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KAI_CUDA(cudaLaunchKernelEx(&cfg, gemm_small_tc_kernel<A_KMAJOR, B_KMAJOR>, p));
    count_launch();
    count_tc_launch();
    return check_launch("gemm_small_tc_kernel");
}

}  // namespace

// Shapes this kernel is meant for: at least half a tile of rows, a few columns, a reduction worth splitting.
bool gemm_small_tc_fits(int64_t M, int64_t N, int64_t K) {
    const int64_t tiles = ((M + ST_BM - 1) / ST_BM) * ((N + ST_BN - 1) / ST_BN);
    return M >= 48 && N >= 16 && K >= 64 && tiles <= 4096;
}

int gemm_small_tc(DeviceState* st, int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
                  int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    const int64_t tiles = ((M + ST_BM - 1) / ST_BM) * ((N + ST_BN - 1) / ST_BN);
    int ranks = 1;
    while (ranks < 8 && tiles * ranks * 2 <= 2 * st->sm_count && K / (ranks * 2) >= 32) ranks *= 2;
    int64_t k_per_rank = ((K + ranks - 1) / ranks + ST_BK - 1) / ST_BK * ST_BK;
    StParams p;
    p.a = a; p.b = b; p.c = c;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc;
    p.bias = ep.bias; p.leaky_alpha = ep.leaky_alpha; p.act = ep.act; p.accumulate = ep.accumulate;
    p.k_per_rank = k_per_rank;
    // promotion interval as in the large kernel: K held in tensor memory <= 2.5 * sqrt(K), in 32-wide blocks
    int64_t kc = 32;
    while (kc * 2 <= 128 && static_cast<double>(kc * 2) <= 2.5 * sqrt(static_cast<double>(K))) kc *= 2;
    p.chunk_blocks = static_cast<int>(kc / ST_BK);
    p.status = st->status_dev;
    // 16-byte loads need K-major rows that start on 16-byte boundaries
    p.vec_a = (layout != KAI_GEMM_TN && (K & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0) ? 1 : 0;
    p.vec_b = (layout == KAI_GEMM_NT && (K & 3) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0) ? 1 : 0;
    dim3 grid(static_cast<unsigned>((N + ST_BN - 1) / ST_BN), static_cast<unsigned>((M + ST_BM - 1) / ST_BM),
              static_cast<unsigned>(ranks));
    int rc;
    switch (layout) {
        case KAI_GEMM_NT: p.sam = K; p.sak = 1; p.sbn = K; p.sbk = 1; rc = launch_small_tc<true, true>(grid, ranks, p, s); break;
        case KAI_GEMM_NN: p.sam = K; p.sak = 1; p.sbn = 1; p.sbk = N; rc = launch_small_tc<true, false>(grid, ranks, p, s); break;
        case KAI_GEMM_TN: p.sam = 1; p.sak = M; p.sbn = 1; p.sbk = N; rc = launch_small_tc<false, false>(grid, ranks, p, s); break;
        default: return fail(KAI_E_INVALID_ARG, "gemm_small_tc: unknown layout %d", layout);
    }
    KAI_TRY(rc);
    if (st->status_host[0] != 0)
        return fail(KAI_E_DEVICE_WAIT, "a device-side wait ran out earlier (where=%d)", st->status_host[1]);
    return KAI_OK;
}

}  // namespace kai
