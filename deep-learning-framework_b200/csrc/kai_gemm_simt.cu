// CUDA-core GEMM kernels of the matmul / Linear path: the shapes the tensor-core kernel is
// not the right tool for.
//
//  * gemm_simt      shared-memory tiled fp32 FMA GEMM with arbitrary operand strides: small
//                   problems (launch-latency regime, e.g. the 128-row MLP configuration),
//                   K = 0, outputs 10 columns wide.  Same three layouts as the reference trio
//                   (source/engine/support/vmath.cu:2961-3093).
//  * gemm_skinny_nt Y[M,N] = X[M,K] . W[N,K]^T for M <= 16 (inference with a handful of
//                   tokens): W is streamed from HBM exactly once with 16-byte loads, X stays
//                   in L1/L2; the kernel is bound by HBM bandwidth, not by math.
//
// Both accumulate in fp32 with fused multiply-add, which is at least as accurate as the
// reference's separately rounded multiply and add.
#include <cooperative_groups.h>

#include "kai_act.cuh"
#include "kai_common.cuh"

namespace kai {
namespace {

// ---------------------------------------------------------------------------------------
// Generic tiled GEMM:  C[m,n] = sum_k A(m,k) B(n,k),  A(m,k) = a[m*sam + k*sak], B likewise.
// ---------------------------------------------------------------------------------------
template <int T, bool A_KMAJOR, bool B_KMAJOR>
__device__ __forceinline__ void
simt_gemm_body(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
               int64_t M, int64_t N, int64_t K, int64_t sam, int64_t sak, int64_t sbn, int64_t sbk,
               int64_t ldc, const float* __restrict__ bias, const float* __restrict__ leaky_alpha,
               int act, int accumulate) {
    constexpr int BKS = 16;
    constexpr int R = T / 16;  // outputs per thread per dimension
    __shared__ float As[BKS][T + 4];
    __shared__ float Bs[BKS][T + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * T;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * T;
    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += BKS) {
        // T x 16 elements per operand, 256 threads.
#pragma unroll
        for (int e = tid; e < T * BKS; e += 256) {
            int kk, mm;
            if (A_KMAJOR) { kk = e & 15; mm = e >> 4; } else { mm = e % T; kk = e / T; }
            const int64_t m = m0 + mm, k = k0 + kk;
            As[kk][mm] = (m < M && k < K) ? a[m * sam + k * sak] : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < T * BKS; e += 256) {
            int kk, nn;
            if (B_KMAJOR) { kk = e & 15; nn = e >> 4; } else { nn = e % T; kk = e / T; }
            const int64_t n = n0 + nn, k = k0 + kk;
            Bs[kk][nn] = (n < N && k < K) ? b[n * sbn + k * sbk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BKS; ++kk) {
            float av[R], bv[R];
#pragma unroll
            for (int i = 0; i < R; ++i) av[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < R; ++j) bv[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int j = 0; j < R; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int64_t m = m0 + ty + 16 * i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int64_t n = n0 + tx + 16 * j;
            if (n >= N) continue;
            float t = acc[i][j];
            float* out = c + m * ldc + n;
            if (accumulate) t = *out + t;
            if (bias) t = t + __ldg(bias + n);
            *out = act_forward(act, t, alpha);
        }
    }
}

template <int T, bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                 int64_t M, int64_t N, int64_t K, int64_t sam, int64_t sak, int64_t sbn, int64_t sbk,
                 int64_t ldc, const float* __restrict__ bias, const float* __restrict__ leaky_alpha,
                 int act, int accumulate) {
    simt_gemm_body<T, A_KMAJOR, B_KMAJOR>(a, b, c, M, N, K, sam, sak, sbn, sbk, ldc, bias, leaky_alpha, act, accumulate);
}

// Grouped form: up to kGroupMax independent products of one shape in one launch (blockIdx.z = group).
// The operand pointers travel in the kernel parameters, so nothing is staged in device memory and the
// launch can be recorded into a call list like any other.
constexpr int kGroupMax = 32;
struct GroupPtrs {
    const float* a[kGroupMax];
    const float* b[kGroupMax];
    float* c[kGroupMax];
};

template <int T, bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(256)
simt_gemm_grouped_kernel(const __grid_constant__ GroupPtrs g, int64_t M, int64_t N, int64_t K, int64_t sam,
                         int64_t sak, int64_t sbn, int64_t sbk, int64_t ldc, const float* __restrict__ bias,
                         const float* __restrict__ leaky_alpha, int act, int accumulate) {
    const int z = blockIdx.z;
    simt_gemm_body<T, A_KMAJOR, B_KMAJOR>(g.a[z], g.b[z], g.c[z], M, N, K, sam, sak, sbn, sbk, ldc, bias, leaky_alpha,
                                          act, accumulate);
}

template <int T>
int launch_simt(int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
                int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    dim3 grid(static_cast<unsigned>((N + T - 1) / T), static_cast<unsigned>((M + T - 1) / T));
    if (grid.y > 65535u) return fail(KAI_E_TOO_LARGE, "gemm_simt: M too large for this kernel");
    switch (layout) {
        case KAI_GEMM_NT:
            simt_gemm_kernel<T, true, true><<<grid, 256, 0, s>>>(a, b, c, M, N, K, K, 1, K, 1, ldc, ep.bias,
                                                                 ep.leaky_alpha, ep.act, ep.accumulate);
            break;
        case KAI_GEMM_NN:
            simt_gemm_kernel<T, true, false><<<grid, 256, 0, s>>>(a, b, c, M, N, K, K, 1, 1, N, ldc, ep.bias,
                                                                  ep.leaky_alpha, ep.act, ep.accumulate);
            break;
        case KAI_GEMM_TN:
            simt_gemm_kernel<T, false, false><<<grid, 256, 0, s>>>(a, b, c, M, N, K, 1, M, 1, N, ldc, ep.bias,
                                                                   ep.leaky_alpha, ep.act, ep.accumulate);
            break;
        default:
            return fail(KAI_E_INVALID_ARG, "gemm_simt: unknown layout %d", layout);
    }
    count_launch();
    return check_launch("simt_gemm_kernel");
}

// ---------------------------------------------------------------------------------------
// The same tiled GEMM for problems with fewer 64 x 64 output tiles than the GPU has SMs (the
// latency regime: 512^3, the 128-row MLP layers).  The reduction dimension is split over the
// CTAs of a thread-block cluster (blockIdx.z = rank, up to 8); every CTA leaves its partial
// tile in its own shared memory and, after a cluster barrier, each rank finishes 64 / S rows of
// the tile by adding the S partials in rank order through distributed shared memory.  One
// launch, no scratch in global memory, and the result does not depend on timing.
// ---------------------------------------------------------------------------------------
template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(256)
simt_gemm_cluster_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                         int64_t M, int64_t N, int64_t K, int64_t sam, int64_t sak, int64_t sbn, int64_t sbk,
                         int64_t ldc, const float* __restrict__ bias, const float* __restrict__ leaky_alpha,
                         int act, int accumulate, int64_t k_per_rank) {
    namespace cg = cooperative_groups;
    constexpr int T = 64, BKS = 16, R = 4;
    __shared__ __align__(16) float As[BKS][T + 4];
    __shared__ __align__(16) float Bs[BKS][T + 4];
    __shared__ float part[T][T + 1];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = static_cast<int>(blockIdx.z);          // cluster = (1, 1, S): rank == blockIdx.z
    const int nrank = static_cast<int>(gridDim.z);
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * T;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * T;
    const int64_t k_begin = rank * k_per_rank;
    const int64_t k_end = (k_begin + k_per_rank < K) ? k_begin + k_per_rank : K;
    float acc[R][R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i][j] = 0.0f;

    // The next K-block's 4 + 4 values per thread are fetched into registers while the current block is
    // multiplied out of shared memory, so the global-load latency is paid once, not once per block.
    float ra[4], rb[4];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = tid + 256 * u;
            int kk, mm;
            if (A_KMAJOR) { kk = e & 15; mm = e >> 4; } else { mm = e % T; kk = e / T; }
            const int64_t m = m0 + mm, k = k0 + kk;
            ra[u] = (m < M && k < k_end) ? a[m * sam + k * sak] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = tid + 256 * u;
            int kk, nn;
            if (B_KMAJOR) { kk = e & 15; nn = e >> 4; } else { nn = e % T; kk = e / T; }
            const int64_t n = n0 + nn, k = k0 + kk;
            rb[u] = (n < N && k < k_end) ? b[n * sbn + k * sbk] : 0.0f;
        }
    };
    if (k_begin < k_end) fetch(k_begin);
    for (int64_t k0 = k_begin; k0 < k_end; k0 += BKS) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = tid + 256 * u;
            if (A_KMAJOR) As[e & 15][e >> 4] = ra[u]; else As[e / T][e % T] = ra[u];
            if (B_KMAJOR) Bs[e & 15][e >> 4] = rb[u]; else Bs[e / T][e % T] = rb[u];
        }
        __syncthreads();
        if (k0 + BKS < k_end) fetch(k0 + BKS);
#pragma unroll
        for (int kk = 0; kk < BKS; ++kk) {
            // the thread's 4 rows and 4 columns are adjacent: one 16-byte shared-memory load each
            const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][4 * ty]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][4 * tx]);
            const float av[R] = {a4.x, a4.y, a4.z, a4.w}, bv[R] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int j = 0; j < R; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) part[4 * ty + i][4 * tx + j] = acc[i][j];
    cluster.sync();

    // rank r finishes rows [r * T / S, (r + 1) * T / S) of the tile
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    const int rows = T / nrank;
    for (int e = tid; e < rows * T; e += 256) {
        const int row = rank * rows + e / T, col = e % T;
        float t = 0.0f;
        for (int z = 0; z < nrank; ++z) t += cluster.map_shared_rank(&part[0][0], z)[row * (T + 1) + col];
        const int64_t m = m0 + row, n = n0 + col;
        if (m < M && n < N) {
            float* out = c + m * ldc + n;
            if (accumulate) t = *out + t;
            if (bias) t = t + __ldg(bias + n);
            *out = act_forward(act, t, alpha);
        }
    }
    cluster.sync();   // nobody leaves while a neighbour may still read its partial tile
}

template <bool A_KMAJOR, bool B_KMAJOR>
int launch_cluster_one(dim3 grid, int ranks, const float* a, const float* b, float* c, int64_t M, int64_t N, int64_t K,
                       int64_t sam, int64_t sak, int64_t sbn, int64_t sbk, int64_t ldc, const Epilogue& ep,
                       int64_t k_per_rank, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = static_cast<unsigned>(ranks);
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    KAI_CUDA(cudaLaunchKernelEx(&cfg, simt_gemm_cluster_kernel<A_KMAJOR, B_KMAJOR>, a, b, c, M, N, K, sam, sak, sbn,
                                sbk, ldc, ep.bias, ep.leaky_alpha, ep.act, ep.accumulate, k_per_rank));
    count_launch();
    return check_launch("simt_gemm_cluster_kernel");
}

int launch_simt_cluster(int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
                        int64_t ldc, const Epilogue& ep, int sm_count, cudaStream_t s) {
    const int64_t tiles = ((M + 63) / 64) * ((N + 63) / 64);
    int ranks = 1;
    while (ranks < 8 && tiles * ranks < sm_count && K / (ranks * 2) >= 32) ranks *= 2;
    int64_t k_per_rank = ((K + ranks - 1) / ranks + 15) / 16 * 16;
    if (k_per_rank < 16) k_per_rank = 16;
    dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64), static_cast<unsigned>(ranks));
    switch (layout) {
        case KAI_GEMM_NT:
            return launch_cluster_one<true, true>(grid, ranks, a, b, c, M, N, K, K, 1, K, 1, ldc, ep, k_per_rank, s);
        case KAI_GEMM_NN:
            return launch_cluster_one<true, false>(grid, ranks, a, b, c, M, N, K, K, 1, 1, N, ldc, ep, k_per_rank, s);
        case KAI_GEMM_TN:
            return launch_cluster_one<false, false>(grid, ranks, a, b, c, M, N, K, 1, M, 1, N, ldc, ep, k_per_rank, s);
        default:
            return fail(KAI_E_INVALID_ARG, "gemm_simt: unknown layout %d", layout);
    }
}

// ---------------------------------------------------------------------------------------
// Skinny NT kernel.  One block = 4 warps = 8 consecutive rows of W; warp w takes the 16-byte
// K-chunks q with (q / 32) % 4 == w, so the block reads each W row front to back with fully
// coalesced 512-byte requests.  MT = rows of X handled (1, 2, 4, 8 or 16).
// ---------------------------------------------------------------------------------------
constexpr int SK_ROWS = 8;
constexpr int SK_WARPS = 4;

template <int MT, int ROWS>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_nt_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                 int64_t M, int64_t N, int64_t K, int64_t ldc, const float* __restrict__ bias,
                 const float* __restrict__ leaky_alpha, int act, int accumulate) {
    __shared__ float red[SK_WARPS][ROWS][MT];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * ROWS;
    const int64_t kq = K >> 2;  // float4 chunks per row (K % 4 == 0 is a launch precondition)

    float acc[ROWS][MT];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    const float4* wrow[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int64_t n = (n0 + r < N) ? (n0 + r) : (N - 1);  // clamp: duplicates are not stored
        wrow[r] = reinterpret_cast<const float4*>(w + n * K);
    }
    const float4* x4 = reinterpret_cast<const float4*>(x);

    for (int64_t q = warp * 32 + lane; q < kq; q += SK_WARPS * 32) {
        float4 wv[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) wv[r] = __ldcs(wrow[r] + q);  // streamed once: evict first
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4 xv = __ldg(x4 + m * kq + q);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    acc[r][m] = fmaf(wv[r].x, xv.x, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].y, xv.y, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].z, xv.z, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].w, xv.w, acc[r][m]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp][r][m] = v;
        }
    __syncthreads();

    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int e = threadIdx.x; e < ROWS * MT; e += SK_WARPS * 32) {
        const int r = e % ROWS, m = e / ROWS;
        const int64_t n = n0 + r;
        if (n >= N || m >= M) continue;
        float t = 0.0f;
#pragma unroll
        for (int ww = 0; ww < SK_WARPS; ++ww) t += red[ww][r][m];
        float* out = y + static_cast<int64_t>(m) * ldc + n;
        if (accumulate) t = *out + t;
        if (bias) t = t + __ldg(bias + n);
        *out = act_forward(act, t, alpha);
    }
}

// ---------------------------------------------------------------------------------------
// Skinny NT kernel for M = 5..16: X lives in registers.
// With 8 or 16 rows of X the row-streaming kernel above re-reads X from L1 for every piece of W
// and becomes load-issue bound.  Here a thread owns one 16-byte K slot of a 1024-wide K chunk and
// keeps the MT values of X for that slot in registers (4 MT registers); the block then walks
// down the rows of W: one 16-byte load of W, 4 MT FMAs, and a halving butterfly over the warp
// (MT + ... + 1 shuffles) that leaves one of the MT sums in every other lane.  Eight rows are
// batched between block-level reductions.  Each (row slab, K chunk) block writes partial sums; a
// small second kernel adds the K chunks in a fixed order and applies the epilogue.
// ---------------------------------------------------------------------------------------
constexpr int SX_THREADS = 256;
constexpr int SX_KC = SX_THREADS * 4;   // 1024 values of K per block
constexpr int SX_BATCH = 8;             // rows between block reductions

template <int MT>
__global__ void __launch_bounds__(SX_THREADS)
skinny_regx_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ part,
                   int64_t M, int64_t N, int64_t K, int64_t rows_per_block) {
    __shared__ float red[SX_BATCH][SX_THREADS / 32][MT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t k = static_cast<int64_t>(blockIdx.y) * SX_KC + 4 * tid;
    const bool kvalid = k < K;            // K % 4 == 0: a slot is inside or outside as a whole
    const int64_t n_begin = static_cast<int64_t>(blockIdx.x) * rows_per_block;
    const int64_t n_end = min(N, n_begin + rows_per_block);

    float4 xr[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m)
        xr[m] = (kvalid && m < M) ? __ldg(reinterpret_cast<const float4*>(x + m * K + k)) : make_float4(0.f, 0.f, 0.f, 0.f);

    // which of the MT sums this lane holds after the butterfly (valid in even lanes for MT = 16,
    // in lanes that are multiples of 4 for MT = 8)
    int my_m = 0;
    {
        int cnt = MT / 2;
        for (int off = 16; cnt >= 1; off >>= 1, cnt >>= 1)
            if (lane & off) my_m += cnt;
    }
    constexpr int LANE_STEP = 32 / MT;    // lanes that end up holding distinct sums are LANE_STEP apart

    const float* wp = w + k;
    auto load_batch = [&](int64_t n0, float4 (&dst)[SX_BATCH]) {
#pragma unroll
        for (int r = 0; r < SX_BATCH; ++r)
            dst[r] = (kvalid && n0 + r < n_end) ? __ldcs(reinterpret_cast<const float4*>(wp + (n0 + r) * K))
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    float4 wnext[SX_BATCH];
    load_batch(n_begin, wnext);
    for (int64_t n0 = n_begin; n0 < n_end; n0 += SX_BATCH) {
        float4 wv[SX_BATCH];
#pragma unroll
        for (int r = 0; r < SX_BATCH; ++r) wv[r] = wnext[r];
        load_batch(n0 + SX_BATCH, wnext);   // in flight while this batch is multiplied and reduced
#pragma unroll
        for (int r = 0; r < SX_BATCH; ++r) {
            float v[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                v[m] = fmaf(wv[r].w, xr[m].w, fmaf(wv[r].z, xr[m].z, fmaf(wv[r].y, xr[m].y, wv[r].x * xr[m].x)));
            // halving butterfly: each step keeps half of the sums and adds the partner's half
            int off = 16;
#pragma unroll
            for (int cnt = MT / 2; cnt >= 1; cnt >>= 1, off >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < cnt; ++i) {
                    const float send = upper ? v[i] : v[i + cnt];
                    const float keep = upper ? v[i + cnt] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            for (; off >= 1; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
            if ((lane & (LANE_STEP - 1)) == 0) red[r][warp][my_m] = v[0];
        }
        __syncthreads();
        // SX_BATCH x MT outputs of this batch: add the eight warps in a fixed order
        for (int e = tid; e < SX_BATCH * MT; e += SX_THREADS) {
            const int r = e / MT, m = e % MT;
            const int64_t n = n0 + r;
            if (n < n_end) {
                float t = 0.0f;
#pragma unroll
                for (int ww = 0; ww < SX_THREADS / 32; ++ww) t += red[r][ww][m];
                part[(static_cast<int64_t>(blockIdx.y) * N + n) * MT + m] = t;
            }
        }
        __syncthreads();
    }
}

template <int MT>
__global__ void skinny_regx_finish_kernel(const float* __restrict__ part, int chunks, float* __restrict__ y,
                                          int64_t M, int64_t N, int64_t ldc, const float* __restrict__ bias,
                                          const float* __restrict__ leaky_alpha, int act, int accumulate) {
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    const int64_t total = N * MT;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t n = i / MT;
        const int m = static_cast<int>(i % MT);
        if (m >= M) continue;
        float t = 0.0f;
        for (int c = 0; c < chunks; ++c) t += part[static_cast<int64_t>(c) * total + i];
        float* out = y + static_cast<int64_t>(m) * ldc + n;
        if (accumulate) t = *out + t;
        if (bias) t = t + __ldg(bias + n);
        *out = act_forward(act, t, alpha);
    }
}

template <int MT>
int launch_skinny_regx(DeviceState* st, const float* x, const float* w, float* c, int64_t M, int64_t N, int64_t K,
                       int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    const int64_t chunks = (K + SX_KC - 1) / SX_KC;
    if (chunks > 65535) return fail(KAI_E_TOO_LARGE, "gemm_skinny_nt: K too large");
    // about four blocks per SM, whole batches of rows per block
    int64_t row_blocks = (static_cast<int64_t>(st->sm_count) * 4 + chunks - 1) / chunks;
    int64_t rows_per_block = (N + row_blocks - 1) / row_blocks;
    rows_per_block = (rows_per_block + SX_BATCH - 1) / SX_BATCH * SX_BATCH;
    row_blocks = (N + rows_per_block - 1) / rows_per_block;
    KAI_TRY(ensure_workspace(st, 0, chunks * N * MT * 4));
    float* part = static_cast<float*>(st->ws);
    dim3 grid(static_cast<unsigned>(row_blocks), static_cast<unsigned>(chunks));
    skinny_regx_kernel<MT><<<grid, SX_THREADS, 0, s>>>(x, w, part, M, N, K, rows_per_block);
    count_launch();
    KAI_TRY(check_launch("skinny_regx_kernel"));
    const int64_t total = N * MT;
    int64_t blocks = (total + 255) / 256;
    if (blocks > st->sm_count * 8) blocks = st->sm_count * 8;
    skinny_regx_finish_kernel<MT><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        part, static_cast<int>(chunks), c, M, N, ldc, ep.bias, ep.leaky_alpha, ep.act, ep.accumulate);
    count_launch();
    return check_launch("skinny_regx_finish_kernel");
}

}  // namespace

int gemm_simt(int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
              int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    const int64_t tiles64 = ((M + 63) / 64) * ((N + 63) / 64);
    if (tiles64 >= 148 || tiles64 > 65535) return launch_simt<64>(layout, c, a, b, M, N, K, ldc, ep, s);
    return launch_simt_cluster(layout, c, a, b, M, N, K, ldc, ep, 148, s);
}

// `count` products C_i (+)= op(A_i).op(B_i) of one shape, kGroupMax per launch.  Outputs of different groups
// must not overlap (they are written concurrently); a group may read what an earlier CALL wrote, not what another
// group of the same call writes.
int gemm_simt_grouped(int layout, int count, float* const* c, const float* const* a, const float* const* b, int64_t M,
                      int64_t N, int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    constexpr int T = 64;
    dim3 grid(static_cast<unsigned>((N + T - 1) / T), static_cast<unsigned>((M + T - 1) / T), 1);
    if (grid.y > 65535u) return fail(KAI_E_TOO_LARGE, "sgemm_grouped: M too large for this kernel");
    for (int g0 = 0; g0 < count; g0 += kGroupMax) {
        const int n = (count - g0 < kGroupMax) ? (count - g0) : kGroupMax;
        GroupPtrs gp;
        for (int i = 0; i < kGroupMax; ++i) {
            const int j = g0 + (i < n ? i : 0);
            gp.a[i] = a[j]; gp.b[i] = b[j]; gp.c[i] = c[j];
        }
        grid.z = static_cast<unsigned>(n);
        switch (layout) {
            case KAI_GEMM_NT:
                simt_gemm_grouped_kernel<T, true, true><<<grid, 256, 0, s>>>(gp, M, N, K, K, 1, K, 1, ldc, ep.bias,
                                                                             ep.leaky_alpha, ep.act, ep.accumulate);
                break;
            case KAI_GEMM_NN:
                simt_gemm_grouped_kernel<T, true, false><<<grid, 256, 0, s>>>(gp, M, N, K, K, 1, 1, N, ldc, ep.bias,
                                                                              ep.leaky_alpha, ep.act, ep.accumulate);
                break;
            case KAI_GEMM_TN:
                simt_gemm_grouped_kernel<T, false, false><<<grid, 256, 0, s>>>(gp, M, N, K, 1, M, 1, N, ldc, ep.bias,
                                                                               ep.leaky_alpha, ep.act, ep.accumulate);
                break;
            default:
                return fail(KAI_E_INVALID_ARG, "sgemm_grouped: unknown layout %d", layout);
        }
        count_launch();
        KAI_TRY(check_launch("simt_gemm_grouped_kernel"));
    }
    return KAI_OK;
}

int gemm_skinny_nt(DeviceState* st, float* c, const float* x, const float* w, int64_t M, int64_t N,
                   int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    if (M < 1 || M > 16) return fail(KAI_E_INVALID_ARG, "gemm_skinny_nt: M=%lld not in 1..16", (long long)M);
    if ((K & 3) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0)
        return fail(KAI_E_INVALID_ARG, "gemm_skinny_nt: needs K %% 4 == 0 and 16-byte aligned operands");
    // Default: the warp-MMA streaming kernel (kai_gemm_skinny.cu).  "skinny_mma" = 0 selects the CUDA-core
    // kernels below, which it replaced (kept for comparison runs).
    if (options().skinny_mma.load() != 0) return gemm_skinny_mma(c, x, w, M, N, K, ldc, ep, s);
    if (M > 4 && options().skinny_regx.load() != 0) {
        if (M <= 8) return launch_skinny_regx<8>(st, x, w, c, M, N, K, ldc, ep, s);
        return launch_skinny_regx<16>(st, x, w, c, M, N, K, ldc, ep, s);
    }
    // Rows of W per block: 8 by default; 4 for M <= 4, which evens out the load over the SMs (4096 rows:
    // 512 blocks are 3.46 per SM, 1024 blocks 6.9).  "skinny_rows": 0 = choose, 2, 4 or 8 = force.
    int rows = SK_ROWS;
    const int64_t forced_rows = options().skinny_rows.load();
    if (forced_rows == 2) rows = 2;
    else if (forced_rows == 4 || (forced_rows == 0 && M <= 4)) rows = 4;
    const int64_t blocks = (N + rows - 1) / rows;
    if (blocks > 0x7fffffffLL) return fail(KAI_E_TOO_LARGE, "gemm_skinny_nt: N too large");
    const unsigned g = static_cast<unsigned>(blocks);
#define KAI_SKINNY(MT)                                                                                        \
    do {                                                                                                      \
        if (rows == 2)                                                                                        \
            skinny_nt_kernel<MT, 2><<<g, SK_WARPS * 32, 0, s>>>(x, w, c, M, N, K, ldc, ep.bias, ep.leaky_alpha, \
                                                                 ep.act, ep.accumulate);                      \
        else if (rows == 4)                                                                                   \
            skinny_nt_kernel<MT, 4><<<g, SK_WARPS * 32, 0, s>>>(x, w, c, M, N, K, ldc, ep.bias, ep.leaky_alpha, \
                                                                 ep.act, ep.accumulate);                      \
        else                                                                                                  \
            skinny_nt_kernel<MT, 8><<<g, SK_WARPS * 32, 0, s>>>(x, w, c, M, N, K, ldc, ep.bias, ep.leaky_alpha, \
                                                                 ep.act, ep.accumulate);                      \
    } while (0)
    if (M == 1) KAI_SKINNY(1);
    else if (M == 2) KAI_SKINNY(2);
    else if (M <= 4) KAI_SKINNY(4);
    else if (M <= 8) KAI_SKINNY(8);
    else KAI_SKINNY(16);
#undef KAI_SKINNY
    count_launch();
    return check_launch("skinny_nt_kernel");
}

}  // namespace kai
