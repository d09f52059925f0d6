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
#include "kai_act.cuh"
#include "kai_common.cuh"

namespace kai {
namespace {

// ---------------------------------------------------------------------------------------
// Generic tiled GEMM:  C[m,n] = sum_k A(m,k) B(n,k),  A(m,k) = a[m*sam + k*sak], B likewise.
// ---------------------------------------------------------------------------------------
template <int T, bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
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
// Skinny NT kernel.  One block = 4 warps = 8 consecutive rows of W; warp w takes the 16-byte
// K-chunks q with (q / 32) % 4 == w, so the block reads each W row front to back with fully
// coalesced 512-byte requests.  MT = rows of X handled (1, 2, 4, 8 or 16).
// ---------------------------------------------------------------------------------------
constexpr int SK_ROWS = 8;
constexpr int SK_WARPS = 4;

template <int MT>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_nt_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y,
                 int64_t M, int64_t N, int64_t K, int64_t ldc, const float* __restrict__ bias,
                 const float* __restrict__ leaky_alpha, int act, int accumulate) {
    __shared__ float red[SK_WARPS][SK_ROWS][MT];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * SK_ROWS;
    const int64_t kq = K >> 2;  // float4 chunks per row (K % 4 == 0 is a launch precondition)

    float acc[SK_ROWS][MT];
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    const float4* wrow[SK_ROWS];
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r) {
        const int64_t n = (n0 + r < N) ? (n0 + r) : (N - 1);  // clamp: duplicates are not stored
        wrow[r] = reinterpret_cast<const float4*>(w + n * K);
    }
    const float4* x4 = reinterpret_cast<const float4*>(x);

    for (int64_t q = warp * 32 + lane; q < kq; q += SK_WARPS * 32) {
        float4 wv[SK_ROWS];
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) wv[r] = __ldcs(wrow[r] + q);  // streamed once: evict first
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4 xv = __ldg(x4 + m * kq + q);
#pragma unroll
                for (int r = 0; r < SK_ROWS; ++r) {
                    acc[r][m] = fmaf(wv[r].x, xv.x, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].y, xv.y, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].z, xv.z, acc[r][m]);
                    acc[r][m] = fmaf(wv[r].w, xv.w, acc[r][m]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp][r][m] = v;
        }
    __syncthreads();

    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int e = threadIdx.x; e < SK_ROWS * MT; e += SK_WARPS * 32) {
        const int r = e % SK_ROWS, m = e / SK_ROWS;
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

}  // namespace

int gemm_simt(int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
              int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    const int64_t tiles64 = ((M + 63) / 64) * ((N + 63) / 64);
    if (tiles64 >= 148) return launch_simt<64>(layout, c, a, b, M, N, K, ldc, ep, s);
    return launch_simt<32>(layout, c, a, b, M, N, K, ldc, ep, s);
}

int gemm_skinny_nt(DeviceState* st, float* c, const float* x, const float* w, int64_t M, int64_t N,
                   int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s) {
    (void)st;
    if (M < 1 || M > 16) return fail(KAI_E_INVALID_ARG, "gemm_skinny_nt: M=%lld not in 1..16", (long long)M);
    if ((K & 3) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0)
        return fail(KAI_E_INVALID_ARG, "gemm_skinny_nt: needs K %% 4 == 0 and 16-byte aligned operands");
    const int64_t blocks = (N + SK_ROWS - 1) / SK_ROWS;
    if (blocks > 0x7fffffffLL) return fail(KAI_E_TOO_LARGE, "gemm_skinny_nt: N too large");
    const unsigned g = static_cast<unsigned>(blocks);
#define KAI_SKINNY(MT)                                                                                  \
    skinny_nt_kernel<MT><<<g, SK_WARPS * 32, 0, s>>>(x, w, c, M, N, K, ldc, ep.bias, ep.leaky_alpha, \
                                                      ep.act, ep.accumulate)
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
