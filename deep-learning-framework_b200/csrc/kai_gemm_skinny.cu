// Skinny NT product of the matmul / Linear path: Y[M,N] = X[M,K] . W[N,K]^T with M <= 16
// (inference with a handful of tokens; VMath::matmul, source/engine/support/vmath.cu:2961-2998).
//
// The call is bound by reading W once from HBM (4.N.K bytes; X and Y are a few hundred KB), so the
// kernel is built around that stream:
//   * a warp owns 16 rows of W and a contiguous range of K; a lane reads 16-byte pieces of "its" two
//     rows straight from global memory into registers, in exactly the layout the warp-level
//     mma.sync.m16n8k8 TF32 instruction wants for its A operand -- W never passes through shared
//     memory and no cross-lane reduction is needed: the 16 x 8 accumulator fragment IS the output;
//   * the loads of the next 64 values of K are in flight while the current 64 are multiplied (two
//     register stages of 8 x 16 bytes per lane, 4 KB per warp, 16 warps per SM);
//   * the eight warps of a block take eight K ranges of the same 16 rows and add their fragments in
//     warp order through shared memory: one launch, no global scratch, the same bits on every run.
// CUDA-core forms of this product need a reduction over lanes (shuffles) or re-read X from shared
// memory for every piece of W and end up bound by those instructions at M = 8..16; the tensor core
// does the 16 x M x 8 block product in one instruction.
//
// Inside a group of 16 values of K the instruction's eight reduction slots are filled in the order
// that makes a lane's operands adjacent in memory: lane (g, t) holds W[row g][k0 + 4t .. 4t+3]; the
// first MMA of the group takes elements .x (slot t) and .y (slot t + 4), the second .z and .w.  X is
// read with the same mapping, so A and B agree on which k sits in which slot; the sum over the group
// is unchanged.
//
// Accuracy: 3xTF32 in registers (hi = rna_tf32(v), lo = rna_tf32(v - hi); lo.hi + hi.lo + hi.hi).  The
// cross terms and the hi.hi chain of 64 values of K are kept in separate zeroed fragments and added
// into the fp32 result with round-to-nearest adds, as the other tensor-core kernels of the library do.
#include "kai_act.cuh"
#include "kai_common.cuh"

namespace kai {
namespace {

constexpr int SKM_WARPS = 8;    // warps per block = K ranges of one 16-row tile
constexpr int SKM_STEP = 64;    // values of K per pipeline step (4 groups of 16)

__device__ __forceinline__ void split_frag(float v, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(v));
    const float rest = v - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(rest));
}

// D(16x8) += A(16x8, row) . B(8x8, col), TF32 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// NT = number of 8-column output tiles: 1 for M <= 8, 2 for M <= 16.
template <int NT>
__global__ void __launch_bounds__(SKM_WARPS * 32, 2)
skinny_mma_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M, int64_t N,
                  int64_t K, int64_t ldc, int64_t k_per_warp, const float* __restrict__ bias,
                  const float* __restrict__ leaky_alpha, int act, int accumulate) {
    __shared__ float red[SKM_WARPS][16][8 * NT + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * 16;
    // rows past N are clamped (their results are never stored)
    const int64_t r0 = (n0 + g < N) ? (n0 + g) : (N - 1);
    const int64_t r1 = (n0 + g + 8 < N) ? (n0 + g + 8) : (N - 1);
    const float* w0 = w + r0 * K + 4 * t;
    const float* w1 = w + r1 * K + 4 * t;
    const float* xrow[NT];
    bool xvalid[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        xvalid[i] = (g + 8 * i) < M;
        xrow[i] = x + static_cast<int64_t>(xvalid[i] ? g + 8 * i : 0) * K + 4 * t;
    }
    const int64_t k_begin = static_cast<int64_t>(warp) * k_per_warp;
    const int64_t k_end = (k_begin + k_per_warp < K) ? (k_begin + k_per_warp) : K;

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.0f;

    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 na[4], nb[4];
    auto load = [&](int64_t k0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + 16 * j;
            const bool in = (k + 4 * t) < k_end;    // K % 4 == 0: a piece is inside or outside as a whole
            na[j] = in ? __ldcs(reinterpret_cast<const float4*>(w0 + k)) : zero4;   // streamed once
            nb[j] = in ? __ldcs(reinterpret_cast<const float4*>(w1 + k)) : zero4;
        }
    };
    if (k_begin < k_end) load(k_begin);
    for (int64_t k0 = k_begin; k0 < k_end; k0 += SKM_STEP) {
        float4 wa[4], wb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { wa[j] = na[j]; wb[j] = nb[j]; }
        if (k0 + SKM_STEP < k_end) load(k0 + SKM_STEP);   // in flight while this step is multiplied

        float cm[NT][4], cx[NT][4];   // hi.hi chain / cross terms of this step
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) { cm[i][e] = 0.0f; cx[i][e] = 0.0f; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + 16 * j;
            const bool in = (k + 4 * t) < k_end;
            float4 xv[NT];
#pragma unroll
            for (int i = 0; i < NT; ++i)
                xv[i] = (in && xvalid[i]) ? __ldg(reinterpret_cast<const float4*>(xrow[i] + k)) : zero4;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t ah[4], al[4];
                split_frag(half ? wa[j].z : wa[j].x, ah[0], al[0]);   // (row g,     slot t)
                split_frag(half ? wb[j].z : wb[j].x, ah[1], al[1]);   // (row g + 8, slot t)
                split_frag(half ? wa[j].w : wa[j].y, ah[2], al[2]);   // (row g,     slot t + 4)
                split_frag(half ? wb[j].w : wb[j].y, ah[3], al[3]);   // (row g + 8, slot t + 4)
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                    uint32_t bh[2], bl[2];
                    split_frag(half ? xv[i].z : xv[i].x, bh[0], bl[0]);   // (slot t,     column g)
                    split_frag(half ? xv[i].w : xv[i].y, bh[1], bl[1]);   // (slot t + 4, column g)
                    mma_tf32(cx[i], al, bh);
                    mma_tf32(cx[i], ah, bl);
                    mma_tf32(cm[i], ah, bh);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][e] += cm[i][e] + cx[i][e];
    }

    // fragment element e of tile i: row g (e = 0, 1) or g + 8 (e = 2, 3), column 8 i + 2 t + (e & 1)
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        red[warp][g][8 * i + 2 * t] = acc[i][0];
        red[warp][g][8 * i + 2 * t + 1] = acc[i][1];
        red[warp][g + 8][8 * i + 2 * t] = acc[i][2];
        red[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();

    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int e = threadIdx.x; e < 16 * 8 * NT; e += SKM_WARPS * 32) {
        const int r = e & 15, m = e >> 4;      // consecutive threads -> consecutive columns of Y
        const int64_t n = n0 + r;
        if (n >= N || m >= M) continue;
        float s = 0.0f;
#pragma unroll
        for (int ww = 0; ww < SKM_WARPS; ++ww) s += red[ww][r][m];
        float* out = y + static_cast<int64_t>(m) * ldc + n;
        if (accumulate) s = *out + s;
        if (bias) s = s + __ldg(bias + n);
        *out = act_forward(act, s, alpha);
    }
}

}  // namespace

int gemm_skinny_mma(float* c, const float* x, const float* w, int64_t M, int64_t N, int64_t K, int64_t ldc,
                    const Epilogue& ep, cudaStream_t s) {
    if (M < 1 || M > 16) return fail(KAI_E_INVALID_ARG, "gemm_skinny_mma: M=%lld not in 1..16", (long long)M);
    if ((K & 3) != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) != 0)
        return fail(KAI_E_INVALID_ARG, "gemm_skinny_mma: needs K %% 4 == 0 and 16-byte aligned operands");
    const int64_t blocks = (N + 15) / 16;
    if (blocks > 0x7fffffffLL) return fail(KAI_E_TOO_LARGE, "gemm_skinny_mma: N too large");
    int64_t k_per_warp = (K + SKM_WARPS - 1) / SKM_WARPS;
    k_per_warp = (k_per_warp + SKM_STEP - 1) / SKM_STEP * SKM_STEP;
    const unsigned grid = static_cast<unsigned>(blocks);
    if (M <= 8)
        skinny_mma_kernel<1><<<grid, SKM_WARPS * 32, 0, s>>>(x, w, c, static_cast<int>(M), N, K, ldc, k_per_warp, ep.bias,
                                                             ep.leaky_alpha, ep.act, ep.accumulate);
    else
        skinny_mma_kernel<2><<<grid, SKM_WARPS * 32, 0, s>>>(x, w, c, static_cast<int>(M), N, K, ldc, k_per_warp, ep.bias,
                                                             ep.leaky_alpha, ep.act, ep.accumulate);
    count_launch();
    return check_launch("skinny_mma_kernel");
}

}  // namespace kai
