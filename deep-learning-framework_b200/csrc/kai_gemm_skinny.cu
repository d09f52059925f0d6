// Skinny NT product of the matmul / Linear path: Y[M,N] = X[M,K] . W[N,K]^T with M <= 16 (M = 5..16 on the warp-level
// tensor-core instruction, M <= 4 with plain FMAs: skinny_fma_kernel below)
// (inference with a handful of tokens; VMath::matmul, source/engine/support/vmath.cu:2961-2998).
//
// The call is bound by reading W once from HBM (4.N.K bytes; X and Y are a few hundred KB), so the
// kernel is built around that stream:
//   * a warp owns 16 rows of W and a contiguous range of K; a lane fetches 16-byte pieces of "its" two
//     rows, exactly the values the warp-level mma.sync.m16n8k8 TF32 instruction wants from that lane for
//     its A operand -- no lane ever needs another lane's piece of W, and no cross-lane reduction is
//     needed: the 16 x 8 accumulator fragment IS the output;
//   * W travels through a ring of shared memory that is private to each lane: a lane's eight 16-byte pieces
//     of one 64-wide step of K are fetched with cp.async (no registers held while they fly), three steps
//     deep, and read back by the same lane -- no barrier, no bank conflict (lane-major layout), and
//     2 steps x 4 KB x 16 warps = 128 KB per SM in flight, which is what HBM's latency x bandwidth asks for
//     (a register double buffer gives half of that and measured 2.6 TB/s);
//   * the eight warps of a block take interleaved 64-wide steps of K over the same 16 rows and add their
//     fragments in warp order through shared memory: one launch, no global scratch, the same bits on every run.
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
// Accuracy: 3xTF32 in registers (hi = v rounded to TF32, lo = v - hi; lo.hi + hi.lo + hi.hi).  The
// cross terms and the hi.hi chain of 64 values of K are kept in separate zeroed fragments and added
// into the fp32 result with round-to-nearest adds, as the other tensor-core kernels of the library do.
#include "kai_act.cuh"
#include "kai_common.cuh"

namespace kai {
namespace {

constexpr int SKM_WARPS = 8;    // warps per block = K ranges of one 16-row tile
constexpr int SKM_STEP = 64;    // values of K per pipeline step (4 groups of 16)
constexpr int SKM_STAGES = 3;   // ring depth: two steps in flight while one is multiplied
constexpr int SKM_RING_BYTES = SKM_WARPS * SKM_STAGES * 8 * 32 * 16;   // 96 KB per block

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// hi = v rounded to TF32 (nearest, ties away from zero) by integer arithmetic on the bits -- a carry out of
// the mantissa ripples into the exponent, which is the correctly rounded result -- and lo = v - hi, which is
// exact in fp32.  lo is handed to the tensor core as it is: whatever the core does with mantissa bits below
// TF32's ten, lo is 2^-11 of v, so the product keeps fp32-grade accuracy.  The conversion instruction
// (cvt.rna.tf32.f32) is avoided on purpose: it issues at a fraction of the rate of integer and add
// instructions, and with two of them per element of W the kernel was bound by that pipe (measured: 25 us
// for a 10 us stream).  Values whose magnitude is within 2^-11 of FLT_MAX, infinities and NaNs give NaN.
__device__ __forceinline__ void split_frag(float v, uint32_t& hi, uint32_t& lo) {
    hi = (__float_as_uint(v) + 0x1000u) & 0xFFFFE000u;
    lo = __float_as_uint(v - __uint_as_float(hi));
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
    // The eight warps interleave their 64-wide steps of K: at step s warp w takes k = (8 s + w) * 64 ..., so the
    // block as a whole reads 2 KB contiguous of each of its 16 rows per round of steps -- a DRAM page is consumed by
    // neighbouring warps at about the same time instead of being revisited over the life of one warp.
    (void)k_per_warp;
    constexpr int64_t kStride = static_cast<int64_t>(SKM_WARPS) * SKM_STEP;
    const int64_t k_begin = static_cast<int64_t>(warp) * SKM_STEP;
    const int64_t k_end = K;

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.0f;

    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    extern __shared__ float4 skm_ring[];          // [warp][stage][piece 0..7][lane]
    float4* ring = skm_ring + static_cast<size_t>(warp) * SKM_STAGES * 8 * 32 + lane;
    auto issue = [&](int64_t k0, int stage) {
        float4* dst = ring + stage * 8 * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + 16 * j;
            const bool in = (k + 4 * t) < k_end;    // K % 4 == 0: a piece is inside or outside as a whole
            cp_async16(dst + (2 * j) * 32, in ? (w0 + k) : w0, in);
            cp_async16(dst + (2 * j + 1) * 32, in ? (w1 + k) : w1, in);
        }
        cp_async_commit();                          // one group per step, also when it is empty
    };
#pragma unroll
    for (int sidx = 0; sidx < SKM_STAGES - 1; ++sidx) issue(k_begin + sidx * kStride, sidx);
    int stage = 0;
    for (int64_t k0 = k_begin; k0 < k_end; k0 += kStride) {
        // this step's pieces of X first (L1 / L2): their latency runs under the wait for the ring
        float4 xq[4][NT];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = k0 + 16 * j;
            const bool in = (k + 4 * t) < k_end;
#pragma unroll
            for (int i = 0; i < NT; ++i)
                xq[j][i] = (in && xvalid[i]) ? __ldg(reinterpret_cast<const float4*>(xrow[i] + k)) : zero4;
        }
        {
            const int nxt = (stage == 0) ? SKM_STAGES - 1 : stage - 1;      // (stage + STAGES - 1) % STAGES
            issue(k0 + (SKM_STAGES - 1) * kStride, nxt);                    // its last reader was the previous step
        }
        cp_async_wait<SKM_STAGES - 1>();                                    // this step's group has landed
        float4 wa[4], wb[4];
        {
            const float4* src = ring + stage * 8 * 32;
#pragma unroll
            for (int j = 0; j < 4; ++j) { wa[j] = src[(2 * j) * 32]; wb[j] = src[(2 * j + 1) * 32]; }
        }
        if (++stage == SKM_STAGES) stage = 0;

        float cm[NT][4], cx[NT][4];   // hi.hi chain / cross terms of this step
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) { cm[i][e] = 0.0f; cx[i][e] = 0.0f; }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float4 xv[NT];
#pragma unroll
            for (int i = 0; i < NT; ++i) xv[i] = xq[j][i];
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

// M <= 4 (and K <= 4096): plain fp32 fused multiply-adds -- with so few rows of X the arithmetic is a few FMAs per
// 16 bytes of W and needs neither the tensor core nor an operand split.  A warp owns a 512-wide range of K: its lanes
// keep their pieces of X in registers for the whole kernel (no load of X inside the loop), and the warp walks down the
// block's rows of W, 2 KB contiguous per row -- one DRAM page, asked for at once -- two rows per step of the same
// per-lane cp.async ring.  Per row a shuffle tree adds the lanes; the eight warps (eight ranges of K) add up through
// shared memory in warp order at the end.
constexpr int SKF_ROWS = 16;       // most rows of W a block takes
constexpr int SKF_KW = 512;        // values of K per warp: 4 pieces x 32 lanes x 4 floats

template <int MF>
__global__ void __launch_bounds__(SKM_WARPS * 32, 2)
skinny_fma_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M, int64_t N,
                  int64_t K, int64_t ldc, int rows_per_block, const float* __restrict__ bias,
                  const float* __restrict__ leaky_alpha, int act, int accumulate) {
    __shared__ float red[SKM_WARPS][SKF_ROWS][MF];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * rows_per_block;
    const int nrows = static_cast<int>((N - r0 < rows_per_block) ? (N - r0) : rows_per_block);
    const int64_t kb = static_cast<int64_t>(warp) * SKF_KW + 4 * lane;      // this lane's first k; pieces are 128 apart
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 xr[MF][4];
#pragma unroll
    for (int m = 0; m < MF; ++m)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            xr[m][i] = (m < M && kb + 128 * i < K) ? __ldg(reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K + kb + 128 * i))
                                                   : zero4;          // K % 4 == 0: a piece is inside or outside as a whole

    extern __shared__ float4 skm_ring[];          // [warp][stage][piece 0..7][lane]; pieces 0-3 = first row of the step
    float4* ring = skm_ring + static_cast<size_t>(warp) * SKM_STAGES * 8 * 32 + lane;
    const int steps = (nrows + 1) >> 1;
    auto issue = [&](int step, int stage) {
        float4* dst = ring + stage * 8 * 32;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const int row = 2 * step + (p >> 2);
            const int64_t k = kb + 128 * (p & 3);
            const bool in = step < steps && row < nrows && k < K;
            cp_async16(dst + p * 32, in ? (w + (r0 + row) * K + k) : w, in);
        }
        cp_async_commit();                          // one group per step, also when it is empty
    };
#pragma unroll
    for (int sidx = 0; sidx < SKM_STAGES - 1; ++sidx) issue(sidx, sidx);
    int stage = 0;
    for (int step = 0; step < steps; ++step) {
        {
            const int nxt = (stage == 0) ? SKM_STAGES - 1 : stage - 1;
            issue(step + SKM_STAGES - 1, nxt);
        }
        cp_async_wait<SKM_STAGES - 1>();
        const float4* src = ring + stage * 8 * 32;
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float4 wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) wv[i] = src[(4 * rr + i) * 32];
#pragma unroll
            for (int m = 0; m < MF; ++m) {
                float v = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    v = fmaf(wv[i].w, xr[m][i].w, fmaf(wv[i].z, xr[m][i].z, fmaf(wv[i].y, xr[m][i].y, fmaf(wv[i].x, xr[m][i].x, v))));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && 2 * step + rr < SKF_ROWS) red[warp][2 * step + rr][m] = v;
            }
        }
        if (++stage == SKM_STAGES) stage = 0;
    }
    __syncthreads();
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int e = threadIdx.x; e < SKF_ROWS * MF; e += SKM_WARPS * 32) {
        const int r = e % SKF_ROWS, m = e / SKF_ROWS;      // consecutive threads -> consecutive columns of Y
        if (r >= nrows || m >= M) continue;
        float sum = 0.0f;
#pragma unroll
        for (int ww = 0; ww < SKM_WARPS; ++ww) sum += red[ww][r][m];
        float* out = y + static_cast<int64_t>(m) * ldc + r0 + r;
        if (accumulate) sum = *out + sum;
        if (bias) sum = sum + __ldg(bias + r0 + r);
        *out = act_forward(act, sum, alpha);
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
    static bool configured[kMaxDevices] = {};
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(skinny_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SKM_RING_BYTES));
        KAI_CUDA(cudaFuncSetAttribute(skinny_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SKM_RING_BYTES));
        KAI_CUDA(cudaFuncSetAttribute(skinny_fma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SKM_RING_BYTES));
        KAI_CUDA(cudaFuncSetAttribute(skinny_fma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SKM_RING_BYTES));
        KAI_CUDA(cudaFuncSetAttribute(skinny_fma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SKM_RING_BYTES));
        configured[dev] = true;
    }
#define KAI_SKM_ARGS x, w, c, static_cast<int>(M), N, K, ldc, k_per_warp, ep.bias, ep.leaky_alpha, ep.act, ep.accumulate
    if (M <= 4 && K <= SKM_WARPS * SKF_KW) {
        // Rows per block (even, at most 16) chosen so that the blocks fill two per SM evenly: 4096 rows on 148 SMs are
        // 14 rows x 293 blocks, where 16 rows x 256 blocks would leave 40 SMs with half the work of the others.
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int64_t rpb = (N + 2 * static_cast<int64_t>(sms) - 1) / (2 * static_cast<int64_t>(sms));
        rpb = (rpb + 1) / 2 * 2;
        if (rpb > SKF_ROWS) rpb = SKF_ROWS;
        if (rpb < 2) rpb = 2;
        const unsigned fgrid = static_cast<unsigned>((N + rpb - 1) / rpb);
#define KAI_SKF_ARGS x, w, c, static_cast<int>(M), N, K, ldc, static_cast<int>(rpb), ep.bias, ep.leaky_alpha, ep.act, ep.accumulate
        if (M == 1) skinny_fma_kernel<1><<<fgrid, SKM_WARPS * 32, SKM_RING_BYTES, s>>>(KAI_SKF_ARGS);
        else if (M == 2) skinny_fma_kernel<2><<<fgrid, SKM_WARPS * 32, SKM_RING_BYTES, s>>>(KAI_SKF_ARGS);
        else skinny_fma_kernel<4><<<fgrid, SKM_WARPS * 32, SKM_RING_BYTES, s>>>(KAI_SKF_ARGS);
#undef KAI_SKF_ARGS
    }
    else if (M <= 8) skinny_mma_kernel<1><<<grid, SKM_WARPS * 32, SKM_RING_BYTES, s>>>(KAI_SKM_ARGS);
    else skinny_mma_kernel<2><<<grid, SKM_WARPS * 32, SKM_RING_BYTES, s>>>(KAI_SKM_ARGS);
#undef KAI_SKM_ARGS
    count_launch();
    return check_launch("skinny_mma_kernel");
}

}  // namespace kai
