// Tensor-core forms of the attention contractions, in the reference's tensor layouts
// (source/engine/support/vmath.cu:6729-6750 mult_on_heads, 6864-6885 softmax_direct_on_axis,
// 6977-6997 mix_values).
//
// The head-minor `probs[b,q,k,h]` tensor makes these GEMMs awkward for bulk tensor copies: the
// reduction index of P.V is strided by nhead, and Q.K^T has to emit all heads of a (q,k) pair
// together to write whole 32-byte runs.  They are therefore written with warp-level
// mma.sync.m16n8k8 TF32 tensor-core instructions, whose operand fragments are gathered from
// shared memory by the threads themselves, and use the same 3xTF32 split as the big GEMM
// (a = hi + lo; a.b ~ lo.hi + hi.lo + hi.hi) with the hi/lo parts formed in registers.
//
// Accumulation: the tensor core's fp32 accumulate truncates (see kai_gemm_tc.cu), so
//   * Q.K^T (reduction over npiece <= 128) keeps the small cross terms in their own accumulator and
//     the hi.hi chain in another, added once at the end;
//   * P.V (reduction over ntimes keys) accumulates 16 keys at a time into a zeroed fragment and adds
//     each finished fragment into fp32 registers with a round-to-nearest add.
//
// Inside each group of eight reduction indices the columns are consumed in the order
// (0,4,1,5,2,6,3,7): a thread's two A (and B) values of one instruction are then adjacent in
// shared memory and load as one 64-bit word; the sum over the group is unchanged.
//
// Every launcher returns kNotApplicable for shapes outside its fast path; the caller then uses
// the CUDA-core kernels of kai_attention.cu.
#include <float.h>

#include "kai_common.cuh"

namespace kai {
namespace {

constexpr int kNotApplicable = 1;

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

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---------------------------------------------------------------------------------------
// mult_on_heads: probs[b,q,k,h] = coef * sum_p K[b,k,h*P+p] * Q[b,q,h*P+p]
// Block = (b, 64 queries, 64 keys), 8 warps as 4 (16 queries) x 2 (32 keys).  Heads are taken
// eight at a time; the Q_h / K_h tiles of the next head arrive by cp.async while the current
// head is multiplied.  A thread ends up with the eight head values of each of its (q,k) pairs
// and stores them as one 32-byte run.
// ---------------------------------------------------------------------------------------
constexpr int MM_T = 64;
constexpr int MM_HG = 8;

__global__ void __launch_bounds__(256, 1)
mult_on_heads_mma_kernel(float* __restrict__ pp, const float* __restrict__ pK, const float* __restrict__ pQ,
                         int ntimes, int nvec, int nhead, int npiece, const float* __restrict__ coef_ptr) {
    extern __shared__ __align__(16) float mm_smem[];
    const int ps = npiece + 4;            // row stride in floats (16-byte multiple)
    const int tile_f = MM_T * ps;         // floats per operand tile
    // layout: [buffer 0: Q tile, K tile][buffer 1: Q tile, K tile]
    const float coef = (coef_ptr != nullptr) ? __ldg(coef_ptr) : 0.0f;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wq = warp & 3, wk = warp >> 2;
    const int b = blockIdx.z;
    const int q0 = blockIdx.y * MM_T, k0 = blockIdx.x * MM_T;
    const float* Qb = pQ + static_cast<int64_t>(b) * ntimes * nvec;
    const float* Kb = pK + static_cast<int64_t>(b) * ntimes * nvec;
    float* Pb = pp + static_cast<int64_t>(b) * ntimes * ntimes * nhead;
    const int quads = npiece >> 2;        // 16-byte pieces per row

    auto prefetch = [&](int head, int buf) {
        float* Qs = mm_smem + buf * 2 * tile_f;
        float* Ks = Qs + tile_f;
        const int col0 = head * npiece;
        for (int e = tid; e < MM_T * quads; e += 256) {
            const int r = e / quads, c4 = (e - r * quads) << 2;
            const bool vq = (q0 + r) < ntimes, vk = (k0 + r) < ntimes;
            cp_async16(Qs + r * ps + c4, Qb + static_cast<int64_t>(vq ? q0 + r : 0) * nvec + col0 + c4, vq);
            cp_async16(Ks + r * ps + c4, Kb + static_cast<int64_t>(vk ? k0 + r : 0) * nvec + col0 + c4, vk);
        }
        cp_async_commit();
    };

    for (int hg = 0; hg < nhead; hg += MM_HG) {
        const int nh = min(MM_HG, nhead - hg);
        float acc[MM_HG][4][4];
#pragma unroll
        for (int h = 0; h < MM_HG; ++h)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[h][nt][i] = 0.0f;

        prefetch(hg, 0);
#pragma unroll
        for (int h = 0; h < MM_HG; ++h) {
            if (h < nh) {
                if (h + 1 < nh) {
                    prefetch(hg + h + 1, (h + 1) & 1);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();
                const float* Qs = mm_smem + (h & 1) * 2 * tile_f;
                const float* Ks = Qs + tile_f;
                float cm[4][4], cx[4][4];  // hi.hi chain / cross terms
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) { cm[nt][i] = 0.0f; cx[nt][i] = 0.0f; }
                const float* qrow0 = Qs + (wq * 16 + g) * ps + 2 * t;
                const float* qrow1 = qrow0 + 8 * ps;
                const float* krow = Ks + (wk * 32 + g) * ps + 2 * t;
                for (int kk = 0; kk < npiece; kk += 8) {
                    const float2 v0 = *reinterpret_cast<const float2*>(qrow0 + kk);
                    const float2 v1 = *reinterpret_cast<const float2*>(qrow1 + kk);
                    uint32_t ah[4], al[4];
                    split_frag(v0.x, ah[0], al[0]);
                    split_frag(v1.x, ah[1], al[1]);
                    split_frag(v0.y, ah[2], al[2]);
                    split_frag(v1.y, ah[3], al[3]);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const float2 w = *reinterpret_cast<const float2*>(krow + nt * 8 * ps + kk);
                        uint32_t bh[2], bl[2];
                        split_frag(w.x, bh[0], bl[0]);
                        split_frag(w.y, bh[1], bl[1]);
                        mma_tf32(cx[nt], al, bh);
                        mma_tf32(cx[nt], ah, bl);
                        mma_tf32(cm[nt], ah, bh);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[h][nt][i] = (cm[nt][i] + cx[nt][i]) * coef;
                __syncthreads();  // the buffer is refilled two heads later
            }
        }

        // C fragment: c0 (row g, col 2t), c1 (g, 2t+1), c2 (g+8, 2t), c3 (g+8, 2t+1)
        const bool vec_out = (nh == MM_HG) && (nhead % 4 == 0) && ((reinterpret_cast<uintptr_t>(pp) & 15) == 0);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int q = q0 + wq * 16 + g + ((i >> 1) << 3);
                const int k = k0 + wk * 32 + nt * 8 + 2 * t + (i & 1);
                if (q < ntimes && k < ntimes) {
                    float* out = Pb + (static_cast<int64_t>(q) * ntimes + k) * nhead + hg;
                    if (vec_out) {
                        reinterpret_cast<float4*>(out)[0] =
                            make_float4(acc[0][nt][i], acc[1][nt][i], acc[2][nt][i], acc[3][nt][i]);
                        reinterpret_cast<float4*>(out)[1] =
                            make_float4(acc[4][nt][i], acc[5][nt][i], acc[6][nt][i], acc[7][nt][i]);
                    } else {
#pragma unroll
                        for (int h = 0; h < MM_HG; ++h)
                            if (h < nh) out[h] = acc[h][nt][i];
                    }
                }
            }
    }
}

// ---------------------------------------------------------------------------------------
// softmax_direct_on_axis for slabs that fit one warp's registers: one warp per row of
// pp[nrow][nvec][NCOL], every lane holds PER_LANE 16-byte pieces (so all loads of a row are in
// flight at once), column maxima and sums by shuffles among the lanes that own the same
// columns.  NCOL in {4, 8, 16, 32}; nvec * NCOL = 128 * PER_LANE.
// ---------------------------------------------------------------------------------------
template <int NCOL, int PER_LANE>
__global__ void __launch_bounds__(256)
softmax_axis_warp_kernel(float* __restrict__ pp, int64_t nrow) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (row >= nrow) return;
    float4* base = reinterpret_cast<float4*>(pp + row * (128 * PER_LANE));
    float4 v[PER_LANE];
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) v[j] = __ldcs(base + lane + 32 * j);
    // piece f = lane + 32 j covers columns (4 f) % NCOL .. +3: the same four columns for every j
    float4 mx = make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        mx.x = fmaxf(mx.x, v[j].x); mx.y = fmaxf(mx.y, v[j].y);
        mx.z = fmaxf(mx.z, v[j].z); mx.w = fmaxf(mx.w, v[j].w);
    }
#pragma unroll
    for (int o = NCOL / 4; o < 32; o <<= 1) {
        mx.x = fmaxf(mx.x, __shfl_xor_sync(0xffffffffu, mx.x, o));
        mx.y = fmaxf(mx.y, __shfl_xor_sync(0xffffffffu, mx.y, o));
        mx.z = fmaxf(mx.z, __shfl_xor_sync(0xffffffffu, mx.z, o));
        mx.w = fmaxf(mx.w, __shfl_xor_sync(0xffffffffu, mx.w, o));
    }
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        v[j].x = expf(v[j].x - mx.x); v[j].y = expf(v[j].y - mx.y);
        v[j].z = expf(v[j].z - mx.z); v[j].w = expf(v[j].w - mx.w);
        sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w;
    }
#pragma unroll
    for (int o = NCOL / 4; o < 32; o <<= 1) {
        sum.x += __shfl_xor_sync(0xffffffffu, sum.x, o);
        sum.y += __shfl_xor_sync(0xffffffffu, sum.y, o);
        sum.z += __shfl_xor_sync(0xffffffffu, sum.z, o);
        sum.w += __shfl_xor_sync(0xffffffffu, sum.w, o);
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        v[j].x /= sum.x; v[j].y /= sum.y; v[j].z /= sum.z; v[j].w /= sum.w;
        base[lane + 32 * j] = v[j];
    }
}

// ---------------------------------------------------------------------------------------
// mix_values: out[b,q,h,p] = sum_k probs[b,q,k,h] * V[b,k,h*P+p]
// Block = (b, 32 queries, up to 8 heads): warp w owns head w and computes its 32 x npiece output
// tile (2 x npiece/8 fragments in registers).  Keys are consumed 16 at a time: the probs slab
// [32 q][16 k][nhead] is regrouped in shared memory as [head][q][k] and the V rows as
// [column][k] (k contiguous for both, row stride 24 floats = conflict-free 64-bit fragment loads);
// the next chunk is fetched into registers while the current one is multiplied.
// ---------------------------------------------------------------------------------------
constexpr int MX_TQ = 32;
constexpr int MX_KC = 16;
constexpr int MX_LD = 24;   // floats per shared-memory row
constexpr int MX_HG = 8;

template <int NT>  // npiece = 8 * NT
__global__ void __launch_bounds__(256, 1)
mix_values_mma_kernel(float* __restrict__ py, const float* __restrict__ pp, const float* __restrict__ pV, int ntimes,
                      int nhead) {
    constexpr int NPIECE = 8 * NT;
    constexpr int COLS = MX_HG * NPIECE;                 // V columns of one head group
    __shared__ __align__(16) float Ps[MX_HG][MX_TQ][MX_LD];
    extern __shared__ __align__(16) float Vt[];          // [COLS][MX_LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z;
    const int q0 = blockIdx.y * MX_TQ;
    const int hg = blockIdx.x * MX_HG;
    const int nh = min(MX_HG, nhead - hg);
    const int nvec = nhead * NPIECE;
    const float* Pb = pp + static_cast<int64_t>(b) * ntimes * ntimes * nhead;
    const float* Vb = pV + static_cast<int64_t>(b) * ntimes * nvec;
    const bool pvec = (nhead % 4 == 0) && ((reinterpret_cast<uintptr_t>(pp) & 15) == 0);

    // Staging registers.  probs: MX_TQ*MX_KC (q,k) pairs x 8 heads = 4096 values, 16 per thread as
    // 2 pairs x 8 heads.  V: MX_KC rows x COLS columns, (COLS/4) 16-byte pieces per row.
    constexpr int V_Q = COLS / 4;                        // pieces per V row
    constexpr int V_PER_THREAD = (MX_KC * V_Q + 255) / 256;
    float pr[2][MX_HG];
    float4 vr[V_PER_THREAD];

    auto fetch = [&](int kc0) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int pair = tid + 256 * i;              // (q, k) pair inside the chunk
            const int qi = pair / MX_KC, kk = pair % MX_KC;
            const int q = q0 + qi, k = kc0 + kk;
            const bool ok = q < ntimes && k < ntimes;
            const float* src = Pb + (static_cast<int64_t>(ok ? q : 0) * ntimes + (ok ? k : 0)) * nhead + hg;
            if (pvec && nh == MX_HG) {   // eight heads = two 16-byte pieces
                const float4 lo4 = ok ? __ldcs(reinterpret_cast<const float4*>(src)) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 hi4 = ok ? __ldcs(reinterpret_cast<const float4*>(src) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                pr[i][0] = lo4.x; pr[i][1] = lo4.y; pr[i][2] = lo4.z; pr[i][3] = lo4.w;
                pr[i][4] = hi4.x; pr[i][5] = hi4.y; pr[i][6] = hi4.z; pr[i][7] = hi4.w;
            } else {
#pragma unroll
                for (int h = 0; h < MX_HG; ++h) pr[i][h] = (ok && h < nh) ? __ldcs(src + h) : 0.0f;
            }
        }
#pragma unroll
        for (int i = 0; i < V_PER_THREAD; ++i) {
            const int e = tid + 256 * i;
            const int kk = e % MX_KC, c4 = (e / MX_KC) << 2;   // lanes run along the keys
            const int k = kc0 + kk;
            const bool ok = e < MX_KC * V_Q && k < ntimes && c4 < nh * NPIECE;
            vr[i] = ok ? __ldg(reinterpret_cast<const float4*>(Vb + static_cast<int64_t>(k) * nvec + hg * NPIECE + c4))
                       : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int pair = tid + 256 * i;
            const int qi = pair / MX_KC, kk = pair % MX_KC;
#pragma unroll
            for (int h = 0; h < MX_HG; ++h) Ps[h][qi][kk] = pr[i][h];
        }
#pragma unroll
        for (int i = 0; i < V_PER_THREAD; ++i) {
            const int e = tid + 256 * i;
            if (e < MX_KC * V_Q) {
                const int kk = e % MX_KC, c4 = (e / MX_KC) << 2;
                Vt[(c4 + 0) * MX_LD + kk] = vr[i].x;
                Vt[(c4 + 1) * MX_LD + kk] = vr[i].y;
                Vt[(c4 + 2) * MX_LD + kk] = vr[i].z;
                Vt[(c4 + 3) * MX_LD + kk] = vr[i].w;
            }
        }
    };

    float acc[2][NT][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.0f;

    fetch(0);
    for (int kc0 = 0; kc0 < ntimes; kc0 += MX_KC) {
        __syncthreads();          // previous chunk fully consumed
        stash();
        __syncthreads();
        if (kc0 + MX_KC < ntimes) fetch(kc0 + MX_KC);
        if (warp < nh) {
            const float* prow = &Ps[warp][g][2 * t];
            const float* vrow = Vt + (warp * NPIECE + g) * MX_LD + 2 * t;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                uint32_t ah[2][4], al[2][4];
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    const float2 v0 = *reinterpret_cast<const float2*>(prow + (mt * 16) * MX_LD + ks * 8);
                    const float2 v1 = *reinterpret_cast<const float2*>(prow + (mt * 16 + 8) * MX_LD + ks * 8);
                    split_frag(v0.x, ah[ks][0], al[ks][0]);
                    split_frag(v1.x, ah[ks][1], al[ks][1]);
                    split_frag(v0.y, ah[ks][2], al[ks][2]);
                    split_frag(v1.y, ah[ks][3], al[ks][3]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        const float2 w = *reinterpret_cast<const float2*>(vrow + nt * 8 * MX_LD + ks * 8);
                        uint32_t bh[2], bl[2];
                        split_frag(w.x, bh[0], bl[0]);
                        split_frag(w.y, bh[1], bl[1]);
                        mma_tf32(c, al[ks], bh);
                        mma_tf32(c, ah[ks], bl);
                        mma_tf32(c, ah[ks], bh);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[mt][nt][i] += c[i];   // round-to-nearest promotion
                }
            }
        }
    }

    if (warp < nh) {
        // out[b,q,h,p]: column index inside a query row = (hg + warp) * NPIECE + p
        float* Ob = py + static_cast<int64_t>(b) * ntimes * nvec + (hg + warp) * NPIECE;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int q = q0 + mt * 16 + g + 8 * half;
                    if (q < ntimes)
                        *reinterpret_cast<float2*>(Ob + static_cast<int64_t>(q) * nvec + nt * 8 + 2 * t) =
                            make_float2(acc[mt][nt][2 * half], acc[mt][nt][2 * half + 1]);
                }
    }
}

template <typename K>
int set_smem(K kernel, size_t bytes, bool* configured) {
    int dev = 0;
    KAI_CUDA(cudaGetDevice(&dev));
    if (dev < kMaxDevices && !configured[dev]) {
        KAI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
        configured[dev] = true;
    }
    return KAI_OK;
}

}  // namespace

int attn_mult_on_heads_mma(float* pp, const float* pK, const float* pQ, int64_t nbat, int64_t ntimes, int64_t nvec,
                           int64_t nhead, int64_t npiece, const float* coef, cudaStream_t s) {
    const bool ok = npiece % 8 == 0 && npiece >= 8 && npiece <= 128 && nvec % 4 == 0 && nbat <= 65535 &&
                    ntimes < (1 << 30) && nhead < (1 << 20) &&
                    ((reinterpret_cast<uintptr_t>(pK) | reinterpret_cast<uintptr_t>(pQ)) & 15) == 0;
    if (!ok) return kNotApplicable;
    const unsigned t = static_cast<unsigned>((ntimes + MM_T - 1) / MM_T);
    if (t > 65535u) return kNotApplicable;
    const size_t smem = 2 * 2 * MM_T * (npiece + 4) * sizeof(float);
    static bool configured[kMaxDevices] = {};
    KAI_TRY(set_smem(mult_on_heads_mma_kernel, 2 * 2 * MM_T * (128 + 4) * sizeof(float), configured));
    dim3 grid(t, t, static_cast<unsigned>(nbat));
    mult_on_heads_mma_kernel<<<grid, 256, smem, s>>>(pp, pK, pQ, static_cast<int>(ntimes), static_cast<int>(nvec),
                                                     static_cast<int>(nhead), static_cast<int>(npiece), coef);
    count_launch();
    return check_launch("mult_on_heads_mma_kernel");
}

template <int NCOL>
static int launch_softmax_warp(float* pp, int64_t nrow, int per_lane, cudaStream_t s) {
    const unsigned blocks = static_cast<unsigned>((nrow * 32 + 255) / 256);
    switch (per_lane) {
        case 1: softmax_axis_warp_kernel<NCOL, 1><<<blocks, 256, 0, s>>>(pp, nrow); break;
        case 2: softmax_axis_warp_kernel<NCOL, 2><<<blocks, 256, 0, s>>>(pp, nrow); break;
        case 4: softmax_axis_warp_kernel<NCOL, 4><<<blocks, 256, 0, s>>>(pp, nrow); break;
        case 8: softmax_axis_warp_kernel<NCOL, 8><<<blocks, 256, 0, s>>>(pp, nrow); break;
        case 16: softmax_axis_warp_kernel<NCOL, 16><<<blocks, 256, 0, s>>>(pp, nrow); break;
        case 32: softmax_axis_warp_kernel<NCOL, 32><<<blocks, 256, 0, s>>>(pp, nrow); break;
        default: return kNotApplicable;
    }
    count_launch();
    return check_launch("softmax_axis_warp_kernel");
}

int attn_softmax_axis_warp(float* pp, int64_t nrow, int64_t nvec, int64_t ncol, cudaStream_t s) {
    const int64_t slab = nvec * ncol;
    if (slab % 128 != 0 || slab > 4096 || (reinterpret_cast<uintptr_t>(pp) & 15) != 0 || nrow > (int64_t(1) << 26))
        return kNotApplicable;
    const int per_lane = static_cast<int>(slab / 128);
    if (per_lane & (per_lane - 1)) return kNotApplicable;
    switch (ncol) {
        case 4: return launch_softmax_warp<4>(pp, nrow, per_lane, s);
        case 8: return launch_softmax_warp<8>(pp, nrow, per_lane, s);
        case 16: return launch_softmax_warp<16>(pp, nrow, per_lane, s);
        case 32: return launch_softmax_warp<32>(pp, nrow, per_lane, s);
        default: return kNotApplicable;
    }
}

template <int NT>
static int launch_mix(float* py, const float* pp, const float* pV, int64_t nbat, int64_t ntimes, int64_t nhead,
                      cudaStream_t s) {
    constexpr size_t smem = static_cast<size_t>(MX_HG) * 8 * NT * MX_LD * sizeof(float);
    static bool configured[kMaxDevices] = {};
    KAI_TRY(set_smem(mix_values_mma_kernel<NT>, smem, configured));
    dim3 grid(static_cast<unsigned>((nhead + MX_HG - 1) / MX_HG), static_cast<unsigned>((ntimes + MX_TQ - 1) / MX_TQ),
              static_cast<unsigned>(nbat));
    mix_values_mma_kernel<NT><<<grid, 256, smem, s>>>(py, pp, pV, static_cast<int>(ntimes), static_cast<int>(nhead));
    count_launch();
    return check_launch("mix_values_mma_kernel");
}

int attn_mix_values_mma(float* py, const float* pp, const float* pV, int64_t nbat, int64_t ntimes, int64_t nvec,
                        int64_t nhead, int64_t npiece, cudaStream_t s) {
    const bool ok = npiece % 8 == 0 && npiece >= 8 && npiece <= 64 && nbat <= 65535 && ntimes < (1 << 30) &&
                    (ntimes + MX_TQ - 1) / MX_TQ <= 65535 && nhead < (1 << 20) && nvec % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pV)) & 15) == 0;
    if (!ok) return kNotApplicable;
    switch (npiece / 8) {
        case 1: return launch_mix<1>(py, pp, pV, nbat, ntimes, nhead, s);
        case 2: return launch_mix<2>(py, pp, pV, nbat, ntimes, nhead, s);
        case 3: return launch_mix<3>(py, pp, pV, nbat, ntimes, nhead, s);
        case 4: return launch_mix<4>(py, pp, pV, nbat, ntimes, nhead, s);
        case 5: return launch_mix<5>(py, pp, pV, nbat, ntimes, nhead, s);
        case 6: return launch_mix<6>(py, pp, pV, nbat, ntimes, nhead, s);
        case 7: return launch_mix<7>(py, pp, pV, nbat, ntimes, nhead, s);
        case 8: return launch_mix<8>(py, pp, pV, nbat, ntimes, nhead, s);
        default: return kNotApplicable;
    }
}

}  // namespace kai
