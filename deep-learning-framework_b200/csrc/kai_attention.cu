// Batched attention contractions of the reference's mh_attention layer, in its own tensor
// layouts (source/engine/support/vmath.cu:6729-7025):
//   Q, K, V  [nbat, ntimes, nvec]             head h owns columns h*npiece .. h*npiece+npiece-1
//   probs    [nbat, ntimes(q), ntimes(k), nhead]   head-minor
//   out      [nbat, ntimes, nhead, npiece]
// The three forward kernels are separate launches because the reference records them as
// separate math calls and keeps `probs` for the backward pass.
#include <float.h>

#include "kai_common.cuh"

namespace kai {
namespace {

// ---------------------------------------------------------------------------------------
// mult_on_heads: probs[b,q,k,h] = coef * sum_p K[b,k,h*P+p] * Q[b,q,h*P+p]
// Block = (b, 64 queries, 64 keys); 16x16 threads, each 4x4 (q,k) pairs for up to 8 heads held
// in registers, so the 8 head values of one (q,k) leave as one contiguous 32-byte run.
// ---------------------------------------------------------------------------------------
constexpr int MH_T = 64;
constexpr int MH_PC = 16;  // reduction chunk
constexpr int MH_HG = 8;   // heads per register group

__global__ void __launch_bounds__(256)
mult_on_heads_kernel(float* __restrict__ pp, const float* __restrict__ pK, const float* __restrict__ pQ,
                     int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece,
                     const float* __restrict__ coef_ptr) {
    __shared__ float Qs[MH_PC][MH_T + 4];
    __shared__ float Ks[MH_PC][MH_T + 4];
    const float coef = (coef_ptr != nullptr) ? __ldg(coef_ptr) : 0.0f;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t b = blockIdx.z;
    const int64_t q0 = static_cast<int64_t>(blockIdx.y) * MH_T;
    const int64_t k0 = static_cast<int64_t>(blockIdx.x) * MH_T;
    const float* Qb = pQ + b * ntimes * nvec;
    const float* Kb = pK + b * ntimes * nvec;
    float* Pb = pp + b * ntimes * ntimes * nhead;
    const bool vec_out = (nhead % 4 == 0) && ((reinterpret_cast<uintptr_t>(pp) & 15) == 0);

    for (int64_t hg = 0; hg < nhead; hg += MH_HG) {
        const int nh = static_cast<int>((nhead - hg < MH_HG) ? (nhead - hg) : MH_HG);
        float acc[MH_HG][4][4];
#pragma unroll
        for (int h = 0; h < MH_HG; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[h][i][j] = 0.0f;

#pragma unroll
        for (int h = 0; h < MH_HG; ++h) {
            if (h < nh) {
                const int64_t col0 = (hg + h) * npiece;
                for (int64_t p0 = 0; p0 < npiece; p0 += MH_PC) {
#pragma unroll
                    for (int e = tid; e < MH_T * MH_PC; e += 256) {
                        const int pc = e & 15, r = e >> 4;
                        const int64_t p = p0 + pc;
                        const int64_t q = q0 + r, k = k0 + r;
                        Qs[pc][r] = (q < ntimes && p < npiece) ? Qb[q * nvec + col0 + p] : 0.0f;
                        Ks[pc][r] = (k < ntimes && p < npiece) ? Kb[k * nvec + col0 + p] : 0.0f;
                    }
                    __syncthreads();
#pragma unroll
                    for (int pc = 0; pc < MH_PC; ++pc) {
                        float qv[4], kv[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) qv[i] = Qs[pc][ty + 16 * i];
#pragma unroll
                        for (int j = 0; j < 4; ++j) kv[j] = Ks[pc][tx + 16 * j];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int j = 0; j < 4; ++j) acc[h][i][j] = fmaf(kv[j], qv[i], acc[h][i][j]);
                    }
                    __syncthreads();
                }
            }
        }

#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t q = q0 + ty + 16 * i;
            if (q >= ntimes) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t k = k0 + tx + 16 * j;
                if (k >= ntimes) continue;
                float* out = Pb + (q * ntimes + k) * nhead + hg;
                if (vec_out && nh == MH_HG) {
                    reinterpret_cast<float4*>(out)[0] = make_float4(acc[0][i][j] * coef, acc[1][i][j] * coef,
                                                                    acc[2][i][j] * coef, acc[3][i][j] * coef);
                    reinterpret_cast<float4*>(out)[1] = make_float4(acc[4][i][j] * coef, acc[5][i][j] * coef,
                                                                    acc[6][i][j] * coef, acc[7][i][j] * coef);
                } else {
#pragma unroll
                    for (int h = 0; h < MH_HG; ++h)
                        if (h < nh) out[h] = acc[h][i][j] * coef;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// set_mh_attention_mask (vmath.cu:6833-6860)
// ---------------------------------------------------------------------------------------
__global__ void attention_mask_kernel(float* __restrict__ pp, int64_t total, int64_t ntimes, int64_t nhead,
                                      int forward) {
    for (int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; n < total;
         n += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t nq = n / (ntimes * nhead) % ntimes;
        const int64_t nk = n / nhead % ntimes;
        if (nq < nk) pp[n] = forward ? -INFINITY : 0.0f;
    }
}

// ---------------------------------------------------------------------------------------
// softmax_direct_on_axis: in-place softmax of pp[nrow, nvec, ncol] over nvec (stride ncol).
// Fast form: one block per row, the nvec x ncol slab staged once in shared memory, so HBM
// sees one read and one write per element.  ncol must be a power of two <= 256.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
softmax_axis_smem_kernel(float* __restrict__ pp, int64_t nvec, int64_t ncol) {
    extern __shared__ float slab[];
    __shared__ float red[256];
    const int tid = threadIdx.x;
    const int64_t n = nvec * ncol;
    float* base = pp + static_cast<int64_t>(blockIdx.x) * n;
    const bool vec = ((n & 3) == 0) && ((reinterpret_cast<uintptr_t>(pp) & 15) == 0);
    if (vec) {
        for (int64_t i = tid; i < (n >> 2); i += 256)
            reinterpret_cast<float4*>(slab)[i] = reinterpret_cast<const float4*>(base)[i];
    } else {
        for (int64_t i = tid; i < n; i += 256) slab[i] = base[i];
    }
    __syncthreads();
    const int c = tid % static_cast<int>(ncol);
    const int g = tid / static_cast<int>(ncol);
    const int groups = 256 / static_cast<int>(ncol);
    // column maxima (seed -FLT_MAX as the reference does)
    float mx = -FLT_MAX;
    for (int64_t v = g; v < nvec; v += groups) mx = fmaxf(mx, slab[v * ncol + c]);
    red[tid] = mx;
    __syncthreads();
    for (int o = 128; o >= ncol; o >>= 1) {
        if (tid < o) red[tid] = fmaxf(red[tid], red[tid + o]);
        __syncthreads();
    }
    mx = red[c];
    __syncthreads();
    // exponentials (kept in the slab) and their column sums
    float sum = 0.f;
    for (int64_t v = g; v < nvec; v += groups) {
        const float e = expf(slab[v * ncol + c] - mx);
        slab[v * ncol + c] = e;
        sum += e;
    }
    red[tid] = sum;
    __syncthreads();
    for (int o = 128; o >= ncol; o >>= 1) {
        if (tid < o) red[tid] += red[tid + o];
        __syncthreads();
    }
    // every thread needs the sums of the columns it writes below
    if (vec) {
        for (int64_t i = tid; i < (n >> 2); i += 256) {
            float4 e = reinterpret_cast<const float4*>(slab)[i];
            const int c0 = static_cast<int>((i << 2) % ncol);
            if (ncol >= 4) {
                e.x /= red[c0]; e.y /= red[c0 + 1]; e.z /= red[c0 + 2]; e.w /= red[c0 + 3];
            } else {
                e.x /= red[c0 % ncol]; e.y /= red[(c0 + 1) % ncol];
                e.z /= red[(c0 + 2) % ncol]; e.w /= red[(c0 + 3) % ncol];
            }
            reinterpret_cast<float4*>(base)[i] = e;
        }
    } else {
        for (int64_t i = tid; i < n; i += 256) base[i] = slab[i] / red[i % ncol];
    }
}

// General form: one thread per (row, column), three strided passes, as the reference does.
__global__ void softmax_axis_generic_kernel(float* __restrict__ pp, int64_t nrow, int64_t nvec, int64_t ncol) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= nrow * ncol) return;
    const int64_t nr = n / ncol, nc = n % ncol;
    float* p = pp + nr * nvec * ncol + nc;
    float mx = -FLT_MAX;
    for (int64_t v = 0; v < nvec; ++v) mx = fmaxf(mx, p[v * ncol]);
    float sum = 0.f;
    for (int64_t v = 0; v < nvec; ++v) sum += expf(p[v * ncol] - mx);
    for (int64_t v = 0; v < nvec; ++v) p[v * ncol] = expf(p[v * ncol] - mx) / sum;
}

// ---------------------------------------------------------------------------------------
// mix_values: out[b,q,h,p] = sum_k probs[b,q,k,h] * V[b,k,h*P+p]
// Block = (b, 16 queries, up to 512 output columns).  Thread = 4 consecutive columns (one head,
// npiece % 4 == 0) x 8 queries.  Per 16-key chunk the probs slab [16 q][16 k][H] and the V rows
// are staged in shared memory with contiguous copies.
// ---------------------------------------------------------------------------------------
constexpr int MV_TQ = 16;
constexpr int MV_KC = 16;
constexpr int MV_COLS = 512;

// TRANSPOSED = true computes the value gradient instead (vmath.cu:7081-7104):
//   out[b,k,h,p] = sum_q probs[b,q,k,h] * gy[b,q,h*P+p]
// i.e. the same contraction with the two time indices of probs exchanged; the names below follow
// the forward case (the "query" tile is the tile of output rows, "keys" are the reduction index).
template <bool TRANSPOSED>
__global__ void __launch_bounds__(256)
mix_values_kernel(float* __restrict__ py, const float* __restrict__ pp, const float* __restrict__ pV,
                  int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece) {
    extern __shared__ float sm[];
    float* Vs = sm;                                  // [MV_KC][MV_COLS]
    float* Ps = sm + MV_KC * MV_COLS;                // [MV_TQ][MV_KC][nhead]
    const int tid = threadIdx.x;
    const int64_t b = blockIdx.z;
    const int64_t q0 = static_cast<int64_t>(blockIdx.y) * MV_TQ;
    const int64_t col0 = static_cast<int64_t>(blockIdx.x) * MV_COLS;
    const int cg = tid & 127;        // column group inside the block
    const int qh = tid >> 7;         // which 8 queries
    const int64_t col = col0 + 4 * cg;
    const bool active = col < nvec;
    const int64_t h = active ? col / npiece : 0;
    const float* Vb = pV + b * ntimes * nvec;
    const float* Pb = pp + b * ntimes * ntimes * nhead;
    const int ncols_blk = static_cast<int>((nvec - col0 < MV_COLS) ? (nvec - col0) : MV_COLS);

    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int64_t k0 = 0; k0 < ntimes; k0 += MV_KC) {
        const int kc = static_cast<int>((ntimes - k0 < MV_KC) ? (ntimes - k0) : MV_KC);
        // V rows k0..k0+kc-1, columns col0..col0+ncols_blk-1 (nvec % 4 == 0 guaranteed by the launcher)
        for (int e = tid; e < MV_KC * (MV_COLS / 4); e += 256) {
            const int kk = e / (MV_COLS / 4), c4 = e % (MV_COLS / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kk < kc && 4 * c4 < ncols_blk)
                v = *reinterpret_cast<const float4*>(Vb + (k0 + kk) * nvec + col0 + 4 * c4);
            reinterpret_cast<float4*>(Vs)[e] = v;
        }
        // forward: probs[q0+qi][k0..k0+kc-1][0..H-1] = kc*H contiguous floats per output row;
        // transposed: probs[k0+kk][q0..q0+15][0..H-1] = 16*H contiguous floats per reduction index.
        // Either way Ps is indexed [output row][reduction index][head].
        const int run = MV_KC * static_cast<int>(nhead);
        for (int e = tid; e < MV_TQ * run; e += 256) {
            float v = 0.f;
            if (!TRANSPOSED) {
                const int qi = e / run, r = e % run;
                const int64_t q = q0 + qi;
                if (q < ntimes && r < kc * nhead) v = Pb[(q * ntimes + k0) * nhead + r];
                Ps[e] = v;
            } else {
                const int run_t = MV_TQ * static_cast<int>(nhead);
                const int kk = e / run_t, r = e % run_t;          // r = qi * H + h
                const int qi = r / static_cast<int>(nhead), hh = r % static_cast<int>(nhead);
                if (kk < kc && q0 + qi < ntimes) v = Pb[((k0 + kk) * ntimes + q0) * nhead + r];
                Ps[(qi * MV_KC + kk) * nhead + hh] = v;
            }
        }
        __syncthreads();
        if (active) {
#pragma unroll 4
            for (int kk = 0; kk < MV_KC; ++kk) {
                const float4 v = reinterpret_cast<const float4*>(Vs)[kk * (MV_COLS / 4) + cg];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float pr = Ps[((qh * 8 + i) * MV_KC + kk) * nhead + h];
                    acc[i][0] = fmaf(pr, v.x, acc[i][0]);
                    acc[i][1] = fmaf(pr, v.y, acc[i][1]);
                    acc[i][2] = fmaf(pr, v.z, acc[i][2]);
                    acc[i][3] = fmaf(pr, v.w, acc[i][3]);
                }
            }
        }
        __syncthreads();
    }
    if (!active) return;
    // out[b,q,h,p] with (h,p) flattened = the same column index as V.
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t q = q0 + qh * 8 + i;
        if (q < ntimes)
            *reinterpret_cast<float4*>(py + (b * ntimes + q) * nvec + col) =
                make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
}

// Fallbacks for shapes the tiled kernels do not cover (npiece % 4 != 0, unaligned bases):
// one thread per output, the reference's own decomposition.
__global__ void mix_values_generic_kernel(float* __restrict__ py, const float* __restrict__ pp,
                                          const float* __restrict__ pV, int64_t total, int64_t ntimes,
                                          int64_t nvec, int64_t nhead, int64_t npiece, int transposed) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= total) return;
    const int64_t np = n % npiece, nh = n / npiece % nhead, nq = n / (npiece * nhead) % ntimes,
                  nb = n / (npiece * nhead * ntimes);
    float sum = 0.f;
    for (int64_t nk = 0; nk < ntimes; ++nk) {
        const int64_t ppos = transposed ? ((nb * ntimes + nk) * ntimes + nq) * nhead + nh
                                        : ((nb * ntimes + nq) * ntimes + nk) * nhead + nh;
        sum = fmaf(pp[ppos], pV[(nb * ntimes + nk) * nvec + nh * npiece + np], sum);
    }
    py[n] = sum;
}

// ---------------------------------------------------------------------------------------
// softmax_direct_on_axis for slabs of EPT x 1024 values with ncol in {4, 8, ..., 128}: one block per
// slab, every thread keeps EPT float4 of it in registers (its four columns are the same in each of
// them because ncol divides 1024), so the slab is read once and written once.  Column maxima and
// sums: xor-shuffles between the lanes that share columns, then across the 8 warps through shared
// memory.  Low register count, full occupancy: the kernel runs at memory speed.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float4 f4_max(float4 a, float4 b) {
    return make_float4(fmaxf(a.x, b.x), fmaxf(a.y, b.y), fmaxf(a.z, b.z), fmaxf(a.w, b.w));
}
__device__ __forceinline__ float4 f4_add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 f4_shfl_xor(float4 a, int o) {
    return make_float4(__shfl_xor_sync(0xffffffffu, a.x, o), __shfl_xor_sync(0xffffffffu, a.y, o),
                       __shfl_xor_sync(0xffffffffu, a.z, o), __shfl_xor_sync(0xffffffffu, a.w, o));
}

template <int EPT>
__global__ void __launch_bounds__(256)
softmax_axis_block_kernel(float* __restrict__ pp, int groups /* ncol / 4: threads tid % groups share columns */) {
    __shared__ float4 red[2][8][32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float4* slab = reinterpret_cast<float4*>(pp) + static_cast<int64_t>(blockIdx.x) * (EPT * 256);
    float4 v[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) v[i] = slab[i * 256 + tid];
    float4 m = v[0];
#pragma unroll
    for (int i = 1; i < EPT; ++i) m = f4_max(m, v[i]);
    for (int o = 16; o >= groups; o >>= 1) m = f4_max(m, f4_shfl_xor(m, o));
    if (lane < groups) red[0][warp][lane] = m;
    __syncthreads();
    const int grp = lane & (groups - 1);
    m = red[0][0][grp];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = f4_max(m, red[0][w][grp]);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        v[i] = make_float4(expf(v[i].x - m.x), expf(v[i].y - m.y), expf(v[i].z - m.z), expf(v[i].w - m.w));
        sum = f4_add(sum, v[i]);
    }
    for (int o = 16; o >= groups; o >>= 1) sum = f4_add(sum, f4_shfl_xor(sum, o));
    if (lane < groups) red[1][warp][lane] = sum;
    __syncthreads();
    sum = red[1][0][grp];
#pragma unroll
    for (int w = 1; w < 8; ++w) sum = f4_add(sum, red[1][w][grp]);
#pragma unroll
    for (int i = 0; i < EPT; ++i)
        slab[i * 256 + tid] = make_float4(v[i].x / sum.x, v[i].y / sum.y, v[i].z / sum.z, v[i].w / sum.w);
}

// Returns 1 when the shape is outside this kernel.
int attn_softmax_axis_block(float* pp, int64_t nrow, int64_t nvec, int64_t ncol, cudaStream_t s) {
    const int64_t slab = nvec * ncol;
    const bool ok = ncol >= 4 && ncol <= 128 && (ncol & (ncol - 1)) == 0 && (slab % 1024) == 0 &&
                    nrow <= 0x7fffffffLL && (reinterpret_cast<uintptr_t>(pp) & 15) == 0;
    if (!ok) return 1;
    const unsigned grid = static_cast<unsigned>(nrow);
    const int groups = static_cast<int>(ncol / 4);
    switch (slab / 1024) {
        case 1: softmax_axis_block_kernel<1><<<grid, 256, 0, s>>>(pp, groups); break;
        case 2: softmax_axis_block_kernel<2><<<grid, 256, 0, s>>>(pp, groups); break;
        case 4: softmax_axis_block_kernel<4><<<grid, 256, 0, s>>>(pp, groups); break;
        case 8: softmax_axis_block_kernel<8><<<grid, 256, 0, s>>>(pp, groups); break;
        case 16: softmax_axis_block_kernel<16><<<grid, 256, 0, s>>>(pp, groups); break;
        default: return 1;
    }
    count_launch();
    return check_launch("softmax_axis_block_kernel");
}

// ---------------------------------------------------------------------------------------
// softmax_direct_on_axis_backward (vmath.cu:6920-6945), in place on gp:
//   gp[b,q,k,h] = coef * pp[b,q,k,h] * (gp[b,q,k,h] - sum_k' pp[b,q,k',h] * gp[b,q,k',h])
// One block per (b,q) slab of ntimes x nhead values; nhead a power of two <= 256.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
softmax_axis_backward_kernel(float* __restrict__ gp, const float* __restrict__ pp, int64_t nvec, int64_t ncol,
                             const float* __restrict__ coef_ptr) {
    __shared__ float red[256];
    const float coef = (coef_ptr != nullptr) ? __ldg(coef_ptr) : 0.0f;
    const int tid = threadIdx.x;
    const int64_t n = nvec * ncol;
    float* g = gp + static_cast<int64_t>(blockIdx.x) * n;
    const float* p = pp + static_cast<int64_t>(blockIdx.x) * n;
    // thread tid always meets column tid % ncol (256 % ncol == 0)
    float sum = 0.f;
    for (int64_t i = tid; i < n; i += 256) sum += p[i] * g[i];
    red[tid] = sum;
    __syncthreads();
    for (int o = 128; o >= ncol; o >>= 1) {
        if (tid < o) red[tid] += red[tid + o];
        __syncthreads();
    }
    const float colsum = red[tid % static_cast<int>(ncol)];
    for (int64_t i = tid; i < n; i += 256) g[i] = coef * p[i] * (g[i] - colsum);
}

__global__ void softmax_axis_backward_generic_kernel(float* __restrict__ gp, const float* __restrict__ pp,
                                                     int64_t nrow, int64_t nvec, int64_t ncol,
                                                     const float* __restrict__ coef_ptr) {
    const float coef = (coef_ptr != nullptr) ? __ldg(coef_ptr) : 0.0f;
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= nrow * ncol) return;
    const int64_t base = (n / ncol) * nvec * ncol + n % ncol;
    float sum = 0.f;
    for (int64_t v = 0; v < nvec; ++v) sum += pp[base + v * ncol] * gp[base + v * ncol];
    for (int64_t v = 0; v < nvec; ++v) gp[base + v * ncol] = coef * pp[base + v * ncol] * (gp[base + v * ncol] - sum);
}

}  // namespace

int attn_softmax_axis_backward(float* gp, const float* pp, int64_t nrow, int64_t nvec, int64_t ncol,
                               const float* coef, cudaStream_t s) {
    const bool pow2 = ncol > 0 && (ncol & (ncol - 1)) == 0 && ncol <= 256;
    if (pow2 && nrow <= 0x7fffffffLL) {
        softmax_axis_backward_kernel<<<static_cast<unsigned>(nrow), 256, 0, s>>>(gp, pp, nvec, ncol, coef);
        count_launch();
        return check_launch("softmax_axis_backward_kernel");
    }
    const int64_t total = nrow * ncol;
    softmax_axis_backward_generic_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(gp, pp, nrow, nvec,
                                                                                                  ncol, coef);
    count_launch();
    return check_launch("softmax_axis_backward_generic_kernel");
}

// tensor-core forms (kai_attention_mma.cu); they return 1 when a shape is outside their fast path
int attn_mult_on_heads_mma(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                           const float*, cudaStream_t);
int attn_softmax_axis_warp(float*, int64_t, int64_t, int64_t, cudaStream_t);
int attn_mix_values_mma(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                        cudaStream_t);

int attn_mult_on_heads(float* pp, const float* pK, const float* pQ, int64_t nbat, int64_t ntimes, int64_t nvec,
                       int64_t nhead, int64_t npiece, const float* coef, cudaStream_t s) {
    if (options().attn_path.load() != 1) {
        const int rc = attn_mult_on_heads_mma(pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, coef, s);
        if (rc != 1) return rc;
    }
    if (nbat > 65535) return fail(KAI_E_TOO_LARGE, "mult_on_heads: nbat > 65535");
    const unsigned t = static_cast<unsigned>((ntimes + MH_T - 1) / MH_T);
    dim3 grid(t, t, static_cast<unsigned>(nbat));
    mult_on_heads_kernel<<<grid, 256, 0, s>>>(pp, pK, pQ, ntimes, nvec, nhead, npiece, coef);
    count_launch();
    return check_launch("mult_on_heads_kernel");
}

int attn_mask(DeviceState* st, float* pp, int64_t ndat, int64_t ntimes, int64_t nhead, int forward,
              cudaStream_t s) {
    const int64_t total = ndat * ntimes * ntimes * nhead;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = static_cast<int64_t>(st->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    attention_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(pp, total, ntimes, nhead, forward);
    count_launch();
    return check_launch("attention_mask_kernel");
}

int attn_softmax_axis(float* pp, int64_t nrow, int64_t nvec, int64_t ncol, cudaStream_t s) {
    if (options().attn_path.load() != 1) {
        const int rcb = attn_softmax_axis_block(pp, nrow, nvec, ncol, s);
        if (rcb != 1) return rcb;
        const int rc = attn_softmax_axis_warp(pp, nrow, nvec, ncol, s);
        if (rc != 1) return rc;
    }
    const bool pow2 = ncol > 0 && (ncol & (ncol - 1)) == 0 && ncol <= 256;
    const int64_t slab_bytes = nvec * ncol * 4;
    if (pow2 && slab_bytes <= 160 * 1024 && nrow <= 0x7fffffffLL) {
        static bool configured[kMaxDevices] = {};
        int dev = 0;
        KAI_CUDA(cudaGetDevice(&dev));
        if (dev < kMaxDevices && !configured[dev]) {
            KAI_CUDA(cudaFuncSetAttribute(softmax_axis_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          160 * 1024));
            configured[dev] = true;
        }
        softmax_axis_smem_kernel<<<static_cast<unsigned>(nrow), 256, static_cast<size_t>(slab_bytes), s>>>(pp, nvec,
                                                                                                            ncol);
        count_launch();
        return check_launch("softmax_axis_smem_kernel");
    }
    const int64_t total = nrow * ncol;
    softmax_axis_generic_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(pp, nrow, nvec, ncol);
    count_launch();
    return check_launch("softmax_axis_generic_kernel");
}

int attn_mix_values(float* py, const float* pp, const float* pV, int64_t nbat, int64_t ntimes, int64_t nvec,
                    int64_t nhead, int64_t npiece, cudaStream_t s, bool transposed) {
    if (!transposed && options().attn_path.load() != 1) {
        const int rc = attn_mix_values_mma(py, pp, pV, nbat, ntimes, nvec, nhead, npiece, s);
        if (rc != 1) return rc;
    }
    const bool tiled = (npiece % 4 == 0) && (nvec % 4 == 0) && nbat <= 65535 &&
                       ((reinterpret_cast<uintptr_t>(py) | reinterpret_cast<uintptr_t>(pV)) & 15) == 0 &&
                       nhead <= 64;
    if (tiled) {
        const size_t smem = (MV_KC * MV_COLS + MV_TQ * MV_KC * static_cast<size_t>(nhead)) * sizeof(float);
        static bool configured[kMaxDevices] = {};
        int dev = 0;
        KAI_CUDA(cudaGetDevice(&dev));
        if (dev < kMaxDevices && !configured[dev]) {
            KAI_CUDA(cudaFuncSetAttribute(mix_values_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (MV_KC * MV_COLS + MV_TQ * MV_KC * 64) * 4));
            KAI_CUDA(cudaFuncSetAttribute(mix_values_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (MV_KC * MV_COLS + MV_TQ * MV_KC * 64) * 4));
            configured[dev] = true;
        }
        dim3 grid(static_cast<unsigned>((nvec + MV_COLS - 1) / MV_COLS),
                  static_cast<unsigned>((ntimes + MV_TQ - 1) / MV_TQ), static_cast<unsigned>(nbat));
        if (transposed) mix_values_kernel<true><<<grid, 256, smem, s>>>(py, pp, pV, ntimes, nvec, nhead, npiece);
        else mix_values_kernel<false><<<grid, 256, smem, s>>>(py, pp, pV, ntimes, nvec, nhead, npiece);
        count_launch();
        return check_launch("mix_values_kernel");
    }
    const int64_t total = nbat * ntimes * nvec;
    mix_values_generic_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
        py, pp, pV, total, ntimes, nvec, nhead, npiece, transposed ? 1 : 0);
    count_launch();
    return check_launch("mix_values_generic_kernel");
}

}  // namespace kai
