// Bias, activation and loss kernels of the matmul / Linear path (HBM-bound passes).
// When a caller can use kai_linear_forward these are fused into the GEMM epilogue; the
// standalone forms exist because the reference engine records them as separate math calls
// (add_bias, activate, ... in source/engine/support/vmath.cu) and replays them one by one.
#include <float.h>

#include "kai_act.cuh"
#include "kai_common.cuh"

namespace kai {
namespace {

inline unsigned grid_for(int64_t items, int per_block, int sm_count, int waves = 8) {
    int64_t blocks = (items + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(sm_count > 0 ? sm_count : 148) * waves;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

// ---- add_bias (vmath.cu:875-897) --------------------------------------------------------
__global__ void add_bias_kernel(float* y, const float* a,  // y may alias a
                                const float* __restrict__ b, int64_t nrow, int64_t ncol, int vec) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (vec) {
        const int64_t qcol = ncol >> 2, total = nrow * qcol;
        for (int64_t i = tid; i < total; i += stride) {
            const int64_t c = (i % qcol) << 2;
            const float4 av = reinterpret_cast<const float4*>(a)[i];
            const float4 bv = *reinterpret_cast<const float4*>(b + c);
            reinterpret_cast<float4*>(y)[i] = make_float4(av.x + bv.x, av.y + bv.y, av.z + bv.z, av.w + bv.w);
        }
    } else {
        const int64_t total = nrow * ncol;
        for (int64_t i = tid; i < total; i += stride) y[i] = a[i] + b[i % ncol];
    }
}

// ---- add_bias_backward_b (vmath.cu:901-932): column sums --------------------------------
// Block = 32 x 8 threads; x covers 32 columns, y covers row lanes.  Row slabs (gridDim.y) write
// partial sums that a second pass adds in slab order, so the result does not depend on
// scheduling.
__global__ void colsum_partial_kernel(const float* __restrict__ gy, int64_t nrow, int64_t ncol,
                                      int64_t rows_per_slab, float* __restrict__ out /*[slabs][ncol]*/) {
    __shared__ float red[8][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + tx;
    const int64_t r_begin = static_cast<int64_t>(blockIdx.y) * rows_per_slab;
    const int64_t r_end = min(nrow, r_begin + rows_per_slab);
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (c < ncol) {
        int64_t r = r_begin + ty;
        for (; r + 24 < r_end; r += 32) {
            s0 += gy[r * ncol + c];
            s1 += gy[(r + 8) * ncol + c];
            s2 += gy[(r + 16) * ncol + c];
            s3 += gy[(r + 24) * ncol + c];
        }
        for (; r < r_end; r += 8) s0 += gy[r * ncol + c];
    }
    red[ty][tx] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (ty == 0 && c < ncol) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][tx];
        out[static_cast<int64_t>(blockIdx.y) * ncol + c] = t;
    }
}

// 16-byte form: a thread owns four adjacent columns, a block 128 columns x 8 row lanes.
__global__ void colsum_partial4_kernel(const float* __restrict__ gy, int64_t nrow, int64_t ncol,
                                       int64_t rows_per_slab, float* __restrict__ out /*[slabs][ncol]*/) {
    __shared__ float4 red[8][32];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t c = (static_cast<int64_t>(blockIdx.x) * 32 + tx) * 4;
    const int64_t r_begin = static_cast<int64_t>(blockIdx.y) * rows_per_slab;
    const int64_t r_end = min(nrow, r_begin + rows_per_slab);
    float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;
    if (c < ncol) {
        int64_t r = r_begin + ty;
        for (; r + 24 < r_end; r += 32) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(gy + r * ncol + c));
            const float4 b = __ldcs(reinterpret_cast<const float4*>(gy + (r + 8) * ncol + c));
            const float4 d = __ldcs(reinterpret_cast<const float4*>(gy + (r + 16) * ncol + c));
            const float4 e = __ldcs(reinterpret_cast<const float4*>(gy + (r + 24) * ncol + c));
            s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
            s1.x += b.x; s1.y += b.y; s1.z += b.z; s1.w += b.w;
            s2.x += d.x; s2.y += d.y; s2.z += d.z; s2.w += d.w;
            s3.x += e.x; s3.y += e.y; s3.z += e.z; s3.w += e.w;
        }
        for (; r < r_end; r += 8) {
            const float4 a = __ldcs(reinterpret_cast<const float4*>(gy + r * ncol + c));
            s0.x += a.x; s0.y += a.y; s0.z += a.z; s0.w += a.w;
        }
    }
    red[ty][tx] = make_float4((s0.x + s1.x) + (s2.x + s3.x), (s0.y + s1.y) + (s2.y + s3.y),
                              (s0.z + s1.z) + (s2.z + s3.z), (s0.w + s1.w) + (s2.w + s3.w));
    __syncthreads();
    if (ty == 0 && c < ncol) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { t.x += red[i][tx].x; t.y += red[i][tx].y; t.z += red[i][tx].z; t.w += red[i][tx].w; }
        *reinterpret_cast<float4*>(out + static_cast<int64_t>(blockIdx.y) * ncol + c) = t;
    }
}

__global__ void colsum_final_kernel(const float* __restrict__ partial, int slabs, int64_t ncol,
                                    float* __restrict__ gb, int acc) {
    const int64_t c = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (c >= ncol) return;
    float t = 0.f;
    for (int s = 0; s < slabs; ++s) t += partial[static_cast<int64_t>(s) * ncol + c];
    gb[c] = acc ? gb[c] + t : t;
}

// ---- activate (vmath.cu:3097-3243) -------------------------------------------------------
__global__ void activate_kernel(float* y, const float* x, int64_t total,  // y may alias x
                                int act, const float* __restrict__ leaky_alpha, int vec) {
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (vec) {  // 16-byte aligned: four elements per thread per step
        const int64_t quads = total >> 2;
        int64_t i = tid;
        for (; i + 3 * stride < quads; i += 4 * stride) {   // four independent 16-byte loads in flight
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = reinterpret_cast<const float4*>(x)[i + u * stride];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                v[u].x = act_forward(act, v[u].x, alpha); v[u].y = act_forward(act, v[u].y, alpha);
                v[u].z = act_forward(act, v[u].z, alpha); v[u].w = act_forward(act, v[u].w, alpha);
                reinterpret_cast<float4*>(y)[i + u * stride] = v[u];
            }
        }
        for (; i < quads; i += stride) {
            float4 v = reinterpret_cast<const float4*>(x)[i];
            v.x = act_forward(act, v.x, alpha); v.y = act_forward(act, v.y, alpha);
            v.z = act_forward(act, v.z, alpha); v.w = act_forward(act, v.w, alpha);
            reinterpret_cast<float4*>(y)[i] = v;
        }
        for (int64_t i = (quads << 2) + tid; i < total; i += stride) y[i] = act_forward(act, x[i], alpha);
    } else {
        for (int64_t i = tid; i < total; i += stride) y[i] = act_forward(act, x[i], alpha);
    }
}

// Row softmax (ActFunc::softmax, vmath.cu:3141-3157): one warp per row, max seeded with -FLT_MAX.
// The row is read completely before anything is written, so y may alias x.
__global__ void softmax_rows_kernel(float* y, const float* x, int64_t nrow,
                                    int64_t ncol) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (row >= nrow) return;
    const float* px = x + row * ncol;
    float mx = -FLT_MAX;
    for (int64_t c = lane; c < ncol; c += 32) mx = fmaxf(mx, px[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int64_t c = lane; c < ncol; c += 32) sum += expf(px[c] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    float* py = y + row * ncol;
    // In-place safe: each lane rewrites only the elements it alone reads below.
    for (int64_t c = lane; c < ncol; c += 32) py[c] = expf(px[c] - mx) / sum;
}

__device__ __forceinline__ float act_grad(int act, float r, float alpha, int from_y) {
    return from_y ? act_grad_from_y(act, r, alpha) : act_grad_from_x(act, r, alpha);
}

__global__ void activate_backward_kernel(float* gx, const float* gy, const float* ref, int64_t total, int act,
                                         const float* __restrict__ leaky_alpha, int from_y, int vec) {
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    if (vec) {
        const int64_t quads = total >> 2;
        for (int64_t i = tid; i < quads; i += stride) {
            const float4 r = reinterpret_cast<const float4*>(ref)[i];
            const float4 g = reinterpret_cast<const float4*>(gy)[i];
            reinterpret_cast<float4*>(gx)[i] =
                make_float4(act_grad(act, r.x, alpha, from_y) * g.x, act_grad(act, r.y, alpha, from_y) * g.y,
                            act_grad(act, r.z, alpha, from_y) * g.z, act_grad(act, r.w, alpha, from_y) * g.w);
        }
        for (int64_t i = (quads << 2) + tid; i < total; i += stride)
            gx[i] = act_grad(act, ref[i], alpha, from_y) * gy[i];
    } else {
        for (int64_t i = tid; i < total; i += stride) gx[i] = act_grad(act, ref[i], alpha, from_y) * gy[i];
    }
}

// ---- softmax_idx_crossentropy (vmath.cu:8916-8965, 9022-9077): one warp per row ----------
__global__ void ce_forward_kernel(float* __restrict__ y, const float* __restrict__ x,
                                  const int* __restrict__ label, int64_t nrow, int64_t ncol,
                                  int* __restrict__ bad_flag) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (row >= nrow) return;
    const float* px = x + row * ncol;
    const int lab = label[row];
    if (lab < 0 || lab >= ncol) {  // the reference throws VERR_OUT_OF_RANGE here (vmath.cu:8918)
        if (lane == 0) { y[row] = nanf(""); atomicExch(bad_flag, 1); }
        return;
    }
    float mx = px[0];
    for (int64_t c = lane; c < ncol; c += 32) mx = fmaxf(mx, px[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int64_t c = lane; c < ncol; c += 32) sum += expf(px[c] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        const float prob = expf(px[lab] - mx) / sum;
        y[row] = -logf(prob + 1.0e-10f);
    }
}

__global__ void ce_backward_kernel(float* __restrict__ gx, const float* __restrict__ gy,
                                   const float* __restrict__ x, const int* __restrict__ label,
                                   int64_t nrow, int64_t ncol) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
    if (row >= nrow) return;
    const float* px = x + row * ncol;
    float mx = px[0];
    for (int64_t c = lane; c < ncol; c += 32) mx = fmaxf(mx, px[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int64_t c = lane; c < ncol; c += 32) sum += expf(px[c] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const int lab = label[row];
    const float g = gy[row];
    for (int64_t c = lane; c < ncol; c += 32) {
        float t = expf(px[c] - mx) / sum;
        if (c == lab) t -= 1.0f;
        gx[row * ncol + c] = t * g;
    }
}

// ---- sum / sum_backward (vmath.cu:9739-9779) ---------------------------------------------
// One block; each thread sums a strided subset, then a fixed shared-memory tree.
__global__ void sum_kernel(float* __restrict__ y, const float* __restrict__ x, int64_t n) {
    __shared__ float red[1024];
    float t = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) t += x[i];
    red[threadIdx.x] = t;
    __syncthreads();
    for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) y[0] = red[0];
}

__global__ void sum_backward_kernel(float* __restrict__ gx, const float* __restrict__ gy, int64_t n) {
    const float v = (gy != nullptr) ? gy[0] : 1.0f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        gx[i] = v;
}

// ---- layernorm (vmath.cu:5977-6085) -------------------------------------------------------
// One warp per row, the row held in registers (Q 16-byte pieces per lane, ncol <= 128 Q): one read and
// one write of the tensor.  avg = sum / ncol; std = sqrtf(mean((x - avg)^2) + 1e-10f);
// y = scale * ((x - avg) / std); ps[row] = (avg, std).  The sums run lane-wise and then over the
// warp, i.e. in another order than the reference's serial loop.
template <int Q>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(float* __restrict__ y, const float* __restrict__ x, float* __restrict__ ps, int64_t nrow,
                      int64_t ncol, const float* __restrict__ scale_ptr) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= nrow) return;
    const float scale = (scale_ptr != nullptr) ? __ldg(scale_ptr) : 0.0f;
    const int64_t quads = ncol >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + row * ncol);
    float4 v[Q];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        const int64_t q = lane + 32 * i;
        v[i] = (q < quads) ? __ldcs(xr + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float avg = sum / static_cast<float>(ncol);
    float dsq = 0.0f;
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        if (lane + 32 * i < quads) {
            const float a = v[i].x - avg, b = v[i].y - avg, c = v[i].z - avg, d = v[i].w - avg;
            dsq += (a * a + b * b) + (c * c + d * d);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dsq += __shfl_xor_sync(0xffffffffu, dsq, o);
    const float sd = sqrtf(dsq / static_cast<float>(ncol) + 1e-10f);
    float4* yr = reinterpret_cast<float4*>(y + row * ncol);
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        const int64_t q = lane + 32 * i;
        if (q < quads)
            __stcs(yr + q, make_float4(scale * ((v[i].x - avg) / sd), scale * ((v[i].y - avg) / sd),
                                       scale * ((v[i].z - avg) / sd), scale * ((v[i].w - avg) / sd)));
    }
    if (lane == 0) {
        ps[2 * row + 0] = avg;
        ps[2 * row + 1] = sd;
    }
}

// Any row length and alignment: one block per row, three passes over the row (the second and third
// hit L1 / L2), block-wide sums through shared memory.
__global__ void __launch_bounds__(256)
layernorm_block_kernel(float* y, const float* x, float* __restrict__ ps, int64_t nrow, int64_t ncol,
                       const float* __restrict__ scale_ptr) {
    __shared__ float red[8];
    __shared__ float bcast;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float scale = (scale_ptr != nullptr) ? __ldg(scale_ptr) : 0.0f;
    for (int64_t row = blockIdx.x; row < nrow; row += gridDim.x) {
        const float* xr = x + row * ncol;
        float part = 0.0f;
        for (int64_t c = threadIdx.x; c < ncol; c += 256) part += xr[c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < 8; ++w) t += red[w];
            bcast = t / static_cast<float>(ncol);
        }
        __syncthreads();
        const float avg = bcast;
        part = 0.0f;
        for (int64_t c = threadIdx.x; c < ncol; c += 256) {
            const float d = xr[c] - avg;
            part += d * d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        __syncthreads();
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (int w = 0; w < 8; ++w) t += red[w];
            bcast = sqrtf(t / static_cast<float>(ncol) + 1e-10f);
        }
        __syncthreads();
        const float sd = bcast;
        for (int64_t c = threadIdx.x; c < ncol; c += 256) y[row * ncol + c] = scale * ((xr[c] - avg) / sd);
        if (threadIdx.x == 0) {
            ps[2 * row + 0] = avg;
            ps[2 * row + 1] = sd;
        }
        __syncthreads();
    }
}

// layernorm_backward (vmath.cu:6056-6085): gx = scale * ((gy - avg) / std) with the saved row statistics.
__global__ void layernorm_backward_kernel(float* gx, const float* gy, const float* __restrict__ ps, int64_t nrow,
                                          int64_t ncol, const float* __restrict__ scale_ptr, int vec) {
    const float scale = (scale_ptr != nullptr) ? __ldg(scale_ptr) : 0.0f;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (vec) {
        const int64_t qcol = ncol >> 2, total = nrow * qcol;
        for (int64_t i = tid; i < total; i += stride) {
            const int64_t r = i / qcol;
            const float avg = __ldg(ps + 2 * r), sd = __ldg(ps + 2 * r + 1);
            const float4 g = reinterpret_cast<const float4*>(gy)[i];
            reinterpret_cast<float4*>(gx)[i] = make_float4(scale * ((g.x - avg) / sd), scale * ((g.y - avg) / sd),
                                                           scale * ((g.z - avg) / sd), scale * ((g.w - avg) / sd));
        }
    } else {
        const int64_t total = nrow * ncol;
        for (int64_t i = tid; i < total; i += stride) {
            const int64_t r = i / ncol;
            gx[i] = scale * ((gy[i] - __ldg(ps + 2 * r)) / __ldg(ps + 2 * r + 1));
        }
    }
}

}  // namespace

// ---- host launchers (called from the C ABI) ------------------------------------------------
int ew_add_bias(DeviceState* st, float* y, const float* a, const float* b, int64_t nrow, int64_t ncol,
                cudaStream_t s) {
    const int vec = ((ncol & 3) == 0 && ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(a) |
                                         reinterpret_cast<uintptr_t>(b)) & 15) == 0) ? 1 : 0;
    const int64_t items = vec ? nrow * (ncol >> 2) : nrow * ncol;
    add_bias_kernel<<<grid_for(items, 256, st->sm_count), 256, 0, s>>>(y, a, b, nrow, ncol, vec);
    count_launch();
    return check_launch("add_bias_kernel");
}

int ew_colsum(DeviceState* st, int device, float* gb, const float* gy, int64_t nrow, int64_t ncol, int acc,
              cudaStream_t s) {
    const bool vec = (ncol & 3) == 0 && (reinterpret_cast<uintptr_t>(gy) & 15) == 0;
    const int64_t col_blocks = vec ? (ncol + 127) / 128 : (ncol + 31) / 32;
    // Enough row slabs to put ~12 blocks on every SM, at least 64 rows each.
    int64_t slabs = (static_cast<int64_t>(st->sm_count) * 12 + col_blocks - 1) / col_blocks;
    const int64_t max_slabs = (nrow + 63) / 64;
    if (slabs > max_slabs) slabs = max_slabs;
    if (slabs < 1) slabs = 1;
    if (slabs > 1024) slabs = 1024;
    const int64_t rows_per_slab = (nrow + slabs - 1) / slabs;
    slabs = (nrow + rows_per_slab - 1) / rows_per_slab;
    if (slabs < 1) slabs = 1;
    KAI_TRY(ensure_workspace(st, device, slabs * ncol * 4));
    float* partial = static_cast<float*>(st->ws);
    dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(slabs));
    if (vec) colsum_partial4_kernel<<<grid, dim3(32, 8), 0, s>>>(gy, nrow, ncol, rows_per_slab, partial);
    else colsum_partial_kernel<<<grid, dim3(32, 8), 0, s>>>(gy, nrow, ncol, rows_per_slab, partial);
    count_launch();
    KAI_TRY(check_launch("colsum_partial_kernel"));
    colsum_final_kernel<<<static_cast<unsigned>((ncol + 255) / 256), 256, 0, s>>>(
        partial, static_cast<int>(slabs), ncol, gb, acc);
    count_launch();
    return check_launch("colsum_final_kernel");
}

int ew_activate(DeviceState* st, float* y, const float* x, int64_t nrow, int64_t ncol, int act,
                const float* alpha, cudaStream_t s) {
    if (act == KAI_ACT_SOFTMAX) {
        const int64_t threads = nrow * 32;
        softmax_rows_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(y, x, nrow, ncol);
        count_launch();
        return check_launch("softmax_rows_kernel");
    }
    const int64_t total = nrow * ncol;
    const int vec = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15) == 0 ? 1 : 0;
    activate_kernel<<<grid_for(vec ? (total + 3) / 4 : total, 256, st->sm_count), 256, 0, s>>>(y, x, total, act, alpha,
                                                                                          vec);
    count_launch();
    return check_launch("activate_kernel");
}

int ew_activate_backward(DeviceState* st, float* gx, const float* gy, const float* ref, int64_t total,
                         int act, const float* alpha, int from_y, cudaStream_t s) {
    const int vec = ((reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(gy) |
                      reinterpret_cast<uintptr_t>(ref)) & 15) == 0 ? 1 : 0;
    activate_backward_kernel<<<grid_for(vec ? (total + 3) / 4 : total, 256, st->sm_count), 256, 0, s>>>(
        gx, gy, ref, total, act, alpha, from_y, vec);
    count_launch();
    return check_launch("activate_backward_kernel");
}

int ew_ce_forward(DeviceState* st, float* y, const float* x, const int* label, int64_t nrow, int64_t ncol,
                  cudaStream_t s) {
    // Inside a stream capture nothing may block: the kernel then raises the second flag word, which stays in
    // device memory until kai_device_status reads (and clears) it.
    int* flag = st->flag_dev + (capturing() ? 1 : 0);
    if (!capturing()) KAI_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), s));
    const int64_t threads = nrow * 32;
    ce_forward_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(y, x, label, nrow, ncol, flag);
    count_launch();
    KAI_TRY(check_launch("ce_forward_kernel"));
    if (capturing()) return KAI_OK;
    int bad = 0;
    KAI_CUDA(cudaMemcpyAsync(&bad, st->flag_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
    KAI_CUDA(cudaStreamSynchronize(s));
    if (bad) return fail(KAI_E_OUT_OF_RANGE, "softmax_idx_crossentropy: label outside [0, %lld)", (long long)ncol);
    return KAI_OK;
}

int ew_ce_backward(DeviceState* st, float* gx, const float* gy, const float* x, const int* label, int64_t nrow,
                   int64_t ncol, cudaStream_t s) {
    (void)st;
    const int64_t threads = nrow * 32;
    ce_backward_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(gx, gy, x, label, nrow, ncol);
    count_launch();
    return check_launch("ce_backward_kernel");
}

int ew_sum(float* y, const float* x, int64_t n, cudaStream_t s) {
    sum_kernel<<<1, 1024, 0, s>>>(y, x, n);
    count_launch();
    return check_launch("sum_kernel");
}

int ew_sum_backward(DeviceState* st, float* gx, const float* gy, int64_t n, cudaStream_t s) {
    sum_backward_kernel<<<grid_for(n, 256, st->sm_count), 256, 0, s>>>(gx, gy, n);
    count_launch();
    return check_launch("sum_backward_kernel");
}

int ew_layernorm(float* y, const float* x, float* ps, int64_t nrow, int64_t ncol, const float* scale, cudaStream_t s) {
    const bool vec = (ncol & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if (vec && ncol <= 128 * 16) {
        const unsigned blocks = static_cast<unsigned>((nrow + 7) / 8);   // 8 warps = 8 rows per block
        const int64_t quads = ncol >> 2;
        if (quads <= 32) layernorm_warp_kernel<1><<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
        else if (quads <= 64) layernorm_warp_kernel<2><<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
        else if (quads <= 128) layernorm_warp_kernel<4><<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
        else if (quads <= 256) layernorm_warp_kernel<8><<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
        else layernorm_warp_kernel<16><<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
        count_launch();
        return check_launch("layernorm_warp_kernel");
    }
    const unsigned blocks = static_cast<unsigned>(nrow < 148 * 8 ? nrow : 148 * 8);
    layernorm_block_kernel<<<blocks, 256, 0, s>>>(y, x, ps, nrow, ncol, scale);
    count_launch();
    return check_launch("layernorm_block_kernel");
}

int ew_layernorm_backward(float* gx, const float* gy, const float* ps, int64_t nrow, int64_t ncol, const float* scale,
                          cudaStream_t s) {
    const int vec = ((ncol & 3) == 0 && ((reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(gy)) & 15) == 0) ? 1 : 0;
    const int64_t items = vec ? nrow * (ncol >> 2) : nrow * ncol;
    layernorm_backward_kernel<<<grid_for(items, 256, 148), 256, 0, s>>>(gx, gy, ps, nrow, ncol, scale, vec);
    count_launch();
    return check_launch("layernorm_backward_kernel");
}

}  // namespace kai
