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
                                int act, const float* __restrict__ leaky_alpha) {
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        y[i] = act_forward(act, x[i], alpha);
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

__global__ void activate_backward_kernel(float* __restrict__ gx, const float* __restrict__ gy,
                                         const float* __restrict__ ref, int64_t total, int act,
                                         const float* __restrict__ leaky_alpha, int from_y) {
    const float alpha = (leaky_alpha != nullptr) ? __ldg(leaky_alpha) : 0.0f;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const float g = from_y ? act_grad_from_y(act, ref[i], alpha) : act_grad_from_x(act, ref[i], alpha);
        gx[i] = g * gy[i];
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
    const int64_t col_blocks = (ncol + 31) / 32;
    // Enough row slabs to put ~4 blocks on every SM, at least 64 rows each.
    int64_t slabs = (static_cast<int64_t>(st->sm_count) * 4 + col_blocks - 1) / col_blocks;
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
    colsum_partial_kernel<<<grid, dim3(32, 8), 0, s>>>(gy, nrow, ncol, rows_per_slab, partial);
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
    activate_kernel<<<grid_for(total, 256, st->sm_count), 256, 0, s>>>(y, x, total, act, alpha);
    count_launch();
    return check_launch("activate_kernel");
}

int ew_activate_backward(DeviceState* st, float* gx, const float* gy, const float* ref, int64_t total,
                         int act, const float* alpha, int from_y, cudaStream_t s) {
    activate_backward_kernel<<<grid_for(total, 256, st->sm_count), 256, 0, s>>>(gx, gy, ref, total, act, alpha,
                                                                               from_y);
    count_launch();
    return check_launch("activate_backward_kernel");
}

int ew_ce_forward(DeviceState* st, float* y, const float* x, const int* label, int64_t nrow, int64_t ncol,
                  cudaStream_t s) {
    KAI_CUDA(cudaMemsetAsync(st->flag_dev, 0, sizeof(int), s));
    const int64_t threads = nrow * 32;
    ce_forward_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, s>>>(y, x, label, nrow, ncol,
                                                                                   st->flag_dev);
    count_launch();
    KAI_TRY(check_launch("ce_forward_kernel"));
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

}  // namespace kai
