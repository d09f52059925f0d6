// conv2d / conv2d_backward_x / conv2d_backward_k of the reference (support/vmath.cu:3490-3744):
// NCHW, stride 1, zero padding, kernel tensor [ychn][xchn / group][kh][kw].
//
// For group == 1 the three are dense contractions over (channel, kr, kc) or over (image, pixel),
// run on the GEMM kernels of this library.  The unfolded input is written in the orientation that
// is a plain copy of shifted image rows,
//     colT[(cn, kr, kc)][(nd, r, c)] = src[nd][cn][r + kr - ph][c + kc - pw]      (0 outside the image)
// so that
//     forward      y'[yn][m]   = k[yn][(xn,kr,kc)]          . colT(x)[(xn,kr,kc)][m]            (NN)
//     backward_x   gx'[xn][m]  = kT[xn][(yn,kr,kc)]         . colT(gy, flipped)[(yn,kr,kc)][m]   (NN)
//     backward_k   gk[yn][(xn,kr,kc)] = gy'[yn][m]          . colT(x)[(xn,kr,kc)][m]^T           (NT)
// with m = (image, pixel) and y', gx', gy' the [channel][image][pixel] forms of the NCHW tensors (a
// strided row copy apart; identical when ndat == 1).  The unfolded matrix and the permuted copies
// live at the front of the per-device workspace, the GEMM's own operand planes behind them.
// group != 1 (where the reference sums every input channel xn against kernel channel xn / group) becomes the
// group-1 convolution of the channel-group sums; the transposed family becomes a plain convolution of the
// row- and column-repeated image (forward) or a strided unfolding plus a GEMM (gradients).  One-thread-per-output
// kernels that repeat the reference's device loops remain behind the "conv_direct" option and for shapes the
// unfolding path does not take.
#include "kai_common.cuh"

namespace kai {

int64_t gemm_tc_scratch_bound(int64_t M, int64_t N, int64_t K);
bool conv_igemm_fits(int64_t M, int64_t K, int64_t nout);
bool conv_igemm_tma_fits(int64_t ndat, int64_t cchn, int64_t oh, int64_t ow, int64_t nout, int64_t kh, int64_t kw,
                         int64_t shP, int64_t swP);
int64_t conv_igemm_tma_bytes(int64_t ndat, int64_t cchn, int64_t nout, int64_t kh, int64_t kw, int64_t shP, int64_t swP);
int conv_igemm_tma(DeviceState* st, float* out, const float* src, const float* wsrc, int64_t wsn, int64_t wsc,
                   void* scratch, int64_t ndat, int64_t cchn, int64_t sh, int64_t sw, int64_t oh, int64_t ow,
                   int64_t nout, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t gh, int64_t gw, int flip,
                   int shP, int swP, int pt, int pl, cudaStream_t s);
int conv_igemm(DeviceState* st, float* out, const float* srcp, const float* wmat, float* w_hi, float* w_lo, int64_t ndat,
               int64_t cchn, int64_t oh, int64_t ow, int64_t nout, int64_t kh, int64_t kw, int64_t ph, int64_t pw,
               int64_t gh, int64_t gw, int flip, int shP, int swP, int pt, int pl, cudaStream_t s);

int taps_tile_channels(int64_t kh);
int64_t gemm_tc_taps_scratch(int64_t M, int64_t chan, int64_t shifts, int64_t kh);
int gemm_tc_taps(DeviceState* st, int device, float* c, const float* a_hi, const float* a_lo, int64_t M, int64_t K,
                 const float* b_hi, const float* b_lo, int64_t chan, int64_t chan_pitch, int64_t shifts, int64_t kh,
                 int64_t row_step, cudaStream_t s);

namespace {

inline int64_t al256(int64_t v) { return (v + 255) / 256 * 256; }

struct ConvDims {
    int64_t ndat, cchn, sh, sw;   // source tensor [ndat][cchn][sh][sw]
    int64_t oh, ow;               // grid of output positions
    int64_t kh, kw, ph, pw;
    int flip;                     // 0: source row = r + (kr - ph) * gh;  1: source row = r - (kr - ph) * gh
    int64_t gh, gw;               // gap between kernel taps (1 = ordinary convolution)
    int64_t strh = 1, strw = 1;   // stride of the output grid over the source (explicit-unfolding "rows" path only)
    int64_t vh = 0, vw = 0;       // valid extent of a source plane when smaller than sh x sw (0 = whole plane)
    int64_t valid_h() const { return vh > 0 ? vh : sh; }
    int64_t valid_w() const { return vw > 0 ? vw : sw; }
    bool plain() const { return strh == 1 && strw == 1 && vh == 0 && vw == 0; }
};

// One thread per (channel, 4 consecutive m): it divides the position (image, row, column) of its first
// output out once and then writes the kh * kw rows of colT that belong to the channel.  Rows of colT are
// `M` floats apart.  32-bit index arithmetic.
__global__ void __launch_bounds__(256)
im2col_t_kernel(float* __restrict__ col, float* __restrict__ col_lo, const float* __restrict__ src, ConvDims d, int M,
                int quads) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int cn = blockIdx.y;
    if (i >= quads) return;
    const int kw = static_cast<int>(d.kw), kh = static_cast<int>(d.kh);
    const int ow = static_cast<int>(d.ow), oh = static_cast<int>(d.oh);
    const int sh = static_cast<int>(d.sh), sw = static_cast<int>(d.sw), cchn = static_cast<int>(d.cchn);
    const int pix = oh * ow;
    const int m = 4 * i;
    // positions of the four outputs
    int nd[4], r[4], c[4];
    {
        int n0 = m / pix;
        int p = m - n0 * pix;
        int r0 = p / ow, c0 = p - r0 * ow;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            nd[e] = n0; r[e] = r0; c[e] = c0;
            if (++c0 == ow) { c0 = 0; if (++r0 == oh) { r0 = 0; ++n0; } }
        }
    }
    const bool vec = (M & 3) == 0;
    const float* pos[4];      // address of the untapped source position of each output
#pragma unroll
    for (int e = 0; e < 4; ++e) pos[e] = src + ((static_cast<int64_t>(nd[e]) * cchn + cn) * sh + r[e]) * sw + c[e];
    for (int kr = 0; kr < kh; ++kr) {
        const int dr = (d.flip ? (static_cast<int>(d.ph) - kr) : (kr - static_cast<int>(d.ph))) * static_cast<int>(d.gh);
        for (int kc = 0; kc < kw; ++kc) {
            const int dc = (d.flip ? (static_cast<int>(d.pw) - kc) : (kc - static_cast<int>(d.pw))) * static_cast<int>(d.gw);
            const int shift = dr * sw + dc;
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int sr = r[e] + dr, sc = c[e] + dc;
                float t = 0.0f;
                if (m + e < M && sr >= 0 && sr < sh && sc >= 0 && sc < sw) t = __ldg(pos[e] + shift);
                v[e] = t;
            }
            float* out = col + (static_cast<int64_t>(cn) * kh * kw + kr * kw + kc) * M + m;
            if (vec) {
                *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
                if (col_lo != nullptr) {
                    // lo plane against the truncated high part: the GEMM then reads colT itself as the hi operand
                    float l[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float t = __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u);
                        const float rest = isfinite(v[e]) ? (v[e] - t) : 0.0f;
                        uint32_t lw;
                        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(rest));
                        l[e] = __uint_as_float(lw);
                    }
                    *reinterpret_cast<float4*>(col_lo + (out - col)) = make_float4(l[0], l[1], l[2], l[3]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (m + e < M) out[e] = v[e];
            }
        }
    }
}

// Zero-padded copy of the source planes: dst[plane][shP][swP], the image at (pt, pl).
__global__ void __launch_bounds__(256)
pad_planes_kernel(float* __restrict__ dst, const float* __restrict__ src, int sh, int sw, int shP, int swP, int pt,
                  int pl, int vh, int vw) {
    const int plane = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= shP * swP) return;
    const int r = i / swP - pt, c = i % swP - pl;
    float v = 0.0f;
    if (r >= 0 && r < vh && c >= 0 && c < vw) v = __ldg(src + (static_cast<int64_t>(plane) * sh + r) * sw + c);
    dst[static_cast<int64_t>(plane) * shP * swP + i] = v;
}

// The other orientation, col[(nd, r, c)][(cn, kr, kc)], written together with its lo plane (against the truncated
// high part): the K-major B operand of an NT GEMM that needs no split pass.  It reads a zero-padded copy of the
// source, so a tap is one table read (the tap's linear offset in the padded tensor) and one load, without bounds
// tests.  A block takes 32 output positions.  K % 4 == 0, K <= 8192.
constexpr int IR_ROWS = 32;
struct PadDims { int shP, swP, pt, pl; };
__global__ void __launch_bounds__(256)
im2col_rows_kernel(float* __restrict__ col, float* __restrict__ col_lo, const float* __restrict__ srcp, ConvDims d,
                   PadDims pd, int M, int K) {
    extern __shared__ int ir_smem[];
    int* tap_lin = ir_smem;            // [K] offset of tap k from an output's own position in the padded tensor
    int* row_pos = ir_smem + K;        // [32] that position, or -1 past the end
    const int kw = static_cast<int>(d.kw), kh = static_cast<int>(d.kh);
    const int ow = static_cast<int>(d.ow), oh = static_cast<int>(d.oh), cchn = static_cast<int>(d.cchn);
    const int plane = pd.shP * pd.swP;
    for (int k = threadIdx.x; k < K; k += 256) {
        const int kc = k % kw, kr = (k / kw) % kh, cn = k / (kw * kh);
        const int dr = (d.flip ? (static_cast<int>(d.ph) - kr) : (kr - static_cast<int>(d.ph))) * static_cast<int>(d.gh);
        const int dc = (d.flip ? (static_cast<int>(d.pw) - kc) : (kc - static_cast<int>(d.pw))) * static_cast<int>(d.gw);
        tap_lin[k] = cn * plane + dr * pd.swP + dc;
    }
    const int m0 = blockIdx.x * IR_ROWS;
    if (threadIdx.x < IR_ROWS) {
        const int m = m0 + threadIdx.x;
        int pos = -1;
        if (m < M) {
            const int pix = oh * ow, nd = m / pix, p = m - nd * pix;
            pos = nd * cchn * plane + ((p / ow) * static_cast<int>(d.strh) + pd.pt) * pd.swP +
                  ((p % ow) * static_cast<int>(d.strw) + pd.pl);
        }
        row_pos[threadIdx.x] = pos;
    }
    __syncthreads();
    const int kq = K >> 2;
    for (int idx = threadIdx.x; idx < IR_ROWS * kq; idx += 256) {
        const int ml = idx / kq, k4 = idx - ml * kq;
        const int pos = row_pos[ml];
        if (pos < 0) continue;
        const int4 tl = *reinterpret_cast<const int4*>(tap_lin + 4 * k4);
        const float v[4] = {__ldg(srcp + pos + tl.x), __ldg(srcp + pos + tl.y), __ldg(srcp + pos + tl.z),
                            __ldg(srcp + pos + tl.w)};
        float l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float hi = __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u);
            const float rest = isfinite(v[e]) ? (v[e] - hi) : 0.0f;
            uint32_t lw;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(rest));
            l[e] = __uint_as_float(lw);
        }
        const int64_t o = static_cast<int64_t>(m0 + ml) * K + 4 * k4;
        *reinterpret_cast<float4*>(col + o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(col_lo + o) = make_float4(l[0], l[1], l[2], l[3]);
    }
}

// dst[b][a][p] = src[a][b][p]: blockIdx.y = a * B + b picks a row of P floats, blockIdx.x a piece of it.
__global__ void __launch_bounds__(256)
swap01_kernel(float* __restrict__ dst, const float* __restrict__ src, int A, int B, int64_t P) {
    const int a = blockIdx.y / B, b = blockIdx.y - a * B;
    const float* s = src + static_cast<int64_t>(blockIdx.y) * P;
    float* d = dst + (static_cast<int64_t>(b) * A + a) * P;
    const int64_t i = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4;
    if (i >= P) return;
    if (i + 3 < P && ((reinterpret_cast<uintptr_t>(s + i) | reinterpret_cast<uintptr_t>(d + i)) & 15) == 0) {
        *reinterpret_cast<float4*>(d + i) = *reinterpret_cast<const float4*>(s + i);
    } else {
        for (int64_t e = i; e < P && e < i + 4; ++e) d[e] = s[e];
    }
}

// col_lo (optional, needs M % 4 == 0): also write the lo plane of colT
int launch_im2col(float* col, const float* src, const ConvDims& d, cudaStream_t s, float* col_lo = nullptr) {
    const int64_t M = d.ndat * d.oh * d.ow, K = d.cchn * d.kh * d.kw;
    const int64_t quads = (M + 3) / 4;
    (void)K;
    if (d.cchn > 65535) return fail(KAI_E_TOO_LARGE, "conv2d: %lld channels exceed 65535", (long long)d.cchn);
    if (M >= (int64_t(1) << 31) - 8) return fail(KAI_E_TOO_LARGE, "conv2d: images * pixels = %lld exceeds 2^31", (long long)M);
    dim3 grid(static_cast<unsigned>((quads + 255) / 256), static_cast<unsigned>(d.cchn));
    im2col_t_kernel<<<grid, 256, 0, s>>>(col, (M & 3) == 0 ? col_lo : nullptr, src, d, static_cast<int>(M),
                                         static_cast<int>(quads));
    count_launch();
    return check_launch("im2col_t_kernel");
}

int launch_swap01(float* dst, const float* src, int64_t A, int64_t B, int64_t P, int sm_count, cudaStream_t s) {
    (void)sm_count;
    if (A * B > 65535) return fail(KAI_E_TOO_LARGE, "conv2d: images * channels = %lld exceeds 65535", (long long)(A * B));
    dim3 grid(static_cast<unsigned>((P + 1023) / 1024), static_cast<unsigned>(A * B));
    swap01_kernel<<<grid, 256, 0, s>>>(dst, src, static_cast<int>(A), static_cast<int>(B), P);
    count_launch();
    return check_launch("swap01_kernel");
}

// Padding that makes every tap of every output position land inside the padded plane.
PadDims pad_dims(const ConvDims& d) {
    const int64_t r_lo = d.flip ? (d.ph - (d.kh - 1)) * d.gh : -d.ph * d.gh;      // smallest and largest row shift
    const int64_t r_hi = d.flip ? d.ph * d.gh : (d.kh - 1 - d.ph) * d.gh;
    const int64_t c_lo = d.flip ? (d.pw - (d.kw - 1)) * d.gw : -d.pw * d.gw;
    const int64_t c_hi = d.flip ? d.pw * d.gw : (d.kw - 1 - d.pw) * d.gw;
    PadDims p;
    p.pt = static_cast<int>(r_lo < 0 ? -r_lo : 0);
    p.pl = static_cast<int>(c_lo < 0 ? -c_lo : 0);
    const int64_t last_r = (d.oh - 1) * d.strh + r_hi + 1, last_c = (d.ow - 1) * d.strw + c_hi + 1;
    const int64_t bottom = (last_r > d.valid_h()) ? last_r : d.valid_h();          // rows [0, bottom) of the source frame
    const int64_t right = (last_c > d.valid_w()) ? last_c : d.valid_w();
    p.shP = static_cast<int>(p.pt + bottom);
    p.swP = static_cast<int>(p.pl + right);
    return p;
}

// Whether the row orientation (and with it the split-free NT GEMM) applies.
bool rows_form_ok(const ConvDims& d) {
    const int64_t M = d.ndat * d.oh * d.ow, K = d.cchn * d.kh * d.kw;
    if ((K & 3) != 0 || K > 8192 || M >= (int64_t(1) << 31) - 64 || d.ndat * d.cchn > 65535) return false;
    if (d.kh * d.gh > 4096 || d.kw * d.gw > 4096 || d.oh > 16384 || d.ow > 16384 || d.sh > 16384 || d.sw > 16384) return false;
    const PadDims p = pad_dims(d);
    return d.ndat * d.cchn * static_cast<int64_t>(p.shP) * p.swP < (int64_t(1) << 31);
}

int64_t padded_bytes(const ConvDims& d) {
    const PadDims p = pad_dims(d);
    return al256(d.ndat * d.cchn * static_cast<int64_t>(p.shP) * p.swP * 4);
}

int launch_pad(float* padded, const float* src, const ConvDims& d, cudaStream_t s) {
    const PadDims p = pad_dims(d);
    dim3 pgrid(static_cast<unsigned>((static_cast<int64_t>(p.shP) * p.swP + 255) / 256), static_cast<unsigned>(d.ndat * d.cchn));
    pad_planes_kernel<<<pgrid, 256, 0, s>>>(padded, src, static_cast<int>(d.sh), static_cast<int>(d.sw), p.shP, p.swP, p.pt, p.pl,
                                            static_cast<int>(d.valid_h()), static_cast<int>(d.valid_w()));
    count_launch();
    return check_launch("pad_planes_kernel");
}

// The implicit-GEMM kernel builds its operand tiles from the padded image itself: no unfolded matrix in memory.
bool igemm_ok(const ConvDims& d, int64_t nout) {
    if (options().conv_igemm.load() == 0) return false;
    const int64_t M = d.ndat * d.oh * d.ow, K = d.cchn * d.kh * d.kw;
    if (!conv_igemm_fits(M, K, nout) || d.ndat * d.cchn > 65535) return false;
    if (d.kh * d.gh > 4096 || d.kw * d.gw > 4096 || d.oh > 16384 || d.ow > 16384 || d.sh > 16384 || d.sw > 16384) return false;
    const PadDims p = pad_dims(d);
    return d.ndat * d.cchn * static_cast<int64_t>(p.shP) * p.swP < (int64_t(1) << 31);
}

int run_igemm(DeviceState* st, int device, float* out, const float* src, const float* wmat, const ConvDims& d, int64_t nout,
              int64_t extra_front, cudaStream_t s) {
    // front of the workspace: [extra_front bytes of the caller][padded image][weight hi][weight lo]
    const int64_t K = d.cchn * d.kh * d.kw, kp = (K + 3) / 4 * 4;
    const int64_t pad_bytes = padded_bytes(d), w_bytes = al256(nout * kp * 4);
    uint8_t* base = static_cast<uint8_t*>(st->ws) + extra_front;
    float* padded = reinterpret_cast<float*>(base);
    float* w_hi = reinterpret_cast<float*>(base + pad_bytes);
    float* w_lo = reinterpret_cast<float*>(base + pad_bytes + w_bytes);
    (void)device;
    KAI_TRY(launch_pad(padded, src, d, s));
    const PadDims p = pad_dims(d);
    return conv_igemm(st, out, padded, wmat, w_hi, w_lo, d.ndat, d.cchn, d.oh, d.ow, nout, d.kh, d.kw, d.ph, d.pw, d.gh,
                      d.gw, d.flip, p.shP, p.swP, p.pt, p.pl, s);
}

// The TMA-fed variant: operand tiles are boxes of a zero-padded channels-last copy of the image.
bool igemm_tma_ok(const ConvDims& d, int64_t nout) {
    if (options().conv_igemm.load() != 1) return false;
    if (d.kh * d.gh > 4096 || d.kw * d.gw > 4096 || d.oh > 16384 || d.ow > 16384 || d.sh > 16384 || d.sw > 16384) return false;
    const PadDims p = pad_dims(d);
    return conv_igemm_tma_fits(d.ndat, d.cchn, d.oh, d.ow, nout, d.kh, d.kw, p.shP, p.swP);
}

// wsn / wsc: strides of the weight tensor over the output channel and the reduced channel (taps are contiguous).
int run_igemm_tma(DeviceState* st, int device, float* out, const float* src, const float* w, int64_t wsn, int64_t wsc,
                  const ConvDims& d, int64_t nout, cudaStream_t s) {
    const PadDims p = pad_dims(d);
    KAI_TRY(ensure_workspace(st, device, conv_igemm_tma_bytes(d.ndat, d.cchn, nout, d.kh, d.kw, p.shP, p.swP) + 256));
    return conv_igemm_tma(st, out, src, w, wsn, wsc, st->ws, d.ndat, d.cchn, d.sh, d.sw, d.oh, d.ow, nout, d.kh, d.kw,
                          d.ph, d.pw, d.gh, d.gw, d.flip, p.shP, p.swP, p.pt, p.pl, s);
}

int64_t igemm_front_bytes(const ConvDims& d, int64_t nout) {
    const int64_t K = d.cchn * d.kh * d.kw, kp = (K + 3) / 4 * 4;
    return padded_bytes(d) + 2 * al256(nout * kp * 4);
}

int launch_im2col_rows(float* col, float* col_lo, float* padded, const float* src, const ConvDims& d, cudaStream_t s) {
    const int64_t M = d.ndat * d.oh * d.ow, K = d.cchn * d.kh * d.kw;
    const PadDims p = pad_dims(d);
    KAI_TRY(launch_pad(padded, src, d, s));
    const unsigned blocks = static_cast<unsigned>((M + IR_ROWS - 1) / IR_ROWS);
    const size_t smem = (static_cast<size_t>(K) + IR_ROWS) * sizeof(int);
    im2col_rows_kernel<<<blocks, 256, smem, s>>>(col, col_lo, padded, d, p, static_cast<int>(M), static_cast<int>(K));
    count_launch();
    return check_launch("im2col_rows_kernel");
}

// The GEMM behind a convolution: tensor cores unless the problem is tiny.
int conv_gemm(DeviceState* st, int device, int layout, float* c, const float* a, const float* b, int64_t M, int64_t N,
              int64_t K, cudaStream_t s, const float* b_lo = nullptr) {
    const Epilogue ep{nullptr, nullptr, KAI_ACT_NONE, 0};
    const double flops = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
    if (flops < static_cast<double>(options().tc_min_flops.load()) || M < 32 || N < 32 || K == 0)
        return gemm_simt(layout, c, a, b, M, N, K, N, ep, s);
    return gemm_tc(st, device, layout, c, a, b, M, N, K, N, ep, s, b_lo);
}

struct FrontGuard {   // reserves the front of the workspace for the lifetime of one convolution
    DeviceState* st;
    FrontGuard(DeviceState* s_, int64_t bytes) : st(s_) { st->ws_front = bytes; }
    ~FrontGuard() { st->ws_front = 0; }
};


// ---- kernel gradient without the unfolded matrix ---------------------------------------------------------
// gk[yn][xn][kr][kc] = sum_{nd,r,c} gy[nd][yn][r][c] * x[nd][xn][r + (kr - ph) gh][c + (kc - pw) gw] is a GEMM whose
// reduction runs over the output positions.  Positions are numbered on a padded grid, m' = (nd * Hp + r) * Wp + c with
// Hp = yh + (kh - 1) gh rows and Wp = round_up(yw, 4) columns, and both operands are written once as K-major planes
// over m' (hi = the values, lo = their TF32 remainders):
//   gy'[yn][m']           = gy[nd][yn][r][c], zero on the padding;
//   xs[kc][xn][m']        = x[nd][xn][r - ph gh][c + (kc - pw) gw], zero outside the image: one copy per kernel COLUMN,
//                           shifted by that column's offset, so that every tile a bulk tensor copy fetches starts
//                           on a 16-byte boundary;
// a kernel ROW is then just a start offset of kr * gh * Wp elements into the same copy.  The GEMM kernel reads a B
// tile as kh boxes (one per kernel row) of 64 channels and accumulates gk for (all kernel rows) x (64 channels) x
// (128 output channels) per tile; the few tiles are range-split over the SMs along m'.  The explicit unfolding wrote
// and re-read kh * kw copies of the input (x its lo plane); this writes kw.
struct WgradDims {
    int ndat, xchn, ychn, xh, xw, yh, yw, kh, kw, ph, pw, gh, gw, hp, wp;
    int64_t k;            // ndat * hp * wp
    int64_t chan_pitch;   // floats per (column shift, channel) row of xs
};

__global__ void __launch_bounds__(256)
wgrad_planes_kernel(float* __restrict__ gy_hi, float* __restrict__ gy_lo, float* __restrict__ xs_hi, float* __restrict__ xs_lo,
                    const float* __restrict__ gy, const float* __restrict__ x, const WgradDims d) {
    // blockIdx.y: 0 .. ychn-1 -> a row of gy'; ychn .. ychn + kw*xchn - 1 -> a row of xs (column shift, channel)
    const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;      // group of 4 consecutive columns
    const int wq = d.wp >> 2;
    const int64_t quads = static_cast<int64_t>(d.ndat) * d.hp * wq;
    const bool is_gy = static_cast<int>(blockIdx.y) < d.ychn;
    const int row = is_gy ? blockIdx.y : blockIdx.y - d.ychn;
    float* hi = is_gy ? gy_hi + static_cast<int64_t>(row) * d.k : xs_hi + static_cast<int64_t>(row) * d.chan_pitch;
    float* lo = is_gy ? gy_lo + static_cast<int64_t>(row) * d.k : xs_lo + static_cast<int64_t>(row) * d.chan_pitch;
    const int64_t tail_quads = is_gy ? quads : (d.chan_pitch >> 2);
    if (q >= tail_quads) return;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (q < quads) {
        const int c0 = static_cast<int>(q % wq) * 4;
        const int rr = static_cast<int>((q / wq) % d.hp);
        const int nd = static_cast<int>(q / (static_cast<int64_t>(wq) * d.hp));
        if (is_gy) {
            if (rr < d.yh) {
                const float* src = gy + ((static_cast<int64_t>(nd) * d.ychn + row) * d.yh + rr) * d.yw;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c0 + e < d.yw) v[e] = __ldg(src + c0 + e);
            }
        } else {
            const int kc = row / d.xchn, xn = row - kc * d.xchn;
            const int sr = rr - d.ph * d.gh;
            if (sr >= 0 && sr < d.xh) {
                const float* src = x + ((static_cast<int64_t>(nd) * d.xchn + xn) * d.xh + sr) * d.xw;
                const int sc0 = c0 + (kc - d.pw) * d.gw;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (sc0 + e >= 0 && sc0 + e < d.xw) v[e] = __ldg(src + sc0 + e);
            }
        }
    }
    float l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float t = __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u);     // the tensor core reads hi truncated
        const float rest = isfinite(v[e]) ? (v[e] - t) : 0.0f;
        uint32_t lw;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lw) : "f"(rest));
        l[e] = __uint_as_float(lw);
    }
    *reinterpret_cast<float4*>(hi + 4 * q) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(lo + 4 * q) = make_float4(l[0], l[1], l[2], l[3]);
}

// gk[yn][xn][kr][kc] = ctmp[yn][((kc * xblocks + xn / xb) * kh + kr) * xb + xn % xb]
__global__ void __launch_bounds__(256)
wgrad_gather_kernel(float* __restrict__ gk, const float* __restrict__ ctmp, int64_t total, int xchn, int kh, int kw, int xb,
                    int xblocks, int64_t ncols) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (i >= total) return;
    const int kc = static_cast<int>(i % kw), kr = static_cast<int>((i / kw) % kh);
    const int xn = static_cast<int>((i / (static_cast<int64_t>(kw) * kh)) % xchn);
    const int64_t yn = i / (static_cast<int64_t>(kw) * kh * xchn);
    gk[i] = __ldg(ctmp + yn * ncols + (static_cast<int64_t>(kc * xblocks + xn / xb) * kh + kr) * xb + xn % xb);
}

// Returns 1 when the shape is outside this path.
int conv_wgrad_taps(DeviceState* st, int device, float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn,
                    int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw, int64_t ph,
                    int64_t pw, int64_t gh, int64_t gw, cudaStream_t s) {
    const int xb = taps_tile_channels(kh);
    if (options().conv_igemm.load() == 0 || xb == 0 || kw > 8 || ychn < 16 || xchn < 8) return 1;
    const int64_t hp = yh + (kh - 1) * gh, wp = (yw + 3) / 4 * 4;
    const int64_t K = ndat * hp * wp;
    const int64_t row_step = gh * wp;
    const int64_t chan_pitch = (K + (kh - 1) * row_step + 3) / 4 * 4;
    if (K >= (int64_t(1) << 31) || chan_pitch >= (int64_t(1) << 31) || ychn + kw * xchn > 65535) return 1;
    const double flops = 2.0 * static_cast<double>(ndat * yh * yw) * static_cast<double>(ychn) * static_cast<double>(xchn * kh * kw);
    if (flops < static_cast<double>(options().tc_min_flops.load())) return 1;
    const int64_t xblocks = (xchn + xb - 1) / xb;
    const int64_t ncols = kw * xblocks * kh * xb;
    const int64_t gy_plane = al256(ychn * K * 4), xs_plane = al256(kw * xchn * chan_pitch * 4), ct_bytes = al256(ychn * ncols * 4);
    const int64_t front = 2 * gy_plane + 2 * xs_plane + ct_bytes;
    KAI_TRY(ensure_workspace(st, device, front + 256 + gemm_tc_taps_scratch(ychn, xchn, kw, kh)));
    FrontGuard guard(st, front);
    uint8_t* base = static_cast<uint8_t*>(st->ws);
    float* gy_hi = reinterpret_cast<float*>(base);
    float* gy_lo = reinterpret_cast<float*>(base + gy_plane);
    float* xs_hi = reinterpret_cast<float*>(base + 2 * gy_plane);
    float* xs_lo = reinterpret_cast<float*>(base + 2 * gy_plane + xs_plane);
    float* ctmp = reinterpret_cast<float*>(base + 2 * gy_plane + 2 * xs_plane);
    WgradDims d;
    d.ndat = static_cast<int>(ndat); d.xchn = static_cast<int>(xchn); d.ychn = static_cast<int>(ychn);
    d.xh = static_cast<int>(xh); d.xw = static_cast<int>(xw); d.yh = static_cast<int>(yh); d.yw = static_cast<int>(yw);
    d.kh = static_cast<int>(kh); d.kw = static_cast<int>(kw); d.ph = static_cast<int>(ph); d.pw = static_cast<int>(pw);
    d.gh = static_cast<int>(gh); d.gw = static_cast<int>(gw); d.hp = static_cast<int>(hp); d.wp = static_cast<int>(wp);
    d.k = K; d.chan_pitch = chan_pitch;
    const dim3 grid(static_cast<unsigned>((chan_pitch / 4 + 255) / 256), static_cast<unsigned>(ychn + kw * xchn));
    wgrad_planes_kernel<<<grid, 256, 0, s>>>(gy_hi, gy_lo, xs_hi, xs_lo, pgy, px, d);
    count_launch();
    KAI_TRY(check_launch("wgrad_planes_kernel"));
    KAI_TRY(gemm_tc_taps(st, device, ctmp, gy_hi, gy_lo, ychn, K, xs_hi, xs_lo, xchn, chan_pitch, kw, kh, row_step, s));
    const int64_t total = ychn * xchn * kh * kw;
    wgrad_gather_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
        pgk, ctmp, total, static_cast<int>(xchn), static_cast<int>(kh), static_cast<int>(kw), xb, static_cast<int>(xblocks), ncols);
    count_launch();
    return check_launch("wgrad_gather_kernel");
}

// ---- rewrites that turn the convolution variants into plain convolutions ----------------------------------
// group != 1: the reference sums EVERY input channel xn against kernel channel xn / group (vmath.cu:3530-3566),
// i.e. `group` adjacent input channels share one kernel channel.  Summing those channels first,
//     x'[nd][c][p] = sum_{g < group} x[nd][c * group + g][p],
// leaves an ordinary convolution over xchn / group channels (forward, kernel gradient); the input gradient of
// channel xn is the plain input gradient of channel xn / group.
__global__ void __launch_bounds__(256)
group_sum_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t total, int64_t pix, int group) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;   // over [nd][kchn][pix]
    if (i >= total) return;
    const int64_t plane = i / pix, p = i - plane * pix;
    const float* s = src + plane * group * pix + p;
    float t = 0.0f;
    for (int g = 0; g < group; ++g) t += __ldg(s + g * pix);
    dst[i] = t;
}
__global__ void __launch_bounds__(256)
group_broadcast_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t total, int64_t pix, int64_t xchn,
                       int group) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;   // over [nd][xchn][pix]
    if (i >= total) return;
    const int64_t plane = i / pix, p = i - plane * pix;
    const int64_t nd = plane / xchn, xn = plane - nd * xchn;
    dst[i] = __ldg(src + (nd * (xchn / group) + xn / group) * pix + p);
}

// conv2d_transposed (vmath.cu:3748-3824) reads, for output row yr and tap kr, the input row
//     xr = (yr - (kr - bh) - (sh - 1) / 2) / sh          (C quotient, no remainder test; skipped unless 0 <= xr < xh)
// Every tap contributes: the map is "repeat every input row sh times, then convolve".  With z = yr + off - kr,
// off = bh - (sh - 1) / 2, the row read is U[z] = x[z / sh]; the C quotient maps z in (-sh, 0) to row 0, so U is
// defined on [-(sh - 1), xh * sh) and zero outside.  V[j] = U[j - h0] (h0 rows of that lead-in kept) is the
// repeated image; y[yr] = sum_kr' V[yr + kr' - ph] * k[kh - 1 - kr'] with ph = (kh - 1) - off - h0 is then the
// forward convolution of V with the flipped kernel and padding ph (columns likewise).
__global__ void __launch_bounds__(256)
repeat_rows_cols_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t total, int xh, int xw, int sh,
                        int sw, int h0, int w0, int vh, int vw) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;   // over [plane][vh][vw]
    if (i >= total) return;
    const int c = static_cast<int>(i % vw), r = static_cast<int>((i / vw) % vh);
    const int64_t plane = i / (static_cast<int64_t>(vw) * vh);
    const int zr = r - h0, zc = c - w0;
    const int xr = zr < 0 ? 0 : zr / sh, xc = zc < 0 ? 0 : zc / sw;
    dst[i] = __ldg(src + (plane * xh + xr) * xw + xc);
}
__global__ void __launch_bounds__(256)
flip_taps_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t total, int kh, int kw) {
    const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;   // over [filters][kh][kw]
    if (i >= total) return;
    const int kc = static_cast<int>(i % kw), kr = static_cast<int>((i / kw) % kh);
    const int64_t f = i / (static_cast<int64_t>(kw) * kh);
    dst[i] = __ldg(src + (f * kh + (kh - 1 - kr)) * kw + (kw - 1 - kc));
}

// ---- group != 1, option "conv_direct": the reference's own decomposition, one thread per output ----
__global__ void conv2d_generic_kernel(float* __restrict__ py, const float* __restrict__ px, const float* __restrict__ pk,
                                      int64_t size, int64_t ychn, int64_t yh, int64_t yw, int64_t xchn, int64_t xh,
                                      int64_t xw, int64_t kh, int64_t kw, int64_t group, int64_t ph, int64_t pw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t yc = n % yw, yr = (n / yw) % yh, yn = (n / (yw * yh)) % ychn, nd = n / (yw * yh * ychn);
    const int64_t kchn = xchn / group;
    float sum = 0.f;
    for (int64_t kr = 0; kr < kh; ++kr)
        for (int64_t kc = 0; kc < kw; ++kc) {
            const int64_t xr = yr + (kr - ph), xc = yc + (kc - pw);
            if (xr < 0 || xr >= xh || xc < 0 || xc >= xw) continue;
            for (int64_t xn = 0; xn < xchn; ++xn)
                sum = fmaf(px[((nd * xchn + xn) * xh + xr) * xw + xc],
                           pk[((yn * kchn + (xn / group)) * kh + kr) * kw + kc], sum);
        }
    py[n] = sum;
}

__global__ void conv2d_backward_x_generic_kernel(float* __restrict__ pgx, const float* __restrict__ pgy,
                                                 const float* __restrict__ pk, int64_t size, int64_t xchn, int64_t xh,
                                                 int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh,
                                                 int64_t kw, int64_t group, int64_t ph, int64_t pw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t xc = n % xw, xr = (n / xw) % xh, xn = (n / (xw * xh)) % xchn, nd = n / (xw * xh * xchn);
    const int64_t kchn = xchn / group;
    float sum = 0.f;
    for (int64_t kr = 0; kr < kh; ++kr) {
        const int64_t yr = xr - (kr - ph);
        if (yr < 0 || yr >= yh) continue;
        for (int64_t kc = 0; kc < kw; ++kc) {
            const int64_t yc = xc - (kc - pw);
            if (yc < 0 || yc >= yw) continue;
            for (int64_t yn = 0; yn < ychn; ++yn)
                sum = fmaf(pgy[((nd * ychn + yn) * yh + yr) * yw + yc],
                           pk[((yn * kchn + (xn / group)) * kh + kr) * kw + kc], sum);
        }
    }
    pgx[n] = sum;
}

__global__ void conv2d_backward_k_generic_kernel(float* __restrict__ pgk, const float* __restrict__ pgy,
                                                 const float* __restrict__ px, int64_t size, int64_t ndat,
                                                 int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh,
                                                 int64_t yw, int64_t kh, int64_t kw, int64_t group, int64_t ph,
                                                 int64_t pw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t kchn = xchn / group;
    const int64_t kc = n % kw, kr = (n / kw) % kh, kn = (n / (kw * kh)) % kchn, yn = n / (kw * kh * kchn);
    float sum = 0.f;
    for (int64_t xr = 0; xr < xh; ++xr) {
        const int64_t yr = xr - (kr - ph);
        if (yr < 0 || yr >= yh) continue;
        for (int64_t xc = 0; xc < xw; ++xc) {
            const int64_t yc = xc - (kc - pw);
            if (yc < 0 || yc >= yw) continue;
            for (int64_t nd = 0; nd < ndat; ++nd)
                for (int64_t ng = 0; ng < group; ++ng)
                    sum = fmaf(pgy[((nd * ychn + yn) * yh + yr) * yw + yc],
                               px[((nd * xchn + kn * group + ng) * xh + xr) * xw + xc], sum);
        }
    }
    pgk[n] = sum;
}

// ---- conv2d_transposed family (support/vmath.cu:3748-3988): the reference's index rules are kept as they
// are (C integer quotient without a remainder test in the forward map; the backward maps test the output
// position against xh / xw), so these follow its loops one thread per output, multiply and add rounded
// separately in the same order: the results are the reference's bit for bit.
__global__ void conv2d_transposed_kernel(float* __restrict__ py, const float* __restrict__ px, const float* __restrict__ pk,
                                         int64_t size, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh,
                                         int64_t kw, int64_t sh, int64_t sw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    const int64_t yc = n % yw, yr = (n / yw) % yh, yn = (n / (yw * yh)) % ychn, nd = n / (yw * yh * ychn);
    float sum = 0.f;
    for (int64_t kr = 0; kr < kh; ++kr) {
        const int64_t xr = (yr - (kr - bh) - (sh - 1) / 2) / sh;
        if (xr < 0 || xr >= xh) continue;
        for (int64_t kc = 0; kc < kw; ++kc) {
            const int64_t xc = (yc - (kc - bw) - (sw - 1) / 2) / sw;
            if (xc < 0 || xc >= xw) continue;
            for (int64_t xn = 0; xn < xchn; ++xn)
                sum = __fadd_rn(sum, __fmul_rn(px[((nd * xchn + xn) * xh + xr) * xw + xc],
                                               pk[((yn * xchn + xn) * kh + kr) * kw + kc]));
        }
    }
    py[n] = sum;
}

__global__ void conv2d_transposed_backward_x_kernel(float* __restrict__ pgx, const float* __restrict__ pgy,
                                                    const float* __restrict__ pk, int64_t size, int64_t xchn,
                                                    int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                                                    int64_t sh, int64_t sw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    const int64_t xc = n % xw, xr = (n / xw) % xh, xn = (n / (xw * xh)) % xchn, nd = n / (xw * xh * xchn);
    float sum = 0.f;
    for (int64_t kr = 0; kr < kh; ++kr) {
        const int64_t yr = xr * sh + (kr - bh) + (sh - 1) / 2;
        if (yr < 0 || yr >= xh) continue;
        for (int64_t kc = 0; kc < kw; ++kc) {
            const int64_t yc = xc * sw + (kc - bw) + (sw - 1) / 2;
            if (yc < 0 || yc >= xw) continue;
            for (int64_t yn = 0; yn < ychn; ++yn)
                sum = __fadd_rn(sum, __fmul_rn(pgy[((nd * ychn + yn) * yh + yr) * yw + yc],
                                               pk[((yn * xchn + xn) * kh + kr) * kw + kc]));
        }
    }
    pgx[n] = sum;
}

__global__ void conv2d_transposed_backward_k_kernel(float* __restrict__ pgk, const float* __restrict__ pgy,
                                                    const float* __restrict__ px, int64_t size, int64_t ndat,
                                                    int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh,
                                                    int64_t kw, int64_t sh, int64_t sw) {
    const int64_t n = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    if (n >= size) return;
    const int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    const int64_t kc = n % kw, kr = (n / kw) % kh, xn = (n / (kw * kh)) % xchn, yn = n / (kw * kh * xchn);
    float sum = 0.f;
    for (int64_t xr = 0; xr < xh; ++xr) {
        const int64_t yr = xr * sh + (kr - bh) + (sh - 1) / 2;
        if (yr < 0 || yr >= xh) continue;
        for (int64_t xc = 0; xc < xw; ++xc) {
            const int64_t yc = xc * sw + (kc - bw) + (sw - 1) / 2;
            if (yc < 0 || yc >= xw) continue;
            for (int64_t nd = 0; nd < ndat; ++nd)
                sum = __fadd_rn(sum, __fmul_rn(pgy[((nd * ychn + yn) * yh + yr) * yw + yc],
                                               px[((nd * xchn + xn) * xh + xr) * xw + xc]));
        }
    }
    pgk[n] = sum;
}

}  // namespace

int conv2d_backward_x(DeviceState* st, int device, float* pgx, const float* pgy, const float* pk, int64_t ndat,
                      int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                      int64_t group, int64_t ph, int64_t pw, int64_t gh, int64_t gw, cudaStream_t s);
int conv2d_backward_k(DeviceState* st, int device, float* pgk, const float* pgy, const float* px, int64_t ndat,
                      int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                      int64_t group, int64_t ph, int64_t pw, int64_t gh, int64_t gw, cudaStream_t s);

static unsigned blocks_for(int64_t total) { return static_cast<unsigned>((total + 255) / 256); }

// strh / strw: stride of the output grid over the source; vh / vw: valid extent of a source plane when it is
// smaller than xh x xw (0 = all of it).  Both exist for the transposed family's gradients and run on the
// explicit-unfolding path only; the call returns 1 ("not applicable") when that path does not take the shape.
int conv2d_forward(DeviceState* st, int device, float* py, const float* px, const float* pk, int64_t ndat, int64_t ychn,
                   int64_t yh, int64_t yw, int64_t xchn, int64_t xh, int64_t xw, int64_t kh, int64_t kw, int64_t group,
                   int64_t ph, int64_t pw, int64_t gh, int64_t gw, cudaStream_t s, int64_t strh, int64_t strw, int64_t vh,
                   int64_t vw) {
    if (group != 1) {
        if (options().conv_direct.load() != 0) {
            const int64_t size = ndat * ychn * yh * yw;
            conv2d_generic_kernel<<<static_cast<unsigned>((size + 255) / 256), 256, 0, s>>>(py, px, pk, size, ychn, yh, yw,
                                                                                            xchn, xh, xw, kh, kw, group, ph, pw);
            count_launch();
            return check_launch("conv2d_generic_kernel");
        }
        const int64_t kchn = xchn / group, total = ndat * kchn * xh * xw;
        KAI_TRY(ensure_aux(st, total * 4));
        float* xs = static_cast<float*>(st->aux);
        group_sum_kernel<<<blocks_for(total), 256, 0, s>>>(xs, px, total, xh * xw, static_cast<int>(group));
        count_launch();
        KAI_TRY(check_launch("group_sum_kernel"));
        return conv2d_forward(st, device, py, xs, pk, ndat, ychn, yh, yw, kchn, xh, xw, kh, kw, 1, ph, pw, gh, gw, s, 1, 1, 0, 0);
    }
    const int64_t M = ndat * yh * yw, K = xchn * kh * kw;
    ConvDims d{ndat, xchn, xh, xw, yh, yw, kh, kw, ph, pw, 0, gh, gw};
    d.strh = strh; d.strw = strw; d.vh = vh; d.vw = vw;
    if (d.plain()) {
        if (igemm_tma_ok(d, ychn)) return run_igemm_tma(st, device, py, px, pk, xchn * kh * kw, kh * kw, d, ychn, s);
        if (igemm_ok(d, ychn)) {
            KAI_TRY(ensure_workspace(st, device, igemm_front_bytes(d, ychn) + 256));
            return run_igemm(st, device, py, px, pk, d, ychn, 0, s);
        }
    }
    const int64_t col_bytes = al256(K * M * 4), tmp_bytes = (ndat > 1) ? al256(ychn * M * 4) : 0;
    if (rows_form_ok(d)) {
        // y'[yn][m] = k[yn][.] . col[m][.]^T with col and its lo plane written in one pass: no split of col
        const int64_t pad_bytes = padded_bytes(d);
        KAI_TRY(ensure_workspace(st, device, 2 * col_bytes + tmp_bytes + pad_bytes + 256 + gemm_tc_scratch_bound(ychn, M, K)));
        FrontGuard front(st, 2 * col_bytes + tmp_bytes + pad_bytes);
        uint8_t* base = static_cast<uint8_t*>(st->ws);
        float* col = reinterpret_cast<float*>(base);
        float* col_lo = reinterpret_cast<float*>(base + col_bytes);
        float* padded = reinterpret_cast<float*>(base + 2 * col_bytes);
        float* tmp = (ndat > 1) ? reinterpret_cast<float*>(base + 2 * col_bytes + pad_bytes) : py;
        KAI_TRY(launch_im2col_rows(col, col_lo, padded, px, d, s));
        KAI_TRY(conv_gemm(st, device, KAI_GEMM_NT, tmp, pk, col, ychn, M, K, s, col_lo));
        if (ndat > 1) KAI_TRY(launch_swap01(py, tmp, ychn, ndat, yh * yw, st->sm_count, s));
        return KAI_OK;
    }
    if (!d.plain()) return 1;
    KAI_TRY(ensure_workspace(st, device, col_bytes + tmp_bytes + 256 + gemm_tc_scratch_bound(ychn, M, K)));
    FrontGuard front(st, col_bytes + tmp_bytes);
    float* col = static_cast<float*>(st->ws);
    float* tmp = (ndat > 1) ? reinterpret_cast<float*>(static_cast<uint8_t*>(st->ws) + col_bytes) : py;
    KAI_TRY(launch_im2col(col, px, d, s));
    KAI_TRY(conv_gemm(st, device, KAI_GEMM_NN, tmp, pk, col, ychn, M, K, s));   // [ychn][ndat][pix]
    if (ndat > 1) KAI_TRY(launch_swap01(py, tmp, ychn, ndat, yh * yw, st->sm_count, s));
    return KAI_OK;
}

int conv2d_backward_x(DeviceState* st, int device, float* pgx, const float* pgy, const float* pk, int64_t ndat,
                      int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                      int64_t group, int64_t ph, int64_t pw, int64_t gh, int64_t gw, cudaStream_t s) {
    if (group != 1) {
        if (options().conv_direct.load() != 0) {
            const int64_t size = ndat * xchn * xh * xw;
            conv2d_backward_x_generic_kernel<<<static_cast<unsigned>((size + 255) / 256), 256, 0, s>>>(
                pgx, pgy, pk, size, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw);
            count_launch();
            return check_launch("conv2d_backward_x_generic_kernel");
        }
        // the input gradient over xchn / group summed channels, then every channel takes its group's gradient
        const int64_t kchn = xchn / group, total = ndat * kchn * xh * xw;
        KAI_TRY(ensure_aux(st, total * 4));
        float* gxs = static_cast<float*>(st->aux);
        KAI_TRY(conv2d_backward_x(st, device, gxs, pgy, pk, ndat, kchn, xh, xw, ychn, yh, yw, kh, kw, 1, ph, pw, gh, gw, s));
        const int64_t full = ndat * xchn * xh * xw;
        group_broadcast_kernel<<<blocks_for(full), 256, 0, s>>>(pgx, gxs, full, xh * xw, xchn, static_cast<int>(group));
        count_launch();
        return check_launch("group_broadcast_kernel");
    }
    const int64_t M = ndat * xh * xw, K = ychn * kh * kw;
    const ConvDims d{ndat, ychn, yh, yw, xh, xw, kh, kw, ph, pw, 1, gh, gw};
    const int64_t kt_bytes = al256(xchn * K * 4);
    if (igemm_tma_ok(d, xchn)) return run_igemm_tma(st, device, pgx, pgy, pk, kh * kw, xchn * kh * kw, d, xchn, s);
    if (igemm_ok(d, xchn)) {
        KAI_TRY(ensure_workspace(st, device, kt_bytes + igemm_front_bytes(d, xchn) + 256));
        float* kt2 = static_cast<float*>(st->ws);
        KAI_TRY(launch_swap01(kt2, pk, ychn, xchn, kh * kw, st->sm_count, s));     // k[yn][xn][.] -> kT[xn][yn][.]
        return run_igemm(st, device, pgx, pgy, kt2, d, xchn, kt_bytes, s);
    }
    const bool rows = rows_form_ok(d);
    const int64_t col_bytes = al256(K * M * 4) * (rows ? 2 : 1), tmp_bytes = (ndat > 1) ? al256(xchn * M * 4) : 0;
    const int64_t pad_bytes = rows ? padded_bytes(d) : 0;
    KAI_TRY(ensure_workspace(st, device, col_bytes + tmp_bytes + kt_bytes + pad_bytes + 256 + gemm_tc_scratch_bound(xchn, M, K)));
    FrontGuard front(st, col_bytes + tmp_bytes + kt_bytes + pad_bytes);
    uint8_t* base = static_cast<uint8_t*>(st->ws);
    float* col = reinterpret_cast<float*>(base);
    float* col_lo = rows ? reinterpret_cast<float*>(base + col_bytes / 2) : nullptr;
    float* kt = reinterpret_cast<float*>(base + col_bytes);
    float* padded = reinterpret_cast<float*>(base + col_bytes + kt_bytes);
    float* tmp = (ndat > 1) ? reinterpret_cast<float*>(base + col_bytes + kt_bytes + pad_bytes) : pgx;
    KAI_TRY(launch_swap01(kt, pk, ychn, xchn, kh * kw, st->sm_count, s));          // k[yn][xn][.] -> kT[xn][yn][.]
    if (rows) {
        KAI_TRY(launch_im2col_rows(col, col_lo, padded, pgy, d, s));
        KAI_TRY(conv_gemm(st, device, KAI_GEMM_NT, tmp, kt, col, xchn, M, K, s, col_lo));
    } else {
        KAI_TRY(launch_im2col(col, pgy, d, s));
        KAI_TRY(conv_gemm(st, device, KAI_GEMM_NN, tmp, kt, col, xchn, M, K, s));  // [xchn][ndat][pix]
    }
    if (ndat > 1) KAI_TRY(launch_swap01(pgx, tmp, xchn, ndat, xh * xw, st->sm_count, s));
    return KAI_OK;
}

int conv2d_backward_k(DeviceState* st, int device, float* pgk, const float* pgy, const float* px, int64_t ndat,
                      int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                      int64_t group, int64_t ph, int64_t pw, int64_t gh, int64_t gw, cudaStream_t s) {
    if (group != 1) {
        if (options().conv_direct.load() != 0) {
            const int64_t size = kh * kw * (xchn / group) * ychn;
            conv2d_backward_k_generic_kernel<<<static_cast<unsigned>((size + 255) / 256), 256, 0, s>>>(
                pgk, pgy, px, size, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw);
            count_launch();
            return check_launch("conv2d_backward_k_generic_kernel");
        }
        const int64_t kchn = xchn / group, total = ndat * kchn * xh * xw;
        KAI_TRY(ensure_aux(st, total * 4));
        float* xs = static_cast<float*>(st->aux);
        group_sum_kernel<<<blocks_for(total), 256, 0, s>>>(xs, px, total, xh * xw, static_cast<int>(group));
        count_launch();
        KAI_TRY(check_launch("group_sum_kernel"));
        return conv2d_backward_k(st, device, pgk, pgy, xs, ndat, kchn, xh, xw, ychn, yh, yw, kh, kw, 1, ph, pw, gh, gw, s);
    }
    {
        const int rc = conv_wgrad_taps(st, device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, ph, pw, gh, gw, s);
        if (rc != 1) return rc;     // 1 = shape outside the tap-row path: explicit unfolding below
    }
    const int64_t M = ndat * yh * yw, K = xchn * kh * kw;      // reduction over M
    const bool with_lo = (M & 3) == 0;                         // unfolding writes the lo plane of colT as well
    const int64_t col_bytes = al256(K * M * 4), gyp_bytes = (ndat > 1) ? al256(ychn * M * 4) : 0;
    const int64_t lo_bytes = with_lo ? col_bytes : 0;
    KAI_TRY(ensure_workspace(st, device, col_bytes + lo_bytes + gyp_bytes + 256 + gemm_tc_scratch_bound(ychn, K, M)));
    FrontGuard front(st, col_bytes + lo_bytes + gyp_bytes);
    uint8_t* base = static_cast<uint8_t*>(st->ws);
    float* col = reinterpret_cast<float*>(base);
    float* col_lo = with_lo ? reinterpret_cast<float*>(base + col_bytes) : nullptr;
    const float* gyp = pgy;
    if (ndat > 1) {
        float* t = reinterpret_cast<float*>(base + col_bytes + lo_bytes);
        KAI_TRY(launch_swap01(t, pgy, ndat, ychn, yh * yw, st->sm_count, s));      // [nd][yn][pix] -> [yn][nd][pix]
        gyp = t;
    }
    const ConvDims d{ndat, xchn, xh, xw, yh, yw, kh, kw, ph, pw, 0, gh, gw};
    KAI_TRY(launch_im2col(col, px, d, s, col_lo));
    return conv_gemm(st, device, KAI_GEMM_NT, pgk, gyp, col, ychn, K, M, s, col_lo);       // gk[ychn][(xn,kr,kc)]
}

// The transposed family on the GEMM kernels.  Returns 1 when a shape is outside what the unfolding path takes.
//   forward       repeat rows / columns of x (see repeat_rows_cols_kernel), flip the kernel, plain conv2d;
//   backward_x    gx[nd,xn,xr,xc] = sum gy[nd,yn, xr*sh + kr - bh + (sh-1)/2, ...] k[yn,xn,kr,kc], the position tested
//                 against xh / xw as the reference does (vmath.cu:3840-3846): a convolution of the top-left xh x xw
//                 window of gy with stride (sh, sw) and the kernel's two channel axes exchanged;
//   backward_k    gk[yn,xn,kr,kc] = sum_m gy(same positions) x[m, xn]: the same strided unfolding of gy, contracted
//                 with the channel-major copy of x over m = (image, pixel).
static int conv2d_transposed_gemm(DeviceState* st, int device, int which, float* out, const float* first,
                                  const float* second, int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn,
                                  int64_t kh, int64_t kw, int64_t sh, int64_t sw, cudaStream_t s) {
    const int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    const int64_t offh = bh - (sh - 1) / 2, offw = bw - (sw - 1) / 2;
    if (ychn * xchn > 65535 || ndat * xchn > 65535 || ndat * ychn > 65535) return 1;     // row-permutation kernel's grid limit
    if (which == 0) {
        const int64_t ah = (kh - 1) - offh, aw = (kw - 1) - offw;          // >= 0: offh <= bh <= kh - 1
        const int64_t h0 = (sh - 1 < ah) ? sh - 1 : ah, w0 = (sw - 1 < aw) ? sw - 1 : aw;
        const int64_t vh = yh + h0, vw = yw + w0;
        const int64_t v_count = ndat * xchn * vh * vw, k_count = ychn * xchn * kh * kw;
        if (vh > 16384 || vw > 16384) return 1;
        KAI_TRY(ensure_aux(st, al256(v_count * 4) + k_count * 4));
        float* v = static_cast<float*>(st->aux);
        float* kf = reinterpret_cast<float*>(static_cast<uint8_t*>(st->aux) + al256(v_count * 4));
        repeat_rows_cols_kernel<<<blocks_for(v_count), 256, 0, s>>>(v, first, v_count, static_cast<int>(xh), static_cast<int>(xw),
                                                                   static_cast<int>(sh), static_cast<int>(sw), static_cast<int>(h0),
                                                                   static_cast<int>(w0), static_cast<int>(vh), static_cast<int>(vw));
        count_launch();
        KAI_TRY(check_launch("repeat_rows_cols_kernel"));
        flip_taps_kernel<<<blocks_for(k_count), 256, 0, s>>>(kf, second, k_count, static_cast<int>(kh), static_cast<int>(kw));
        count_launch();
        KAI_TRY(check_launch("flip_taps_kernel"));
        return conv2d_forward(st, device, out, v, kf, ndat, ychn, yh, yw, xchn, vh, vw, kh, kw, 1, ah - h0, aw - w0, 1, 1, s,
                              1, 1, 0, 0);
    }
    if (which == 1) {
        const int64_t k_count = ychn * xchn * kh * kw;
        KAI_TRY(ensure_aux(st, k_count * 4));
        float* w2 = static_cast<float*>(st->aux);
        KAI_TRY(launch_swap01(w2, second, ychn, xchn, kh * kw, st->sm_count, s));      // k[yn][xn][.] -> [xn][yn][.]
        // source = gy (ychn channels, planes yh x yw, valid window xh x xw), outputs on the xh x xw grid with stride
        return conv2d_forward(st, device, out, first, w2, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, 1, offh, offw, 1, 1, s, sh,
                              sw, xh, xw);
    }
    ConvDims d{ndat, ychn, yh, yw, xh, xw, kh, kw, offh, offw, 0, 1, 1};
    d.strh = sh; d.strw = sw; d.vh = xh; d.vw = xw;
    if (!rows_form_ok(d)) return 1;
    const int64_t M = ndat * xh * xw, K = ychn * kh * kw;
    const int64_t xcm_bytes = al256(xchn * M * 4), res_bytes = al256(xchn * K * 4);
    KAI_TRY(ensure_aux(st, xcm_bytes + res_bytes));
    float* xcm = static_cast<float*>(st->aux);
    float* res = reinterpret_cast<float*>(static_cast<uint8_t*>(st->aux) + xcm_bytes);
    const int64_t col_bytes = al256(K * M * 4), pad_bytes = padded_bytes(d);
    KAI_TRY(ensure_workspace(st, device, 2 * col_bytes + pad_bytes + 256 + gemm_tc_scratch_bound(xchn, K, M)));
    FrontGuard front(st, 2 * col_bytes + pad_bytes);
    uint8_t* base = static_cast<uint8_t*>(st->ws);
    float* col = reinterpret_cast<float*>(base);
    float* col_lo = reinterpret_cast<float*>(base + col_bytes);
    float* padded = reinterpret_cast<float*>(base + 2 * col_bytes);
    const float* xsrc = second;
    if (ndat > 1) {
        KAI_TRY(launch_swap01(xcm, second, ndat, xchn, xh * xw, st->sm_count, s));      // [nd][xn][pix] -> [xn][nd][pix]
        xsrc = xcm;
    }
    KAI_TRY(launch_im2col_rows(col, col_lo, padded, first, d, s));
    KAI_TRY(conv_gemm(st, device, KAI_GEMM_NN, res, xsrc, col, xchn, K, M, s));        // res[xn][(yn,kr,kc)]
    return launch_swap01(out, res, xchn, ychn, kh * kw, st->sm_count, s);              // -> gk[yn][xn][kr][kc]
}

// which: 0 forward, 1 backward_x, 2 backward_k
int conv2d_transposed_any(DeviceState* st, int device, int which, float* out, const float* first, const float* second,
                          int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                          int64_t sh, int64_t sw, cudaStream_t s) {
    const int64_t size = which == 0 ? ndat * ychn * xh * sh * xw * sw : which == 1 ? ndat * xchn * xh * xw : ychn * xchn * kh * kw;
    if (size == 0) return KAI_OK;
    if (size > (int64_t(1) << 39)) return fail(KAI_E_TOO_LARGE, "conv2d_transposed: output too large");
    if (options().conv_direct.load() == 0 && ndat * xchn * xh * xw > 0 && ychn > 0) {
        const int rc = conv2d_transposed_gemm(st, device, which, out, first, second, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, s);
        if (rc != 1) return rc;     // 1 = shape outside the unfolding path: the per-output kernels below take it
    }
    const unsigned blocks = static_cast<unsigned>((size + 255) / 256);
    if (which == 0) conv2d_transposed_kernel<<<blocks, 256, 0, s>>>(out, first, second, size, xchn, xh, xw, ychn, kh, kw, sh, sw);
    else if (which == 1) conv2d_transposed_backward_x_kernel<<<blocks, 256, 0, s>>>(out, first, second, size, xchn, xh, xw, ychn, kh, kw, sh, sw);
    else conv2d_transposed_backward_k_kernel<<<blocks, 256, 0, s>>>(out, first, second, size, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw);
    count_launch();
    return check_launch("conv2d_transposed kernels");
}

}  // namespace kai
