/*
 * TEST INFRASTRUCTURE -- not product code.  Nothing under the package may include, link or
 * call this file; only tests/, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * CPU restatement, in plain C, of the reference engine's host loops for the matmul / Linear
 * path (konantech-ai/deep-learning-framework, source/engine/support/vmath.cu).  Each function
 * names the lines it follows.  Loop order, the order of floating-point operations and the
 * libm calls are the reference's, and the file is compiled with -ffp-contract=off (the
 * reference builds with -fmad=false / -ffp-contract=off, engine/CMakeLists.txt:189-208), so
 * the results are bit-identical to the reference's `device = -1` branch.  That identity is
 * checked by tests/test_oracle.py against the reference itself (oracle/_ref, built from the
 * reference sources by oracle/build_ref.sh) whenever that library is present, and against the
 * committed vectors under tests/golden/ (generated from the reference) everywhere.
 *
 * The reference ships no golden vectors or known-answer tests of its own for this path.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>

#define HYPER_ACCESS(x) ((x) ? *(x) : 0)   /* local_objects/vhypermanager.h:9 */

/* vmath.cu:2961-2977  matmul_host: py[nd,ny] (+)= sum_nx pw[ny,nx] * px[nd,nx] */
void orc_matmul(float* py, const float* pw, const float* px, int64_t yvec, int64_t ndat, int64_t xvec, int acc) {
    for (int64_t nd = 0, n = 0; nd < ndat; nd++) {
        for (int64_t ny = 0; ny < yvec; ny++, n++) {
            float dotsum = 0;
            int64_t wpos = ny * xvec;
            int64_t xpos = nd * xvec;
            for (int64_t nx = 0; nx < xvec; nx++) dotsum += pw[wpos++] * px[xpos++];
            if (acc) py[n] += dotsum; else py[n] = dotsum;
        }
    }
}

/* vmath.cu:3007-3022  matmul_backward_x_host: pgx[nd,nx] (+)= sum_ny pw[ny,nx] * pgy[nd,ny] */
void orc_matmul_backward_x(float* pgx, const float* pgy, const float* pw, int64_t yvec, int64_t ndat, int64_t xvec,
                           int acc) {
    for (int64_t nd = 0, n = 0; nd < ndat; nd++) {
        for (int64_t nx = 0; nx < xvec; nx++, n++) {
            float dotsum = 0;
            for (int64_t ny = 0; ny < yvec; ny++) dotsum += pw[ny * xvec + nx] * pgy[nd * yvec + ny];
            if (acc) pgx[n] += dotsum; else pgx[n] = dotsum;
        }
    }
}

/* vmath.cu:3051-3067  matmul_backward_w_host: pgw[ny,nx] (+)= sum_nd px[nd,nx] * pgy[nd,ny] */
void orc_matmul_backward_w(float* pgw, const float* pgy, const float* px, int64_t yvec, int64_t ndat, int64_t xvec,
                           int acc) {
    for (int64_t ny = 0, n = 0; ny < yvec; ny++) {
        for (int64_t nx = 0; nx < xvec; nx++, n++) {
            float dotsum = 0;
            for (int64_t nd = 0; nd < ndat; nd++) dotsum += px[nd * xvec + nx] * pgy[nd * yvec + ny];
            if (acc) pgw[n] += dotsum; else pgw[n] = dotsum;
        }
    }
}

/* vmath.cu:875-881  add_bias_host */
void orc_add_bias(float* py, const float* pa, const float* pb, int64_t nrow, int64_t ncol) {
    for (int64_t nr = 0; nr < nrow; nr++)
        for (int64_t nc = 0; nc < ncol; nc++) py[nr * ncol + nc] = pa[nr * ncol + nc] + pb[nc];
}

/* vmath.cu:901-911  add_bias_backward_b_host */
void orc_add_bias_backward_b(float* pgb, const float* pgy, int64_t nrow, int64_t ncol, int acc) {
    for (int64_t nc = 0; nc < ncol; nc++) {
        float sum = 0;
        for (int64_t nr = 0; nr < nrow; nr++) sum += pgy[nr * ncol + nc];
        if (acc) pgb[nc] += sum; else pgb[nc] = sum;
    }
}

/* vmath.cu:297-311 */
static float orc_sigmoid(float x) { return (x > 0) ? (1.0f / (1.0f + expf(-x))) : (expf(x) / (expf(x) + 1.0f)); }
static float orc_tanh(float x) { return 2 * orc_sigmoid(2 * x) - 1; }

/* vmath.cu:3097-3167  activate_host; returns -1 for an unknown function (the reference throws) */
int orc_activate(float* py, const float* px, int64_t nrow, int64_t ncol, int actFunc, const float* hLeakyAlpha) {
    float leaky_alpha = HYPER_ACCESS(hLeakyAlpha);
    for (int64_t nr = 0, n = 0; nr < nrow; nr++) {
        for (int64_t nc = 0; nc < ncol; nc++, n++) {
            float x = px[n];
            float y, t;
            switch (actFunc) {
            case 0: y = x; break;
            case 1: y = (x > 0) ? x : 0; break;
            case 2: y = (x > 0) ? x : x * leaky_alpha; break;
            case 3: y = orc_sigmoid(x); break;
            case 4: y = orc_tanh(x); break;
            case 5: y = x * 0.5f * (1.0f + erff(x / sqrtf(2.0f))); break;
            case 6: {
                float lambda = 1.0507009f, alpha = 1.6732632f;
                y = (x > 0) ? lambda * x : lambda * alpha * (expf(x) - 1);
            } break;
            case 7:
                t = logf(1.0f + expf(x)) * 2;
                t = (float)((t > 0) ? ((1.0f - expf(-t)) / (1.0f + expf(-t))) : ((expf(t) - 1.0f) / (expf(t) + 1.0f)));
                y = x * t;
                break;
            case 8:
                t = (float)((x > 0) ? (1.0f / (1.0f + expf(-x))) : (expf(x) / (expf(x) + 1.0f)));
                y = x * t;
                break;
            case 9: {
                /* Row softmax.  The reference forms the row base as `px - (n % ncol)` (vmath.cu:3145,
                 * 3218) with px the ARRAY base, which reads in front of the array for every column
                 * but the first; the intended row base `px + n - n % ncol` is used here, and this
                 * one case is therefore never compared with the compiled reference. */
                float max_term = -FLT_MAX, exp_sum = 0;
                const float* pp = px + (n - n % ncol);
                for (int64_t nn = 0; nn < ncol; nn++) if (pp[nn] > max_term) max_term = pp[nn];
                for (int64_t nn = 0; nn < ncol; nn++) exp_sum += expf(pp[nn] - max_term);
                y = expf(x - max_term) / exp_sum;
            } break;
            default: return -1;
            }
            py[n] = y;
        }
    }
    return 0;
}

/* vmath.cu:3247-3330  activate_backward_host (px = pre-activation) */
int orc_activate_backward(float* pgx, const float* pgy, const float* px, int64_t nrow, int64_t ncol, int actFunc,
                          const float* hLeakyAlpha) {
    float leaky_alpha = HYPER_ACCESS(hLeakyAlpha);
    const long double PI_L = 3.1415926535897931L;
    for (int64_t n = 0; n < nrow * ncol; n++) {
        float gy = pgy[n], x = px[n];
        float gx, y, s, t, u, v;
        switch (actFunc) {
        case 0: gx = 1.0f; break;
        case 1: gx = (x > 0) ? 1.0f : 0.0f; break;
        case 2: gx = (x > 0) ? 1.0f : leaky_alpha; break;
        case 3: y = orc_sigmoid(x); gx = y * (1.0f - y); break;
        case 4: y = orc_tanh(x); gx = 1.0f - y * y; break;
        case 5:
            s = 0.5f * (1.0f + erff(x / sqrtf(2.0f)));
            t = 0.5f * x * sqrtf(2.0f / (float)PI_L) * expf(-x * x / 2.0f);
            gx = s + t;
            break;
        case 6: {
            float lambda = 1.0507009f, alpha = 1.6732632f;
            gx = (x > 0) ? lambda : lambda * alpha * expf(x);
        } break;
        case 7:
            s = logf(1.0f + expf(x));
            t = (x > 0) ? (1.0f / (1.0f + expf(-x))) : (expf(x) / (1.0f + expf(x)));
            s = s * 2.0f;
            u = (float)((s > 0) ? ((1.0f - expf(-s)) / (1.0f + expf(-s))) : ((expf(s) - 1.0f) / (expf(s) + 1.0f)));
            v = (1.0f - u * u);
            gx = u + x * v * t;
            break;
        case 8:
            s = orc_sigmoid(x);
            t = s * (1.0f - s);
            gx = s + x * t;
            break;
        default: return -1;
        }
        pgx[n] = gx * gy;
    }
    return 0;
}

/* vmath.cu:3411-3444  activate_backward_with_y_host (py = output) */
int orc_activate_backward_with_y(float* pgx, const float* pgy, const float* py, int64_t nrow, int64_t ncol,
                                 int actFunc, const float* hLeakyAlpha) {
    float leaky_alpha = HYPER_ACCESS(hLeakyAlpha);
    for (int64_t n = 0; n < nrow * ncol; n++) {
        float gy = pgy[n], y = py[n], gx;
        switch (actFunc) {
        case 0: gx = 1.0f; break;
        case 1: gx = (y > 0) ? 1.0f : 0; break;
        case 2: gx = (y > 0) ? 1.0f : leaky_alpha; break;
        case 3: gx = y * (1 - y); break;
        case 4: gx = 1 - y * y; break;
        default: return -1;
        }
        pgx[n] = gx * gy;
    }
    return 0;
}

/* vmath.cu:6729-6750  mult_on_heads_host */
void orc_mult_on_heads(float* pp, const float* pK, const float* pQ, int64_t nbat, int64_t ntimes, int64_t nvec,
                       int64_t nhead, int64_t npiece, const float* hCoef) {
    float coef = HYPER_ACCESS(hCoef);
    for (int64_t nb = 0, n = 0; nb < nbat; nb++)
        for (int64_t nq = 0; nq < ntimes; nq++)
            for (int64_t nk = 0; nk < ntimes; nk++)
                for (int64_t nh = 0; nh < nhead; nh++, n++) {
                    int64_t kpos = (nb * ntimes + nk) * nvec + nh * npiece;
                    int64_t qpos = (nb * ntimes + nq) * nvec + nh * npiece;
                    float sum = 0;
                    for (int64_t np = 0; np < npiece; np++) sum += pK[kpos++] * pQ[qpos++];
                    pp[n] = sum * coef;
                }
}

/* vmath.cu:6833-6845  set_mh_attention_mask_host */
void orc_set_mh_attention_mask(float* pp, int64_t ndat, int64_t ntimes, int64_t nhead, int forward) {
    for (int64_t nd = 0; nd < ndat; nd++)
        for (int64_t nh = 0; nh < nhead; nh++)
            for (int64_t nq = 0; nq < ntimes; nq++)
                for (int64_t nk = nq + 1; nk < ntimes; nk++)
                    pp[((nd * ntimes + nq) * ntimes + nk) * nhead + nh] = forward ? -INFINITY : 0;
}

/* vmath.cu:6864-6885  softmax_direct_on_axis_host */
void orc_softmax_direct_on_axis(float* pp, int64_t nrow, int64_t nvec, int64_t ncol) {
    for (int64_t nr = 0; nr < nrow; nr++)
        for (int64_t nc = 0; nc < ncol; nc++) {
            float max_term = -FLT_MAX, exp_sum = 0;
            int64_t ppos0 = nr * nvec * ncol + nc;
            for (int64_t nv = 0, ppos = ppos0; nv < nvec; nv++, ppos += ncol)
                if (pp[ppos] > max_term) max_term = pp[ppos];
            for (int64_t nv = 0, ppos = ppos0; nv < nvec; nv++, ppos += ncol) exp_sum += expf(pp[ppos] - max_term);
            for (int64_t nv = 0, ppos = ppos0; nv < nvec; nv++, ppos += ncol)
                pp[ppos] = expf(pp[ppos] - max_term) / exp_sum;
        }
}

/* vmath.cu:6977-6997  mix_values_host */
void orc_mix_values(float* py, const float* pp, const float* pV, int64_t nbat, int64_t ntimes, int64_t nvec,
                    int64_t nhead, int64_t npiece) {
    for (int64_t nb = 0; nb < nbat; nb++)
        for (int64_t nq = 0; nq < ntimes; nq++)
            for (int64_t nh = 0; nh < nhead; nh++)
                for (int64_t np = 0; np < npiece; np++) {
                    float sum = 0;
                    for (int64_t nk = 0; nk < ntimes; nk++)
                        sum += pp[((nb * ntimes + nq) * ntimes + nk) * nhead + nh] *
                               pV[(nb * ntimes + nk) * nvec + nh * npiece + np];
                    py[(((nb * ntimes) + nq) * nhead + nh) * npiece + np] = sum;
                }
}

/* vmath.cu:6782-6801  mult_on_heads_backward_host (called once per operand, vtensor.cpp:3153-3154) */
void orc_mult_on_heads_backward(float* pgQK, const float* pgp, const float* pKQ, int64_t nbat, int64_t ntimes,
                                int64_t nvec, int64_t nhead, int64_t npiece) {
    for (int64_t nb = 0; nb < nbat; nb++)
        for (int64_t nt = 0; nt < ntimes; nt++)
            for (int64_t nh = 0; nh < nhead; nh++)
                for (int64_t np = 0; np < npiece; np++) {
                    float sum = 0;
                    for (int64_t nk = 0; nk < ntimes; nk++)
                        sum += pgp[((nb * ntimes + nt) * ntimes + nk) * nhead + nh] *
                               pKQ[(nb * ntimes + nk) * nvec + nh * npiece + np];
                    pgQK[(nb * ntimes + nt) * nvec + nh * npiece + np] = sum;
                }
}

/* vmath.cu:6919-6943  softmax_direct_on_axis_backward_host (in place on pgp) */
void orc_softmax_direct_on_axis_backward(float* pgp, const float* pp, int64_t nbat, int64_t ntimes, int64_t nhead,
                                         const float* hCoef) {
    float coef = HYPER_ACCESS(hCoef);
    for (int64_t nb = 0; nb < nbat; nb++)
        for (int64_t nq = 0; nq < ntimes; nq++)
            for (int64_t nh = 0; nh < nhead; nh++) {
                int64_t p0 = ((nb * ntimes + nq) * ntimes) * nhead + nh;
                float sum = 0;
                for (int64_t nk = 0, ppos = p0; nk < ntimes; nk++, ppos += nhead) sum += pp[ppos] * pgp[ppos];
                for (int64_t nk = 0, ppos = p0; nk < ntimes; nk++, ppos += nhead)
                    pgp[ppos] = coef * pp[ppos] * (pgp[ppos] - sum);
            }
}

/* vmath.cu:7028-7049  mix_values_backward_prop_host */
void orc_mix_values_backward_prop(float* pgp, const float* pgy, const float* pV, int64_t nbat, int64_t ntimes,
                                  int64_t nvec, int64_t nhead, int64_t npiece) {
    for (int64_t nb = 0, n = 0; nb < nbat; nb++)
        for (int64_t nq = 0; nq < ntimes; nq++)
            for (int64_t nk = 0; nk < ntimes; nk++)
                for (int64_t nh = 0; nh < nhead; nh++, n++) {
                    int64_t ypos = ((nb * ntimes + nq) * nhead + nh) * npiece;
                    int64_t vpos = (nb * ntimes + nk) * nvec + nh * npiece;
                    float sum = 0;
                    for (int64_t np = 0; np < npiece; np++) sum += pgy[ypos++] * pV[vpos++];
                    pgp[n] = sum;
                }
}

/* vmath.cu:7080-7101  mix_values_backward_value_host */
void orc_mix_values_backward_value(float* pgV, const float* pgy, const float* pp, int64_t nbat, int64_t ntimes,
                                   int64_t nvec, int64_t nhead, int64_t npiece) {
    for (int64_t nb = 0; nb < nbat; nb++)
        for (int64_t nk = 0; nk < ntimes; nk++)
            for (int64_t nh = 0; nh < nhead; nh++)
                for (int64_t np = 0; np < npiece; np++) {
                    float sum = 0;
                    for (int64_t nq = 0; nq < ntimes; nq++)
                        sum += pp[((nb * ntimes + nq) * ntimes + nk) * nhead + nh] *
                               pgy[((nb * ntimes + nq) * nhead + nh) * npiece + np];
                    pgV[(nb * ntimes + nk) * nvec + nh * npiece + np] = sum;
                }
}

/* vmath.cu:3490-3529  conv2d_host (NCHW, stride 1, zero padding; every input channel xn is summed
 * with kernel channel xn / group, as the reference does) */
void orc_conv2d(float* py, const float* px, const float* pk, int64_t ndat, int64_t ychn, int64_t yh, int64_t yw,
                int64_t xchn, int64_t xh, int64_t xw, int64_t kh, int64_t kw, int64_t group, int64_t ph, int64_t pw) {
    int64_t kchn = xchn / group;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t yn = 0; yn < ychn; yn++)
            for (int64_t yr = 0; yr < yh; yr++)
                for (int64_t yc = 0; yc < yw; yc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++)
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t xr = yr + (kr - ph), xc = yc + (kc - pw);
                            if (xr < 0 || xr >= xh || xc < 0 || xc >= xw) continue;
                            for (int64_t xn = 0; xn < xchn; xn++)
                                sum += px[((nd * xchn + xn) * xh + xr) * xw + xc] *
                                       pk[((yn * kchn + (xn / group)) * kh + kr) * kw + kc];
                        }
                    py[n] = sum;
                }
}

/* vmath.cu:3580-3611  conv2d_backward_x_host */
void orc_conv2d_backward_x(float* pgx, const float* pgy, const float* pk, int64_t ndat, int64_t xchn, int64_t xh,
                           int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw, int64_t group,
                           int64_t ph, int64_t pw) {
    int64_t kchn = xchn / group;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t xn = 0; xn < xchn; xn++)
            for (int64_t xr = 0; xr < xh; xr++)
                for (int64_t xc = 0; xc < xw; xc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++) {
                        int64_t yr = xr - (kr - ph);
                        if (yr < 0 || yr >= yh) continue;
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t yc = xc - (kc - pw);
                            if (yc < 0 || yc >= yw) continue;
                            for (int64_t yn = 0; yn < ychn; yn++)
                                sum += pgy[((nd * ychn + yn) * yh + yr) * yw + yc] *
                                       pk[((yn * kchn + (xn / group)) * kh + kr) * kw + kc];
                        }
                    }
                    pgx[n] = sum;
                }
}

/* vmath.cu:3659-3695  conv2d_backward_k_host, with the column offset of the reference's device kernel
 * (vmath.cu:3717: yc = xc - (kc - pw)); the host loop writes `kc - yw` there (vmath.cu:3676), which
 * only agrees when yw == pw. */
void orc_conv2d_backward_k(float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn, int64_t xh,
                           int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw, int64_t group,
                           int64_t ph, int64_t pw) {
    int64_t kchn = xchn / group;
    for (int64_t kr = 0; kr < kh; kr++)
        for (int64_t kc = 0; kc < kw; kc++)
            for (int64_t kn = 0; kn < kchn; kn++)
                for (int64_t yn = 0; yn < ychn; yn++) {
                    float sum = 0;
                    for (int64_t xr = 0; xr < xh; xr++) {
                        int64_t yr = xr - (kr - ph);
                        if (yr < 0 || yr >= yh) continue;
                        for (int64_t xc = 0; xc < xw; xc++) {
                            int64_t yc = xc - (kc - pw);
                            if (yc < 0 || yc >= yw) continue;
                            for (int64_t nd = 0; nd < ndat; nd++)
                                for (int64_t ng = 0; ng < group; ng++) {
                                    int64_t xn = kn * group + ng;
                                    sum += pgy[((nd * ychn + yn) * yh + yr) * yw + yc] *
                                           px[((nd * xchn + xn) * xh + xr) * xw + xc];
                                }
                        }
                    }
                    pgk[((yn * kchn + kn) * kh + kr) * kw + kc] = sum;
                }
}

/* vmath.cu:3748-3783  conv2d_transposed_host: output (xh*sh) x (xw*sw); the source position is the C integer
 * quotient (truncating toward zero) of the shifted output position by the stride, without a remainder test */
void orc_conv2d_transposed(float* py, const float* px, const float* pk, int64_t ndat, int64_t xchn, int64_t xh,
                           int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t sh, int64_t sw) {
    int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t yn = 0; yn < ychn; yn++)
            for (int64_t yr = 0; yr < yh; yr++)
                for (int64_t yc = 0; yc < yw; yc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++) {
                        int64_t xr = (yr - (kr - bh) - (sh - 1) / 2) / sh;
                        if (xr < 0 || xr >= xh) continue;
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t xc = (yc - (kc - bw) - (sw - 1) / 2) / sw;
                            if (xc < 0 || xc >= xw) continue;
                            for (int64_t xn = 0; xn < xchn; xn++)
                                sum += px[((nd * xchn + xn) * xh + xr) * xw + xc] * pk[((yn * xchn + xn) * kh + kr) * kw + kc];
                        }
                    }
                    py[n] = sum;
                }
}

/* vmath.cu:3828-3861  conv2d_transposed_backward_x_host (bounds tested against xh / xw, as the reference does) */
void orc_conv2d_transposed_backward_x(float* pgx, const float* pgy, const float* pk, int64_t ndat, int64_t xchn,
                                      int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t sh,
                                      int64_t sw) {
    int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t xn = 0; xn < xchn; xn++)
            for (int64_t xr = 0; xr < xh; xr++)
                for (int64_t xc = 0; xc < xw; xc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++) {
                        int64_t yr = xr * sh + (kr - bh) + (sh - 1) / 2;
                        if (yr < 0 || yr >= xh) continue;
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t yc = xc * sw + (kc - bw) + (sw - 1) / 2;
                            if (yc < 0 || yc >= xw) continue;
                            for (int64_t yn = 0; yn < ychn; yn++)
                                sum += pgy[((nd * ychn + yn) * yh + yr) * yw + yc] * pk[((yn * xchn + xn) * kh + kr) * kw + kc];
                        }
                    }
                    pgx[n] = sum;
                }
}

/* vmath.cu:3909-3944  conv2d_transposed_backward_k_host */
void orc_conv2d_transposed_backward_k(float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn,
                                      int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t sh,
                                      int64_t sw) {
    int64_t yh = xh * sh, yw = xw * sw, bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t kr = 0; kr < kh; kr++)
        for (int64_t kc = 0; kc < kw; kc++)
            for (int64_t xn = 0; xn < xchn; xn++)
                for (int64_t yn = 0; yn < ychn; yn++) {
                    float sum = 0;
                    for (int64_t xr = 0; xr < xh; xr++) {
                        int64_t yr = xr * sh + (kr - bh) + (sh - 1) / 2;
                        if (yr < 0 || yr >= xh) continue;
                        for (int64_t xc = 0; xc < xw; xc++) {
                            int64_t yc = xc * sw + (kc - bw) + (sw - 1) / 2;
                            if (yc < 0 || yc >= xw) continue;
                            for (int64_t nd = 0; nd < ndat; nd++)
                                sum += pgy[((nd * ychn + yn) * yh + yr) * yw + yc] * px[((nd * xchn + xn) * xh + xr) * xw + xc];
                        }
                    }
                    pgk[((yn * xchn + xn) * kh + kr) * kw + kc] = sum;
                }
}

/* vmath.cu:3992-4023  conv2d_dilated_host: same-size output, taps (kr - (kh-1)/2) * gh apart */
void orc_conv2d_dilated(float* py, const float* px, const float* pk, int64_t ndat, int64_t xchn, int64_t xh,
                        int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh, int64_t gw) {
    int64_t bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t yn = 0; yn < ychn; yn++)
            for (int64_t yr = 0; yr < xh; yr++)
                for (int64_t yc = 0; yc < xw; yc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++) {
                        int64_t xr = yr + (kr - bh) * gh;
                        if (xr < 0 || xr >= xh) continue;
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t xc = yc + (kc - bw) * gw;
                            if (xc < 0 || xc >= xw) continue;
                            for (int64_t xn = 0; xn < xchn; xn++)
                                sum += px[((nd * xchn + xn) * xh + xr) * xw + xc] * pk[((yn * xchn + xn) * kh + kr) * kw + kc];
                        }
                    }
                    py[n] = sum;
                }
}

/* vmath.cu:4066-4097  conv2d_dilated_backward_x_host */
void orc_conv2d_dilated_backward_x(float* pgx, const float* pgy, const float* pk, int64_t ndat, int64_t xchn,
                                   int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh,
                                   int64_t gw) {
    int64_t bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t nd = 0, n = 0; nd < ndat; nd++)
        for (int64_t xn = 0; xn < xchn; xn++)
            for (int64_t xr = 0; xr < xh; xr++)
                for (int64_t xc = 0; xc < xw; xc++, n++) {
                    float sum = 0;
                    for (int64_t kr = 0; kr < kh; kr++) {
                        int64_t yr = xr - (kr - bh) * gh;
                        if (yr < 0 || yr >= xh) continue;
                        for (int64_t kc = 0; kc < kw; kc++) {
                            int64_t yc = xc - (kc - bw) * gw;
                            if (yc < 0 || yc >= xw) continue;
                            for (int64_t yn = 0; yn < ychn; yn++)
                                sum += pgy[((nd * ychn + yn) * xh + yr) * xw + yc] * pk[((yn * xchn + xn) * kh + kr) * kw + kc];
                        }
                    }
                    pgx[n] = sum;
                }
}

/* vmath.cu:4140-4173  conv2d_dilated_backward_k_host */
void orc_conv2d_dilated_backward_k(float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn,
                                   int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh,
                                   int64_t gw) {
    int64_t bh = (kh - 1) / 2, bw = (kw - 1) / 2;
    for (int64_t kr = 0; kr < kh; kr++)
        for (int64_t kc = 0; kc < kw; kc++)
            for (int64_t xn = 0; xn < xchn; xn++)
                for (int64_t yn = 0; yn < ychn; yn++) {
                    float sum = 0;
                    for (int64_t xr = 0; xr < xh; xr++) {
                        int64_t yr = xr - (kr - bh) * gh;
                        if (yr < 0 || yr >= xh) continue;
                        for (int64_t xc = 0; xc < xw; xc++) {
                            int64_t yc = xc - (kc - bw) * gw;
                            if (yc < 0 || yc >= xw) continue;
                            for (int64_t nd = 0; nd < ndat; nd++)
                                sum += pgy[((nd * ychn + yn) * xh + yr) * xw + yc] * px[((nd * xchn + xn) * xh + xr) * xw + xc];
                        }
                    }
                    pgk[((yn * xchn + xn) * kh + kr) * kw + kc] = sum;
                }
}

/* vmath.cu:8916-8936  softmax_idx_crossentropy_host; returns -1 on a label outside [0,ncol) */
int orc_softmax_idx_crossentropy(float* py, const float* px, const int* pc, int64_t nrow, int64_t ncol) {
    for (int64_t n = 0; n < nrow; n++) {
        if (pc[n] < 0 || pc[n] >= ncol) return -1;
        float max_term = px[n * ncol], exp_sum = 0;
        for (int64_t m = 0; m < ncol; m++) if (px[n * ncol + m] > max_term) max_term = px[n * ncol + m];
        for (int64_t m = 0; m < ncol; m++) exp_sum += expf(px[n * ncol + m] - max_term);
        float prob = expf(px[n * ncol + pc[n]] - max_term) / exp_sum;
        py[n] = -logf(prob + 1.0e-10f);
    }
    return 0;
}

/* vmath.cu:9022-9045  softmax_idx_crossentropy_backward_x_host */
void orc_softmax_idx_crossentropy_backward_x(float* pgx, const float* pgy, const float* px, const int* pz,
                                             int64_t nrow, int64_t ncol) {
    for (int64_t nr = 0; nr < nrow; nr++) {
        float* g = pgx + nr * ncol;
        const float* x = px + nr * ncol;
        float max_term = x[0], exp_sum = 0;
        for (int64_t m = 0; m < ncol; m++) if (x[m] > max_term) max_term = x[m];
        for (int64_t m = 0; m < ncol; m++) exp_sum += expf(x[m] - max_term);
        for (int64_t m = 0; m < ncol; m++) {
            g[m] = expf(x[m] - max_term) / exp_sum;
            if (m == pz[nr]) g[m] -= 1.0f;
            g[m] *= pgy[nr];
        }
    }
}

/* vmath.cu:9739-9743  sum_host */
void orc_sum(float* py, const float* px, int64_t nrow) {
    float sum = 0;
    for (int64_t n = 0; n < nrow; n++) sum += px[n];
    py[0] = sum;
}

/* vmath.cu:9761-9765  sum_backward_host */
void orc_sum_backward(float* pgx, const float* pgy, int64_t nrow) {
    for (int64_t n = 0; n < nrow; n++) pgx[n] = pgy ? pgy[0] : 1.0f;
}

/* vmath.cu:5977-6009  layernorm_host: per row, mean, then the mean of squared deviations, then
 * y = scale * ((x - avg) / std) with std = sqrtf(var + 1e-10f); ps keeps (avg, std) per row. */
void orc_layernorm(float* py, const float* px, float* ps, int64_t nrow, int64_t ncol, const float* hScale) {
    float scale = HYPER_ACCESS(hScale);
    for (int64_t nr = 0; nr < nrow; nr++) {
        float sum = 0;
        float dsqsum = 0;
        for (int64_t nc = 0; nc < ncol; nc++) sum += px[nr * ncol + nc];
        float avg = sum / ncol;
        for (int64_t nc = 0; nc < ncol; nc++) {
            float diff = px[nr * ncol + nc] - avg;
            dsqsum += diff * diff;
        }
        float var = dsqsum / ncol;
        float std = sqrtf(var + 1e-10f);
        for (int64_t nc = 0; nc < ncol; nc++) py[nr * ncol + nc] = scale * ((px[nr * ncol + nc] - avg) / std);
        ps[2 * nr + 0] = avg;
        ps[2 * nr + 1] = std;
    }
}

/* vmath.cu:6056-6067  layernorm_backward_host: the reference applies the forward's affine map to the
 * incoming gradient, pgx = scale * ((pgy - avg) / std), with the row statistics saved by the forward. */
void orc_layernorm_backward(float* pgx, const float* pgy, const float* ps, int64_t nrow, int64_t ncol,
                            const float* hScale) {
    float scale = HYPER_ACCESS(hScale);
    for (int64_t nr = 0, n = 0; nr < nrow; nr++) {
        for (int64_t nc = 0; nc < ncol; nc++, n++) {
            float avg = ps[2 * nr + 0];
            float std = ps[2 * nr + 1];
            pgx[n] = scale * ((pgy[n] - avg) / std);
        }
    }
}
