// See vmath_shim.h.  Plain C++ (no CUDA headers): everything device-side is behind the C ABI.
#include "vmath_shim.h"

#include "../../include/kai_b200.h"

namespace kai_shim {

namespace {

#ifndef KAI_SHIM_THROW
#define KAI_SHIM_THROW(code, status, text) throw VMathError((code), (status), (text))
#endif

// Non-zero status -> the exception VMath::cudaCheck would have raised.
inline void check(int rc) {
    if (rc == KAI_OK) return;
    std::string msg = kai_last_error_string();
    if (msg.compare(0, 5, "cuda:") != 0) msg = "cuda:" + msg;
    KAI_SHIM_THROW(rc == KAI_E_OUT_OF_RANGE ? kVerrOutOfRange : kVerrCudaError, rc, msg);
}

}  // namespace

void* VMath::mem_alloc(int device, int64 size) {
    void* p = nullptr;
    check(kai_mem_alloc(device, size, &p));
    return p;
}
void VMath::mem_free(int device, void* ptr) { check(kai_mem_free(device, ptr)); }

void VMath::add_bias(int device, float* py, float* pa, float* pb, int64 nrow, int64 ncol) {
    check(kai_add_bias(device, py, pa, pb, nrow, ncol, nullptr));
}
void VMath::add_bias_backward_b(int device, float* pgb, float* pgy, int64 nrow, int64 ncol, bool acc) {
    check(kai_add_bias_backward_b(device, pgb, pgy, nrow, ncol, acc, nullptr));
}

void VMath::layernorm(int device, float* py, float* px, float* ps, int64 nrow, int64 ncol, HYPER hScale) {
    check(kai_layernorm(device, py, px, ps, nrow, ncol, hScale, nullptr));
}
void VMath::layernorm_backward(int device, float* pgx, float* pgy, float* ps, int64 nrow, int64 ncol, HYPER hScale) {
    check(kai_layernorm_backward(device, pgx, pgy, ps, nrow, ncol, hScale, nullptr));
}

void VMath::matmul(int device, float* py, float* pw, float* px, int64 yvec, int64 ndat, int64 xvec, bool acc) {
    check(kai_matmul(device, py, pw, px, yvec, ndat, xvec, acc, nullptr));
}
void VMath::matmul_backward_x(int device, float* pgx, float* pgy, float* pw, int64 yvec, int64 ndat, int64 xvec, bool acc) {
    check(kai_matmul_backward_x(device, pgx, pgy, pw, yvec, ndat, xvec, acc, nullptr));
}
void VMath::matmul_backward_w(int device, float* pgw, float* pgy, float* px, int64 yvec, int64 ndat, int64 xvec, bool acc) {
    check(kai_matmul_backward_w(device, pgw, pgy, px, yvec, ndat, xvec, acc, nullptr));
}

void VMath::activate(int device, float* py, float* px, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha) {
    check(kai_activate(device, py, px, nrow, ncol, actFunc, hLeakyAlpha, nullptr));
}
void VMath::activate_backward(int device, float* pgx, float* pgy, float* px, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha) {
    check(kai_activate_backward(device, pgx, pgy, px, nrow, ncol, actFunc, hLeakyAlpha, nullptr));
}
void VMath::activate_backward_with_y(int device, float* pgx, float* pgy, float* py, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha) {
    check(kai_activate_backward_with_y(device, pgx, pgy, py, nrow, ncol, actFunc, hLeakyAlpha, nullptr));
}

void VMath::mult_on_heads(int device, float* pp, float* pK, float* pQ, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece, HYPER hCoef) {
    check(kai_mult_on_heads(device, pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, hCoef, nullptr));
}
void VMath::set_mh_attention_mask(int device, float* pp, int64 ndat, int64 ntimes, int64 nhead, bool forward) {
    check(kai_set_mh_attention_mask(device, pp, ndat, ntimes, nhead, forward, nullptr));
}
void VMath::softmax_direct_on_axis(int device, float* pp, int64 nrow, int64 nvec, int64 ncol) {
    check(kai_softmax_direct_on_axis(device, pp, nrow, nvec, ncol, nullptr));
}
void VMath::mix_values(int device, float* py, float* pp, float* pV, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece) {
    check(kai_mix_values(device, py, pp, pV, nbat, ntimes, nvec, nhead, npiece, nullptr));
}
void VMath::conv2d(int device, float* py, float* px, float* pk, int64 ndat, int64 ychn, int64 yh, int64 yw, int64 xchn, int64 xh, int64 xw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw, int pmode) {
    check(kai_conv2d(device, py, px, pk, ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, group, ph, pw, pmode, nullptr));
}
void VMath::conv2d_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 yh, int64 yw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw) {
    check(kai_conv2d_backward_x(device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, nullptr));
}
void VMath::conv2d_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 yh, int64 yw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw) {
    check(kai_conv2d_backward_k(device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, nullptr));
}
void VMath::conv2d_transposed(int device, float* py, float* px, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw) {
    check(kai_conv2d_transposed(device, py, px, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, nullptr));
}
void VMath::conv2d_transposed_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw) {
    check(kai_conv2d_transposed_backward_x(device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, nullptr));
}
void VMath::conv2d_transposed_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw) {
    check(kai_conv2d_transposed_backward_k(device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, nullptr));
}
void VMath::conv2d_dilated(int device, float* py, float* px, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw) {
    check(kai_conv2d_dilated(device, py, px, pk, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw, nullptr));
}
void VMath::conv2d_dilated_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw) {
    check(kai_conv2d_dilated_backward_x(device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw, nullptr));
}
void VMath::conv2d_dilated_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw) {
    check(kai_conv2d_dilated_backward_k(device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw, nullptr));
}
void VMath::mult_on_heads_backward(int device, float* pgQK, float* pgp, float* pKQ, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece) {
    check(kai_mult_on_heads_backward(device, pgQK, pgp, pKQ, nbat, ntimes, nvec, nhead, npiece, nullptr));
}
void VMath::softmax_direct_on_axis_backward(int device, float* pgp, float* pp, int64 nbat, int64 ntimes, int64 nhead, HYPER hCoef) {
    check(kai_softmax_direct_on_axis_backward(device, pgp, pp, nbat, ntimes, nhead, hCoef, nullptr));
}
void VMath::mix_values_backward_prop(int device, float* pgp, float* pgy, float* pV, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece) {
    check(kai_mix_values_backward_prop(device, pgp, pgy, pV, nbat, ntimes, nvec, nhead, npiece, nullptr));
}
void VMath::mix_values_backward_value(int device, float* pgV, float* pgy, float* pp, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece) {
    check(kai_mix_values_backward_value(device, pgV, pgy, pp, nbat, ntimes, nvec, nhead, npiece, nullptr));
}

void VMath::softmax_idx_crossentropy(int device, float* py, float* px, int* pz, int64 nrow, int64 ncol) {
    check(kai_softmax_idx_crossentropy(device, py, px, pz, nrow, ncol, nullptr));
}
void VMath::softmax_idx_crossentropy_backward_x(int device, float* pgx, float* pgy, float* px, int* pz, int64 nrow, int64 ncol) {
    check(kai_softmax_idx_crossentropy_backward_x(device, pgx, pgy, px, pz, nrow, ncol, nullptr));
}
void VMath::sum(int device, float* py, float* px, int64 nrow) { check(kai_sum(device, py, px, nrow, nullptr)); }
void VMath::sum_backward(int device, float* pgx, float* pgy, int64 nrow) {
    check(kai_sum_backward(device, pgx, pgy, nrow, nullptr));
}

void VMath::linear_forward(int device, float* py, float* pw, float* px, float* pb, int64 yvec, int64 ndat, int64 xvec, int actFunc, HYPER hLeakyAlpha) {
    check(kai_linear_forward(device, py, pw, px, pb, yvec, ndat, xvec, yvec, actFunc, hLeakyAlpha, nullptr));
}

}  // namespace kai_shim
