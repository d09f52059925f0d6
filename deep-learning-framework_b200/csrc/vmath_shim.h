// C++ host side of the drop-in: the static methods of the reference engine's `class VMath`
// (source/engine/support/vmath.h:18-19, 65-66, 137-143, 234-241, 299-301, 325-326) for the
// matmul / Linear path, with the reference's names, argument order and types, implemented on
// top of the C ABI in include/kai_b200.h.
//
// Behaviour kept from the reference:
//   * void return; failure is an exception carrying the code VERR_CUDA_ERROR (50002,
//     include/verrors.h:164) and the text "cuda:<message>", which is what VMath::cudaCheck
//     raises (support/vmath.cu:64-87).  Inside the engine the exception type is VException
//     (define KAI_SHIM_THROW before including this header to raise it); stand-alone builds
//     get kai_shim::VMathError.
//   * kernels run on the legacy default stream and rely on the caller's current device for
//     ordering with the engine's cudaMemcpy calls; `device` is honoured as well.
// Difference, by contract of this path: there is no host branch.  device < 0 raises; the
// engine keeps its own `_host` loops for that case.
#pragma once

#include <stdint.h>

#include <stdexcept>
#include <string>

namespace kai_shim {

constexpr int kVerrCudaError = 50002;        // VERR_CUDA_ERROR
constexpr int kVerrOutOfRange = 4;           // VERR_OUT_OF_RANGE (label outside [0, ncol))

struct VMathError : std::runtime_error {
    int code;      // the reference's error code
    int status;    // the C ABI's status (KAI_E_* or cudaError_t)
    VMathError(int code_, int status_, const std::string& what) : std::runtime_error(what), code(code_), status(status_) {}
};

typedef int64_t int64;   // include/vtypes.h:18-22 on Linux
typedef float* HYPER;    // local_objects/vhypermanager.h:6 -- a float in the device's memory, or NULL

class VMath {
public:
    static void* mem_alloc(int device, int64 size);
    static void mem_free(int device, void* ptr);

    static void add_bias(int device, float* py, float* pa, float* pb, int64 nrow, int64 ncol);
    static void add_bias_backward_b(int device, float* pgb, float* pgy, int64 nrow, int64 ncol, bool acc);

    static void matmul(int device, float* py, float* pw, float* px, int64 yvec, int64 ndat, int64 xvec, bool acc);
    static void matmul_backward_x(int device, float* pgx, float* pgy, float* pw, int64 yvec, int64 ndat, int64 xvec, bool acc);
    static void matmul_backward_w(int device, float* pgw, float* pgy, float* px, int64 yvec, int64 ndat, int64 xvec, bool acc);

    static void activate(int device, float* py, float* px, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha);
    static void activate_backward(int device, float* pgx, float* pgy, float* px, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha);
    static void activate_backward_with_y(int device, float* pgx, float* pgy, float* py, int64 nrow, int64 ncol, int actFunc, HYPER hLeakyAlpha);

    static void mult_on_heads(int device, float* pp, float* pK, float* pQ, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece, HYPER hCoef);
    static void set_mh_attention_mask(int device, float* pp, int64 ndat, int64 ntimes, int64 nhead, bool forward);
    static void softmax_direct_on_axis(int device, float* pp, int64 nrow, int64 nvec, int64 ncol);
    static void mix_values(int device, float* py, float* pp, float* pV, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece);
    static void conv2d(int device, float* py, float* px, float* pk, int64 ndat, int64 ychn, int64 yh, int64 yw, int64 xchn, int64 xh, int64 xw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw, int pmode);
    static void conv2d_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 yh, int64 yw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw);
    static void conv2d_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 yh, int64 yw, int64 kh, int64 kw, int64 group, int64 ph, int64 pw);
    static void conv2d_transposed(int device, float* py, float* px, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw);
    static void conv2d_transposed_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw);
    static void conv2d_transposed_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 sh, int64 sw);
    static void conv2d_dilated(int device, float* py, float* px, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw);
    static void conv2d_dilated_backward_x(int device, float* pgx, float* pgy, float* pk, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw);
    static void conv2d_dilated_backward_k(int device, float* pgk, float* pgy, float* px, int64 ndat, int64 xchn, int64 xh, int64 xw, int64 ychn, int64 kh, int64 kw, int64 gh, int64 gw);
    static void mult_on_heads_backward(int device, float* pgQK, float* pgp, float* pKQ, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece);
    static void softmax_direct_on_axis_backward(int device, float* pgp, float* pp, int64 nbat, int64 ntimes, int64 nhead, HYPER hCoef);
    static void mix_values_backward_prop(int device, float* pgp, float* pgy, float* pV, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece);
    static void mix_values_backward_value(int device, float* pgV, float* pgy, float* pp, int64 nbat, int64 ntimes, int64 nvec, int64 nhead, int64 npiece);

    static void layernorm(int device, float* py, float* px, float* ps, int64 nrow, int64 ncol, HYPER hScale);
    static void layernorm_backward(int device, float* pgx, float* pgy, float* ps, int64 nrow, int64 ncol, HYPER hScale);

    static void softmax_idx_crossentropy(int device, float* py, float* px, int* pz, int64 nrow, int64 ncol);
    static void softmax_idx_crossentropy_backward_x(int device, float* pgx, float* pgy, float* px, int* pz, int64 nrow, int64 ncol);
    static void sum(int device, float* py, float* px, int64 nrow);
    static void sum_backward(int device, float* pgx, float* pgy, int64 nrow);

    // Not in the reference: its `linear` / `dense` formulas (api/vconst.cpp:10-11) as one launch.
    static void linear_forward(int device, float* py, float* pw, float* px, float* pb, int64 yvec, int64 ndat, int64 xvec, int actFunc, HYPER hLeakyAlpha);
};

}  // namespace kai_shim
