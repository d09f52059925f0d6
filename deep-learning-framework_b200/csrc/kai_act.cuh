// Elementwise activation math shared by the GEMM epilogues and the standalone kernels.
// Formulas follow the reference's activate / activate_backward / activate_backward_with_y
// (source/engine/support/vmath.cu:297-311, 3097-3167, 3247-3330, 3411-3444): the same
// branch structure and the same libm calls, so results agree with its host loops to a few
// ulp of expf/erff/logf.
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include "../../include/kai_b200.h"

namespace kai {

__device__ __forceinline__ float act_sigmoid(float x) {
    // two-branch stable form (vmath.cu:297-303)
    return (x > 0) ? (1.0f / (1.0f + expf(-x))) : (expf(x) / (expf(x) + 1.0f));
}

__device__ __forceinline__ float act_tanh(float x) {
    return 2 * act_sigmoid(2 * x) - 1;  // vmath.cu:305-311
}

// Forward value for the elementwise activations (everything except softmax).
__device__ __forceinline__ float act_forward(int act, float x, float leaky_alpha) {
    switch (act) {
        case KAI_ACT_NONE: return x;
        case KAI_ACT_RELU: return (x > 0) ? x : 0.0f;
        case KAI_ACT_LEAKY: return (x > 0) ? x : x * leaky_alpha;
        case KAI_ACT_SIGMOID: return act_sigmoid(x);
        case KAI_ACT_TANH: return act_tanh(x);
        case KAI_ACT_GELU: return x * 0.5f * (1.0f + erff(x / sqrtf(2.0f)));
        case KAI_ACT_SELU: {
            const float lambda = 1.0507009f, alpha = 1.6732632f;
            return (x > 0) ? lambda * x : lambda * alpha * (expf(x) - 1);
        }
        case KAI_ACT_MISH: {
            float t = logf(1.0f + expf(x)) * 2;
            t = (t > 0) ? ((1.0f - expf(-t)) / (1.0f + expf(-t)))
                        : ((expf(t) - 1.0f) / (expf(t) + 1.0f));
            return x * t;
        }
        case KAI_ACT_SWISH: return x * act_sigmoid(x);
        default: return x;
    }
}

// d act / d x evaluated on the pre-activation x (vmath.cu:3247-3330).
__device__ __forceinline__ float act_grad_from_x(int act, float x, float leaky_alpha) {
    float y, s, t, u, v;
    switch (act) {
        case KAI_ACT_NONE: return 1.0f;
        case KAI_ACT_RELU: return (x > 0) ? 1.0f : 0.0f;
        case KAI_ACT_LEAKY: return (x > 0) ? 1.0f : leaky_alpha;
        case KAI_ACT_SIGMOID: y = act_sigmoid(x); return y * (1.0f - y);
        case KAI_ACT_TANH: y = act_tanh(x); return 1.0f - y * y;
        case KAI_ACT_GELU:
            s = 0.5f * (1.0f + erff(x / sqrtf(2.0f)));
            t = 0.5f * x * sqrtf(2.0f / 3.14159265358979323846f) * expf(-x * x / 2.0f);
            return s + t;
        case KAI_ACT_SELU: {
            const float lambda = 1.0507009f, alpha = 1.6732632f;
            return (x > 0) ? lambda : lambda * alpha * expf(x);
        }
        case KAI_ACT_MISH:
            s = logf(1.0f + expf(x));
            t = act_sigmoid(x);
            s = s * 2.0f;
            u = (s > 0) ? ((1.0f - expf(-s)) / (1.0f + expf(-s)))
                        : ((expf(s) - 1.0f) / (expf(s) + 1.0f));
            v = 1.0f - u * u;
            return u + x * v * t;
        case KAI_ACT_SWISH:
            s = act_sigmoid(x);
            t = s * (1.0f - s);
            return s + x * t;
        default: return 1.0f;
    }
}

// d act / d x evaluated on the OUTPUT y (vmath.cu:3411-3444); only these five exist there.
__device__ __forceinline__ float act_grad_from_y(int act, float y, float leaky_alpha) {
    switch (act) {
        case KAI_ACT_NONE: return 1.0f;
        case KAI_ACT_RELU: return (y > 0) ? 1.0f : 0.0f;
        case KAI_ACT_LEAKY: return (y > 0) ? 1.0f : leaky_alpha;
        case KAI_ACT_SIGMOID: return y * (1 - y);
        case KAI_ACT_TANH: return 1 - y * y;
        default: return 1.0f;
    }
}

}  // namespace kai
