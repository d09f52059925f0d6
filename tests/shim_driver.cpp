// Test driver of the C++ VMath shim: `shim_driver cpu` checks the error convention without a GPU;
// `shim_driver gpu` runs a Linear forward/backward through VMath::* and prints the results for the
// Python test to compare with the oracle.
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "vmath_shim.h"

using kai_shim::VMath;
using kai_shim::VMathError;

static int run_cpu() {
    int fails = 0;
    try {
        VMath::matmul(-1, nullptr, nullptr, nullptr, 4, 4, 4, false);
        printf("FAIL: device -1 did not raise\n"); fails++;
    } catch (const VMathError& e) {
        printf("host branch: code=%d status=%d what=%s\n", e.code, e.status, e.what());
        if (e.code != 50002 || strncmp(e.what(), "cuda:", 5) != 0) fails++;
    }
    return fails;
}

static int run_gpu() {
    const int64_t ndat = 48, xvec = 40, yvec = 72;
    std::vector<float> x(ndat * xvec), w(yvec * xvec), gy(ndat * yvec), b(yvec);
    unsigned s = 12345u;
    auto rnd = [&]() { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = rnd();
    for (auto& v : w) v = rnd();
    for (auto& v : gy) v = rnd();
    for (auto& v : b) v = rnd();
    auto up = [](const std::vector<float>& h) {
        float* d = static_cast<float*>(VMath::mem_alloc(0, h.size() * 4));
        cudaMemcpy(d, h.data(), h.size() * 4, cudaMemcpyHostToDevice);
        return d;
    };
    float *dx = up(x), *dw = up(w), *dgy = up(gy), *db = up(b);
    float* dy = static_cast<float*>(VMath::mem_alloc(0, ndat * yvec * 4));
    float* dgx = static_cast<float*>(VMath::mem_alloc(0, ndat * xvec * 4));
    float* dgw = static_cast<float*>(VMath::mem_alloc(0, yvec * xvec * 4));
    float* dgb = static_cast<float*>(VMath::mem_alloc(0, yvec * 4));
    VMath::matmul(0, dy, dw, dx, yvec, ndat, xvec, false);
    VMath::add_bias(0, dy, dy, db, ndat, yvec);
    VMath::activate(0, dy, dy, ndat, yvec, 1, nullptr);
    VMath::matmul_backward_x(0, dgx, dgy, dw, yvec, ndat, xvec, false);
    VMath::matmul_backward_w(0, dgw, dgy, dx, yvec, ndat, xvec, false);
    VMath::add_bias_backward_b(0, dgb, dgy, ndat, yvec, false);
    auto dump = [](const char* name, float* d, int64_t n) {
        std::vector<float> h(n);
        cudaMemcpy(h.data(), d, n * 4, cudaMemcpyDeviceToHost);
        printf("%s", name);
        for (float v : h) printf(" %.9g", v);
        printf("\n");
    };
    dump("x", dx, ndat * xvec); dump("w", dw, yvec * xvec); dump("gy", dgy, ndat * yvec); dump("b", db, yvec);
    dump("y", dy, ndat * yvec); dump("gx", dgx, ndat * xvec); dump("gw", dgw, yvec * xvec); dump("gb", dgb, yvec);
    int fails = 0;
    try {
        VMath::mem_free(0, reinterpret_cast<void*>(0x1000));
        fails++;
    } catch (const VMathError& e) {
        if (e.code != 50002) fails++;
    }
    for (float* p : {dx, dw, dgy, db, dy, dgx, dgw, dgb}) VMath::mem_free(0, p);
    return fails;
}

int main(int argc, char** argv) {
    const bool gpu = argc > 1 && !strcmp(argv[1], "gpu");
    const int fails = gpu ? run_gpu() : run_cpu();
    printf("fails=%d\n", fails);
    return fails ? 1 : 0;
}
