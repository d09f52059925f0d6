// Shared host-side plumbing of the sm_100a matmul library: per-thread error text,
// per-device state (status word, workspaces), launch accounting and option storage.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/kai_b200.h"

namespace kai {

constexpr int kMaxDevices = 16;

// ---- error text (thread local) ---------------------------------------------------------
void set_error(const char* fmt, ...);
int  fail(int code, const char* fmt, ...);
int  cuda_fail(cudaError_t e, const char* what);

#define KAI_CUDA(expr)                                                     \
    do {                                                                   \
        cudaError_t e__ = (expr);                                          \
        if (e__ != cudaSuccess) return ::kai::cuda_fail(e__, #expr);       \
    } while (0)

#define KAI_TRY(expr)                                                      \
    do {                                                                   \
        int rc__ = (expr);                                                 \
        if (rc__ != KAI_OK) return rc__;                                   \
    } while (0)

// ---- options ---------------------------------------------------------------------------
struct Options {
    std::atomic<int64_t> tc_bn{256};
    std::atomic<int64_t> tc_bk{16};
    std::atomic<int64_t> tc_min_flops{int64_t(1) << 29};  // below: SIMT kernel
    std::atomic<int64_t> split_k{0};                      // 0 = automatic
    std::atomic<int64_t> path{KAI_PATH_AUTO};
    std::atomic<int64_t> tc_group_m{16};                  // rasterisation group (tiles along M)
    std::atomic<int64_t> tc_raw_hi{0};                    // K-major operands as their own hi plane: 0 by shape, 1 always, 2 never
    std::atomic<int64_t> attn_path{0};                    // 0 = tcgen05, then warp-MMA, then CUDA-core kernels by shape; 2 = no tcgen05; 1 = CUDA-core only
    std::atomic<int64_t> skinny_rows{0};                  // rows of W per block of the M <= 4 skinny kernel: 0 = by shape, 4, 8
    std::atomic<int64_t> conv_wide{1};                    // implicit-GEMM convolution: one operand box per kernel row (0 = one per tap)
    std::atomic<int64_t> conv_igemm{1};                   // implicit-GEMM convolution kernels where they fit: 1 = TMA-fed, then converter-fed; 2 = converter-fed only; 0 = none
    std::atomic<int64_t> tc_balance{0};                   // 1 = also range-split the tiles of an uneven last round
    std::atomic<int64_t> skinny_regx{1};                  // 1 = X-in-registers skinny kernel for M = 5..16
    std::atomic<int64_t> conv_direct{0};                  // 1 = transposed family and group != 1 on the one-thread-per-output kernels (the reference's loops, bit for bit)
    std::atomic<int64_t> tc_kc{0};                        // K per TMEM accumulation chunk (0 = from K)
    std::atomic<int64_t> tc_cross_bf16{1};                // 1 = products with a reduction of 2048 or more form their two cross terms with one BF16 MMA
    std::atomic<int64_t> tc_pair_bk{32};                  // K block of the CTA-pair kernel (16 | 32)
    std::atomic<int64_t> tc_pair{1};                      // 1 = large products run on CTA pairs (cta_group::2, 256 x 256 tiles)
    std::atomic<int64_t> tc_max_ctas{0};                  // CTAs of the persistent GEMM grid (0 = one per SM): leaves SMs to kernels that run beside it
    std::atomic<int64_t> skinny_mma{1};                   // 1 = M <= 16 NT products on the warp-MMA streaming kernel
};
Options& options();

// ---- launch accounting -----------------------------------------------------------------
extern std::atomic<int64_t> g_launches;
extern std::atomic<int64_t> g_tc_launches;   // launches of kernels that issue tcgen05.mma
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }
inline void count_tc_launch(int n = 1) { g_tc_launches.fetch_add(n, std::memory_order_relaxed); }
extern std::atomic<int64_t> g_tc_pair_launches;   // of those, launches of the CTA-pair GEMM kernel
inline void count_tc_pair_launch() { g_tc_pair_launches.fetch_add(1, std::memory_order_relaxed); }

// Checks the launch like the reference's CUDA_CALL does (cudaGetLastError after <<<>>>,
// support/vmath.cu:46-55).
int check_launch(const char* kernel);

// ---- per-device state ------------------------------------------------------------------
// The status word lives in mapped pinned host memory: kernels whose bounded waits give up
// write a code there, and the host can read it without a synchronisation.
struct DeviceState {
    std::mutex mu;
    bool       ready = false;
    int        sm_count = 0;
    int*       status_host = nullptr;   // host view  (2 ints: code, detail)
    int*       status_dev = nullptr;    // device view of the same words
    // Operand-split workspace (hi/lo planes of both GEMM operands, split-K partials).
    void*      ws = nullptr;
    int64_t    ws_bytes = 0;
    // Bytes at the start of the workspace that the current caller keeps for itself (the im2col
    // matrices of a convolution); the GEMM's own planes start behind them.
    int64_t    ws_front = 0;
    // Second scratch block: inputs that a convolution variant rewrites before it calls the plain convolution
    // (channel-group sums, the upsampled image of a transposed convolution, permuted kernels), which uses `ws`.
    void*      aux = nullptr;
    int64_t    aux_bytes = 0;
    int*       flag_dev = nullptr;      // small device scratch (label range flag)
    // Once a stream capture has recorded kernels that point into the workspace, a block that is
    // outgrown later is kept (a recorded graph may still be replayed) instead of being freed.
    bool       ws_recorded = false;
    bool       ws_recorded_foreign = false;   // recorded by a capture that kai_replay_* does not own
    std::vector<void*> ws_retired;
};

// Makes `device` current for the calling thread if it is not already and returns its
// lazily created state.  The reference's kernels rely on the caller's cudaSetDevice
// (local_objects/vdevicemanager.cpp:112-124); honouring the argument as well makes the
// entry points safe to call from a thread that has another device current.
int get_device(int device, DeviceState** out);

// Grows the per-device workspace to at least `bytes` (stream-ordered: the old block is
// released only after work already queued on the device has drained).
int ensure_workspace(DeviceState* st, int device, int64_t bytes);

// The same for the second scratch block.
int ensure_aux(DeviceState* st, int64_t bytes);

// RAII: switch to a device, restore the previous one on scope exit.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    int enter(int device);
    ~DeviceGuard();
};

// Converts the `stream` argument of an entry point and notes, for the calling thread, whether that
// stream is being captured into a CUDA graph (capturing() below).  Inside a capture the entry points
// make no blocking call and never move the workspace.
cudaStream_t as_stream(void* s);
bool capturing();

// ---- epilogue description shared by every GEMM kernel -----------------------------------
struct Epilogue {
    const float* bias;         // length N or nullptr
    const float* leaky_alpha;  // device scalar or nullptr
    int          act;          // KAI_ACT_*
    int          accumulate;   // C += instead of C =
};

// K-major hi/lo planes [rows][kp] of one GEMM operand, ready for the tensor-core kernel
// (kp = round_up(K, 4); hi may be the caller's own matrix when that already has this form).
struct PlanePair {
    const float* hi;
    const float* lo;
    int64_t kp;
    int xfmt;      // form of the second plane: 0 = TF32 lo values, 1 / 2 = bf16 cross-term plane of a left / right operand
};

// ---- kernel families (defined in their own translation units) ---------------------------
int gemm_tc(DeviceState* st, int device, int layout, float* c, const float* a, const float* b,
            int64_t M, int64_t N, int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s,
            const float* b_lo_given = nullptr, const PlanePair* a_prep = nullptr,
            const PlanePair* b_prep = nullptr);
// hi/lo planes of one operand into caller-provided memory: src is [rows][k] (transpose == false) or
// [k][rows] (transpose == true) with row stride ld; hi == nullptr writes only lo (against the truncated value)
int split_operand(const float* src, int64_t rows, int64_t k, int64_t ld, bool transpose, float* hi, float* lo,
                  int sm_count, cudaStream_t s, int xside = 0);
// status words of kai_linear_forward_static on `device` (zeros if never used there)
void static_status_peek(int device, int out[2], bool clear);
int gemm_simt(int layout, float* c, const float* a, const float* b, int64_t M, int64_t N,
              int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s);
// lo planes (against the truncated high part) of one (b == nullptr) or two dense 16-byte aligned tensors
int split_lo_pair(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, cudaStream_t s);
int gemm_skinny_mma(float* c, const float* x, const float* w, int64_t M, int64_t N, int64_t K, int64_t ldc,
                    const Epilogue& ep, cudaStream_t s);
int gemm_skinny_nt(DeviceState* st, float* c, const float* x, const float* w, int64_t M,
                   int64_t N, int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s);

}  // namespace kai
