// C ABI of the sm_100a matmul / Linear path: argument checks, device state, dispatch to the
// kernel families, and the device allocator.  See include/kai_b200.h for the contract.
#include <string.h>

#include <map>
#include <vector>

#include "kai_common.cuh"

namespace kai {

// launchers defined in kai_elementwise.cu / kai_attention.cu
int ew_add_bias(DeviceState*, float*, const float*, const float*, int64_t, int64_t, cudaStream_t);
int ew_colsum(DeviceState*, int, float*, const float*, int64_t, int64_t, int, cudaStream_t);
int ew_activate(DeviceState*, float*, const float*, int64_t, int64_t, int, const float*, cudaStream_t);
int ew_activate_backward(DeviceState*, float*, const float*, const float*, int64_t, int, const float*, int,
                         cudaStream_t);
int ew_ce_forward(DeviceState*, float*, const float*, const int*, int64_t, int64_t, cudaStream_t);
int ew_ce_backward(DeviceState*, float*, const float*, const float*, const int*, int64_t, int64_t, cudaStream_t);
int ew_sum(float*, const float*, int64_t, cudaStream_t);
int ew_sum_backward(DeviceState*, float*, const float*, int64_t, cudaStream_t);
int attn_mult_on_heads(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                       const float*, cudaStream_t);
int split_lo_pair(const float* a, const float* b, int64_t count, float* lo_a, float* lo_b, cudaStream_t s);
int attn_mult_on_heads_tc(DeviceState*, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                          int64_t, const float*, cudaStream_t);
int attn_mix_values_tc(DeviceState*, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                       int64_t, cudaStream_t, bool transposed = false);
int attn_fused_forward_tc(DeviceState*, int, float*, const float*, const float*, const float*, int64_t, int64_t,
                          int64_t, int64_t, int64_t, const float*, int, cudaStream_t);
int conv2d_forward(DeviceState*, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                   int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, cudaStream_t,
                   int64_t strh = 1, int64_t strw = 1, int64_t vh = 0, int64_t vw = 0);
int conv2d_backward_x(DeviceState*, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                      int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                      cudaStream_t);
int conv2d_backward_k(DeviceState*, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                      int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                      cudaStream_t);
int conv2d_transposed_any(DeviceState*, int, int, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int64_t, int64_t, int64_t, int64_t, cudaStream_t);
int attn_mask(DeviceState*, float*, int64_t, int64_t, int64_t, int, cudaStream_t);
int attn_softmax_axis(float*, int64_t, int64_t, int64_t, cudaStream_t);
int attn_mix_values(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                    cudaStream_t, bool transposed = false);
int attn_softmax_axis_backward(float*, const float*, int64_t, int64_t, int64_t, const float*, cudaStream_t);

int selftest_bounded_wait(DeviceState*, int64_t, cudaStream_t);
int ew_layernorm(float*, const float*, float*, int64_t, int64_t, const float*, cudaStream_t);
int ew_layernorm_backward(float*, const float*, const float*, int64_t, int64_t, const float*, cudaStream_t);
int gemm_simt_grouped(int layout, int count, float* const* c, const float* const* a, const float* const* b, int64_t M,
                      int64_t N, int64_t K, int64_t ldc, const Epilogue& ep, cudaStream_t s);
void profile_enable(bool on);
int profile_read(double ms[3], int64_t launches[3]);

// ---- errors ------------------------------------------------------------------------------
static thread_local char tl_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
}
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    // Same text the reference's cudaCheck raises: "cuda:" + cudaGetErrorString (vmath.cu:64-87).
    snprintf(tl_error, sizeof(tl_error), "cuda:%s (%s)", cudaGetErrorString(e), what);
    return static_cast<int>(e);
}
int check_launch(const char* kernel) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, kernel);
    return KAI_OK;
}

// ---- globals -----------------------------------------------------------------------------
Options& options() {
    static Options o;
    return o;
}
std::atomic<int64_t> g_launches{0};
std::atomic<int64_t> g_tc_launches{0};
std::atomic<int64_t> g_tc_pair_launches{0};

static DeviceState g_devices[kMaxDevices];
static std::atomic<int> g_live_replays[kMaxDevices];

// Workspace blocks that were kept alive because a recorded call list pointed into them can go once no
// recorded list exists on the device any more.
static void release_retired_workspaces(DeviceState* st) {
    std::lock_guard<std::mutex> lock(st->mu);
    if (st->ws_recorded_foreign) return;          // a graph the caller captured itself may still be replayed
    for (void* p : st->ws_retired) cudaFree(p);   // waits for queued work that still uses the block
    st->ws_retired.clear();
    st->ws_recorded = false;
}

int DeviceGuard::enter(int device) {
    int cur = -1;
    KAI_CUDA(cudaGetDevice(&cur));
    if (cur != device) {
        KAI_CUDA(cudaSetDevice(device));
        prev = cur;
        switched = true;
    }
    return KAI_OK;
}
DeviceGuard::~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
}

int get_device(int device, DeviceState** out) {
    if (device < 0) return fail(KAI_E_NO_HOST_PATH, "device %d: this library has no CPU branch", device);
    if (device >= kMaxDevices) return fail(KAI_E_INVALID_ARG, "device %d out of range", device);
    DeviceState* st = &g_devices[device];
    std::lock_guard<std::mutex> lock(st->mu);
    if (!st->ready) {
        int count = 0;
        KAI_CUDA(cudaGetDeviceCount(&count));
        if (device >= count) return fail(KAI_E_INVALID_ARG, "device %d but only %d visible", device, count);
        DeviceGuard g;
        KAI_TRY(g.enter(device));
        cudaDeviceProp prop;
        KAI_CUDA(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            return fail(KAI_E_INVALID_ARG, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                        prop.major, prop.minor);
        st->sm_count = prop.multiProcessorCount;
        KAI_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&st->status_host), 2 * sizeof(int), cudaHostAllocMapped));
        st->status_host[0] = 0;
        st->status_host[1] = 0;
        KAI_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&st->status_dev), st->status_host, 0));
        KAI_CUDA(cudaMalloc(reinterpret_cast<void**>(&st->flag_dev), 64));
        KAI_CUDA(cudaMemset(st->flag_dev, 0, 64));
        const float one = 1.0f;   // a device-resident 1.0f for ops whose reference form has no coefficient
        KAI_CUDA(cudaMemcpy(reinterpret_cast<float*>(st->flag_dev) + 8, &one, sizeof(one), cudaMemcpyHostToDevice));
        st->ready = true;
    }
    *out = st;
    return KAI_OK;
}

thread_local bool tl_capturing = false;

cudaStream_t as_stream(void* s) {
    cudaStream_t cs = reinterpret_cast<cudaStream_t>(s);
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    // On the legacy stream this query fails while another stream captures in global mode; the launch
    // that follows reports that error, so the result is only used when the query succeeds.
    if (cudaStreamIsCapturing(cs, &status) != cudaSuccess) {
        cudaGetLastError();
        status = cudaStreamCaptureStatusNone;
    }
    tl_capturing = (status == cudaStreamCaptureStatusActive);
    return cs;
}
bool capturing() { return tl_capturing; }

int ensure_workspace(DeviceState* st, int device, int64_t bytes) {
    (void)device;
    std::lock_guard<std::mutex> lock(st->mu);
    if (capturing()) {
        st->ws_recorded = true;
        if (g_live_replays[st - g_devices].load() == 0) st->ws_recorded_foreign = true;   // not one of kai_replay_*'s captures
    }
    if (bytes <= st->ws_bytes) return KAI_OK;
    if (capturing())
        return fail(KAI_E_ALLOC,
                    "the scratch workspace would have to grow to %lld bytes inside a stream capture; run the call "
                    "list once outside the capture first", (long long)bytes);
    if (st->ws && st->ws_recorded) {
        st->ws_retired.push_back(st->ws);   // a recorded graph may still point into it
        st->ws = nullptr;
        st->ws_bytes = 0;
    }
    if (st->ws) {
        // cudaFree waits for work already queued on the device, so kernels still reading the old
        // block finish first.
        KAI_CUDA(cudaFree(st->ws));
        st->ws = nullptr;
        st->ws_bytes = 0;
    }
    const int64_t want = (bytes + (int64_t(1) << 21) - 1) >> 21 << 21;  // 2 MiB granules
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, static_cast<size_t>(want));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(KAI_E_ALLOC, "workspace of %lld bytes: %s", (long long)want, cudaGetErrorString(e));
    }
    st->ws = p;
    st->ws_bytes = want;
    return KAI_OK;
}

int ensure_aux(DeviceState* st, int64_t bytes) {
    std::lock_guard<std::mutex> lock(st->mu);
    if (capturing()) {
        st->ws_recorded = true;
        if (g_live_replays[st - g_devices].load() == 0) st->ws_recorded_foreign = true;
    }
    if (bytes <= st->aux_bytes) return KAI_OK;
    if (capturing())
        return fail(KAI_E_ALLOC,
                    "the scratch block of this convolution would have to grow to %lld bytes inside a stream capture; run "
                    "the call list once outside the capture first", (long long)bytes);
    if (st->aux) {
        if (st->ws_recorded) st->ws_retired.push_back(st->aux);   // a recorded graph may still point into it
        else KAI_CUDA(cudaFree(st->aux));                         // waits for queued work that still reads it
        st->aux = nullptr;
        st->aux_bytes = 0;
    }
    const int64_t want = (bytes + (int64_t(1) << 21) - 1) >> 21 << 21;
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, static_cast<size_t>(want));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(KAI_E_ALLOC, "scratch block of %lld bytes: %s", (long long)want, cudaGetErrorString(e));
    }
    st->aux = p;
    st->aux_bytes = want;
    return KAI_OK;
}

// ---- allocator ---------------------------------------------------------------------------
// Size-class cache in front of cudaMalloc: a freed block goes to the free list of its
// (rounded) size and the next request of that size takes it back without a driver call.
// The reference calls cudaMalloc/cudaFree for every tensor (vmath.cu:169-208, 243-264), each
// of which synchronises the device.
struct Pool {
    std::mutex mu;
    std::map<void*, int64_t> live;                    // ptr -> rounded size
    std::map<int64_t, std::vector<void*>> free_list;  // rounded size -> blocks
    int64_t live_bytes = 0, cached_bytes = 0, driver_allocs = 0;
};
static Pool g_pools[kMaxDevices];

static int64_t size_class(int64_t size) {
    if (size < 1) size = 1;
    if (size <= (int64_t(1) << 20)) return (size + 511) / 512 * 512;
    return (size + (int64_t(1) << 20) - 1) >> 20 << 20;
}

static int pool_alloc(int device, int64_t size, void** out) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    if (size < 0) return fail(KAI_E_INVALID_ARG, "mem_alloc: negative size");
    const int64_t cls = size_class(size);
    Pool& pool = g_pools[device];
    std::lock_guard<std::mutex> lock(pool.mu);
    auto it = pool.free_list.find(cls);
    if (it != pool.free_list.end() && !it->second.empty()) {
        void* p = it->second.back();
        it->second.pop_back();
        pool.cached_bytes -= cls;
        pool.live[p] = cls;
        pool.live_bytes += cls;
        *out = p;
        return KAI_OK;
    }
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, static_cast<size_t>(cls));
    if (e != cudaSuccess) {
        // Give the cache back to the driver and retry once.
        cudaGetLastError();
        for (auto& kv : pool.free_list) {
            for (void* q : kv.second) cudaFree(q);
            kv.second.clear();
        }
        pool.cached_bytes = 0;
        e = cudaMalloc(&p, static_cast<size_t>(cls));
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(KAI_E_ALLOC, "cuda:%s (cudaMalloc of %lld bytes)", cudaGetErrorString(e), (long long)cls);
        }
    }
    pool.driver_allocs++;
    pool.live[p] = cls;
    pool.live_bytes += cls;
    *out = p;
    return KAI_OK;
}

}  // namespace kai

using namespace kai;

// ==========================================================================================
// extern "C"
// ==========================================================================================
extern "C" {

const char* kai_version(void) { return "kai_b200 0.1 (sm_100a, 3xTF32 tcgen05)"; }
const char* kai_last_error_string(void) { return tl_error; }
int64_t kai_launch_count(void) { return g_launches.load(); }
int64_t kai_tc_launch_count(void) { return g_tc_launches.load(); }
int64_t kai_tc_pair_launch_count(void) { return g_tc_pair_launches.load(); }

int kai_device_status(int device, int* detail) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    KAI_CUDA(cudaDeviceSynchronize());
    if (detail) *detail = st->status_host[1];
    if (st->status_host[0] != 0)
        return fail(st->status_host[0], "device-side bounded wait ran out (where=%d)", st->status_host[1]);
    // the allocation-free entry point keeps its own status words (its kernels may have run from a replayed list)
    int stat[2];
    static_status_peek(device, stat, false);
    if (stat[0] != 0) {
        if (detail) *detail = stat[1];
        return fail(stat[0], "device-side bounded wait ran out in kai_linear_forward_static (where=%d)", stat[1]);
    }
    // label-range flag of softmax_idx_crossentropy calls that ran from a recorded graph
    int bad = 0;
    KAI_CUDA(cudaMemcpy(&bad, st->flag_dev + 1, sizeof(int), cudaMemcpyDeviceToHost));
    if (bad) {
        KAI_CUDA(cudaMemset(st->flag_dev + 1, 0, sizeof(int)));
        return fail(KAI_E_OUT_OF_RANGE, "softmax_idx_crossentropy (replayed): label outside [0, ncol)");
    }
    return KAI_OK;
}

int kai_device_status_clear(int device) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    KAI_CUDA(cudaDeviceSynchronize());      // a kernel that is still giving up would set the word again
    st->status_host[0] = 0;
    st->status_host[1] = 0;
    int stat[2];
    static_status_peek(device, stat, true);
    KAI_CUDA(cudaMemset(st->flag_dev + 1, 0, sizeof(int)));
    return KAI_OK;
}

int kai_selftest_bounded_wait(int device, int64_t limit_ns, void* stream) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    if (limit_ns < 1000 || limit_ns > 1000000000)
        return fail(KAI_E_INVALID_ARG, "selftest_bounded_wait: limit must be between 1 us and 1 s");
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    return selftest_bounded_wait(st, limit_ns, as_stream(stream));
}

// ---- recorded call lists ---------------------------------------------------------------------
namespace {
struct Replay {
    int device = -1;
    cudaStream_t stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    bool recording = false;
};
}  // namespace

int kai_replay_begin(int device, void** out_handle, void** out_stream) {
    if (!out_handle || !out_stream) return fail(KAI_E_INVALID_ARG, "replay_begin: null output pointer");
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));   // first-use set-up of the device happens before the capture starts
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    Replay* r = new Replay();
    r->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamBeginCapture(r->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (r->stream) cudaStreamDestroy(r->stream);
        delete r;
        return fail(static_cast<int>(e), "cuda:%s", cudaGetErrorString(e));
    }
    r->recording = true;
    g_live_replays[device].fetch_add(1);
    *out_handle = r;
    *out_stream = r->stream;
    return KAI_OK;
}

int kai_replay_end(void* handle) {
    Replay* r = static_cast<Replay*>(handle);
    if (!r || !r->recording) return fail(KAI_E_INVALID_ARG, "replay_end: not recording");
    DeviceGuard g;
    KAI_TRY(g.enter(r->device));
    r->recording = false;
    cudaError_t e = cudaStreamEndCapture(r->stream, &r->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&r->exec, r->graph, 0);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(static_cast<int>(e), "cuda:%s", cudaGetErrorString(e));
    }
    return KAI_OK;
}

int kai_replay_launch(void* handle, void* stream) {
    Replay* r = static_cast<Replay*>(handle);
    if (!r || !r->exec) return fail(KAI_E_INVALID_ARG, "replay_launch: nothing recorded");
    DeviceGuard g;
    KAI_TRY(g.enter(r->device));
    KAI_CUDA(cudaGraphLaunch(r->exec, reinterpret_cast<cudaStream_t>(stream)));
    return KAI_OK;
}

int kai_replay_destroy(void* handle) {
    Replay* r = static_cast<Replay*>(handle);
    if (!r) return KAI_OK;
    DeviceGuard g;
    KAI_TRY(g.enter(r->device));
    if (r->recording) {   // abandon the capture
        cudaGraph_t dropped = nullptr;
        cudaStreamEndCapture(r->stream, &dropped);
        if (dropped) cudaGraphDestroy(dropped);
        cudaGetLastError();
    }
    if (r->exec) cudaGraphExecDestroy(r->exec);
    if (r->graph) cudaGraphDestroy(r->graph);
    if (r->stream) cudaStreamDestroy(r->stream);
    const int device = r->device;
    delete r;
    if (g_live_replays[device].fetch_sub(1) == 1 && g_devices[device].ready) release_retired_workspaces(&g_devices[device]);
    return KAI_OK;
}

int kai_profile_enable(int on) {
    profile_enable(on != 0);
    return KAI_OK;
}

int kai_profile_read(double* ms3, int64_t* launches3) {
    if (!ms3 || !launches3) return fail(KAI_E_INVALID_ARG, "profile_read: null output");
    return profile_read(ms3, launches3);
}

int kai_set_option(const char* name, int64_t value) {
    if (!name) return fail(KAI_E_INVALID_ARG, "set_option: null name");
    Options& o = options();
    if (!strcmp(name, "tc_bn")) {
        if (value != 128 && value != 256) return fail(KAI_E_INVALID_ARG, "tc_bn must be 128 or 256");
        o.tc_bn = value;
    } else if (!strcmp(name, "tc_bk")) {
        if (value != 16 && value != 32) return fail(KAI_E_INVALID_ARG, "tc_bk must be 16 or 32");
        o.tc_bk = value;
    } else if (!strcmp(name, "tc_min_flops")) {
        if (value < 0) return fail(KAI_E_INVALID_ARG, "tc_min_flops must be >= 0");
        o.tc_min_flops = value;
    } else if (!strcmp(name, "split_k")) {
        if (value < 0 || value > 64) return fail(KAI_E_INVALID_ARG, "split_k must be in 0..64");
        o.split_k = value;
    } else if (!strcmp(name, "path")) {
        if (value < KAI_PATH_AUTO || value > KAI_PATH_SKINNY) return fail(KAI_E_INVALID_ARG, "unknown path");
        o.path = value;
    } else if (!strcmp(name, "tc_kc")) {
        if (value != 0 && (value < 16 || value > (1 << 20) || (value & (value - 1)) != 0))
            return fail(KAI_E_INVALID_ARG, "tc_kc must be 0 or a power of two >= 16");
        o.tc_kc = value;
    } else if (!strcmp(name, "tc_raw_hi")) {
        if (value < 0 || value > 2) return fail(KAI_E_INVALID_ARG, "tc_raw_hi must be 0, 1 or 2");
        o.tc_raw_hi = value;
    } else if (!strcmp(name, "conv_wide")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "conv_wide must be 0 or 1");
        o.conv_wide = value;
    } else if (!strcmp(name, "conv_igemm")) {
        if (value < 0 || value > 2) return fail(KAI_E_INVALID_ARG, "conv_igemm must be 0, 1 or 2");
        o.conv_igemm = value;
    } else if (!strcmp(name, "conv_direct")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "conv_direct must be 0 or 1");
        o.conv_direct = value;
    } else if (!strcmp(name, "skinny_rows")) {
        if (value != 0 && value != 2 && value != 4 && value != 8) return fail(KAI_E_INVALID_ARG, "skinny_rows must be 0, 2, 4 or 8");
        o.skinny_rows = value;
    } else if (!strcmp(name, "attn_path")) {
        if (value < 0 || value > 2) return fail(KAI_E_INVALID_ARG, "attn_path must be 0, 1 or 2");
        o.attn_path = value;
    } else if (!strcmp(name, "tc_balance")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "tc_balance must be 0 or 1");
        o.tc_balance = value;
    } else if (!strcmp(name, "skinny_regx")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "skinny_regx must be 0 or 1");
        o.skinny_regx = value;
    } else if (!strcmp(name, "tc_cross_bf16")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "tc_cross_bf16 must be 0 or 1");
        o.tc_cross_bf16 = value;
    } else if (!strcmp(name, "tc_pair_bk")) {
        if (value != 16 && value != 32) return fail(KAI_E_INVALID_ARG, "tc_pair_bk must be 16 or 32");
        o.tc_pair_bk = value;
    } else if (!strcmp(name, "tc_pair")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "tc_pair must be 0 or 1");
        o.tc_pair = value;
    } else if (!strcmp(name, "tc_max_ctas")) {
        if (value < 0 || value > 1024) return fail(KAI_E_INVALID_ARG, "tc_max_ctas must be in 0..1024 (0 = one CTA per SM)");
        o.tc_max_ctas = value;
    } else if (!strcmp(name, "skinny_mma")) {
        if (value != 0 && value != 1) return fail(KAI_E_INVALID_ARG, "skinny_mma must be 0 or 1");
        o.skinny_mma = value;
    } else if (!strcmp(name, "tc_group_m")) {
        if (value < 1 || value > 1024) return fail(KAI_E_INVALID_ARG, "tc_group_m must be in 1..1024");
        o.tc_group_m = value;
    } else {
        return fail(KAI_E_INVALID_ARG, "unknown option '%s'", name);
    }
    return KAI_OK;
}

int64_t kai_get_option(const char* name) {
    if (!name) return -1;
    Options& o = options();
    if (!strcmp(name, "tc_bn")) return o.tc_bn;
    if (!strcmp(name, "tc_bk")) return o.tc_bk;
    if (!strcmp(name, "tc_min_flops")) return o.tc_min_flops;
    if (!strcmp(name, "split_k")) return o.split_k;
    if (!strcmp(name, "path")) return o.path;
    if (!strcmp(name, "tc_group_m")) return o.tc_group_m;
    if (!strcmp(name, "tc_kc")) return o.tc_kc;
    if (!strcmp(name, "skinny_regx")) return o.skinny_regx;
    if (!strcmp(name, "tc_balance")) return o.tc_balance;
    if (!strcmp(name, "attn_path")) return o.attn_path;
    if (!strcmp(name, "skinny_rows")) return o.skinny_rows;
    if (!strcmp(name, "conv_wide")) return o.conv_wide;
    if (!strcmp(name, "conv_igemm")) return o.conv_igemm;
    if (!strcmp(name, "conv_direct")) return o.conv_direct;
    if (!strcmp(name, "tc_raw_hi")) return o.tc_raw_hi;
    if (!strcmp(name, "tc_cross_bf16")) return o.tc_cross_bf16;
    if (!strcmp(name, "tc_pair_bk")) return o.tc_pair_bk;
    if (!strcmp(name, "tc_pair")) return o.tc_pair;
    if (!strcmp(name, "tc_max_ctas")) return o.tc_max_ctas;
    if (!strcmp(name, "skinny_mma")) return o.skinny_mma;
    return -1;
}

// ---- allocator ---------------------------------------------------------------------------
int kai_mem_alloc(int device, int64_t size, void** out_ptr) {
    if (!out_ptr) return fail(KAI_E_INVALID_ARG, "mem_alloc: null out_ptr");
    *out_ptr = nullptr;
    return pool_alloc(device, size, out_ptr);
}

int kai_mem_alloc_pitched(int device, int64_t rows, int64_t row_bytes, void** out_ptr, int64_t* out_pitch_bytes) {
    if (!out_ptr || !out_pitch_bytes) return fail(KAI_E_INVALID_ARG, "mem_alloc_pitched: null output");
    if (rows < 0 || row_bytes < 0) return fail(KAI_E_INVALID_ARG, "mem_alloc_pitched: negative extent");
    const int64_t pitch = (row_bytes + 127) / 128 * 128;
    *out_pitch_bytes = pitch;
    *out_ptr = nullptr;
    return pool_alloc(device, rows * pitch, out_ptr);
}

int kai_mem_free(int device, void* ptr) {
    if (!ptr) return KAI_OK;
    if (device < 0) return fail(KAI_E_NO_HOST_PATH, "mem_free: no CPU branch");
    if (device >= kMaxDevices) return fail(KAI_E_INVALID_ARG, "device %d out of range", device);
    Pool& pool = g_pools[device];
    std::lock_guard<std::mutex> lock(pool.mu);
    auto it = pool.live.find(ptr);
    if (it == pool.live.end()) return fail(KAI_E_INVALID_ARG, "mem_free: %p was not allocated by kai_mem_alloc", ptr);
    const int64_t cls = it->second;
    pool.live.erase(it);
    pool.live_bytes -= cls;
    pool.free_list[cls].push_back(ptr);
    pool.cached_bytes += cls;
    return KAI_OK;
}

int kai_mem_trim(int device) {
    if (device < 0 || device >= kMaxDevices) return fail(KAI_E_INVALID_ARG, "device %d out of range", device);
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    {
        Pool& pool = g_pools[device];
        std::lock_guard<std::mutex> lock(pool.mu);
        for (auto& kv : pool.free_list) {
            for (void* q : kv.second) KAI_CUDA(cudaFree(q));
            kv.second.clear();
        }
        pool.cached_bytes = 0;
    }
    // The scratch workspace goes too, unless a recorded call list points into it.
    DeviceState* st = &g_devices[device];
    if (st->ready && g_live_replays[device].load() == 0) release_retired_workspaces(st);
    std::lock_guard<std::mutex> lock(st->mu);
    if (st->ready && st->ws && !st->ws_recorded) {
        KAI_CUDA(cudaFree(st->ws));   // waits for queued work that still uses it
        st->ws = nullptr;
        st->ws_bytes = 0;
    }
    if (st->ready && st->aux && !st->ws_recorded) {
        KAI_CUDA(cudaFree(st->aux));
        st->aux = nullptr;
        st->aux_bytes = 0;
    }
    return KAI_OK;
}

int kai_mem_stats(int device, int64_t* live_bytes, int64_t* cached_bytes, int64_t* driver_allocs) {
    if (device < 0 || device >= kMaxDevices) return fail(KAI_E_INVALID_ARG, "device %d out of range", device);
    Pool& pool = g_pools[device];
    std::lock_guard<std::mutex> lock(pool.mu);
    if (live_bytes) *live_bytes = pool.live_bytes;
    if (cached_bytes) *cached_bytes = pool.cached_bytes;
    if (driver_allocs) *driver_allocs = pool.driver_allocs;
    return KAI_OK;
}

// ---- GEMM --------------------------------------------------------------------------------
int kai_sgemm(int device, int layout, float* c, const float* a, const float* b, int64_t M, int64_t N, int64_t K,
              int64_t ldc, int accumulate, const float* bias, int act, const float* leaky_alpha, int path,
              void* stream) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    if (layout < KAI_GEMM_NT || layout > KAI_GEMM_TN) return fail(KAI_E_INVALID_ARG, "sgemm: unknown layout %d", layout);
    if (M < 0 || N < 0 || K < 0) return fail(KAI_E_INVALID_ARG, "sgemm: negative dimension");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "sgemm: activation %d is not an elementwise epilogue", act);
    if (M == 0 || N == 0) return KAI_OK;
    if (!c || ((!a || !b) && K > 0)) return fail(KAI_E_INVALID_ARG, "sgemm: null operand");
    if (ldc < N) return fail(KAI_E_INVALID_ARG, "sgemm: ldc=%lld < N=%lld", (long long)ldc, (long long)N);
    if (path < KAI_PATH_AUTO || path > KAI_PATH_SKINNY) return fail(KAI_E_INVALID_ARG, "sgemm: unknown path %d", path);
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    cudaStream_t s = as_stream(stream);
    Epilogue ep{bias, leaky_alpha, act, accumulate ? 1 : 0};

    if (path == KAI_PATH_AUTO) path = static_cast<int>(options().path.load());
    if (path == KAI_PATH_AUTO) {
        const bool skinny_ok = layout == KAI_GEMM_NT && M <= 16 && K >= 256 && (K & 3) == 0 &&
                               ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
        const double flops = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
        if (skinny_ok) path = KAI_PATH_SKINNY;
        else if (K == 0 || flops < static_cast<double>(options().tc_min_flops.load()) || M < 32 || N < 32)
            path = KAI_PATH_SIMT;
        else path = KAI_PATH_TC;
    }
    switch (path) {
        case KAI_PATH_SKINNY:
            if (layout != KAI_GEMM_NT) return fail(KAI_E_INVALID_ARG, "sgemm: the skinny path is NT only");
            return gemm_skinny_nt(st, c, a, b, M, N, K, ldc, ep, s);
        case KAI_PATH_SIMT:
            return gemm_simt(layout, c, a, b, M, N, K, ldc, ep, s);
        default:
            if (K == 0) return gemm_simt(layout, c, a, b, M, N, K, ldc, ep, s);
            return gemm_tc(st, device, layout, c, a, b, M, N, K, ldc, ep, s);
    }
}

// ---- prepared operand handle ---------------------------------------------------------------
namespace {
constexpr uint32_t kPrepMagic = 0x4b505250u;   // "KPRP"
struct Prepared {
    uint32_t magic = kPrepMagic;
    int device = -1;
    int64_t rows = 0, k = 0, kp = 0, ld = 0;
    int transpose = 0;
    bool raw_hi = false;          // hi is the caller's own matrix (not owned)
    int xfmt = 0;                 // second plane: 0 = TF32 lo values, 1 / 2 = bf16 cross-term plane of a left / right operand
    float* hi = nullptr;
    float* lo = nullptr;
    void* block = nullptr;        // the planes, one block of the caching allocator
};
// Live handles.  A handle is only dereferenced after it has been found here, so a pointer that never came
// from kai_operand_prepare (or was released) is refused instead of being read.
std::mutex g_prepared_mu;
std::vector<void*> g_prepared;
Prepared* as_prepared(void* h) {
    if (!h) return nullptr;
    std::lock_guard<std::mutex> lock(g_prepared_mu);
    for (void* q : g_prepared)
        if (q == h) return static_cast<Prepared*>(h);
    return nullptr;
}
void register_prepared(Prepared* p, bool add) {
    std::lock_guard<std::mutex> lock(g_prepared_mu);
    if (add) { g_prepared.push_back(p); return; }
    for (size_t i = 0; i < g_prepared.size(); ++i)
        if (g_prepared[i] == p) { g_prepared[i] = g_prepared.back(); g_prepared.pop_back(); return; }
}
}  // namespace

// ---- GEMM on host buffers -------------------------------------------------------------------
namespace {
struct HostPipe {            // per device: two copy streams and the events that order them with the compute stream
    bool ready = false;
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t in_done[2] = {nullptr, nullptr}, mm_done[2] = {nullptr, nullptr}, out_done[2] = {nullptr, nullptr};
    cudaEvent_t b_done = nullptr;
};
HostPipe g_pipes[kMaxDevices];
std::mutex g_pipe_mu;

int pipe_for(int device, HostPipe** out) {
    std::lock_guard<std::mutex> lock(g_pipe_mu);
    HostPipe& hp = g_pipes[device];
    if (!hp.ready) {
        KAI_CUDA(cudaStreamCreateWithFlags(&hp.s_in, cudaStreamNonBlocking));
        KAI_CUDA(cudaStreamCreateWithFlags(&hp.s_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            KAI_CUDA(cudaEventCreateWithFlags(&hp.in_done[i], cudaEventDisableTiming));
            KAI_CUDA(cudaEventCreateWithFlags(&hp.mm_done[i], cudaEventDisableTiming));
            KAI_CUDA(cudaEventCreateWithFlags(&hp.out_done[i], cudaEventDisableTiming));
        }
        KAI_CUDA(cudaEventCreateWithFlags(&hp.b_done, cudaEventDisableTiming));
        hp.ready = true;
    }
    *out = &hp;
    return KAI_OK;
}
}  // namespace

static int matmul_host_impl(int device, float* py_host, const float* pw_host, const Prepared* wp, const float* px_host,
                            int64_t yvec, int64_t ndat, int64_t xvec, const float* pb_host, int act, float leaky_alpha) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    const int64_t M = ndat, N = yvec, K = xvec;
    if (M < 0 || N < 0 || K < 0) return fail(KAI_E_INVALID_ARG, "matmul_host: negative dimension");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "matmul_host: activation %d is not an elementwise epilogue", act);
    if (M == 0 || N == 0) return KAI_OK;
    if (!py_host || ((!(pw_host || wp) || !px_host) && K > 0)) return fail(KAI_E_INVALID_ARG, "matmul_host: null operand");
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    HostPipe* hp = nullptr;
    KAI_TRY(pipe_for(device, &hp));

    // Row chunks of X: the upload of chunk i+1 and the download of chunk i-1 run while chunk i is multiplied.
    int64_t chunk = M;
    if (M >= 4096 && N * K >= (int64_t(1) << 22)) chunk = 512;    // measured against 1024 and 2048 at 8192^3: 95.8 / 93.1 / 87.8 TFLOP/s
    // Row ranges: `chunk` rows each, except that the last range is cut into 1/2, 1/4, 1/4 -- the upload is the longest
    // leg, and what remains after its last byte is the product and the download of the final range (8192^3: about
    // 0.1 ms of 11.3, within the spread between boxes).  Ranges that start large (M/4 rows, whole device buffers for X
    // and Y) measured clearly slower, 12.3 ms: the downloads then bunch up behind the late first products and
    // outlast the upload.
    std::vector<int64_t> starts;
    for (int64_t r = 0; r < M; ) {
        starts.push_back(r);
        const int64_t left = M - r;
        int64_t rows = chunk;
        if (chunk < M && left <= chunk && left >= 256) rows = (left * 4 > chunk) ? left / 2 : left;
        if (rows > left) rows = left;
        r += rows;
    }
    starts.push_back(M);
    const int64_t nchunks = static_cast<int64_t>(starts.size()) - 1;
    void *dW = nullptr, *dWlo = nullptr, *dX[2] = {nullptr, nullptr}, *dY[2] = {nullptr, nullptr}, *dB = nullptr, *dAlpha = nullptr;
    const bool w_lo = !wp && (K & 3) == 0 && K > 0 && nchunks > 1;      // split W once for all chunks
    int rc = KAI_OK;
    auto alloc = [&](void** p, int64_t bytes) { if (rc == KAI_OK) rc = kai_mem_alloc(device, bytes > 0 ? bytes : 4, p); };
    if (!wp) alloc(&dW, N * K * 4);
    if (w_lo) alloc(&dWlo, N * K * 4);
    for (int i = 0; i < (nchunks > 1 ? 2 : 1); ++i) { alloc(&dX[i], chunk * K * 4); alloc(&dY[i], chunk * N * 4); }
    if (pb_host) alloc(&dB, N * 4);
    alloc(&dAlpha, 4);
    cudaStream_t s_mm = nullptr;     // legacy default stream: ordered with the caller's other work on it
    if (rc == KAI_OK) {
        cudaError_t e = cudaSuccess;
        auto chk = [&](cudaError_t x) { if (e == cudaSuccess) e = x; };
        // uploads of W (and bias) start after work already queued on the compute stream
        chk(cudaEventRecord(hp->b_done, s_mm));
        chk(cudaStreamWaitEvent(hp->s_in, hp->b_done, 0));
        if (K > 0 && !wp) chk(cudaMemcpyAsync(dW, pw_host, N * K * 4, cudaMemcpyHostToDevice, hp->s_in));
        if (pb_host) chk(cudaMemcpyAsync(dB, pb_host, N * 4, cudaMemcpyHostToDevice, hp->s_in));
        chk(cudaMemcpyAsync(dAlpha, &leaky_alpha, 4, cudaMemcpyHostToDevice, hp->s_in));
        chk(cudaEventRecord(hp->b_done, hp->s_in));
        chk(cudaStreamWaitEvent(s_mm, hp->b_done, 0));
        if (e == cudaSuccess && w_lo) {
            rc = split_lo_pair(static_cast<const float*>(dW), nullptr, N * K, static_cast<float*>(dWlo), nullptr, s_mm);
        }
        const Epilogue ep{static_cast<const float*>(dB), static_cast<const float*>(dAlpha), act, 0};
        PlanePair wplanes{nullptr, nullptr, 0, 0};
        if (wp) wplanes = PlanePair{wp->hi, wp->lo, wp->kp, wp->xfmt};
        for (int64_t i = 0; i < nchunks && rc == KAI_OK && e == cudaSuccess; ++i) {
            const int buf = static_cast<int>(i & 1);
            const int64_t r0 = starts[i], rows = starts[i + 1] - r0;
            // the buffer pair is free once chunk i-2 has been multiplied (X) and downloaded (Y)
            if (i >= 2) {
                chk(cudaStreamWaitEvent(hp->s_in, hp->mm_done[buf], 0));
                chk(cudaStreamWaitEvent(s_mm, hp->out_done[buf], 0));
            }
            if (K > 0) chk(cudaMemcpyAsync(dX[buf], px_host + r0 * K, rows * K * 4, cudaMemcpyHostToDevice, hp->s_in));
            chk(cudaEventRecord(hp->in_done[buf], hp->s_in));
            chk(cudaStreamWaitEvent(s_mm, hp->in_done[buf], 0));
            if (e != cudaSuccess) break;
            as_stream(s_mm);    // refresh the capture state for this thread (none: legacy stream)
            const double flops = 2.0 * static_cast<double>(rows) * static_cast<double>(N) * static_cast<double>(K);
            if (wp)
                rc = gemm_tc(st, device, KAI_GEMM_NT, static_cast<float*>(dY[buf]), static_cast<const float*>(dX[buf]),
                             nullptr, rows, N, K, N, ep, s_mm, nullptr, nullptr, &wplanes);
            else if (K == 0 || flops < static_cast<double>(options().tc_min_flops.load()) || rows < 32 || N < 32)
                rc = gemm_simt(KAI_GEMM_NT, static_cast<float*>(dY[buf]), static_cast<const float*>(dX[buf]),
                               static_cast<const float*>(dW), rows, N, K, N, ep, s_mm);
            else
                rc = gemm_tc(st, device, KAI_GEMM_NT, static_cast<float*>(dY[buf]), static_cast<const float*>(dX[buf]),
                             static_cast<const float*>(dW), rows, N, K, N, ep, s_mm,
                             w_lo ? static_cast<const float*>(dWlo) : nullptr);
            chk(cudaEventRecord(hp->mm_done[buf], s_mm));
            chk(cudaStreamWaitEvent(hp->s_out, hp->mm_done[buf], 0));
            chk(cudaMemcpyAsync(py_host + r0 * N, dY[buf], rows * N * 4, cudaMemcpyDeviceToHost, hp->s_out));
            chk(cudaEventRecord(hp->out_done[buf], hp->s_out));
        }
        // the call returns when the result is in host memory
        chk(cudaStreamSynchronize(hp->s_out));
        chk(cudaStreamSynchronize(s_mm));
        chk(cudaStreamSynchronize(hp->s_in));
        if (e != cudaSuccess && rc == KAI_OK) {
            cudaGetLastError();
            rc = fail(static_cast<int>(e), "cuda:%s", cudaGetErrorString(e));
        }
    }
    for (void* p : {dW, dWlo, dX[0], dX[1], dY[0], dY[1], dB, dAlpha})
        if (p) kai_mem_free(device, p);
    return rc;
}

int kai_matmul_host(int device, float* py_host, const float* pw_host, const float* px_host, int64_t yvec, int64_t ndat,
                    int64_t xvec, const float* pb_host, int act, float leaky_alpha) {
    return matmul_host_impl(device, py_host, pw_host, nullptr, px_host, yvec, ndat, xvec, pb_host, act, leaky_alpha);
}

int kai_linear_forward_host(int device, float* py_host, void* w_prep, const float* px_host, int64_t ndat,
                            const float* pb_host, int act, float leaky_alpha) {
    const Prepared* wp = as_prepared(w_prep);
    if (!wp) return fail(KAI_E_INVALID_ARG, "linear_forward_host: not a prepared operand");
    if (wp->device != device) return fail(KAI_E_INVALID_ARG, "linear_forward_host: operand prepared on another device");
    return matmul_host_impl(device, py_host, nullptr, wp, px_host, wp->rows, ndat, wp->k, pb_host, act, leaky_alpha);
}

int kai_matmul(int device, float* py, const float* pw, const float* px, int64_t yvec, int64_t ndat, int64_t xvec,
               int acc, void* stream) {
    return kai_sgemm(device, KAI_GEMM_NT, py, px, pw, ndat, yvec, xvec, yvec, acc, nullptr, KAI_ACT_NONE, nullptr,
                     KAI_PATH_AUTO, stream);
}

int kai_matmul_backward_x(int device, float* pgx, const float* pgy, const float* pw, int64_t yvec, int64_t ndat,
                          int64_t xvec, int acc, void* stream) {
    // pgx[ndat,xvec] = pgy[ndat,yvec] . pw[yvec,xvec]: M = ndat, N = xvec, K = yvec
    return kai_sgemm(device, KAI_GEMM_NN, pgx, pgy, pw, ndat, xvec, yvec, xvec, acc, nullptr, KAI_ACT_NONE, nullptr,
                     KAI_PATH_AUTO, stream);
}

int kai_matmul_backward_w(int device, float* pgw, const float* pgy, const float* px, int64_t yvec, int64_t ndat,
                          int64_t xvec, int acc, void* stream) {
    // pgw[yvec,xvec] = pgy[ndat,yvec]^T . px[ndat,xvec]: M = yvec, N = xvec, K = ndat
    return kai_sgemm(device, KAI_GEMM_TN, pgw, pgy, px, yvec, xvec, ndat, xvec, acc, nullptr, KAI_ACT_NONE, nullptr,
                     KAI_PATH_AUTO, stream);
}

int kai_linear_forward(int device, float* py, const float* pw, const float* px, const float* pb, int64_t yvec,
                       int64_t ndat, int64_t xvec, int64_t ldy, int act, const float* leaky_alpha, void* stream) {
    return kai_sgemm(device, KAI_GEMM_NT, py, px, pw, ndat, yvec, xvec, ldy, 0, pb, act, leaky_alpha, KAI_PATH_AUTO,
                     stream);
}

// ---- prepared operands ------------------------------------------------------------------------

int kai_operand_prepare(int device, const float* src, int64_t rows, int64_t k, int64_t ld, int transpose, int flags,
                        void** out_handle, void* stream) {
    if (!out_handle) return fail(KAI_E_INVALID_ARG, "operand_prepare: null out_handle");
    *out_handle = nullptr;
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    if (!src || rows < 1 || k < 1) return fail(KAI_E_INVALID_ARG, "operand_prepare: null source or empty extent");
    if (rows >= (int64_t(1) << 31) || k >= (int64_t(1) << 31)) return fail(KAI_E_TOO_LARGE, "operand_prepare: extent exceeds 2^31-1");
    if (ld < (transpose ? rows : k)) return fail(KAI_E_INVALID_ARG, "operand_prepare: ld smaller than a source row");
    if (flags & ~(KAI_PREP_RAW_HI | KAI_PREP_LEFT | KAI_PREP_TF32_LO))
        return fail(KAI_E_INVALID_ARG, "operand_prepare: unknown flag");
    const bool raw = (flags & KAI_PREP_RAW_HI) != 0;
    if (raw && (transpose || ld != k || (k & 3) != 0 || (reinterpret_cast<uintptr_t>(src) & 15) != 0))
        return fail(KAI_E_INVALID_ARG, "operand_prepare: KAI_PREP_RAW_HI needs a dense, 16-byte aligned, untransposed "
                                       "source with k %% 4 == 0");
    if (capturing()) return fail(KAI_E_ALLOC, "operand_prepare: allocates; call it outside a stream capture");
    const int64_t kp = (k + 3) / 4 * 4;
    const int64_t plane = (rows * kp * 4 + 255) / 256 * 256;
    Prepared* p = new Prepared();
    p->device = device; p->rows = rows; p->k = k; p->kp = kp; p->ld = ld; p->transpose = transpose ? 1 : 0;
    p->raw_hi = raw;
    // long reductions take the mixed scheme (cross terms as one BF16 MMA): the second plane is then written for
    // the side of the product the operand will stand on
    // (not next to a raw hi plane: the lo part against a truncated hi is too large for bf16)
    if (!raw && !(flags & KAI_PREP_TF32_LO) && options().tc_cross_bf16.load() != 0 && k >= 2048 && (k & 7) == 0)
        p->xfmt = (flags & KAI_PREP_LEFT) ? 1 : 2;
    int rc = kai_mem_alloc(device, raw ? plane : 2 * plane, &p->block);
    if (rc != KAI_OK) { delete p; return rc; }
    p->lo = static_cast<float*>(p->block);
    p->hi = raw ? const_cast<float*>(src) : reinterpret_cast<float*>(static_cast<uint8_t*>(p->block) + plane);
    register_prepared(p, true);
    rc = kai_operand_refresh(p, src, stream);
    if (rc != KAI_OK) { register_prepared(p, false); kai_mem_free(device, p->block); delete p; return rc; }
    *out_handle = p;
    return KAI_OK;
}

int kai_operand_refresh(void* handle, const float* src, void* stream) {
    Prepared* p = as_prepared(handle);
    if (!p) return fail(KAI_E_INVALID_ARG, "operand_refresh: not a prepared operand");
    if (!src) return fail(KAI_E_INVALID_ARG, "operand_refresh: null source");
    if (p->raw_hi && src != p->hi)
        return fail(KAI_E_INVALID_ARG, "operand_refresh: a KAI_PREP_RAW_HI operand is tied to the matrix it was prepared from");
    DeviceState* st = nullptr;
    KAI_TRY(get_device(p->device, &st));
    DeviceGuard g;
    KAI_TRY(g.enter(p->device));
    cudaStream_t s = as_stream(stream);
    return split_operand(src, p->rows, p->k, p->ld, p->transpose != 0, p->raw_hi ? nullptr : p->hi, p->lo, st->sm_count, s,
                         p->xfmt);
}

int kai_operand_release(void* handle) {
    if (!handle) return KAI_OK;
    Prepared* p = as_prepared(handle);
    if (!p) return fail(KAI_E_INVALID_ARG, "operand_release: not a prepared operand");
    // The block returns to the caching allocator; work that reuses it is ordered behind queued kernels only
    // on the same stream, so wait for the device before handing it out again.
    DeviceGuard g;
    KAI_TRY(g.enter(p->device));
    KAI_CUDA(cudaDeviceSynchronize());
    const int rc = kai_mem_free(p->device, p->block);
    register_prepared(p, false);
    p->magic = 0;
    delete p;
    return rc;
}

int kai_sgemm_prepared(int device, float* c, void* a_prep, int64_t a_row0, int64_t M, void* b_prep, int64_t b_row0,
                       int64_t N, int64_t ldc, int accumulate, const float* bias, int act, const float* leaky_alpha,
                       void* stream) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    Prepared* pa = as_prepared(a_prep);
    Prepared* pb = as_prepared(b_prep);
    if (!pa || !pb) return fail(KAI_E_INVALID_ARG, "sgemm_prepared: not a prepared operand");
    if (pa->device != device || pb->device != device) return fail(KAI_E_INVALID_ARG, "sgemm_prepared: operand prepared on another device");
    if (pa->k != pb->k) return fail(KAI_E_INVALID_ARG, "sgemm_prepared: reduction lengths differ (%lld vs %lld)", (long long)pa->k, (long long)pb->k);
    if (M < 0 || N < 0 || a_row0 < 0 || b_row0 < 0 || a_row0 + M > pa->rows || b_row0 + N > pb->rows)
        return fail(KAI_E_INVALID_ARG, "sgemm_prepared: row range outside the prepared operand");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "sgemm_prepared: activation %d is not an elementwise epilogue", act);
    if (M == 0 || N == 0) return KAI_OK;
    if (!c) return fail(KAI_E_INVALID_ARG, "sgemm_prepared: null output");
    if (ldc < N) return fail(KAI_E_INVALID_ARG, "sgemm_prepared: ldc < N");
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    cudaStream_t s = as_stream(stream);
    const Epilogue ep{bias, leaky_alpha, act, accumulate ? 1 : 0};
    if (pa->xfmt == 2)
        return fail(KAI_E_INVALID_ARG, "sgemm_prepared: a_prep was prepared as a right operand; prepare it with KAI_PREP_LEFT");
    if (pb->xfmt == 1)
        return fail(KAI_E_INVALID_ARG, "sgemm_prepared: b_prep was prepared with KAI_PREP_LEFT");
    const PlanePair a{pa->hi + a_row0 * pa->kp, pa->lo + a_row0 * pa->kp, pa->kp, pa->xfmt};
    const PlanePair b{pb->hi + b_row0 * pb->kp, pb->lo + b_row0 * pb->kp, pb->kp, pb->xfmt};
    return gemm_tc(st, device, KAI_GEMM_NT, c, nullptr, nullptr, M, N, pa->k, ldc, ep, s, nullptr, &a, &b);
}

int kai_linear_forward_prepared(int device, float* py, void* w_prep, const float* px, const float* pb, int64_t ndat,
                                int64_t ldy, int act, const float* leaky_alpha, void* stream) {
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    Prepared* pw = as_prepared(w_prep);
    if (!pw) return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: not a prepared operand");
    if (pw->device != device) return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: operand prepared on another device");
    if (ndat < 0) return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: negative ndat");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: activation %d is not an elementwise epilogue", act);
    if (ndat == 0) return KAI_OK;
    if (!py || !px) return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: null operand");
    if (ldy < pw->rows) return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: ldy < yvec");
    DeviceGuard g;
    KAI_TRY(g.enter(device));
    cudaStream_t s = as_stream(stream);
    const Epilogue ep{pb, leaky_alpha, act, 0};
    if (pw->xfmt == 1)
        return fail(KAI_E_INVALID_ARG, "linear_forward_prepared: the weight was prepared with KAI_PREP_LEFT");
    const PlanePair b{pw->hi, pw->lo, pw->kp, pw->xfmt};
    return gemm_tc(st, device, KAI_GEMM_NT, py, px, nullptr, ndat, pw->rows, pw->k, ldy, ep, s, nullptr, nullptr, &b);
}

// ---- elementwise -------------------------------------------------------------------------
#define KAI_ENTER(device)                     \
    DeviceState* st = nullptr;                \
    KAI_TRY(get_device(device, &st));         \
    DeviceGuard guard__;                      \
    KAI_TRY(guard__.enter(device));           \
    cudaStream_t s = as_stream(stream)

int kai_add_bias(int device, float* py, const float* pa, const float* pb, int64_t nrow, int64_t ncol, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "add_bias: negative extent");
    if (nrow * ncol == 0) return KAI_OK;
    if (!py || !pa || !pb) return fail(KAI_E_INVALID_ARG, "add_bias: null pointer");
    return ew_add_bias(st, py, pa, pb, nrow, ncol, s);
}

int kai_add_bias_backward_b(int device, float* pgb, const float* pgy, int64_t nrow, int64_t ncol, int acc,
                            void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "add_bias_backward_b: negative extent");
    if (ncol == 0) return KAI_OK;
    if (!pgb || (!pgy && nrow > 0)) return fail(KAI_E_INVALID_ARG, "add_bias_backward_b: null pointer");
    return ew_colsum(st, device, pgb, pgy, nrow, ncol, acc ? 1 : 0, s);
}

int kai_activate(int device, float* py, const float* px, int64_t nrow, int64_t ncol, int act,
                 const float* leaky_alpha, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "activate: negative extent");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SOFTMAX) return fail(KAI_E_INVALID_ARG, "activate: unknown function %d", act);
    if (nrow * ncol == 0) return KAI_OK;
    if (!py || !px) return fail(KAI_E_INVALID_ARG, "activate: null pointer");
    return ew_activate(st, py, px, nrow, ncol, act, leaky_alpha, s);
}

int kai_activate_backward(int device, float* pgx, const float* pgy, const float* px, int64_t nrow, int64_t ncol,
                          int act, const float* leaky_alpha, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "activate_backward: negative extent");
    // The reference has no softmax case here (vmath.cu:3247-3330 falls into its default: throw).
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "activate_backward: unknown function %d", act);
    if (nrow * ncol == 0) return KAI_OK;
    if (!pgx || !pgy || !px) return fail(KAI_E_INVALID_ARG, "activate_backward: null pointer");
    return ew_activate_backward(st, pgx, pgy, px, nrow * ncol, act, leaky_alpha, 0, s);
}

int kai_activate_backward_with_y(int device, float* pgx, const float* pgy, const float* py, int64_t nrow,
                                 int64_t ncol, int act, const float* leaky_alpha, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "activate_backward_with_y: negative extent");
    if (act < KAI_ACT_NONE || act > KAI_ACT_TANH)
        return fail(KAI_E_INVALID_ARG, "activate_backward_with_y: function %d has no from-output gradient", act);
    if (nrow * ncol == 0) return KAI_OK;
    if (!pgx || !pgy || !py) return fail(KAI_E_INVALID_ARG, "activate_backward_with_y: null pointer");
    return ew_activate_backward(st, pgx, pgy, py, nrow * ncol, act, leaky_alpha, 1, s);
}

// ---- layernorm ----------------------------------------------------------------------------
int kai_layernorm(int device, float* py, const float* px, float* ps, int64_t nrow, int64_t ncol, const float* scale,
                  void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "layernorm: negative extent");
    if (nrow == 0) return KAI_OK;
    if (ncol == 0) return fail(KAI_E_INVALID_ARG, "layernorm: rows of length 0 have no mean");
    if (!py || !px || !ps) return fail(KAI_E_INVALID_ARG, "layernorm: null pointer");
    return ew_layernorm(py, px, ps, nrow, ncol, scale, s);
}

int kai_layernorm_backward(int device, float* pgx, const float* pgy, const float* ps, int64_t nrow, int64_t ncol,
                           const float* scale, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "layernorm_backward: negative extent");
    if (nrow * ncol == 0) return KAI_OK;
    if (!pgx || !pgy || !ps) return fail(KAI_E_INVALID_ARG, "layernorm_backward: null pointer");
    return ew_layernorm_backward(pgx, pgy, ps, nrow, ncol, scale, s);
}

// ---- grouped GEMM -------------------------------------------------------------------------
int kai_sgemm_grouped(int device, int layout, int count, float* const* c, const float* const* a, const float* const* b,
                      int64_t M, int64_t N, int64_t K, int64_t ldc, int accumulate, const float* bias, int act,
                      const float* leaky_alpha, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (layout < KAI_GEMM_NT || layout > KAI_GEMM_TN) return fail(KAI_E_INVALID_ARG, "sgemm_grouped: unknown layout %d", layout);
    if (count < 0 || M < 0 || N < 0 || K < 0) return fail(KAI_E_INVALID_ARG, "sgemm_grouped: negative count or dimension");
    if (act < KAI_ACT_NONE || act > KAI_ACT_SWISH)
        return fail(KAI_E_INVALID_ARG, "sgemm_grouped: activation %d is not an elementwise epilogue", act);
    if (count == 0 || M == 0 || N == 0) return KAI_OK;
    if (!c || !a || !b) return fail(KAI_E_INVALID_ARG, "sgemm_grouped: null pointer list");
    for (int i = 0; i < count; ++i)
        if (!c[i] || ((!a[i] || !b[i]) && K > 0)) return fail(KAI_E_INVALID_ARG, "sgemm_grouped: null operand in group %d", i);
    if (ldc < N) return fail(KAI_E_INVALID_ARG, "sgemm_grouped: ldc < N");
    const Epilogue ep{bias, leaky_alpha, act, accumulate ? 1 : 0};
    return gemm_simt_grouped(layout, count, c, a, b, M, N, K, ldc, ep, s);
}

// ---- attention ---------------------------------------------------------------------------
int kai_mult_on_heads(int device, float* pp, const float* pK, const float* pQ, int64_t nbat, int64_t ntimes,
                      int64_t nvec, int64_t nhead, int64_t npiece, const float* coef, void* stream) {
    KAI_ENTER(device);
    if (nbat < 0 || ntimes < 0 || nhead < 0 || npiece < 0) return fail(KAI_E_INVALID_ARG, "mult_on_heads: negative extent");
    if (nvec != nhead * npiece) return fail(KAI_E_INVALID_ARG, "mult_on_heads: nvec != nhead * npiece");
    if (nbat * ntimes * nhead == 0) return KAI_OK;
    if (!pp || !pK || !pQ) return fail(KAI_E_INVALID_ARG, "mult_on_heads: null pointer");
    if (options().attn_path.load() == 0) {
        const int rc = attn_mult_on_heads_tc(st, device, pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, coef, s);
        if (rc != 1) return rc;   // 1 = shape outside the tcgen05 fast path
    }
    return attn_mult_on_heads(pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, coef, s);
}

int kai_set_mh_attention_mask(int device, float* pp, int64_t ndat, int64_t ntimes, int64_t nhead, int forward,
                              void* stream) {
    KAI_ENTER(device);
    if (ndat < 0 || ntimes < 0 || nhead < 0) return fail(KAI_E_INVALID_ARG, "set_mh_attention_mask: negative extent");
    if (ndat * ntimes * nhead == 0) return KAI_OK;
    if (!pp) return fail(KAI_E_INVALID_ARG, "set_mh_attention_mask: null pointer");
    return attn_mask(st, pp, ndat, ntimes, nhead, forward ? 1 : 0, s);
}

int kai_softmax_direct_on_axis(int device, float* pp, int64_t nrow, int64_t nvec, int64_t ncol, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nrow < 0 || nvec < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "softmax_direct_on_axis: negative extent");
    if (nrow * nvec * ncol == 0) return KAI_OK;
    if (!pp) return fail(KAI_E_INVALID_ARG, "softmax_direct_on_axis: null pointer");
    return attn_softmax_axis(pp, nrow, nvec, ncol, s);
}

int kai_mix_values(int device, float* py, const float* pp, const float* pV, int64_t nbat, int64_t ntimes,
                   int64_t nvec, int64_t nhead, int64_t npiece, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nbat < 0 || ntimes < 0 || nhead < 0 || npiece < 0) return fail(KAI_E_INVALID_ARG, "mix_values: negative extent");
    if (nvec != nhead * npiece) return fail(KAI_E_INVALID_ARG, "mix_values: nvec != nhead * npiece");
    if (nbat * ntimes * nvec == 0) return KAI_OK;
    if (!py || !pp || !pV) return fail(KAI_E_INVALID_ARG, "mix_values: null pointer");
    if (options().attn_path.load() == 0) {
        const int rc = attn_mix_values_tc(st, device, py, pp, pV, nbat, ntimes, nvec, nhead, npiece, s);
        if (rc != 1) return rc;   // 1 = shape outside the tcgen05 fast path
    }
    return attn_mix_values(py, pp, pV, nbat, ntimes, nvec, nhead, npiece, s);
}

// ---- convolution -----------------------------------------------------------------------------
static int conv_check(const char* name, int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh,
                      int64_t yw, int64_t kh, int64_t kw, int64_t group) {
    if (ndat < 0 || xchn < 0 || xh < 0 || xw < 0 || ychn < 0 || yh < 0 || yw < 0 || kh < 0 || kw < 0)
        return fail(KAI_E_INVALID_ARG, "%s: negative extent", name);
    if (group < 1 || xchn % group != 0) return fail(KAI_E_INVALID_ARG, "%s: xchn %% group != 0", name);
    return KAI_OK;
}

int kai_conv2d(int device, float* py, const float* px, const float* pk, int64_t ndat, int64_t ychn, int64_t yh,
               int64_t yw, int64_t xchn, int64_t xh, int64_t xw, int64_t kh, int64_t kw, int64_t group, int64_t ph,
               int64_t pw, int pmode, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_check("conv2d", ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group));
    (void)pmode;   // the reference skips out-of-range taps whatever the mode (vmath.cu:3509-3512, 3552-3555): zero padding
    if (ndat * ychn * yh * yw == 0) return KAI_OK;
    if (!py || ((!px || !pk) && xchn * kh * kw > 0)) return fail(KAI_E_INVALID_ARG, "conv2d: null pointer");
    return conv2d_forward(st, device, py, px, pk, ndat, ychn, yh, yw, xchn, xh, xw, kh, kw, group, ph, pw, 1, 1, s);
}

int kai_conv2d_backward_x(int device, float* pgx, const float* pgy, const float* pk, int64_t ndat, int64_t xchn,
                          int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                          int64_t group, int64_t ph, int64_t pw, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_check("conv2d_backward_x", ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group));
    if (ndat * xchn * xh * xw == 0) return KAI_OK;
    if (!pgx || ((!pgy || !pk) && ychn * kh * kw > 0)) return fail(KAI_E_INVALID_ARG, "conv2d_backward_x: null pointer");
    return conv2d_backward_x(st, device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, 1, 1, s);
}

int kai_conv2d_backward_k(int device, float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn,
                          int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw, int64_t kh, int64_t kw,
                          int64_t group, int64_t ph, int64_t pw, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_check("conv2d_backward_k", ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group));
    if (ychn * (xchn / group) * kh * kw == 0) return KAI_OK;
    if (!pgk || ((!pgy || !px) && ndat * yh * yw > 0)) return fail(KAI_E_INVALID_ARG, "conv2d_backward_k: null pointer");
    return conv2d_backward_k(st, device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, yh, yw, kh, kw, group, ph, pw, 1, 1, s);
}

static int conv_variant_check(const char* name, const void* out, const void* a, const void* b, int64_t ndat,
                              int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t p0,
                              int64_t p1) {
    if (ndat < 0 || xchn < 0 || xh < 0 || xw < 0 || ychn < 0 || kh < 1 || kw < 1)
        return fail(KAI_E_INVALID_ARG, "%s: bad extent", name);
    if (p0 < 1 || p1 < 1) return fail(KAI_E_INVALID_ARG, "%s: stride / gap must be >= 1", name);
    if (!out || !a || !b) return fail(KAI_E_INVALID_ARG, "%s: null pointer", name);
    return KAI_OK;
}

int kai_conv2d_transposed(int device, float* py, const float* px, const float* pk, int64_t ndat, int64_t xchn,
                          int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                          void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_transposed", py, px, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw));
    return conv2d_transposed_any(st, device, 0, py, px, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, s);
}
int kai_conv2d_transposed_backward_x(int device, float* pgx, const float* pgy, const float* pk, int64_t ndat,
                                     int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                                     int64_t sh, int64_t sw, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_transposed_backward_x", pgx, pgy, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw));
    return conv2d_transposed_any(st, device, 1, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, s);
}
int kai_conv2d_transposed_backward_k(int device, float* pgk, const float* pgy, const float* px, int64_t ndat,
                                     int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                                     int64_t sh, int64_t sw, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_transposed_backward_k", pgk, pgy, px, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw));
    return conv2d_transposed_any(st, device, 2, pgk, pgy, px, ndat, xchn, xh, xw, ychn, kh, kw, sh, sw, s);
}

// conv2d_dilated family: an ordinary same-size convolution whose taps are gh / gw apart, centred on (kh-1)/2.
int kai_conv2d_dilated(int device, float* py, const float* px, const float* pk, int64_t ndat, int64_t xchn, int64_t xh,
                       int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh, int64_t gw, void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_dilated", py, px, pk, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw));
    if (ndat * ychn * xh * xw == 0) return KAI_OK;
    return conv2d_forward(st, device, py, px, pk, ndat, ychn, xh, xw, xchn, xh, xw, kh, kw, 1, (kh - 1) / 2, (kw - 1) / 2,
                          gh, gw, s);
}
int kai_conv2d_dilated_backward_x(int device, float* pgx, const float* pgy, const float* pk, int64_t ndat, int64_t xchn,
                                  int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh, int64_t gw,
                                  void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_dilated_backward_x", pgx, pgy, pk, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw));
    if (ndat * xchn * xh * xw == 0) return KAI_OK;
    return conv2d_backward_x(st, device, pgx, pgy, pk, ndat, xchn, xh, xw, ychn, xh, xw, kh, kw, 1, (kh - 1) / 2,
                             (kw - 1) / 2, gh, gw, s);
}
int kai_conv2d_dilated_backward_k(int device, float* pgk, const float* pgy, const float* px, int64_t ndat, int64_t xchn,
                                  int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw, int64_t gh, int64_t gw,
                                  void* stream) {
    KAI_ENTER(device);
    KAI_TRY(conv_variant_check("conv2d_dilated_backward_k", pgk, pgy, px, ndat, xchn, xh, xw, ychn, kh, kw, gh, gw));
    if (ychn * xchn * kh * kw == 0) return KAI_OK;
    return conv2d_backward_k(st, device, pgk, pgy, px, ndat, xchn, xh, xw, ychn, xh, xw, kh, kw, 1, (kh - 1) / 2,
                             (kw - 1) / 2, gh, gw, s);
}

// ---- fused attention forward ----------------------------------------------------------------
int kai_mh_attention_forward(int device, float* py, const float* pK, const float* pQ, const float* pV,
                             int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece,
                             const float* coef, int causal_mask, void* stream) {
    KAI_ENTER(device);
    if (nbat < 0 || ntimes < 0 || nhead < 0 || npiece < 0)
        return fail(KAI_E_INVALID_ARG, "mh_attention_forward: negative extent");
    if (nvec != nhead * npiece) return fail(KAI_E_INVALID_ARG, "mh_attention_forward: nvec != nhead * npiece");
    if (nbat * ntimes * nvec == 0) return KAI_OK;
    if (!py || !pK || !pQ || !pV) return fail(KAI_E_INVALID_ARG, "mh_attention_forward: null pointer");
    if (options().attn_path.load() == 0) {
        const int rc = attn_fused_forward_tc(st, device, py, pK, pQ, pV, nbat, ntimes, nvec, nhead, npiece, coef,
                                             causal_mask, s);
        if (rc != 1) return rc;   // 1 = shape outside the fused path
    }
    // Other shapes: the three reference steps through a probs block from the caching allocator.  The block
    // goes back to the cache right away; work that reuses it is ordered behind these kernels on `stream`.
    if (capturing())
        return fail(KAI_E_ALLOC, "mh_attention_forward: this shape needs a scratch block and cannot be recorded");
    void* probs = nullptr;
    KAI_TRY(kai_mem_alloc(device, nbat * ntimes * ntimes * nhead * 4, &probs));
    float* pp = static_cast<float*>(probs);
    int rc = kai_mult_on_heads(device, pp, pK, pQ, nbat, ntimes, nvec, nhead, npiece, coef, stream);
    if (rc == KAI_OK && causal_mask) rc = kai_set_mh_attention_mask(device, pp, nbat, ntimes, nhead, 1, stream);
    if (rc == KAI_OK) rc = kai_softmax_direct_on_axis(device, pp, nbat * ntimes, ntimes, nhead, stream);
    if (rc == KAI_OK) rc = kai_mix_values(device, py, pp, pV, nbat, ntimes, nvec, nhead, npiece, stream);
    const int rc_free = kai_mem_free(device, probs);
    return rc != KAI_OK ? rc : rc_free;
}

// ---- attention backward -------------------------------------------------------------------
int kai_mult_on_heads_backward(int device, float* pgQK, const float* pgp, const float* pKQ, int64_t nbat,
                               int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, void* stream) {
    // pgQK[b,t,h,p] = sum_k pgp[b,t,k,h] * pKQ[b,k,h*P+p]: index for index the mix_values contraction.
    return kai_mix_values(device, pgQK, pgp, pKQ, nbat, ntimes, nvec, nhead, npiece, stream);
}

int kai_mix_values_backward_prop(int device, float* pgp, const float* pgy, const float* pV, int64_t nbat,
                                 int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, void* stream) {
    // pgp[b,q,k,h] = sum_p pgy[b,q,h,p] * pV[b,k,h*P+p]: the mult_on_heads contraction with coef = 1.
    DeviceState* st = nullptr;
    KAI_TRY(get_device(device, &st));
    return kai_mult_on_heads(device, pgp, pV, pgy, nbat, ntimes, nvec, nhead, npiece,
                             reinterpret_cast<const float*>(st->flag_dev) + 8, stream);
}

int kai_mix_values_backward_value(int device, float* pgV, const float* pgy, const float* pp, int64_t nbat,
                                  int64_t ntimes, int64_t nvec, int64_t nhead, int64_t npiece, void* stream) {
    KAI_ENTER(device);
    if (nbat < 0 || ntimes < 0 || nhead < 0 || npiece < 0)
        return fail(KAI_E_INVALID_ARG, "mix_values_backward_value: negative extent");
    if (nvec != nhead * npiece) return fail(KAI_E_INVALID_ARG, "mix_values_backward_value: nvec != nhead * npiece");
    if (nbat * ntimes * nvec == 0) return KAI_OK;
    if (!pgV || !pgy || !pp) return fail(KAI_E_INVALID_ARG, "mix_values_backward_value: null pointer");
    if (options().attn_path.load() == 0) {
        const int rc = attn_mix_values_tc(st, device, pgV, pp, pgy, nbat, ntimes, nvec, nhead, npiece, s, true);
        if (rc != 1) return rc;
    }
    return attn_mix_values(pgV, pp, pgy, nbat, ntimes, nvec, nhead, npiece, s, true);
}

int kai_softmax_direct_on_axis_backward(int device, float* pgp, const float* pp, int64_t nbat, int64_t ntimes,
                                        int64_t nhead, const float* coef, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nbat < 0 || ntimes < 0 || nhead < 0)
        return fail(KAI_E_INVALID_ARG, "softmax_direct_on_axis_backward: negative extent");
    if (nbat * ntimes * nhead == 0) return KAI_OK;
    if (!pgp || !pp) return fail(KAI_E_INVALID_ARG, "softmax_direct_on_axis_backward: null pointer");
    return attn_softmax_axis_backward(pgp, pp, nbat * ntimes, ntimes, nhead, coef, s);
}

// ---- loss --------------------------------------------------------------------------------
int kai_softmax_idx_crossentropy(int device, float* py, const float* px, const int* pz, int64_t nrow, int64_t ncol,
                                 void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "softmax_idx_crossentropy: negative extent");
    if (nrow == 0) return KAI_OK;
    if (ncol == 0) return fail(KAI_E_OUT_OF_RANGE, "softmax_idx_crossentropy: no classes");
    if (!py || !px || !pz) return fail(KAI_E_INVALID_ARG, "softmax_idx_crossentropy: null pointer");
    return ew_ce_forward(st, py, px, pz, nrow, ncol, s);
}

int kai_softmax_idx_crossentropy_backward_x(int device, float* pgx, const float* pgy, const float* px,
                                            const int* pz, int64_t nrow, int64_t ncol, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0 || ncol < 0) return fail(KAI_E_INVALID_ARG, "softmax_idx_crossentropy_backward_x: negative extent");
    if (nrow * ncol == 0) return KAI_OK;
    if (!pgx || !pgy || !px || !pz) return fail(KAI_E_INVALID_ARG, "softmax_idx_crossentropy_backward_x: null pointer");
    return ew_ce_backward(st, pgx, pgy, px, pz, nrow, ncol, s);
}

int kai_sum(int device, float* py, const float* px, int64_t nrow, void* stream) {
    KAI_ENTER(device);
    (void)st;
    if (nrow < 0) return fail(KAI_E_INVALID_ARG, "sum: negative extent");
    if (!py || (!px && nrow > 0)) return fail(KAI_E_INVALID_ARG, "sum: null pointer");
    return ew_sum(py, px, nrow, s);
}

int kai_sum_backward(int device, float* pgx, const float* pgy, int64_t nrow, void* stream) {
    KAI_ENTER(device);
    if (nrow < 0) return fail(KAI_E_INVALID_ARG, "sum_backward: negative extent");
    if (nrow == 0) return KAI_OK;
    if (!pgx) return fail(KAI_E_INVALID_ARG, "sum_backward: null pointer");
    return ew_sum_backward(st, pgx, pgy, nrow, s);
}

}  // extern "C"
