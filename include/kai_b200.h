/*
 * kai_b200.h -- C ABI of the B200 (sm_100a) matmul / Linear path.
 *
 * This is the boundary a host program binds to (ctypes, a C++ shim, ...).  Every entry
 * point takes plain pointers and sizes, returns 0 on success or a negative KAI_E_* /
 * positive cudaError_t value, and never throws.  The message of the last failure on the
 * calling thread is available through kai_last_error_string().
 *
 * Argument names, order and meaning follow the static methods of the reference engine's
 * `class VMath` (source/engine/support/vmath.h) that each entry point replaces; the
 * reference file:line is given beside each declaration.  In the reference notation
 *     ndat = rows of X (batch x tokens), xvec = input width, yvec = output width,
 * all matrices are dense row-major fp32, and `acc` means `+=` instead of `=`.
 *
 * `device` is the CUDA ordinal the pointers live on (the reference's `device >= 0`
 * branch).  There is no host branch: device < 0 returns KAI_E_NO_HOST_PATH.
 * `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream, which
 * is what the reference's kernels run on.
 *
 * HYPER arguments (`leaky_alpha`, `coef`) are `const float*` in the device's memory, as
 * in the reference (local_objects/vhypermanager.h:6-9); NULL reads as 0.
 */
#ifndef KAI_B200_H
#define KAI_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KAI_API __attribute__((visibility("default")))

/* ---- status codes -------------------------------------------------------------------- */
#define KAI_OK                 0
#define KAI_E_INVALID_ARG     -1   /* null pointer, negative size, unknown enum            */
#define KAI_E_NO_HOST_PATH    -2   /* device < 0: this library has no CPU branch           */
#define KAI_E_NO_DRIVER       -3   /* libcuda entry point (tensor-map encode) unavailable  */
#define KAI_E_TENSOR_MAP      -4   /* cuTensorMapEncodeTiled rejected the operand          */
#define KAI_E_DEVICE_WAIT     -5   /* a bounded device-side wait ran out (status word set) */
#define KAI_E_OUT_OF_RANGE    -6   /* label outside [0, ncol)                              */
#define KAI_E_TOO_LARGE       -7   /* size beyond a documented fixed limit                 */
#define KAI_E_ALLOC           -8   /* device allocation failed                             */

/* ---- enums --------------------------------------------------------------------------- */
/* Operand layouts of the three reference GEMMs. */
#define KAI_GEMM_NT 0   /* C[M,N] = A[M,K] . B[N,K]^T   (VMath::matmul)            */
#define KAI_GEMM_NN 1   /* C[M,N] = A[M,K] . B[K,N]     (VMath::matmul_backward_x) */
#define KAI_GEMM_TN 2   /* C[M,N] = A[K,M]^T . B[K,N]   (VMath::matmul_backward_w) */

/* Activation codes = the reference's enum ActFunc (include/vtypes.h:37-39). */
#define KAI_ACT_NONE    0
#define KAI_ACT_RELU    1
#define KAI_ACT_LEAKY   2
#define KAI_ACT_SIGMOID 3
#define KAI_ACT_TANH    4
#define KAI_ACT_GELU    5
#define KAI_ACT_SELU    6
#define KAI_ACT_MISH    7
#define KAI_ACT_SWISH   8
#define KAI_ACT_SOFTMAX 9

/* Kernel families kai_sgemm can be pinned to (KAI_PATH_AUTO picks by shape). */
#define KAI_PATH_AUTO   0
#define KAI_PATH_TC     1   /* TMA + tcgen05 split-fp32 tensor-core kernel      */
#define KAI_PATH_SIMT   2   /* shared-memory tiled fp32 FMA kernel (small/odd)  */
#define KAI_PATH_SKINNY 3   /* HBM-bound row-streaming kernel, M <= 16, NT only */

/* ---- library ------------------------------------------------------------------------- */
KAI_API const char* kai_version(void);
KAI_API const char* kai_last_error_string(void);
/* Synchronises `device` and returns the device-side status word (0, or KAI_E_DEVICE_WAIT
 * with the place a bounded wait gave up encoded in *detail when detail != NULL). */
KAI_API int kai_device_status(int device, int* detail);
/* Clears the status word after a reported KAI_E_DEVICE_WAIT (synchronises the device first), so that
 * one expired wait does not fail every later call of the process.  The reference has no such state:
 * its error convention is the synchronous cudaGetLastError after each launch (support/vmath.cu:64-87). */
KAI_API int kai_device_status_clear(int device);
/* Test hook of the failure-detection path (no counterpart in the reference): launches one small kernel
 * that waits -- with the bounded wait every kernel of this library uses -- on a barrier nothing arrives
 * at.  After `limit_ns` (1 us .. 1 s) the wait gives up and records KAI_E_DEVICE_WAIT with location
 * code 99; the kernel returns by itself and the context stays usable.  kai_device_status then reports
 * the code and kai_device_status_clear resets it. */
KAI_API int kai_selftest_bounded_wait(int device, int64_t limit_ns, void* stream);
/* Tuning switches, by name: "tc_bn" (128|256), "tc_bk" (16|32), "tc_min_flops",
 * "split_k" (0 = automatic), "path" (KAI_PATH_*), "tc_kc" (K per tensor-memory
 * accumulation chunk, 0 = chosen from K), "tc_group_m" (tile rasterisation), "tc_raw_hi",
 * "tc_balance", "tc_max_ctas" (CTAs of the persistent GEMM grid, 0 = one per SM; fewer leaves SMs to
 * kernels that must run beside it, e.g. a collective), "attn_path" (0 tensor-core kernels by shape,
 * 2 no tcgen05, 1 CUDA cores only), "skinny_mma" (1 = warp-MMA streaming kernel for M <= 16),
 * "skinny_rows", "skinny_regx", "conv_igemm" (1 = implicit-GEMM convolution kernels where they fit, 2 = only the one whose
 * tiles are formed by converter warps, 0 = explicit unfolding), "conv_wide" (1, the default: the TMA-fed kernel fetches
 * one operand box per kernel row and reads the row's taps from it through shifted descriptors; 0 = one box per tap), "conv_direct" (1 = the transposed family and
 * group != 1 on one-thread-per-output kernels that repeat the reference's loops bit for bit; 0 = on the GEMM kernels),
 * "tc_cross_bf16" (1, the default: products whose reduction has 2048 values or more, K % 8 == 0, form the
 * two cross terms hi.lo + lo.hi of every K step with one BF16 MMA -- 2^-21 of the product, measured 5.6e-7
 * relative, below the error of a sequential fp32 sum of that length; 0 = three TF32 MMAs per step always),
 * "tc_pair" (1, the default: products whose 256 x 256 tiles fill at least half a round of the SM pairs run on
 * pairs of CTAs with cta_group::2 MMAs -- 8192^3: 3.65 ms against 4.35 ms with one CTA per 128 x 256 tile; 0 = one
 * CTA per tile always), "tc_pair_bk" (K block of the pair kernel, 32 or 16).
 * Returns KAI_E_INVALID_ARG for an unknown name or value. */
KAI_API int kai_set_option(const char* name, int64_t value);
KAI_API int64_t kai_get_option(const char* name);
/* Number of kernels this library has launched since it was loaded (all devices). */
KAI_API int64_t kai_launch_count(void);
/* ... and how many of them were kernels that issue tcgen05.mma (the tensor-core GEMM, convolution and
 * attention kernels): lets a caller check which path a call took. */
KAI_API int64_t kai_tc_launch_count(void);
/* ... and how many of those were the CTA-pair form of the GEMM kernel (cta_group::2, option tc_pair). */
KAI_API int64_t kai_tc_pair_launch_count(void);
/* Kernel timing for benchmarks.  While enabled, every tensor-core GEMM call records CUDA
 * events on its stream around (0) the GEMM kernel, (1) the operand-split kernels and (2) the
 * split-K reduction.  kai_profile_read waits for the recorded events, returns the summed
 * milliseconds and the number of spans per kind in ms3[3] / launches3[3], and clears them. */
KAI_API int kai_profile_enable(int on);
KAI_API int kai_profile_read(double* ms3, int64_t* launches3);

/* ---- recorded call lists ------------------------------------------------------------------
 * The reference records the math calls of the first pass and replays that fixed list on every
 * later pass with the same pointers (local_objects/vexectracer.cpp:496-550, replay switch
 * :586-1192).  Here the list becomes one CUDA graph: kai_replay_begin starts a stream capture and
 * returns the stream to pass as `stream` to every call to be recorded (nothing executes while
 * recording); kai_replay_end closes the list; kai_replay_launch enqueues the whole list on
 * `stream` (NULL = legacy default stream) as a single launch.  Every compute entry point of this header
 * may be recorded except the synchronous ones (kai_matmul_host, kai_device_status, the allocator, and
 * kai_mh_attention_forward on shapes that fall back to the separate steps).  Run the list once un-recorded first: scratch memory is sized on that pass and may
 * not grow while recording (KAI_E_ALLOC).  A label outside its range in a replayed
 * kai_softmax_idx_crossentropy is reported by kai_device_status.  A capture the caller started on
 * its own stream is honoured the same way. */
KAI_API int kai_replay_begin(int device, void** out_handle, void** out_stream);
KAI_API int kai_replay_end(void* handle);
KAI_API int kai_replay_launch(void* handle, void* stream);
KAI_API int kai_replay_destroy(void* handle);

/* ---- allocator: VMath::mem_alloc / mem_free (support/vmath.cu:169-208, 243-264) ------- */
/* Blocks are >= 256-byte aligned and come from a per-device cache of freed blocks, so a
 * steady-state alloc/free pair makes no cudaMalloc/cudaFree call. */
KAI_API int kai_mem_alloc(int device, int64_t size, void** out_ptr);
KAI_API int kai_mem_free(int device, void* ptr);
/* Row-pitched block: *out_pitch_bytes is a multiple of 128, so every row start satisfies
 * the 16-byte rule of TMA descriptors. */
KAI_API int kai_mem_alloc_pitched(int device, int64_t rows, int64_t row_bytes,
                                  void** out_ptr, int64_t* out_pitch_bytes);
/* Returns cached blocks to the driver (cudaFree). */
KAI_API int kai_mem_trim(int device);
/* live_bytes / cached_bytes / number of cudaMalloc calls so far. */
KAI_API int kai_mem_stats(int device, int64_t* live_bytes, int64_t* cached_bytes,
                          int64_t* driver_allocs);

/* ---- the GEMM trio -------------------------------------------------------------------- */
/* VMath::matmul (vmath.h:137; vmath.cu:2961-3003):
 *   py[ndat,yvec] (+)= px[ndat,xvec] . pw[yvec,xvec]^T */
KAI_API int kai_matmul(int device, float* py, const float* pw, const float* px,
                       int64_t yvec, int64_t ndat, int64_t xvec, int acc, void* stream);
/* VMath::matmul_backward_x (vmath.h:138; vmath.cu:3007-3047):
 *   pgx[ndat,xvec] (+)= pgy[ndat,yvec] . pw[yvec,xvec] */
KAI_API int kai_matmul_backward_x(int device, float* pgx, const float* pgy, const float* pw,
                                  int64_t yvec, int64_t ndat, int64_t xvec, int acc,
                                  void* stream);
/* VMath::matmul_backward_w (vmath.h:139; vmath.cu:3051-3093):
 *   pgw[yvec,xvec] (+)= pgy[ndat,yvec]^T . px[ndat,xvec] */
KAI_API int kai_matmul_backward_w(int device, float* pgw, const float* pgy, const float* px,
                                  int64_t yvec, int64_t ndat, int64_t xvec, int acc,
                                  void* stream);
/* The `linear` / `dense` layer formulas, add(matmul(x,w),b) and activate(add(matmul(...)))
 * (api/vconst.cpp:10-11), as one launch:
 *   py[ndat,yvec] = act( px . pw^T + pb )       pb may be NULL, act may be KAI_ACT_NONE.
 * `ldy` is the row stride of py in floats (>= yvec); it lets a column-sharded caller write
 * its block straight into a full-width output.  KAI_ACT_SOFTMAX is not an epilogue
 * (row-wise): it returns KAI_E_INVALID_ARG; call kai_activate afterwards instead. */
KAI_API int kai_linear_forward(int device, float* py, const float* pw, const float* px,
                               const float* pb, int64_t yvec, int64_t ndat, int64_t xvec,
                               int64_t ldy, int act, const float* leaky_alpha, void* stream);
/* No counterpart in the reference (its engine uploads whole tensors with cudaMemcpy before a math call and
 * downloads results afterwards, e.g. graph_core/vgraph_node.cpp:177): py = act(px . pw^T + pb) with ALL buffers
 * in HOST memory (pinned memory gives asynchronous copies).  The rows of px are processed in chunks so that the
 * upload of the next chunk and the download of the previous one overlap the multiplication; pw is uploaded and
 * split once.  Synchronous: returns when py_host holds the result.  pb_host may be NULL. */
KAI_API int kai_matmul_host(int device, float* py_host, const float* pw_host, const float* px_host, int64_t yvec,
                            int64_t ndat, int64_t xvec, const float* pb_host, int act, float leaky_alpha);
/* kai_matmul_host with the weight device-resident as a prepared operand (kai_operand_prepare): only the
 * rows of px go up and the rows of py come down.  The reference re-uploads every parameter on each
 * forward pass (graph_core/vgraph_node.cpp:177); a parameter that stays on the device between calls is
 * uploaded and split once. */
KAI_API int kai_linear_forward_host(int device, float* py_host, void* w_prep, const float* px_host,
                                    int64_t ndat, const float* pb_host, int act, float leaky_alpha);
/* No counterpart in the reference: kai_linear_forward for callers that must not allocate.
 *
 * Same arguments and result as kai_linear_forward, computed by the same tensor-core kernel,
 * but the call makes no cudaMalloc / cudaFree (nor any other allocating call): the operand
 * planes the kernel needs as scratch live in a 32 MiB array that is part of the library image.
 * It is meant for hosts that cannot allocate while they run -- a recorded call list being
 * replayed with fixed pointers, or a process that has given all device memory to its own pool.
 *   - Limit: 8 * (ndat + yvec) * round_up(xvec, 4) bytes (+ 256-byte rounding per plane) must
 *     fit in 32 MiB, e.g. ndat = yvec = 1024 with xvec = 2048.  Larger problems return
 *     KAI_E_TOO_LARGE and compute nothing.  No split-K is used (it would need more scratch).
 *   - Cost: every GPU that loads the library carries the 32 MiB from load until exit.
 *   - The first call on a device looks up the device address of that array
 *     (cudaGetSymbolAddress) and sets a kernel attribute; make that first call before starting
 *     any stream capture.
 *   - All calls on a device share the one array, which keeps the last call's planes; each call
 *     overwrites everything it reads.  Two calls whose kernels overlap on the GPU (different
 *     streams, different host threads) race on it: keep calls on one device ordered.
 *   - xvec must be >= 1 (kai_linear_forward computes act(bias) for xvec == 0; this entry point
 *     returns KAI_E_INVALID_ARG).
 *   - A kernel of an EARLIER call that gave up a bounded wait is reported by the next call and by
 *     kai_device_status (KAI_E_DEVICE_WAIT); the status word lives in one page of the library's own
 *     host memory that the first call page-locks and maps (cudaHostRegister: nothing is allocated). */
KAI_API int kai_linear_forward_static(int device, float* py, const float* pw, const float* px,
                                      const float* pb, int64_t yvec, int64_t ndat,
                                      int64_t xvec, int64_t ldy, int act,
                                      const float* leaky_alpha, void* stream);
/* ---- prepared operands (no counterpart in the reference) -----------------------------------
 * The tensor-core kernel reads each operand as two K-major planes (hi / lo halves of every fp32 value).
 * A plain call writes them into scratch on every call; an operand that does not change between calls --
 * a Linear layer's weight changes only at the optimiser step -- can be prepared once:
 *   kai_operand_prepare   src is [rows][k] (transpose = 0) or [k][rows] (transpose != 0), row stride ld
 *                         floats; writes the planes into a block of the caching allocator and returns a
 *                         handle.  flags: KAI_PREP_RAW_HI keeps no hi plane and reads the caller's own
 *                         matrix instead (dense, 16-byte aligned, untransposed, k % 4 == 0; the matrix
 *                         must stay unchanged while the handle is used; half the memory).
 *                         For k >= 2048 (k % 8 == 0, option tc_cross_bf16 = 1, the default) the second
 *                         plane holds the bf16 cross-term operands of the mixed scheme, whose layout
 *                         depends on the side of the product: handles are written for the RIGHT side
 *                         (the weight of kai_linear_forward_prepared, b_prep) unless KAI_PREP_LEFT says
 *                         the handle will be passed as a_prep; the other side is refused.
 *                         KAI_PREP_TF32_LO keeps TF32 lo values whatever the length (such a handle works
 *                         on either side and makes its calls use three TF32 MMAs per step); so does
 *                         KAI_PREP_RAW_HI.
 *   kai_operand_refresh   re-splits new values of the same shape into the same planes (after an update
 *                         of the weights); capture-safe.
 *   kai_operand_release   returns the planes (synchronises the device).
 *   kai_linear_forward_prepared   kai_linear_forward with the weight given as a handle: yvec = rows,
 *                         xvec = k of the handle.
 *   kai_sgemm_prepared    C[M,N] (+)= A'[a_row0 .. +M) . B'[b_row0 .. +N)^T on two handles -- also the
 *                         way to compute a GEMM in row slabs of the output without splitting the
 *                         operands again for every slab.
 * Handles are explicit on purpose: nothing is cached by pointer value, so a recorded call list that is
 * replayed with the same arguments always computes on the planes its handles name. */
#define KAI_PREP_RAW_HI 1
#define KAI_PREP_LEFT 2
#define KAI_PREP_TF32_LO 4
KAI_API int kai_operand_prepare(int device, const float* src, int64_t rows, int64_t k, int64_t ld,
                                int transpose, int flags, void** out_handle, void* stream);
KAI_API int kai_operand_refresh(void* handle, const float* src, void* stream);
KAI_API int kai_operand_release(void* handle);
KAI_API int kai_linear_forward_prepared(int device, float* py, void* w_prep, const float* px,
                                        const float* pb, int64_t ndat, int64_t ldy, int act,
                                        const float* leaky_alpha, void* stream);
KAI_API int kai_sgemm_prepared(int device, float* c, void* a_prep, int64_t a_row0, int64_t M,
                               void* b_prep, int64_t b_row0, int64_t N, int64_t ldc, int accumulate,
                               const float* bias, int act, const float* leaky_alpha, void* stream);
/* `count` products of one shape in one launch: C_i (+)= op(A_i).op(B_i), i < count, pointer lists in
 * HOST memory (they are copied into the kernel's parameters).  This is the form of the recurrent
 * layers' input products (api_objects/vtensor.cpp:2456-2470: one VMath::matmul with acc = true per
 * timestep, each into its own interior slice): the T calls that do not depend on each other become
 * one launch.  The recurrent products (state of step t-1 -> step t) depend on each other and stay
 * single calls.  The outputs of one call must not overlap.  CUDA-core kernel (these products are a
 * few hundred MFLOP each); when the slices are contiguous, one kai_matmul over [T*ndat, ninp] on the
 * tensor-core path is the faster form. */
KAI_API int kai_sgemm_grouped(int device, int layout, int count, float* const* c, const float* const* a,
                              const float* const* b, int64_t M, int64_t N, int64_t K, int64_t ldc,
                              int accumulate, const float* bias, int act, const float* leaky_alpha,
                              void* stream);
/* General form all of the above reduce to.  C[M,N] (+)= op(A).op(B) with the layouts of
 * KAI_GEMM_*; `ldc` in floats; bias (length N) and act as in kai_linear_forward;
 * `path` = KAI_PATH_*.  A, B and C may be interior pointers (4-byte aligned). */
KAI_API int kai_sgemm(int device, int layout, float* c, const float* a, const float* b,
                      int64_t M, int64_t N, int64_t K, int64_t ldc, int accumulate,
                      const float* bias, int act, const float* leaky_alpha, int path,
                      void* stream);

/* ---- bias and activation -------------------------------------------------------------- */
/* VMath::add_bias (vmath.h:65; vmath.cu:875-897): py[r,c] = pa[r,c] + pb[c]; py may alias pa. */
KAI_API int kai_add_bias(int device, float* py, const float* pa, const float* pb,
                         int64_t nrow, int64_t ncol, void* stream);
/* VMath::add_bias_backward_b (vmath.h:66; vmath.cu:901-932): pgb[c] (+)= sum_r pgy[r,c]. */
KAI_API int kai_add_bias_backward_b(int device, float* pgb, const float* pgy, int64_t nrow,
                                    int64_t ncol, int acc, void* stream);
/* VMath::activate (vmath.h:141; vmath.cu:3097-3243); py may alias px. */
KAI_API int kai_activate(int device, float* py, const float* px, int64_t nrow, int64_t ncol,
                         int act, const float* leaky_alpha, void* stream);
/* VMath::activate_backward (vmath.h:142; vmath.cu:3247-3407): px is the PRE-activation. */
KAI_API int kai_activate_backward(int device, float* pgx, const float* pgy, const float* px,
                                  int64_t nrow, int64_t ncol, int act,
                                  const float* leaky_alpha, void* stream);
/* VMath::activate_backward_with_y (vmath.h:143; vmath.cu:3411-3486): py is the output;
 * only none/relu/leaky/sigmoid/tanh exist in the reference. */
KAI_API int kai_activate_backward_with_y(int device, float* pgx, const float* pgy,
                                         const float* py, int64_t nrow, int64_t ncol, int act,
                                         const float* leaky_alpha, void* stream);

/* VMath::layernorm (vmath.h:214; vmath.cu:5977-6053): per row r of px[nrow,ncol]
 *   avg = mean(x), std = sqrtf(mean((x - avg)^2) + 1e-10f), py = scale * ((px - avg) / std),
 *   ps[2r] = avg, ps[2r+1] = std.   `scale` is a HYPER (device pointer, NULL reads as 0). */
KAI_API int kai_layernorm(int device, float* py, const float* px, float* ps, int64_t nrow,
                          int64_t ncol, const float* scale, void* stream);
/* VMath::layernorm_backward (vmath.h:215; vmath.cu:6056-6087): pgx = scale * ((pgy - avg) / std) with the
 * statistics the forward saved in ps (the reference applies the forward's affine map to the gradient). */
KAI_API int kai_layernorm_backward(int device, float* pgx, const float* pgy, const float* ps,
                                   int64_t nrow, int64_t ncol, const float* scale, void* stream);

/* ---- attention (batched contractions) -------------------------------------------------- */
/* VMath::mult_on_heads (vmath.h:234; vmath.cu:6729-6779):
 *   pp[b,q,k,h] = coef * sum_p pK[b,k,h*npiece+p] * pQ[b,q,h*npiece+p]    (nvec = nhead*npiece) */
KAI_API int kai_mult_on_heads(int device, float* pp, const float* pK, const float* pQ,
                              int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                              int64_t npiece, const float* coef, void* stream);
/* VMath::set_mh_attention_mask (vmath.h:236; vmath.cu:6833-6860): pp[b,q,k,h] = -inf (forward)
 * or 0 (backward) where k > q. */
KAI_API int kai_set_mh_attention_mask(int device, float* pp, int64_t ndat, int64_t ntimes,
                                      int64_t nhead, int forward, void* stream);
/* VMath::softmax_direct_on_axis (vmath.h:237; vmath.cu:6864-6916): in-place softmax of
 * pp[nrow, nvec, ncol] over the middle axis. */
KAI_API int kai_softmax_direct_on_axis(int device, float* pp, int64_t nrow, int64_t nvec,
                                       int64_t ncol, void* stream);
/* VMath::mix_values (vmath.h:239; vmath.cu:6977-7025):
 *   py[b,q,h,p] = sum_k pp[b,q,k,h] * pV[b,k,h*npiece+p] */
KAI_API int kai_mix_values(int device, float* py, const float* pp, const float* pV,
                           int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                           int64_t npiece, void* stream);

/* No single-call counterpart in the reference: the attention core of VTensor::mh_attention
 * (api_objects/vtensor.cpp:3036-3044) as one call for callers that do not need probs afterwards
 * (inference / no_grad),
 *   py = mix_values(softmax_direct_on_axis(mask?(mult_on_heads(pK, pQ, coef))), pV)
 * with py laid out like the output of kai_mix_values.  causal_mask != 0 applies
 * set_mh_attention_mask(forward) to the scores first.  For npiece == 64 the probs tensor is never
 * written to memory (one fused tcgen05 kernel); other shapes run the separate steps through a
 * block taken from kai_mem_alloc. */
KAI_API int kai_mh_attention_forward(int device, float* py, const float* pK, const float* pQ, const float* pV,
                                     int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                                     int64_t npiece, const float* coef, int causal_mask, void* stream);

/* Attention backward.  Argument order as in the reference; all follow its index conventions.
 * VMath::mult_on_heads_backward (vmath.h:235; vmath.cu:6783-6829):
 *   pgQK[b,t,h*P+p] = sum_k pgp[b,t,k,h] * pKQ[b,k,h*P+p]
 * (the engine calls it twice, once per operand of mult_on_heads: api_objects/vtensor.cpp:3153-3154) */
KAI_API int kai_mult_on_heads_backward(int device, float* pgQK, const float* pgp, const float* pKQ,
                                       int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                                       int64_t npiece, void* stream);
/* VMath::softmax_direct_on_axis_backward (vmath.h:238; vmath.cu:6920-6973), in place on pgp:
 *   pgp[b,q,k,h] = coef * pp[b,q,k,h] * (pgp[b,q,k,h] - sum_k' pp[b,q,k',h] * pgp[b,q,k',h]) */
KAI_API int kai_softmax_direct_on_axis_backward(int device, float* pgp, const float* pp, int64_t nbat,
                                                int64_t ntimes, int64_t nhead, const float* coef,
                                                void* stream);
/* VMath::mix_values_backward_prop (vmath.h:240; vmath.cu:7029-7077):
 *   pgp[b,q,k,h] = sum_p pgy[b,q,h,p] * pV[b,k,h*P+p] */
KAI_API int kai_mix_values_backward_prop(int device, float* pgp, const float* pgy, const float* pV,
                                         int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                                         int64_t npiece, void* stream);
/* VMath::mix_values_backward_value (vmath.h:241; vmath.cu:7081-7129):
 *   pgV[b,k,h*P+p] = sum_q pp[b,q,k,h] * pgy[b,q,h,p] */
KAI_API int kai_mix_values_backward_value(int device, float* pgV, const float* pgy, const float* pp,
                                          int64_t nbat, int64_t ntimes, int64_t nvec, int64_t nhead,
                                          int64_t npiece, void* stream);

/* ---- convolution (NCHW, stride 1, zero padding; kernel tensor [ychn][xchn / group][kh][kw]) -----
 * VMath::conv2d (vmath.h:146; vmath.cu:3490-3576):
 *   py[nd,yn,yr,yc] = sum_{kr,kc,xn} px[nd,xn,yr+kr-ph,yc+kc-pw] * pk[yn, xn / group, kr, kc]
 * pmode is accepted and ignored: the reference skips out-of-range taps whatever the mode
 * (vmath.cu:3509-3512, 3552-3555), i.e. every mode is zero padding. */
KAI_API int kai_conv2d(int device, float* py, const float* px, const float* pk, int64_t ndat, int64_t ychn,
                       int64_t yh, int64_t yw, int64_t xchn, int64_t xh, int64_t xw, int64_t kh, int64_t kw,
                       int64_t group, int64_t ph, int64_t pw, int pmode, void* stream);
/* VMath::conv2d_backward_x (vmath.h:149; vmath.cu:3580-3655) */
KAI_API int kai_conv2d_backward_x(int device, float* pgx, const float* pgy, const float* pk, int64_t ndat,
                                  int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw,
                                  int64_t kh, int64_t kw, int64_t group, int64_t ph, int64_t pw, void* stream);
/* VMath::conv2d_backward_k (vmath.h:152; device kernel vmath.cu:3697-3735, wrapper :3737-3744).  The
 * reference's host loop offsets columns by yw instead of pw (vmath.cu:3676); this follows the device
 * kernel, which is the adjoint of conv2d. */
KAI_API int kai_conv2d_backward_k(int device, float* pgk, const float* pgy, const float* px, int64_t ndat,
                                  int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t yh, int64_t yw,
                                  int64_t kh, int64_t kw, int64_t group, int64_t ph, int64_t pw, void* stream);

/* VMath::conv2d_transposed / _backward_x / _backward_k (vmath.h:156-158; vmath.cu:3748-3988): output
 * (xh*sh) x (xw*sw).  The reference's index rules are kept exactly (integer quotient by the stride without a
 * remainder test; the backward maps bound the output position by xh / xw); results equal the reference's host
 * loops bit for bit.  Kernel tensor [ychn][xchn][kh][kw]. */
KAI_API int kai_conv2d_transposed(int device, float* py, const float* px, const float* pk, int64_t ndat,
                                  int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                                  int64_t sh, int64_t sw, void* stream);
KAI_API int kai_conv2d_transposed_backward_x(int device, float* pgx, const float* pgy, const float* pk,
                                             int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn,
                                             int64_t kh, int64_t kw, int64_t sh, int64_t sw, void* stream);
KAI_API int kai_conv2d_transposed_backward_k(int device, float* pgk, const float* pgy, const float* px,
                                             int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn,
                                             int64_t kh, int64_t kw, int64_t sh, int64_t sw, void* stream);
/* VMath::conv2d_dilated / _backward_x / _backward_k (vmath.h:160-162; vmath.cu:3992-4210): same-size output,
 * kernel taps (kr - (kh-1)/2) * gh rows and (kc - (kw-1)/2) * gw columns from the centre. */
KAI_API int kai_conv2d_dilated(int device, float* py, const float* px, const float* pk, int64_t ndat,
                               int64_t xchn, int64_t xh, int64_t xw, int64_t ychn, int64_t kh, int64_t kw,
                               int64_t gh, int64_t gw, void* stream);
KAI_API int kai_conv2d_dilated_backward_x(int device, float* pgx, const float* pgy, const float* pk,
                                          int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn,
                                          int64_t kh, int64_t kw, int64_t gh, int64_t gw, void* stream);
KAI_API int kai_conv2d_dilated_backward_k(int device, float* pgk, const float* pgy, const float* px,
                                          int64_t ndat, int64_t xchn, int64_t xh, int64_t xw, int64_t ychn,
                                          int64_t kh, int64_t kw, int64_t gh, int64_t gw, void* stream);

/* ---- loss kernels of the MLP configuration --------------------------------------------- */
/* VMath::softmax_idx_crossentropy (vmath.h:299; vmath.cu:8916-8965):
 *   py[r] = -logf(softmax(px[r,:])[pz[r]] + 1e-10f).  Labels are checked on the device; an
 * out-of-range label leaves py[r] = NaN and the call returns KAI_E_OUT_OF_RANGE (it
 * synchronises the stream to read that flag, like the reference's host-side throw). */
KAI_API int kai_softmax_idx_crossentropy(int device, float* py, const float* px, const int* pz,
                                         int64_t nrow, int64_t ncol, void* stream);
/* VMath::softmax_idx_crossentropy_backward_x (vmath.h:301; vmath.cu:9022-9077):
 *   pgx[r,c] = (softmax(px[r,:])[c] - (c == pz[r])) * pgy[r] */
KAI_API int kai_softmax_idx_crossentropy_backward_x(int device, float* pgx, const float* pgy,
                                                    const float* px, const int* pz,
                                                    int64_t nrow, int64_t ncol, void* stream);
/* VMath::sum (vmath.h:325; vmath.cu:9739-9757): py[0] = sum px[0..nrow). */
KAI_API int kai_sum(int device, float* py, const float* px, int64_t nrow, void* stream);
/* VMath::sum_backward (vmath.h:326; vmath.cu:9761-9779): pgx[i] = pgy ? pgy[0] : 1. */
KAI_API int kai_sum_backward(int device, float* pgx, const float* pgy, int64_t nrow,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KAI_B200_H */
