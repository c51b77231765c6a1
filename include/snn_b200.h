/*
 * snn_b200.h - C ABI of libsnn_b200.so: the LIF "fire" forward / BPTT backward hot path
 * of liangling76/snn_gpu_training_bptt's `snnlib`, as hand-written sm_100a kernels.
 *
 * Conventions
 *   - plain C types only; every buffer is DEVICE memory owned by the caller; outputs are
 *     written in full; the library never calls cudaMalloc / cudaFree. The only state it keeps
 *     between calls is documented where it applies: the 64 MiB built-in scratch array and its
 *     cached device address (snn_lif_bwd_noalloc), and a small host-side cache of encoded
 *     tensor maps plus a device error word (snn_linear_lif_*);
 *   - tensors are time-major and contiguous: [T, N] with element (t, n) at t*N + n, where
 *     N = B*C*H*W is the reference's per-time-step element count (its `BCHW`,
 *     snnlib/cuda/snn_kernel_fp.cu:60-63); neurons are independent, so B and CHW need not
 *     be passed separately;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is
 *     where the reference launches: snn_kernel_fp.cu:68);
 *   - every entry point validates its arguments BEFORE launching and returns an
 *     snn_status; on any non-zero status nothing was launched. The reference has no error
 *     convention at all (no checks in snnlib/cuda/snn.cpp), so this is a strict superset;
 *   - work is enqueued asynchronously; a launch failure reported by the runtime is
 *     returned as SNN_ERR_CUDA (detail via snn_last_cuda_error()).
 */
#ifndef SNN_B200_H
#define SNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum snn_status {
    SNN_OK = 0,
    SNN_ERR_NULL = 1,        /* a required pointer is NULL */
    SNN_ERR_SHAPE = 2,       /* T < 1, N < 0, or a size that does not fit the kernels' index types */
    SNN_ERR_DTYPE = 3,       /* dtype is not one of snn_dtype */
    SNN_ERR_ALIGN = 4,       /* a pointer is not aligned to its element size */
    SNN_ERR_UNSUPPORTED = 5, /* valid request this build cannot serve (e.g. spike words with T > 32) */
    SNN_ERR_WORKSPACE = 6,   /* scratch buffer missing or too small */
    SNN_ERR_CUDA = 7,        /* the CUDA runtime reported an error at launch */
    SNN_ERR_TOO_LARGE = 8    /* problem does not fit the library's built-in scratch array */
} snn_status;

/* Element type of the tensors in global memory. State is always carried in fp32
 * (fp64 for SNN_F64), whatever the I/O type. */
typedef enum snn_dtype {
    SNN_F32 = 0,
    SNN_BF16 = 1,
    SNN_F16 = 2,
    SNN_F64 = 3
} snn_dtype;

/* Library version (major*10000 + minor*100 + patch). */
int snn_version(void);

/* Human-readable name of a status code (static string). */
const char *snn_status_string(int status);

/* cudaError_t of the most recent SNN_ERR_CUDA on this host thread (0 if none). */
int snn_last_cuda_error(void);

/*
 * LIF forward:  u_t = (alpha*u_{t-1})*(1 - s_{t-1}) + x_t ;  s_t = (u_t > thresh) ; u, s start at 0.
 *
 * Replaces `fire_s_fp(spatial, alpha, thresh) -> spike` (snnlib/cuda/snn.cpp:11-17 ->
 * fire_s_fp_cuda, snnlib/cuda/snn_kernel_fp.cu:55-73, kernel :15-53), and, through the
 * optional `mem` output, the membrane re-materialisation kernels fire_u_fp_kernel /
 * fire_us_fp_kernel (snnlib/cuda/snn_kernel_bp.cu:15-93).
 *
 *   x      [T, N] dtype            input currents
 *   spike  [T, N] dtype  or NULL   0/1 spikes
 *   mem    [T, N] fp32 (fp64 for SNN_F64) or NULL   membrane potentials u_t
 *   bits   [N] words or NULL       packed spikes: bit t of word n = s(t, n); word is uint8 for
 *                                  T <= 8, uint16 for T <= 16, uint32 for T <= 32
 *                                  (SNN_ERR_UNSUPPORTED beyond 32)
 * At least one of spike / mem / bits must be given.
 */
int snn_lif_fwd(const void *x, void *spike, void *mem, void *bits, int64_t T, int64_t N,
                int dtype, float alpha, float thresh, void *stream);

/*
 * Scratch bytes snn_lif_bwd needs for this (T, N, dtype): 0 while the time axis fits in
 * registers (T <= 32), else T*N*sizeof(state type) for a stored membrane tensor.
 * Returns a negative snn_status on invalid arguments.
 */
int64_t snn_lif_bwd_workspace_bytes(int64_t T, int64_t N, int dtype);

/*
 * LIF backward through time with the rectangular surrogate, walking t = T-1 .. 0:
 *   inside = (u_t - thresh < interval) && (thresh - u_t < interval)
 *   gs = inside ? g_t - (gu*alpha)*u_t : 0 ;  gu = gs*beta + (gu*alpha)*(u_t <= thresh) ;  grad_x_t = gu
 *
 * Replaces `fire_bp(spatial, grad_spike, alpha, thresh, beta, interval) -> grad_spatial`
 * (snnlib/cuda/snn.cpp:270-279 -> fire_bp_cuda, snnlib/cuda/snn_kernel_bp.cu:141-168, which
 * allocates a membrane tensor, runs fire_u_fp_kernel :15-52, then fire_bp_kernel :95-139).
 * Here u_t is rebuilt in registers from x inside one kernel.
 *
 *   x, grad_spike  [T, N] dtype   saved input currents, upstream gradient w.r.t. the spikes
 *   grad_x         [T, N] dtype   output
 *   workspace      device scratch of at least snn_lif_bwd_workspace_bytes() bytes, 256-byte
 *                  aligned; may be NULL when that is 0
 */
int snn_lif_bwd(const void *x, const void *grad_spike, void *grad_x, int64_t T, int64_t N,
                int dtype, float alpha, float thresh, float beta, float interval,
                void *workspace, size_t workspace_bytes, void *stream);

/*
 * Expand packed spike words (as written by snn_lif_fwd's `bits`) into a dense [T, N] 0/1
 * tensor of `dtype`. No counterpart in the reference, which stores spikes densely.
 */
int snn_spike_unpack(const void *bits, void *spike, int64_t T, int64_t N, int dtype,
                     void *stream);

/*
 * Copy `rows` rows of `row_bytes` bytes between (pinned) host memory and device memory in one
 * pitched transfer: row r goes from src + r*src_pitch to dst + r*dst_pitch. to_device != 0 =
 * host -> device, 0 = device -> host. One call moves a [T, chunk] slab of a time-major [T, N]
 * host tensor (pitch N*element size) to or from a dense staging buffer: it is what the
 * host-buffer pipeline uses instead of T separate row copies. No counterpart in the reference
 * (its tensors are created on the device).
 */
int snn_copy_rows_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch,
                        size_t row_bytes, int64_t rows, int to_device, void *stream);

/* ----------------------------------------------------------------------------------------
 * Batch-norm family. Tensors are [T, N] time-major with N = B * C * inner; the channel of flat
 * neuron index n is (n / inner) % C: inner = H*W for contiguous [T,B,C,H,W], inner = 1 for
 * [T,B,C] and for channels-last images. weight / bias / var / mean / ivar / sums are fp32
 * arrays of length C for every I/O dtype (SNN_F64 is not offered here: SNN_ERR_UNSUPPORTED).
 * `fire` != 0 selects the BN+LIF form, 0 the plain time-major batch-norm.
 * -------------------------------------------------------------------------------------- */

/*
 * Forward. w' = weight/sqrt(var + eps); ivar_out[c] = w'/weight[c];
 * current = (x - mean)*w' + bias; fire: out = LIF spikes of the current (mem = u, optional);
 * else out = current. If `var` is NULL, `ivar_out` is read as an INPUT and w' = weight*ivar:
 * that is how the reference rebuilds spikes inside its backward functions
 * (bn_fire_us_fp_kernel, snn_kernel_bp.cu:481-530).
 * Replaces bn_fire_s_fp (snnlib/cuda/snn.cpp:55-66 -> snn_kernel_fp.cu:212-240, kernel
 * :157-210) and bn_fp (snn.cpp:30-39 -> snn_kernel_fp.cu:124-150, kernel :80-122).
 */
int snn_bn_lif_fwd(const void *x, const float *weight, const float *bias, const float *var,
                   const float *mean, float eps, void *out, float *mem, float *ivar_out,
                   int64_t T, int64_t N, int64_t C, int64_t inner, int dtype, int fire,
                   float alpha, float thresh, void *stream);

/*
 * Backward pass 1: per-channel sums over all (t, b, position) of the gradient w.r.t. the
 * normalised current: sum_g[c] = sum gu (= grad_bias), sum_gx[c] = sum gu*xhat (= grad_weight),
 * gu = BPTT gradient (fire) or the upstream gradient (plain BN). Both arrays are zeroed by the
 * call (on `stream`) and accumulated with atomics. T <= 32 when fire.
 * Replaces the sums half of bn_fire_bp / bn_fire_bp_dist1 (snn.cpp:373-387, :405-421 ->
 * snn_kernel_bp.cu:679-750, :753-806; kernels :432-479 and :533-610) and of bn_bp / bn_bp_dist1
 * (snn.cpp:293-303, :317-327 -> snn_kernel_bp.cu:288-345, :348-392; kernel :175-236).
 */
int snn_bn_lif_bwd_sums(const void *x, const void *grad, const float *weight, const float *bias,
                        const float *ivar, const float *mean, float *sum_g, float *sum_gx,
                        int64_t T, int64_t N, int64_t C, int64_t inner, int dtype, int fire,
                        float alpha, float thresh, float beta, float interval, void *stream);

/*
 * gxhat[c] = weight[c]*sum_g[c]/count, gxhatx[c] = weight[c]*sum_gx[c]/count: the per-channel
 * means the reference forms with at::mean over its per-position partial sums
 * (snn_kernel_bp.cu:738-744). count = T*B*inner (times the world size after a sync-BN
 * all-reduce of the sums).
 */
int snn_bn_channel_means(const float *sum_g, const float *sum_gx, const float *weight,
                         float *gxhat, float *gxhatx, int64_t C, double count, void *stream);

/*
 * Backward pass 2: grad_x = gu*weight*ivar - ivar*(xhat*gxhatx[c] + gxhat[c]).
 * Replaces the input-gradient half of bn_fire_bp / bn_fire_bp_dist2 (snn.cpp:442-460 ->
 * snn_kernel_bp.cu:808-854; kernel :613-677) and of bn_bp / bn_bp_dist2 (snn.cpp:343-355 ->
 * snn_kernel_bp.cu:394-425; kernel :239-285).
 */
int snn_bn_lif_bwd_input(const void *x, const void *grad, const float *weight, const float *bias,
                         const float *ivar, const float *mean, const float *gxhat,
                         const float *gxhatx, void *grad_x, int64_t T, int64_t N, int64_t C,
                         int64_t inner, int dtype, int fire, float alpha, float thresh, float beta,
                         float interval, void *stream);

/* ----------------------------------------------------------------------------------------
 * LIF followed by AvgPool2d(2) on every time step, fused. No counterpart in the reference's
 * native table: its models place `Fire` in front of pooling-free strided convolutions, while the
 * VGG-style benchmark network pools after LIF (torch AvgPool2d per time step). Fusing keeps the
 * full-resolution spikes and their gradient out of HBM.
 * x is [T][B][H][W][C] in memory (channels-last images), outputs [T][B][H/2][W/2][C];
 * H and W even, T <= 16, dtype f32 / bf16 / f16.
 *   forward   out = mean over each 2x2 window of the LIF spikes of x        (values k/4, exact)
 *   backward  grad_x = LIF reverse pass with upstream gradient grad_out/4 at each window position
 * -------------------------------------------------------------------------------------- */
int snn_lif_pool_fwd(const void *x, void *out, int64_t T, int64_t B, int64_t H, int64_t W,
                     int64_t C, int dtype, float alpha, float thresh, void *stream);
int snn_lif_pool_bwd(const void *x, const void *grad_out, void *grad_x, int64_t T, int64_t B,
                     int64_t H, int64_t W, int64_t C, int dtype, float alpha, float thresh,
                     float beta, float interval, void *stream);

/* ----------------------------------------------------------------------------------------
 * LIF of the sum of two currents (residual networks: block output + shortcut, then LIF). No
 * counterpart in the reference's native table (its residual scripts add with torch and then call
 * the plain LIF op, snnlib_func.py:22-36). The sum is rounded to the I/O type before it enters
 * the recurrence, so results equal "a + b in the I/O type, then snn_lif_fwd / snn_lif_bwd" bit for
 * bit, without the sum ever being written to memory. a, b, spike, grad_spike, grad: [T][N], same
 * layout; dtype f32 / bf16 / f16.
 *   forward   spike = LIF(a + b)
 *   backward  grad  = dL/d(a + b) (= dL/da = dL/db); T <= 16, else SNN_ERR_UNSUPPORTED
 * -------------------------------------------------------------------------------------- */
int snn_lif_add_fwd(const void *a, const void *b, void *spike, int64_t T, int64_t N, int dtype,
                    float alpha, float thresh, void *stream);
int snn_lif_add_bwd(const void *a, const void *b, const void *grad_spike, void *grad, int64_t T,
                    int64_t N, int dtype, float alpha, float thresh, float beta, float interval,
                    void *stream);

/* ----------------------------------------------------------------------------------------
 * Per-channel bias of a synaptic layer. Element (o, c, i) at (o*C + c)*inner + i: inner = 1 for
 * channels-last images and [rows, C] matrices, inner = H*W for contiguous [N, C, H, W].
 *   snn_channel_bias_add   y[o, c, i] += bias[c], in place
 *   snn_channel_sum        out[c] = sum over o, i of grad[o, c, i]   (out is zeroed by the call)
 * They stand in for the bias handling inside the reference's per-time-step at::linear /
 * at::cudnn_convolution calls (snnlib/cuda/snn_kernel_fp.cu:346-352, :445) and for its
 * at::sum(grad, dims) bias gradients (snnlib/cuda/snn_kernel_bp.cu:1127, :1172, :1401, :1435).
 * -------------------------------------------------------------------------------------- */
int snn_channel_bias_add(void *y, const float *bias, int64_t outer, int64_t C, int64_t inner,
                         int dtype, void *stream);
int snn_channel_sum(const void *grad, float *out, int64_t outer, int64_t C, int64_t inner,
                    int dtype, void *stream);

/* ----------------------------------------------------------------------------------------
 * Fused synaptic linear + LIF forward on the tcgen05 tensor cores (bf16 operands, fp32
 * accumulation in tensor memory, LIF recurrence in the GEMM epilogue):
 *   current[t, b, :] = bf16( x[t, b, :] @ weight^T + bias ) ;  spike = LIF over t of current
 * Replaces `Fc` followed by `Fire` of the reference: fc_fp (snnlib/cuda/snn.cpp:130-136 ->
 * snn_kernel_fp.cu:332-357, T cuBLAS calls) then fire_s_fp (snn.cpp:11-17).
 *   x [T, B, K] bf16, weight [M, K] bf16 (both 16-byte aligned), bias [M] fp32 or NULL,
 *   current [T, B, M] bf16 or NULL (the LIF input; backward re-reads it), spike [T, B, M] bf16.
 * Supported when snn_linear_lif_fwd_supported() returns 1: SNN_BF16, 2 <= T <= 16,
 * B % (128/Tt) == 0 with Tt = the smallest of 2, 4, 8, 16 that is >= T (the kernels work on
 * tiles of Tt steps; a tensor with fewer steps - the reference's default T is 6 - leaves the
 * rest of the tile empty), K % 64 == 0, M % 128 == 0; otherwise SNN_ERR_UNSUPPORTED (use
 * snn_lif_fwd after a library GEMM). Outputs that are not 16-byte aligned are accepted for
 * T = 4 and T = 8 only (SNN_ERR_ALIGN otherwise). Waits inside the kernel are bounded; snn_linear_lif_error() returns 0,
 * or the code of the FIRST wait that expired (1 producer, 2 / 4 MMA issuer, 3 epilogue; 11-14 the
 * same roles of the CTA-pair kernel) after synchronising with the device, and clears it when
 * `reset` is non-zero. While the word is non-zero, waits of later launches give up early and
 * their results are undefined: clear it before going on.
 * -------------------------------------------------------------------------------------- */
int snn_linear_lif_fwd_supported(int64_t T, int64_t B, int64_t K, int64_t M, int dtype);
/* Which kernel snn_linear_lif_fwd runs for this problem on a device with `sm_count` SMs (no GPU
 * needed, nothing launched; no counterpart in the reference): 0 = persistent kernel with 128 x 128
 * tiles, 1 = with 128 x 256 tiles (the batch allows them and they save a round of tiles),
 * 2 = CTA-pair kernel, 256 x 256 per pair (every CTA would get two or more wide tiles);
 * -1 = unsupported problem. The environment override SNN_LINEAR_LIF_VARIANT is not applied. */
int snn_linear_lif_fwd_plan(int64_t T, int64_t B, int64_t K, int64_t M, int dtype, int sm_count);
int snn_linear_lif_fwd(const void *x, const void *weight, const float *bias, void *current,
                       void *spike, int64_t T, int64_t B, int64_t K, int64_t M, int dtype,
                       float alpha, float thresh, void *stream);
int snn_linear_lif_error(int reset);

/*
 * Backward through time of the fused synaptic linear + LIF layer on the tcgen05 tensor cores:
 *   dU = LIF reverse pass of (current, grad_spike)   (same arithmetic as snn_lif_bwd, bf16 I/O)
 *   grad_x[t, b, :] = dU[t, b, :] @ weight ;  grad_weight = sum_(t,b) dU[t,b,:]^T x[t,b,:] ;
 *   grad_bias = sum_(t,b) dU[t,b,:]
 * Replaces fire_bp followed by fc_bp of the reference (snnlib/cuda/snn.cpp:270-279 ->
 * snn_kernel_bp.cu:141-168, and snn.cpp:594-602 -> fc_bp_cuda, snn_kernel_bp.cu:1131-1173: 2*T
 * at::mm calls plus at::sum). Two launches: one kernel writes dU (bf16) and per-block partial
 * bias sums into the workspace; one persistent tcgen05 kernel computes both gradient GEMMs,
 * reading weight, x and dU in place (no transposed copies) and summing the bias partials in a
 * fixed order (results are reproducible run to run).
 *   x [T, B, K] bf16, weight [M, K] bf16, current / grad_spike [T, B, M] bf16 (current is the
 *   LIF input that snn_linear_lif_fwd wrote), all 16-byte aligned;
 *   grad_x [T, B, K] bf16 or NULL (skipped); grad_weight [M, K] of grad_weight_dtype (SNN_BF16 or
 *   SNN_F32) or NULL (skipped); grad_bias [M] fp32 or NULL (needs grad_weight);
 *   workspace: snn_linear_lif_bwd_workspace_bytes() bytes of device scratch, 256-byte aligned.
 * Supported when snn_linear_lif_bwd_supported() returns 1: SNN_BF16, 1 <= T <= 16, T*B >= 128,
 * K >= 64, M >= 128, K % 64 == 0, M % 64 == 0; otherwise SNN_ERR_UNSUPPORTED (use snn_lif_bwd and
 * library GEMMs). Bounded waits report through snn_linear_lif_error() with codes 21 (producer),
 * 22 / 24 (MMA issuer), 23 (epilogue).
 */
int snn_linear_lif_bwd_supported(int64_t T, int64_t B, int64_t K, int64_t M, int dtype);
int64_t snn_linear_lif_bwd_workspace_bytes(int64_t T, int64_t B, int64_t K, int64_t M, int dtype);
int snn_linear_lif_bwd(const void *x, const void *weight, const void *current,
                       const void *grad_spike, void *grad_x, void *grad_weight, float *grad_bias,
                       int64_t T, int64_t B, int64_t K, int64_t M, int dtype,
                       int grad_weight_dtype, float alpha, float thresh, float beta, float interval,
                       void *workspace, size_t workspace_bytes, void *stream);

/*
 * LIF backward through time for callers that may not allocate device memory.
 *
 * No counterpart in the reference (its fire_bp allocates two tensors per call,
 * snnlib/cuda/snn_kernel_bp.cu:154,160). Same arithmetic and same result as snn_lif_bwd, but
 * this variant always takes the stored-membrane route (write u_t for all T steps, then walk
 * them in reverse) and keeps the membrane tensor in an array that is compiled into the
 * library instead of in caller-provided scratch. It is meant for hosts that cannot call
 * cudaMalloc at the point where the backward runs: a serving or training process whose own
 * allocator was handed the whole GPU up front, a latency-critical loop in which the implicit
 * device synchronisation of cudaMalloc/cudaFree is not acceptable, or a plugin sandbox that
 * only passes buffers in and out. Such callers still own x, grad_spike and grad_x; the
 * library calls no cudaMalloc, cudaFree or other allocating routine here, for any T.
 *
 * Limits and rules
 *   - the built-in array is SNN_STATIC_SCRATCH_BYTES (64 MiB) per GPU; every GPU on which the
 *     library's device code is loaded holds it until the process exits;
 *   - T * N * (4 bytes, or 8 for SNN_F64) must fit in it, otherwise SNN_ERR_TOO_LARGE is
 *     returned and nothing is launched (e.g. fp32: T*N <= 16 Mi neuron-steps; split the neuron
 *     axis into several calls for more);
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress, with that device current) and caches it for the life of the
 *     process. Make that first call during set-up, before any stream capture is begun on that
 *     device. A cudaDeviceReset() invalidates the cached address: do not call this entry point
 *     on a device after resetting it;
 *   - all calls on one GPU share the one array. It keeps whatever the previous call left; this
 *     entry point overwrites every element it later reads, so nothing needs clearing, but two
 *     calls that can overlap on the GPU (different streams, no dependency) race on it. Issue
 *     them on one stream or order them with events.
 */
#define SNN_STATIC_SCRATCH_BYTES (64u * 1024u * 1024u)
int snn_lif_bwd_noalloc(const void *x, const void *grad_spike, void *grad_x, int64_t T,
                        int64_t N, int dtype, float alpha, float thresh, float beta,
                        float interval, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SNN_B200_H */
