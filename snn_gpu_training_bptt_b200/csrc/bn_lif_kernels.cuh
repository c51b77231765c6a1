// Batch-norm affine (per channel) in front of the LIF recurrence, and plain time-major
// batch-norm: device code for sm_100a.
//
// Reference behaviour (liangling76/snn_gpu_training_bptt):
//   forward   snnlib/cuda/snn_kernel_fp.cu:157-210 (bn_fire_s_fp_kernel), :80-122 (bn_fp_kernel)
//               w' = weight[c] / sqrt(var[c] + eps) ;  ivar[c] = w' / weight[c]
//               current_t = (x_t - mean[c]) * w' + bias[c] ;  LIF on current_t  (or y = current)
//   backward  snnlib/cuda/snn_kernel_bp.cu:432-479 (u rebuilt with w' = weight[c]*ivar[c]),
//             :533-610 (per-channel sums), :613-677 (input gradient); plain BN :175-285
//               gu_t  = BPTT gradient w.r.t. current_t      (= upstream gradient for plain BN)
//               xhat  = (x_t - mean[c]) * ivar[c]
//               grad_bias[c] = sum gu ;  grad_weight[c] = sum gu*xhat
//               gxhat[c] = mean(gu*weight[c]) ;  gxhatx[c] = mean(gu*weight[c]*xhat)
//               grad_x_t = gu*weight[c]*ivar[c] - ivar[c]*(xhat*gxhatx[c] + gxhat[c])
//
// The reference runs backward as three full passes (rebuild u into a tensor, a sums pass that
// runs BPTT, an input-gradient pass that runs BPTT again: 36 B per neuron-step in fp32). Here
// it is two passes that each rebuild u and gu in registers: the sums pass reads x and g (8 B),
// the input-gradient pass reads x and g and writes grad_x (12 B). Between the two passes sits
// the only cross-thread dependency, the per-channel means; that is also exactly where the
// sync-BN variants all-reduce them across GPUs.
//
// Layout: [T, N] time-major; the channel of neuron n (flat index inside one time step) is
// (n / inner) % C: inner = H*W for contiguous [T,B,C,H,W], inner = 1 for [T,B,C] and for
// channels-last images. BN parameters and statistics are fp32 arrays of length C whatever the
// I/O type; sums are accumulated hierarchically (registers over T and the thread's neurons,
// warp shuffles when a warp sits inside one channel, shared-memory atomics per CTA, then one
// global atomicAdd per (CTA, channel)).
#pragma once
#include "lif_kernels.cuh"

namespace snn {

struct BnParams {
    const float* mean;     // [C]
    const float* weight;   // [C]
    const float* bias;     // [C]  (forward / u rebuild only)
    const float* var;      // [C]  forward only
    const float* ivar;     // [C]  backward only
    float eps;
    long long inner;       // neurons per channel run
    int C;
};

// 64-bit integer division is emulated with ~100 instructions; every practical size fits 32 bits.
__device__ __forceinline__ long long run_of(long long n, long long inner) {
    if (n <= 0xffffffffLL && inner <= 0xffffffffLL)
        return static_cast<long long>(static_cast<unsigned int>(n) / static_cast<unsigned int>(inner));
    return n / inner;
}
__device__ __forceinline__ int channel_of_run(long long q, int C) {
    if (q <= 0xffffffffLL) return static_cast<int>(static_cast<unsigned int>(q) % static_cast<unsigned int>(C));
    return static_cast<int>(q % C);
}
__device__ __forceinline__ int channel_of(long long n, long long inner, int C) {
    return channel_of_run(run_of(n, inner), C);
}

// current = ((leak + (x - m) * w) + b), operations rounded one by one, association as in
// the reference expression `alpha*u*(1-s) + (x - m)*w + b` read left to right.
__device__ __forceinline__ float bn_lif_step(float u, float gate, float x, float m, float w, float b,
                                             float alpha) {
    const float leak = mul_rn(mul_rn(alpha, u), gate);
    return add_rn(add_rn(leak, mul_rn(sub_rn(x, m), w)), b);
}

// ---------------------------------------------------------------------------------------
// Forward: FIRE=true -> spikes (and optionally u); FIRE=false -> y = (x-m)*w' + b.
// With p.var given it also writes ivar[c] (by the thread that owns the first neuron of channel
// c in batch 0); with p.var == nullptr it reads p.ivar instead and uses w' = weight*ivar, which
// is how the reference rebuilds spikes inside its backward functions.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TC, bool FIRE>
__global__ void bn_lif_fwd_kernel(const IO* __restrict__ x, IO* __restrict__ out,
                                  float* __restrict__ mem, float* __restrict__ ivar_out,
                                  BnParams p, int T, long long N, float alpha, float thresh)
{
    const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    float m[VEC], w[VEC], b[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const int c = channel_of(i + v, p.inner, p.C);
        const float wt = p.weight[c];
        m[v] = p.mean[c];
        b[v] = p.bias[c];
        if (p.var != nullptr) {
            w[v] = wt / sqrtf(p.var[c] + p.eps);      // IEEE division and square root
            if (ivar_out != nullptr && (i + v) < p.inner * p.C &&
                run_of(i + v, p.inner) * p.inner == (i + v))
                ivar_out[c] = w[v] / wt;
        } else {
            w[v] = mul_rn(wt, p.ivar[c]);             // backward-time rebuild: w' = weight*ivar
        }
    }
    float u[VEC], gate[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { u[v] = 0.f; gate[v] = 1.f; }

    for (int t0 = 0; t0 < T; t0 += TC) {
        Pack<IO, VEC> xin[TC];
#pragma unroll
        for (int k = 0; k < TC; ++k)
            if (t0 + k < T) xin[k] = ld_stream<IO, VEC>(x + static_cast<long long>(t0 + k) * N + i);
#pragma unroll
        for (int k = 0; k < TC; ++k) {
            if (t0 + k < T) {
                Pack<IO, VEC> o;
                Pack<float, VEC> mm;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float xv = Elem<IO>::load(xin[k].v[v]);
                    if (FIRE) {
                        u[v] = bn_lif_step(u[v], gate[v], xv, m[v], w[v], b[v], alpha);
                        const bool s = u[v] > thresh;
                        gate[v] = s ? 0.f : 1.f;
                        o.v[v] = Elem<IO>::store(s ? 1.f : 0.f);
                        mm.v[v] = u[v];
                    } else {
                        o.v[v] = Elem<IO>::store(add_rn(mul_rn(sub_rn(xv, m[v]), w[v]), b[v]));
                    }
                }
                const long long off = static_cast<long long>(t0 + k) * N + i;
                if (out != nullptr) st_stream<IO, VEC>(out + off, o);
                if (FIRE && mem != nullptr) st_stream<float, VEC>(mem + off, mm);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Shared by both backward passes: rebuild u (w' = weight*ivar, as the reference's backward
// does), run the reverse-time recurrence and hand each gu(t, v) to `emit` as soon as it is
// known, so no array of gradients has to stay live beside x and u.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX, bool FIRE, bool EXACT, typename Emit>
__device__ __forceinline__ void bn_lif_grad_current(const Pack<IO, VEC> (&xin)[TMAX],
                                                    const Pack<IO, VEC> (&gin)[TMAX], int T,
                                                    const float (&m)[VEC], const float (&wiv)[VEC],
                                                    const float (&b)[VEC], float alpha, float thresh,
                                                    float beta, float interval, Emit&& emit)
{
    if constexpr (!FIRE) {
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) emit(t, v, Elem<IO>::load(gin[t].v[v]));
            }
    } else {
        float u[TMAX][VEC];
        float uu[VEC], gate[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { uu[v] = 0.f; gate[v] = 1.f; }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (EXACT || t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    uu[v] = bn_lif_step(uu[v], gate[v], Elem<IO>::load(xin[t].v[v]), m[v], wiv[v], b[v], alpha);
                    gate[v] = (uu[v] > thresh) ? 0.f : 1.f;
                    u[t][v] = uu[v];
                }
            }
        }
        float gu[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) gu[v] = 0.f;
#pragma unroll
        for (int t = TMAX - 1; t >= 0; --t) {
            if (EXACT || t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float ut = u[t][v];
                    const float ga = mul_rn(gu[v], alpha);
                    const bool inside = inside_window(ut, thresh, interval);
                    float gs = 0.f;
                    if (inside) gs = sub_rn(Elem<IO>::load(gin[t].v[v]), mul_rn(ga, ut));
                    const float keep = (ut <= thresh) ? 1.f : 0.f;
                    gu[v] = add_rn(mul_rn(gs, beta), mul_rn(ga, keep));
                    emit(t, v, gu[v]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Backward pass 1: per-channel sums  sum_g[c] += gu ,  sum_gx[c] += gu * xhat.
// sums must be zero before the launch.
//   WARP_RUN = true : every warp lies inside one channel run (inner % (32*VEC) == 0): warp
//                     butterfly, then one global atomicAdd pair per warp; no shared memory.
//   WARP_RUN = false: shared-memory accumulators, one slot per channel run a CTA can touch
//                     (dynamic shared memory 2*nq floats, nq = (span + inner - 1)/inner + 1),
//                     then one global atomicAdd pair per (CTA, run). When a CTA touches more runs
//                     than there are channels (short runs: channels-last images and [T,B,C]
//                     inputs have inner = 1, every neuron its own run) the slots are indexed by
//                     channel instead (nq = C, slot = (run - first run) mod C), so the CTA still
//                     reduces in shared memory and issues at most C global atomic pairs.
// ---------------------------------------------------------------------------------------
// EXACT = (T == TMAX): the time loops then carry no per-step bound checks.
template <typename IO, int VEC, int TMAX, bool FIRE, bool WARP_RUN, bool EXACT>
__device__ __forceinline__ void bn_lif_bwd_sums_body(const IO* __restrict__ x, const IO* __restrict__ g,
                                       float* __restrict__ sum_g, float* __restrict__ sum_gx,
                                       const BnParams& p, int T, long long N, int nq, float alpha,
                                       float thresh, float beta, float interval)
{
    extern __shared__ float sacc[];                       // [2][nq]   (unused when WARP_RUN)
    if (!WARP_RUN) {
        for (int j = threadIdx.x; j < 2 * nq; j += blockDim.x) sacc[j] = 0.f;
        __syncthreads();
    }

    const long long blk0 = static_cast<long long>(blockIdx.x) * blockDim.x * VEC;
    const long long q0 = run_of(blk0, p.inner);
    const long long i = blk0 + static_cast<long long>(threadIdx.x) * VEC;
    const bool active = i < N;

    float s1[VEC], s2[VEC];
    long long q[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { s1[v] = 0.f; s2[v] = 0.f; q[v] = q0; }

    if (active) {
        float m[VEC], wiv[VEC], b[VEC], iv[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            q[v] = (WARP_RUN && v > 0) ? q[0] : run_of(i + v, p.inner);
            const int c = channel_of_run(q[v], p.C);
            m[v] = p.mean[c];
            iv[v] = p.ivar[c];
            wiv[v] = mul_rn(p.weight[c], iv[v]);
            b[v] = FIRE ? p.bias[c] : 0.f;
        }
        Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * N + i);
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<long long>(t) * N + i);
        bn_lif_grad_current<IO, VEC, TMAX, FIRE, EXACT>(
            xin, gin, T, m, wiv, b, alpha, thresh, beta, interval, [&](int t, int v, float gu) {
                const float xhat = mul_rn(sub_rn(Elem<IO>::load(xin[t].v[v]), m[v]), iv[v]);
                s1[v] += gu;
                s2[v] = fmaf(gu, xhat, s2[v]);
            });
    }

    if (WARP_RUN) {
        float a = 0.f, c2 = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) { a += s1[v]; c2 += s2[v]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        }
        // lane 0 of a warp is active whenever any lane of the warp is (N is a multiple of inner)
        if ((threadIdx.x & 31) == 0 && active) {
            const int c = channel_of_run(q[0], p.C);
            atomicAdd(&sum_g[c], a);
            atomicAdd(&sum_gx[c], c2);
        }
        return;
    }

    // slot of a run: its offset from the CTA's first run, folded onto the channels when the CTA
    // covers more runs than channels (nq == C then, and slot j belongs to channel_of_run(q0 + j))
    const bool by_channel = nq == p.C;
    auto slot_of = [&](long long run) {
        const unsigned int d = static_cast<unsigned int>(run - q0);
        return static_cast<int>(by_channel ? d % static_cast<unsigned int>(nq) : d);
    };
    // warp inside one channel run: butterfly, one shared atomic per warp; otherwise per lane
    const long long q_first = __shfl_sync(0xffffffffu, q[0], 0);
    const bool same = __all_sync(0xffffffffu, (!active) || (q[0] == q_first && q[VEC - 1] == q_first));
    if (same) {
        float a = 0.f, c2 = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) { a += s1[v]; c2 += s2[v]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        }
        if ((threadIdx.x & 31) == 0) {
            const int j = slot_of(q_first);
            atomicAdd(&sacc[j], a);
            atomicAdd(&sacc[nq + j], c2);
        }
    } else if (active) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            const int j = slot_of(q[v]);
            atomicAdd(&sacc[j], s1[v]);
            atomicAdd(&sacc[nq + j], s2[v]);
        }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < nq; j += blockDim.x) {
        const float a = sacc[j], c2 = sacc[nq + j];
        if (a != 0.f || c2 != 0.f) {
            const int c = channel_of_run(q0 + j, p.C);
            atomicAdd(&sum_g[c], a);
            atomicAdd(&sum_gx[c], c2);
        }
    }
}

template <typename IO, int VEC, int TMAX, bool FIRE, bool WARP_RUN>
__global__ void __launch_bounds__(256, (VEC * TMAX <= 16) ? 4 : ((VEC * TMAX <= 32) ? 2 : 1))
bn_lif_bwd_sums_kernel(const IO* __restrict__ x, const IO* __restrict__ g, float* __restrict__ sum_g,
                       float* __restrict__ sum_gx, BnParams p, int T, long long N, int nq, float alpha,
                       float thresh, float beta, float interval)
{
    if (T == TMAX)
        bn_lif_bwd_sums_body<IO, VEC, TMAX, FIRE, WARP_RUN, true>(x, g, sum_g, sum_gx, p, T, N, nq, alpha, thresh, beta, interval);
    else
        bn_lif_bwd_sums_body<IO, VEC, TMAX, FIRE, WARP_RUN, false>(x, g, sum_g, sum_gx, p, T, N, nq, alpha, thresh, beta, interval);
}

// ---------------------------------------------------------------------------------------
// Backward pass 1 for runs of ONE neuron (inner == 1: channels-last images, [T, B, C] inputs)
// when the CTA's span of blockDim.x * VEC consecutive neurons is a multiple of C: neuron n has
// channel n % C, so a thread that steps through the tensor in strides of whole spans sees the same
// VEC channels every time. It keeps its channel parameters and its two sums in registers across
// all its slabs, and the CTA folds them into C shared-memory slots and issues C global atomic pairs
// ONCE at the end. (With one slab per CTA, as in the kernel above, the flush alone is C pairs per
// 256 * VEC neurons: 67 M global atomics for a 2^26-neuron tensor with C = 256.)
// Dynamic shared memory: 2 * C floats. The grid is a few CTAs per SM.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX, bool FIRE, bool EXACT>
__device__ __forceinline__ void bn_lif_bwd_sums_cl_body(const IO* __restrict__ x, const IO* __restrict__ g,
                                                        float* __restrict__ sum_g, float* __restrict__ sum_gx,
                                                        const BnParams& p, int T, long long N, float alpha,
                                                        float thresh, float beta, float interval)
{
    extern __shared__ float sacc[];                       // [2][C]
    const int C = p.C;
    for (int j = threadIdx.x; j < 2 * C; j += blockDim.x) sacc[j] = 0.f;
    __syncthreads();

    const long long span = static_cast<long long>(blockDim.x) * VEC;
    const int c0 = static_cast<int>((static_cast<long long>(threadIdx.x) * VEC) % C);   // span % C == 0
    float m[VEC], wiv[VEC], b[VEC], iv[VEC], s1[VEC], s2[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const int c = (c0 + v) % C;
        m[v] = p.mean[c];
        iv[v] = p.ivar[c];
        wiv[v] = mul_rn(p.weight[c], iv[v]);
        b[v] = FIRE ? p.bias[c] : 0.f;
        s1[v] = 0.f;
        s2[v] = 0.f;
    }
    for (long long base = static_cast<long long>(blockIdx.x) * span; base < N; base += static_cast<long long>(gridDim.x) * span) {
        const long long i = base + static_cast<long long>(threadIdx.x) * VEC;
        if (i >= N) break;                                // N is a multiple of VEC (checked by the host)
        Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * N + i);
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<long long>(t) * N + i);
        bn_lif_grad_current<IO, VEC, TMAX, FIRE, EXACT>(
            xin, gin, T, m, wiv, b, alpha, thresh, beta, interval, [&](int t, int v, float gu) {
                const float xhat = mul_rn(sub_rn(Elem<IO>::load(xin[t].v[v]), m[v]), iv[v]);
                s1[v] += gu;
                s2[v] = fmaf(gu, xhat, s2[v]);
            });
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const int c = (c0 + v) % C;
        atomicAdd(&sacc[c], s1[v]);
        atomicAdd(&sacc[C + c], s2[v]);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        atomicAdd(&sum_g[c], sacc[c]);
        atomicAdd(&sum_gx[c], sacc[C + c]);
    }
}

template <typename IO, int VEC, int TMAX, bool FIRE>
__global__ void __launch_bounds__(256, (VEC * TMAX <= 16) ? 4 : ((VEC * TMAX <= 32) ? 2 : 1))
bn_lif_bwd_sums_cl_kernel(const IO* __restrict__ x, const IO* __restrict__ g, float* __restrict__ sum_g,
                          float* __restrict__ sum_gx, BnParams p, int T, long long N, float alpha, float thresh,
                          float beta, float interval)
{
    if (T == TMAX)
        bn_lif_bwd_sums_cl_body<IO, VEC, TMAX, FIRE, true>(x, g, sum_g, sum_gx, p, T, N, alpha, thresh, beta, interval);
    else
        bn_lif_bwd_sums_cl_body<IO, VEC, TMAX, FIRE, false>(x, g, sum_g, sum_gx, p, T, N, alpha, thresh, beta, interval);
}

// ---------------------------------------------------------------------------------------
// Backward pass 1 for LONG runs (inner >= the CTA span, e.g. contiguous 32 x 32 images): the grid is
// a multiple of C and a CTA walks channel runs q = blockIdx.x, blockIdx.x + gridDim.x, ... - all of
// ONE channel - so the channel parameters are loaded once, the two sums stay in registers across
// every run the CTA visits, and the CTA ends with one block reduction and ONE global atomic pair.
// The same idea as the short-run kernel above; measured 6.6 TB/s there against 4.9 TB/s for the
// one-slab-per-CTA kernel (a butterfly and an atomic pair per warp and slab).
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX, bool FIRE, bool EXACT>
__device__ __forceinline__ void bn_lif_bwd_sums_run_body(const IO* __restrict__ x, const IO* __restrict__ g,
                                                         float* __restrict__ sum_g, float* __restrict__ sum_gx,
                                                         const BnParams& p, int T, long long N, long long runs,
                                                         float alpha, float thresh, float beta, float interval)
{
    __shared__ float red[2][8];
    const int c = static_cast<int>(blockIdx.x % p.C);     // gridDim.x % C == 0: the same channel on every visit
    float m[VEC], wiv[VEC], b[VEC], iv[VEC];
    {
        const float m0 = p.mean[c], iv0 = p.ivar[c], w0 = mul_rn(p.weight[c], iv0), b0 = FIRE ? p.bias[c] : 0.f;
#pragma unroll
        for (int v = 0; v < VEC; ++v) { m[v] = m0; iv[v] = iv0; wiv[v] = w0; b[v] = b0; }
    }
    float a1 = 0.f, a2 = 0.f;
    const long long inner = p.inner;
    for (long long q = blockIdx.x; q < runs; q += gridDim.x) {
        const long long base = q * inner;
        for (long long j = static_cast<long long>(threadIdx.x) * VEC; j < inner; j += static_cast<long long>(blockDim.x) * VEC) {
            const long long i = base + j;
            Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
            for (int t = 0; t < TMAX; ++t)
                if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * N + i);
#pragma unroll
            for (int t = 0; t < TMAX; ++t)
                if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<long long>(t) * N + i);
            bn_lif_grad_current<IO, VEC, TMAX, FIRE, EXACT>(
                xin, gin, T, m, wiv, b, alpha, thresh, beta, interval, [&](int t, int v, float gu) {
                    const float xhat = mul_rn(sub_rn(Elem<IO>::load(xin[t].v[v]), m[v]), iv[v]);
                    a1 += gu;
                    a2 = fmaf(gu, xhat, a2);
                });
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a1 += __shfl_xor_sync(0xffffffffu, a1, o);
        a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a1; red[1][threadIdx.x >> 5] = a2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t1 = 0.f, t2 = 0.f;
        for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) { t1 += red[0][w]; t2 += red[1][w]; }
        atomicAdd(&sum_g[c], t1);
        atomicAdd(&sum_gx[c], t2);
    }
}

template <typename IO, int VEC, int TMAX, bool FIRE>
__global__ void __launch_bounds__(256, (VEC * TMAX <= 16) ? 4 : ((VEC * TMAX <= 32) ? 2 : 1))
bn_lif_bwd_sums_run_kernel(const IO* __restrict__ x, const IO* __restrict__ g, float* __restrict__ sum_g,
                           float* __restrict__ sum_gx, BnParams p, int T, long long N, long long runs, float alpha,
                           float thresh, float beta, float interval)
{
    if (T == TMAX)
        bn_lif_bwd_sums_run_body<IO, VEC, TMAX, FIRE, true>(x, g, sum_g, sum_gx, p, T, N, runs, alpha, thresh, beta, interval);
    else
        bn_lif_bwd_sums_run_body<IO, VEC, TMAX, FIRE, false>(x, g, sum_g, sum_gx, p, T, N, runs, alpha, thresh, beta, interval);
}

// ---------------------------------------------------------------------------------------
// Backward pass 2: grad_x = gu*w*ivar - ivar*(xhat*gxhatx[c] + gxhat[c]).
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX, bool FIRE, bool EXACT>
__device__ __forceinline__ void bn_lif_bwd_input_body(const IO* __restrict__ x, const IO* __restrict__ g,
                                        const float* __restrict__ gxhat,
                                        const float* __restrict__ gxhatx, IO* __restrict__ gx,
                                        const BnParams& p, int T, long long N, float alpha, float thresh,
                                        float beta, float interval)
{
    const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    float m[VEC], wiv[VEC], b[VEC], iv[VEC], wt[VEC], gh[VEC], ghx[VEC];
    const bool one_channel = (p.inner % VEC) == 0;        // i is a multiple of VEC
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
        const int c = (one_channel && v > 0) ? 0 : channel_of(i + v, p.inner, p.C);
        if (one_channel && v > 0) {
            m[v] = m[0]; iv[v] = iv[0]; wt[v] = wt[0]; wiv[v] = wiv[0]; b[v] = b[0]; gh[v] = gh[0]; ghx[v] = ghx[0];
        } else {
            m[v] = p.mean[c];
            iv[v] = p.ivar[c];
            wt[v] = p.weight[c];
            wiv[v] = mul_rn(wt[v], iv[v]);
            b[v] = FIRE ? p.bias[c] : 0.f;
            gh[v] = gxhat[c];
            ghx[v] = gxhatx[c];
        }
    }
    Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * N + i);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<long long>(t) * N + i);
    Pack<IO, VEC> o;
    bn_lif_grad_current<IO, VEC, TMAX, FIRE, EXACT>(
        xin, gin, T, m, wiv, b, alpha, thresh, beta, interval, [&](int t, int v, float gu) {
            const float xhat = mul_rn(sub_rn(Elem<IO>::load(xin[t].v[v]), m[v]), iv[v]);
            const float lhs = mul_rn(mul_rn(gu, wt[v]), iv[v]);
            const float rhs = mul_rn(iv[v], add_rn(mul_rn(xhat, ghx[v]), gh[v]));
            o.v[v] = Elem<IO>::store(sub_rn(lhs, rhs));
            if (v == VEC - 1) st_stream<IO, VEC>(gx + static_cast<long long>(t) * N + i, o);   // row t complete
        });
}

template <typename IO, int VEC, int TMAX, bool FIRE>
__global__ void __launch_bounds__(256, (VEC * TMAX <= 16) ? 4 : ((VEC * TMAX <= 32) ? 2 : 1))
bn_lif_bwd_input_kernel(const IO* __restrict__ x, const IO* __restrict__ g, const float* __restrict__ gxhat,
                        const float* __restrict__ gxhatx, IO* __restrict__ gx, BnParams p, int T, long long N,
                        float alpha, float thresh, float beta, float interval)
{
    if (T == TMAX)
        bn_lif_bwd_input_body<IO, VEC, TMAX, FIRE, true>(x, g, gxhat, gxhatx, gx, p, T, N, alpha, thresh, beta, interval);
    else
        bn_lif_bwd_input_body<IO, VEC, TMAX, FIRE, false>(x, g, gxhat, gxhatx, gx, p, T, N, alpha, thresh, beta, interval);
}

// gxhat[c] = weight[c]*sum_g[c]/count ; gxhatx[c] = weight[c]*sum_gx[c]/count  (C threads)
__global__ void bn_channel_means_kernel(const float* __restrict__ sum_g,
                                        const float* __restrict__ sum_gx,
                                        const float* __restrict__ weight, float* __restrict__ gxhat,
                                        float* __restrict__ gxhatx, int C, float inv_count)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) {
        gxhat[c] = weight[c] * sum_g[c] * inv_count;
        gxhatx[c] = weight[c] * sum_gx[c] * inv_count;
    }
}

}  // namespace snn
