// LIF on the SUM of two input currents: spike = LIF(a + b), as one pass each way.
//
// Residual spiking networks add a shortcut current to a block's output current and feed the sum to
// a LIF layer ("LIF after each residual add"). Done as a tensor add followed by the LIF kernel, the
// sum is written, re-read by the forward kernel, kept for backward and re-read there. Here the
// forward kernel reads both addends and the backward kernel rebuilds the membrane potential from
// them, so the sum never exists in memory: per neuron-step (in elements) forward moves 3 instead of
// 5, backward 4 instead of 3. The sum is rounded to the I/O type before it enters the recurrence,
// exactly as a separate add would leave it, so spikes and gradients equal those of add -> LIF bit
// for bit. The gradient w.r.t. the sum is the gradient w.r.t. each addend: one output.
// Same recurrence and reverse pass as lif_kernels.cuh (reference: snnlib/cuda/snn_kernel_fp.cu:37-52,
// snn_kernel_bp.cu:117-138); the reference itself has no fused form of this.
#pragma once
#include "lif_kernels.cuh"

namespace snn {

template <typename IO>
__device__ __forceinline__ typename Elem<IO>::CT rounded_sum(IO a, IO b) {
    using CT = typename Elem<IO>::CT;
    const CT s = add_rn(Elem<IO>::load(a), Elem<IO>::load(b));
    return Elem<IO>::load(Elem<IO>::store(s));
}

template <typename IO, int VEC, int TC>
__global__ void lif_add_fwd_kernel(const IO* __restrict__ a, const IO* __restrict__ b, IO* __restrict__ spike,
                                   int T, int64_t N, float alpha_f, float thresh_f)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const CT alpha = static_cast<CT>(alpha_f), thresh = static_cast<CT>(thresh_f);
    CT u[VEC], gate[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { u[v] = CT(0); gate[v] = CT(1); }
    for (int t0 = 0; t0 < T; t0 += TC) {
        Pack<IO, VEC> ain[TC], bin[TC];
#pragma unroll
        for (int k = 0; k < TC; ++k)
            if (t0 + k < T) {
                ain[k] = ld_stream<IO, VEC>(a + static_cast<int64_t>(t0 + k) * N + i);
                bin[k] = ld_stream<IO, VEC>(b + static_cast<int64_t>(t0 + k) * N + i);
            }
#pragma unroll
        for (int k = 0; k < TC; ++k) {
            if (t0 + k < T) {
                Pack<IO, VEC> sp;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const CT leak = mul_rn(mul_rn(alpha, u[v]), gate[v]);
                    u[v] = add_rn(leak, rounded_sum<IO>(ain[k].v[v], bin[k].v[v]));
                    const bool s = u[v] > thresh;
                    gate[v] = s ? CT(0) : CT(1);
                    sp.v[v] = Elem<IO>::store(s ? CT(1) : CT(0));
                }
                st_stream<IO, VEC>(spike + static_cast<int64_t>(t0 + k) * N + i, sp);
            }
        }
    }
}

// register-resident backward, T <= TMAX; EXACT = (T == TMAX)
template <typename IO, int VEC, int TMAX, bool EXACT>
__global__ void lif_add_bwd_kernel(const IO* __restrict__ a, const IO* __restrict__ b, const IO* __restrict__ g,
                                   IO* __restrict__ gx, int T, int64_t N, float alpha_f, float thresh_f,
                                   float beta_f, float interval_f)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const CT alpha = static_cast<CT>(alpha_f), thresh = static_cast<CT>(thresh_f);
    const CT beta = static_cast<CT>(beta_f), interval = static_cast<CT>(interval_f);

    Pack<IO, VEC> ain[TMAX], bin[TMAX], gin[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) ain[t] = ld_stream<IO, VEC>(a + static_cast<int64_t>(t) * N + i);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) bin[t] = ld_stream<IO, VEC>(b + static_cast<int64_t>(t) * N + i);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<int64_t>(t) * N + i);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) { keep_loaded(ain[t]); keep_loaded(bin[t]); keep_loaded(gin[t]); }

    CT u[TMAX][VEC];
    {
        CT uu[VEC], gate[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { uu[v] = CT(0); gate[v] = CT(1); }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (EXACT || t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const CT leak = mul_rn(mul_rn(alpha, uu[v]), gate[v]);
                    uu[v] = add_rn(leak, rounded_sum<IO>(ain[t].v[v], bin[t].v[v]));
                    gate[v] = (uu[v] > thresh) ? CT(0) : CT(1);
                    u[t][v] = uu[v];
                }
            }
        }
    }
    CT gu[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) gu[v] = CT(0);
#pragma unroll
    for (int t = TMAX - 1; t >= 0; --t) {
        if (EXACT || t < T) {
            Pack<IO, VEC> out;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const CT ut = u[t][v];
                const CT ga = mul_rn(gu[v], alpha);
                CT gs = CT(0);
                if (inside_window(ut, thresh, interval)) gs = sub_rn(Elem<IO>::load(gin[t].v[v]), mul_rn(ga, ut));
                const CT keep = (ut <= thresh) ? CT(1) : CT(0);
                gu[v] = add_rn(mul_rn(gs, beta), mul_rn(ga, keep));
                out.v[v] = Elem<IO>::store(gu[v]);
            }
            st_stream<IO, VEC>(gx + static_cast<int64_t>(t) * N + i, out);
        }
    }
}

}  // namespace snn
