// LIF followed by 2x2 average pooling (stride 2) in one pass, for channels-last activations.
//
// In the spiking CNNs this library serves, a LIF layer is often followed by AvgPool2d(2) on
// every time step (the pooled spikes feed the next convolution; nothing else reads the
// full-resolution spikes). Run as two ops that costs, per full-resolution neuron-step in bf16,
// 2 B read + 2 B write (LIF) + 2 B read + 0.5 B write (pool) forward, and the same pattern
// mirrored backward. Fused, the full-resolution spike tensor and the full-resolution spike
// gradient never exist: forward reads x and writes pooled spikes (2 + 0.5 B), backward reads x
// and the pooled gradient and writes grad_x (2 + 0.5 + 2 B).
//
// Arithmetic is the LIF recurrence / reverse pass of lif_kernels.cuh (reference
// snnlib/cuda/snn_kernel_fp.cu:37-52, snn_kernel_bp.cu:117-138) composed with average pooling:
//   out(t, b, ho, wo, c)  = (1/4) * sum_{dy,dx} s(t, b, 2ho+dy, 2wo+dx, c)        (exact: k/4)
//   g_s(t, b, h, w, c)    = (1/4) * g_out(t, b, h/2, w/2, c)                      (exact scaling)
//
// Layout: x is [T][B][H][W][C] in memory (a channels-last batch of T*B images), out / g_out are
// [T][B][H/2][W/2][C]. One thread owns VEC consecutive channels of one pooled position for all T
// steps. The loads of all four window positions (4 x T vectors) are issued before any of them is
// used - processed position by position, each thread went through four dependent rounds of memory
// latency with only T small loads in flight, and the kernels ran at a quarter of the bandwidth.
#pragma once
#include "lif_kernels.cuh"

namespace snn {

// id -> (b, ho, wo, cv); 32-bit arithmetic whenever the thread count fits (64-bit division is
// emulated with ~100 instructions and there are three of them per thread)
__device__ __forceinline__ void decompose(long long id, long long total, int Cv, int Wo, int Ho,
                                          int& cv, int& wo, int& ho, int& b) {
    if (total <= 0xffffffffLL) {
        unsigned int r = static_cast<unsigned int>(id);
        cv = static_cast<int>(r % Cv); r /= Cv;
        wo = static_cast<int>(r % Wo); r /= Wo;
        ho = static_cast<int>(r % Ho);
        b = static_cast<int>(r / Ho);
    } else {
        long long r = id;
        cv = static_cast<int>(r % Cv); r /= Cv;
        wo = static_cast<int>(r % Wo); r /= Wo;
        ho = static_cast<int>(r % Ho);
        b = static_cast<int>(r / Ho);
    }
}

template <typename IO, int VEC, int TMAX>
__global__ void lif_pool_fwd_kernel(const IO* __restrict__ x, IO* __restrict__ out, int T, int B,
                                    int H, int W, int C, float alpha, float thresh)
{
    const int Ho = H / 2, Wo = W / 2, Cv = C / VEC;
    const long long total = static_cast<long long>(B) * Ho * Wo * Cv;
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (id >= total) return;
    int cv, wo, ho, b;
    decompose(id, total, Cv, Wo, Ho, cv, wo, ho, b);
    const long long n_full = static_cast<long long>(B) * H * W * C;      // neurons per time step
    const long long n_pool = static_cast<long long>(B) * Ho * Wo * C;
    const long long o_off = ((static_cast<long long>(b) * Ho + ho) * Wo + wo) * C + cv * VEC;

    float acc[TMAX][VEC];
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[t][v] = 0.f;

    Pack<IO, VEC> xin[4][TMAX];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int h = 2 * ho + (p >> 1), w = 2 * wo + (p & 1);
        const long long off = ((static_cast<long long>(b) * H + h) * W + w) * C + cv * VEC;
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (t < T) xin[p][t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * n_full + off);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (t < T) keep_loaded(xin[p][t]);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        float u[VEC], gate[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { u[v] = 0.f; gate[v] = 1.f; }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float leak = mul_rn(mul_rn(alpha, u[v]), gate[v]);
                    u[v] = add_rn(leak, Elem<IO>::load(xin[p][t].v[v]));
                    const bool s = u[v] > thresh;
                    gate[v] = s ? 0.f : 1.f;
                    acc[t][v] += s ? 0.25f : 0.f;
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
        if (t < T) {
            Pack<IO, VEC> o;
#pragma unroll
            for (int v = 0; v < VEC; ++v) o.v[v] = Elem<IO>::store(acc[t][v]);
            st_stream<IO, VEC>(out + static_cast<long long>(t) * n_pool + o_off, o);
        }
    }
}

template <typename IO, int VEC, int TMAX>
__global__ void lif_pool_bwd_kernel(const IO* __restrict__ x, const IO* __restrict__ g_out,
                                    IO* __restrict__ gx, int T, int B, int H, int W, int C,
                                    float alpha, float thresh, float beta, float interval)
{
    const int Ho = H / 2, Wo = W / 2, Cv = C / VEC;
    const long long total = static_cast<long long>(B) * Ho * Wo * Cv;
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (id >= total) return;
    int cv, wo, ho, b;
    decompose(id, total, Cv, Wo, Ho, cv, wo, ho, b);
    const long long n_full = static_cast<long long>(B) * H * W * C;
    const long long n_pool = static_cast<long long>(B) * Ho * Wo * C;
    const long long o_off = ((static_cast<long long>(b) * Ho + ho) * Wo + wo) * C + cv * VEC;

    float gs[TMAX][VEC];                       // gradient w.r.t. each of the four spikes: g_out / 4
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
        if (t < T) {
            const Pack<IO, VEC> gin = ld_stream<IO, VEC>(g_out + static_cast<long long>(t) * n_pool + o_off);
#pragma unroll
            for (int v = 0; v < VEC; ++v) gs[t][v] = mul_rn(Elem<IO>::load(gin.v[v]), 0.25f);
        }
    }
    Pack<IO, VEC> xin[4][TMAX];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int h = 2 * ho + (p >> 1), w = 2 * wo + (p & 1);
        const long long off = ((static_cast<long long>(b) * H + h) * W + w) * C + cv * VEC;
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (t < T) xin[p][t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * n_full + off);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (t < T) keep_loaded(xin[p][t]);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int h = 2 * ho + (p >> 1), w = 2 * wo + (p & 1);
        const long long off = ((static_cast<long long>(b) * H + h) * W + w) * C + cv * VEC;
        float u[TMAX][VEC];
        float uu[VEC], gate[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { uu[v] = 0.f; gate[v] = 1.f; }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float leak = mul_rn(mul_rn(alpha, uu[v]), gate[v]);
                    uu[v] = add_rn(leak, Elem<IO>::load(xin[p][t].v[v]));
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
            if (t < T) {
                Pack<IO, VEC> o;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float ut = u[t][v];
                    const float ga = mul_rn(gu[v], alpha);
                    const bool inside = inside_window(ut, thresh, interval);
                    float g1 = 0.f;
                    if (inside) g1 = sub_rn(gs[t][v], mul_rn(ga, ut));
                    const float keep = (ut <= thresh) ? 1.f : 0.f;
                    gu[v] = add_rn(mul_rn(g1, beta), mul_rn(ga, keep));
                    o.v[v] = Elem<IO>::store(gu[v]);
                }
                st_stream<IO, VEC>(gx + static_cast<long long>(t) * n_full + off, o);
            }
        }
    }
}

// Backward with one thread per FULL-resolution position (VEC channels, all T steps): the plain LIF
// reverse pass whose upstream gradient is gathered from the pooled tensor (each pooled vector is read
// by the four threads of its window; it is a quarter of the bytes and stays in L1 / L2). Four times
// the threads of the kernel above at ~60 registers each; same arithmetic, same results.
template <typename IO, int VEC, int TMAX>
__global__ void lif_pool_bwd_flat_kernel(const IO* __restrict__ x, const IO* __restrict__ g_out,
                                         IO* __restrict__ gx, int T, int B, int H, int W, int C,
                                         float alpha, float thresh, float beta, float interval)
{
    const int Ho = H / 2, Wo = W / 2, Cv = C / VEC;
    const long long total = static_cast<long long>(B) * H * W * Cv;
    const long long id = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (id >= total) return;
    int cv, w, h, b;
    decompose(id, total, Cv, W, H, cv, w, h, b);
    const long long n_full = static_cast<long long>(B) * H * W * C;
    const long long n_pool = static_cast<long long>(B) * Ho * Wo * C;
    const long long off = id * VEC;                                    // ((b*H + h)*W + w)*C + cv*VEC
    const long long o_off = ((static_cast<long long>(b) * Ho + (h >> 1)) * Wo + (w >> 1)) * C + cv * VEC;

    Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<long long>(t) * n_full + off);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (t < T) gin[t] = ld_stream<IO, VEC>(g_out + static_cast<long long>(t) * n_pool + o_off);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (t < T) { keep_loaded(xin[t]); keep_loaded(gin[t]); }

    float u[TMAX][VEC];
    {
        float uu[VEC], gate[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { uu[v] = 0.f; gate[v] = 1.f; }
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
            if (t < T) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float leak = mul_rn(mul_rn(alpha, uu[v]), gate[v]);
                    uu[v] = add_rn(leak, Elem<IO>::load(xin[t].v[v]));
                    gate[v] = (uu[v] > thresh) ? 0.f : 1.f;
                    u[t][v] = uu[v];
                }
            }
        }
    }
    float gu[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) gu[v] = 0.f;
#pragma unroll
    for (int t = TMAX - 1; t >= 0; --t) {
        if (t < T) {
            Pack<IO, VEC> o;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float ut = u[t][v];
                const float ga = mul_rn(gu[v], alpha);
                float g1 = 0.f;
                if (inside_window(ut, thresh, interval))
                    g1 = sub_rn(mul_rn(Elem<IO>::load(gin[t].v[v]), 0.25f), mul_rn(ga, ut));
                const float keep = (ut <= thresh) ? 1.f : 0.f;
                gu[v] = add_rn(mul_rn(g1, beta), mul_rn(ga, keep));
                o.v[v] = Elem<IO>::store(gu[v]);
            }
            st_stream<IO, VEC>(gx + static_cast<long long>(t) * n_full + off, o);
        }
    }
}

}  // namespace snn
