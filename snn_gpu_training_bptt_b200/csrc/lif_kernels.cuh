// LIF "fire" forward recurrence and BPTT backward pass: device code for sm_100a.
//
// What is computed (reference: liangling76/snn_gpu_training_bptt,
// snnlib/cuda/snn_kernel_fp.cu:37-52 forward, snnlib/cuda/snn_kernel_bp.cu:117-138 backward):
//
//   forward   u_t = (alpha * u_{t-1}) * (1 - s_{t-1}) + x_t ,  s_t = (u_t > thresh),  u_-1 = s_-1 = 0
//   backward  for t = T-1 .. 0, gu = 0 initially:
//               inside = (u_t - thresh < interval) && (thresh - u_t < interval)
//               gs     = inside ? g_t - (gu * alpha) * u_t : 0
//               gu     = gs * beta + (gu * alpha) * (u_t <= thresh)
//               grad_x_t = gu
//
// Every product and sum is rounded on its own (__fmul_rn / __fadd_rn, never contracted
// to an FMA) so results match the reference's PyTorch twin (snnlib/example/gold_op.py)
// bit for bit in fp32.
//
// Layout: time-major [T, N], element (t, n) at t*N + n; N = B*C*H*W flattened (neurons are
// independent). One thread owns VEC consecutive neurons for ALL T steps: state stays in
// registers, every global access is one VEC-wide vector (8 or 16 bytes), consecutive threads
// touch consecutive vectors (fully coalesced), and every byte is touched exactly once.
// The backward kernel recomputes u_t in registers from x instead of reading a stored
// membrane tensor: 12 bytes per neuron-step (fp32) instead of the reference's 8 + 12.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace snn {

// ---------------------------------------------------------------------------------------
// element traits: IO type in global memory, CT = type the state is carried in
// ---------------------------------------------------------------------------------------
template <typename IO> struct Elem;
template <> struct Elem<float> {
    using CT = float;
    static __device__ __forceinline__ float load(float v) { return v; }
    static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Elem<double> {
    using CT = double;
    static __device__ __forceinline__ double load(double v) { return v; }
    static __device__ __forceinline__ double store(double v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
    using CT = float;
    static __device__ __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
    using CT = float;
    static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};

// separately rounded arithmetic (no FMA contraction)
__device__ __forceinline__ float  mul_rn(float a, float b)   { return __fmul_rn(a, b); }
__device__ __forceinline__ float  add_rn(float a, float b)   { return __fadd_rn(a, b); }
__device__ __forceinline__ float  sub_rn(float a, float b)   { return __fsub_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }

// Rectangular surrogate window of the reference, (u - th < iv) && (th - u < iv)
// (snn_kernel_bp.cu:126). IEEE subtraction is antisymmetric, th - u == -(u - th) bit for bit,
// so the pair of tests is exactly |u - th| < iv: one subtract and one compare.
__device__ __forceinline__ bool inside_window(float u, float th, float iv) { return fabsf(sub_rn(u, th)) < iv; }
__device__ __forceinline__ bool inside_window(double u, double th, double iv) { return fabs(sub_rn(u, th)) < iv; }

// ---------------------------------------------------------------------------------------
// VEC-wide packs moved with one instruction
// ---------------------------------------------------------------------------------------
template <int BYTES> struct RawVec;
template <> struct RawVec<16> { using type = uint4; };
template <> struct RawVec<8>  { using type = uint2; };
template <> struct RawVec<4>  { using type = unsigned int; };
template <> struct RawVec<2>  { using type = unsigned short; };
template <> struct RawVec<1>  { using type = unsigned char; };

template <typename E, int VEC>
struct alignas(sizeof(E) * VEC <= 16 ? sizeof(E) * VEC : 16) Pack {
    E v[VEC];
};

// Packs wider than 16 bytes (e.g. 8 fp32 membrane values beside 8 bf16 inputs) move as
// several 16-byte pieces.
// Cache policy of the global accesses (compile-time switch). Default = plain: on B200 plain
// accesses measured 1-2 % faster than the evict-first hints at T=8, N=2^26 (fwd 6.84 vs
// 6.71 TB/s, bwd 7.00 vs 6.85 TB/s), and they leave the freshly written spikes / gradients in
// the 126 MB L2 for the layer that consumes them next.
//   SNN_CACHE_STREAM  ld.global.cs / st.global.cs   evict-first
//   SNN_CACHE_PLAIN   default ld / st
//   SNN_CACHE_NC      ld.global.nc (read-only path) / default st
#define SNN_CACHE_STREAM 0
#define SNN_CACHE_PLAIN 1
#define SNN_CACHE_NC 2
#ifndef SNN_CACHE_POLICY
#define SNN_CACHE_POLICY SNN_CACHE_PLAIN
#endif

template <typename R>
__device__ __forceinline__ R ld_raw(const R* p) {
#if SNN_CACHE_POLICY == SNN_CACHE_STREAM
    return __ldcs(p);
#elif SNN_CACHE_POLICY == SNN_CACHE_NC
    return __ldg(p);
#else
    return *p;
#endif
}
template <typename R>
__device__ __forceinline__ void st_raw(R* p, R v) {
#if SNN_CACHE_POLICY == SNN_CACHE_STREAM
    __stcs(p, v);
#else
    *p = v;
#endif
}

template <typename E, int VEC>
__device__ __forceinline__ Pack<E, VEC> ld_stream(const E* p) {
    constexpr int BYTES = sizeof(E) * VEC;
    if constexpr (BYTES <= 16) {
        using R = typename RawVec<BYTES>::type;
        union { R r; Pack<E, VEC> p; } cvt;
        cvt.r = ld_raw(reinterpret_cast<const R*>(p));
        return cvt.p;
    } else {
        static_assert(BYTES % 16 == 0, "wide packs must be multiples of 16 bytes");
        union { uint4 r[BYTES / 16]; Pack<E, VEC> p; } cvt;
#pragma unroll
        for (int j = 0; j < BYTES / 16; ++j) cvt.r[j] = ld_raw(reinterpret_cast<const uint4*>(p) + j);
        return cvt.p;
    }
}
template <typename E, int VEC>
__device__ __forceinline__ void st_stream(E* p, const Pack<E, VEC>& v) {
    constexpr int BYTES = sizeof(E) * VEC;
    if constexpr (BYTES <= 16) {
        using R = typename RawVec<BYTES>::type;
        union { R r; Pack<E, VEC> p; } cvt;
        cvt.p = v;
        st_raw(reinterpret_cast<R*>(p), cvt.r);
    } else {
        static_assert(BYTES % 16 == 0, "wide packs must be multiples of 16 bytes");
        union { uint4 r[BYTES / 16]; Pack<E, VEC> p; } cvt;
        cvt.p = v;
#pragma unroll
        for (int j = 0; j < BYTES / 16; ++j) st_raw(reinterpret_cast<uint4*>(p) + j, cvt.r[j]);
    }
}

// Makes every word of a freshly loaded pack an operand of an (empty) volatile statement placed
// right after the load loops: the loads cannot be sunk below it. Used by the 16-bit backward,
// where the compiler otherwise postpones the gradient loads until after the forward recurrence to
// save registers and their latency is exposed (measured: 4.6 instead of 6.4 TB/s at T=8).
template <typename P>
__device__ __forceinline__ void keep_loaded(P& p) {
    if constexpr (sizeof(P) >= 4) {
        unsigned int* w = reinterpret_cast<unsigned int*>(&p);
#pragma unroll
        for (int i = 0; i < static_cast<int>(sizeof(P) / 4); ++i) asm volatile("" : "+r"(w[i]));
    }
}

// ---------------------------------------------------------------------------------------
// Forward. Runtime T walked in chunks of TC steps: the TC loads of a chunk are issued
// before any of them is consumed. Outputs, each skipped when its pointer is null (the
// tests are warp-uniform): spikes (IO type), membrane potential (compute type), and one
// packed spike word per neuron (bit t = spike at step t; word_bytes = 1, 2 or 4).
// ---------------------------------------------------------------------------------------
template <typename W, int VEC>
__device__ __forceinline__ void store_words(void* bits, int64_t i, const unsigned int (&word)[VEC]) {
    Pack<W, VEC> w;
#pragma unroll
    for (int v = 0; v < VEC; ++v) w.v[v] = static_cast<W>(word[v]);
    st_stream<W, VEC>(reinterpret_cast<W*>(bits) + i, w);
}

// EXACT = T is a multiple of TC (no per-step bound checks); BITS = packed words requested.
template <typename IO, int VEC, int TC, bool EXACT, bool BITS>
__device__ __forceinline__ void lif_fwd_body(const IO* __restrict__ x, IO* __restrict__ spike,
                                             typename Elem<IO>::CT* __restrict__ mem,
                                             void* __restrict__ bits, int word_bytes, int T, int64_t N,
                                             float alpha_f, float thresh_f)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const CT alpha = static_cast<CT>(alpha_f), thresh = static_cast<CT>(thresh_f);

    CT u[VEC], gate[VEC];
    unsigned int word[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { u[v] = CT(0); gate[v] = CT(1); word[v] = 0u; }

    for (int t0 = 0; t0 < T; t0 += TC) {
        Pack<IO, VEC> xin[TC];
#pragma unroll
        for (int k = 0; k < TC; ++k)
            if (EXACT || t0 + k < T) xin[k] = ld_stream<IO, VEC>(x + static_cast<int64_t>(t0 + k) * N + i);
#pragma unroll
        for (int k = 0; k < TC; ++k) {
            if (EXACT || t0 + k < T) {
                Pack<IO, VEC> sp;
                Pack<CT, VEC> mm;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    CT leak = mul_rn(mul_rn(alpha, u[v]), gate[v]);
                    u[v] = add_rn(leak, Elem<IO>::load(xin[k].v[v]));
                    const bool s = u[v] > thresh;
                    gate[v] = s ? CT(0) : CT(1);
                    sp.v[v] = Elem<IO>::store(s ? CT(1) : CT(0));
                    mm.v[v] = u[v];
                    if (BITS) word[v] |= (s ? 1u : 0u) << ((t0 + k) & 31);
                }
                const int64_t off = static_cast<int64_t>(t0 + k) * N + i;
                if (spike != nullptr) st_stream<IO, VEC>(spike + off, sp);
                if (mem != nullptr) st_stream<CT, VEC>(mem + off, mm);
            }
        }
    }
    if (BITS) {
        if (word_bytes == 1) store_words<unsigned char, VEC>(bits, i, word);
        else if (word_bytes == 2) store_words<unsigned short, VEC>(bits, i, word);
        else store_words<unsigned int, VEC>(bits, i, word);
    }
}

template <typename IO, int VEC, int TC>
__global__ void lif_fwd_kernel(const IO* __restrict__ x, IO* __restrict__ spike,
                               typename Elem<IO>::CT* __restrict__ mem,
                               void* __restrict__ bits, int word_bytes, int T, int64_t N,
                               float alpha_f, float thresh_f)
{
    if (bits != nullptr)
        lif_fwd_body<IO, VEC, TC, false, true>(x, spike, mem, bits, word_bytes, T, N, alpha_f, thresh_f);
    else if (T % TC == 0)
        lif_fwd_body<IO, VEC, TC, true, false>(x, spike, mem, bits, word_bytes, T, N, alpha_f, thresh_f);
    else
        lif_fwd_body<IO, VEC, TC, false, false>(x, spike, mem, bits, word_bytes, T, N, alpha_f, thresh_f);
}

// ---------------------------------------------------------------------------------------
// Backward, register-resident: T <= TMAX. Loads x[0..T) and g[0..T) up front (2*T vector
// loads in flight per thread), rebuilds u_t in registers, then walks time in reverse and
// stores grad_x. No membrane tensor is read or written.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX, bool EXACT>
__device__ __forceinline__ void lif_bwd_body(const IO* __restrict__ x, const IO* __restrict__ g,
                                             IO* __restrict__ gx, int T, int64_t N, float alpha_f,
                                             float thresh_f, float beta_f, float interval_f)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const CT alpha = static_cast<CT>(alpha_f), thresh = static_cast<CT>(thresh_f);
    const CT beta = static_cast<CT>(beta_f), interval = static_cast<CT>(interval_f);

    Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(x + static_cast<int64_t>(t) * N + i);
#pragma unroll
    for (int t = 0; t < TMAX; ++t)
        if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(g + static_cast<int64_t>(t) * N + i);
    if constexpr (sizeof(IO) == 2) {
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) { keep_loaded(xin[t]); keep_loaded(gin[t]); }
    }

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
                    CT leak = mul_rn(mul_rn(alpha, uu[v]), gate[v]);
                    uu[v] = add_rn(leak, Elem<IO>::load(xin[t].v[v]));
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
                const bool inside = inside_window(ut, thresh, interval);
                CT gs = CT(0);
                if (inside) gs = sub_rn(Elem<IO>::load(gin[t].v[v]), mul_rn(ga, ut));
                const CT keep = (ut <= thresh) ? CT(1) : CT(0);
                gu[v] = add_rn(mul_rn(gs, beta), mul_rn(ga, keep));
                out.v[v] = Elem<IO>::store(gu[v]);
            }
            st_stream<IO, VEC>(gx + static_cast<int64_t>(t) * N + i, out);
        }
    }
}

// ---------------------------------------------------------------------------------------
// EXACT = (T == TMAX), chosen by the host (the common case: 4, 6, 8, 12, 16 steps): that
// instantiation carries no per-step bound checks. Two kernels instead of two bodies in one keep
// each at its own register count (16-bit I/O at 16 steps: 8 neurons x 16 steps of state per thread).
template <typename IO, int VEC, int TMAX, bool EXACT>
__global__ void
lif_bwd_kernel(const IO* __restrict__ x, const IO* __restrict__ g,
               IO* __restrict__ gx, int T, int64_t N, float alpha_f,
               float thresh_f, float beta_f, float interval_f)
{
    lif_bwd_body<IO, VEC, TMAX, EXACT>(x, g, gx, T, N, alpha_f, thresh_f, beta_f, interval_f);
}


// Backward for long T (beyond what fits in registers): reads a stored membrane tensor
// (written by lif_fwd_kernel's `mem` output into caller-provided scratch) and walks time in
// reverse in chunks of TC steps. Same arithmetic as above.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, int TC>
__global__ void lif_bwd_mem_kernel(const typename Elem<IO>::CT* __restrict__ mem,
                                   const IO* __restrict__ g, IO* __restrict__ gx, int T,
                                   int64_t N, float alpha_f, float thresh_f, float beta_f,
                                   float interval_f)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const CT alpha = static_cast<CT>(alpha_f), thresh = static_cast<CT>(thresh_f);
    const CT beta = static_cast<CT>(beta_f), interval = static_cast<CT>(interval_f);

    CT gu[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) gu[v] = CT(0);

    for (int t1 = T; t1 > 0; t1 -= TC) {       // chunk covers steps t1-1 .. max(t1-TC, 0)
        Pack<CT, VEC> uin[TC];
        Pack<IO, VEC> gin[TC];
#pragma unroll
        for (int k = 0; k < TC; ++k) {
            const int t = t1 - 1 - k;
            if (t >= 0) {
                const int64_t off = static_cast<int64_t>(t) * N + i;
                uin[k] = ld_stream<CT, VEC>(mem + off);
                gin[k] = ld_stream<IO, VEC>(g + off);
            }
        }
#pragma unroll
        for (int k = 0; k < TC; ++k) {
            const int t = t1 - 1 - k;
            if (t >= 0) {
                Pack<IO, VEC> out;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const CT ut = uin[k].v[v];
                    const CT ga = mul_rn(gu[v], alpha);
                    const bool inside = inside_window(ut, thresh, interval);
                    CT gs = CT(0);
                    if (inside) gs = sub_rn(Elem<IO>::load(gin[k].v[v]), mul_rn(ga, ut));
                    const CT keep = (ut <= thresh) ? CT(1) : CT(0);
                    gu[v] = add_rn(mul_rn(gs, beta), mul_rn(ga, keep));
                    out.v[v] = Elem<IO>::store(gu[v]);
                }
                st_stream<IO, VEC>(gx + static_cast<int64_t>(t) * N + i, out);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Expand packed spike words back to a dense [T, N] 0/1 tensor of type IO.
// ---------------------------------------------------------------------------------------
template <typename IO, int VEC, typename WORD>
__global__ void spike_unpack_kernel(const WORD* __restrict__ bits, IO* __restrict__ spike, int T,
                                    int64_t N)
{
    using CT = typename Elem<IO>::CT;
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= N) return;
    const Pack<WORD, VEC> w = ld_stream<WORD, VEC>(bits + i);
    for (int t = 0; t < T; ++t) {
        Pack<IO, VEC> sp;
#pragma unroll
        for (int v = 0; v < VEC; ++v)
            sp.v[v] = Elem<IO>::store(((static_cast<unsigned int>(w.v[v]) >> t) & 1u) ? CT(1) : CT(0));
        st_stream<IO, VEC>(spike + static_cast<int64_t>(t) * N + i, sp);
    }
}

}  // namespace snn
