// C ABI for the batch-norm + LIF family (declarations and the reference interfaces they
// replace: include/snn_b200.h): argument checks, launch configuration, kernel launches.
#include "../../include/snn_b200.h"
#include "bn_lif_kernels.cuh"

#include <type_traits>

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int kBlock = 256;

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int io_size(int dtype) {
    switch (dtype) {
        case SNN_F32: return 4;
        case SNN_BF16: case SNN_F16: return 2;
        default: return 0;               // fp64 is not offered for the BN family
    }
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snn_internal::set_last_cuda_error(static_cast<int>(e));
        return SNN_ERR_CUDA;
    }
    return SNN_OK;
}

inline unsigned grid_for(int64_t N, int vec) {
    const int64_t threads = (N + vec - 1) / vec;
    return static_cast<unsigned>((threads + kBlock - 1) / kBlock);
}

inline int check_geometry(int64_t T, int64_t N, int64_t C, int64_t inner, int dtype) {
    if (dtype == SNN_F64) return SNN_ERR_UNSUPPORTED;
    if (io_size(dtype) == 0) return SNN_ERR_DTYPE;
    if (T < 1 || N < 0 || C < 1 || inner < 1 || T > INT32_MAX || C > INT32_MAX) return SNN_ERR_SHAPE;
    if (N % (C * inner) != 0) return SNN_ERR_SHAPE;          // N = B * C * inner
    if (N > 0 && T > INT64_MAX / 16 / N) return SNN_ERR_SHAPE;
    if ((N + 127) / 128 > 0x7fffffffLL) return SNN_ERR_SHAPE;
    return SNN_OK;
}

// widest vector (elements) the pointers and the row stride allow, capped by `pref`
inline int pick_vec(int pref, int64_t N, int es, std::initializer_list<const void*> ptrs) {
    for (int vec = pref; vec > 1; vec >>= 1) {
        if (N % vec) continue;
        bool ok = true;
        for (const void* p : ptrs)
            if (p && !aligned(p, static_cast<size_t>(es) * vec)) ok = false;
        if (ok) return vec;
    }
    return 1;
}

inline int tmax_for(int T) {
    const int steps[] = {2, 4, 6, 8, 12, 16, 24, 32};
    for (int s : steps) if (T <= s) return s;
    return 0;
}
inline int vec_pref(int dtype, int tmax) {
    if (dtype == SNN_F32) return tmax <= 16 ? 2 : 1;
    return tmax <= 8 ? 4 : (tmax <= 16 ? 2 : 1);
}

template <typename F>
inline void with_io(int dtype, F&& f) {
    if (dtype == SNN_F32) f(float{});
    else if (dtype == SNN_BF16) f(__nv_bfloat16{});
    else f(__half{});
}
template <typename F>
inline void with_vec4(int vec, F&& f) {
    if (vec >= 4) f(std::integral_constant<int, 4>{});
    else if (vec >= 2) f(std::integral_constant<int, 2>{});
    else f(std::integral_constant<int, 1>{});
}
template <typename F>
inline void with_tmax(int tmax, F&& f) {
    switch (tmax) {
        case 2: return f(std::integral_constant<int, 2>{});
        case 4: return f(std::integral_constant<int, 4>{});
        case 6: return f(std::integral_constant<int, 6>{});
        case 8: return f(std::integral_constant<int, 8>{});
        case 12: return f(std::integral_constant<int, 12>{});
        case 16: return f(std::integral_constant<int, 16>{});
        case 24: return f(std::integral_constant<int, 24>{});
        default: return f(std::integral_constant<int, 32>{});
    }
}
// VEC * TMAX bounded so x, g, u and gu of all steps stay in registers
template <int TMAX> constexpr int max_vec() { return TMAX <= 8 ? 4 : (TMAX <= 16 ? 2 : 1); }

}  // namespace

extern "C" {

int snn_bn_lif_fwd(const void* x, const float* weight, const float* bias, const float* var,
                   const float* mean, float eps, void* out, float* mem, float* ivar_out,
                   int64_t T, int64_t N, int64_t C, int64_t inner, int dtype, int fire,
                   float alpha, float thresh, void* stream) {
    int rc = check_geometry(T, N, C, inner, dtype);
    if (rc) return rc;
    if (!weight || !bias || !mean) return SNN_ERR_NULL;
    if (!var && !ivar_out) return SNN_ERR_NULL;      // without var, ivar_out is the INPUT ivar
    if (N == 0) return SNN_OK;
    if (!x || (!out && !(fire && mem))) return SNN_ERR_NULL;
    const int es = io_size(dtype);
    if (!aligned(x, es) || !aligned(out, es) || !aligned(mem, 4)) return SNN_ERR_ALIGN;
    const int pref = dtype == SNN_F32 ? 2 : 4;
    int vec = pick_vec(pref, N, es, {x, out});
    if (mem && !aligned(mem, 4 * static_cast<size_t>(vec) > 16 ? 16 : 4 * static_cast<size_t>(vec))) vec = 1;
    snn::BnParams p{mean, weight, bias, var, var ? nullptr : ivar_out, eps, static_cast<long long>(inner),
                    static_cast<int>(C)};
    if (!var) ivar_out = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // plain BN has no recurrence: walk it as one long time step
    const int Ti = fire ? static_cast<int>(T) : 1;
    const long long Ni = fire ? N : T * N;
    with_io(dtype, [&](auto tag) {
        using IO = decltype(tag);
        with_vec4(vec, [&](auto v) {
            constexpr int VEC = decltype(v)::value;
            const unsigned grid = grid_for(Ni, VEC);
            if (fire) {
                if (Ti <= 4)
                    snn::bn_lif_fwd_kernel<IO, VEC, 4, true><<<grid, kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<IO*>(out), mem, ivar_out, p, Ti, Ni, alpha, thresh);
                else
                    snn::bn_lif_fwd_kernel<IO, VEC, 8, true><<<grid, kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<IO*>(out), mem, ivar_out, p, Ti, Ni, alpha, thresh);
            } else {
                snn::bn_lif_fwd_kernel<IO, VEC, 4, false><<<grid, kBlock, 0, st>>>(
                    static_cast<const IO*>(x), static_cast<IO*>(out), nullptr, ivar_out, p, Ti, Ni, alpha, thresh);
            }
        });
    });
    return launch_status();
}

int snn_bn_lif_bwd_sums(const void* x, const void* grad, const float* weight, const float* bias,
                        const float* ivar, const float* mean, float* sum_g, float* sum_gx,
                        int64_t T, int64_t N, int64_t C, int64_t inner, int dtype, int fire,
                        float alpha, float thresh, float beta, float interval, void* stream) {
    int rc = check_geometry(T, N, C, inner, dtype);
    if (rc) return rc;
    if (!weight || !ivar || !mean || !sum_g || !sum_gx || (fire && !bias)) return SNN_ERR_NULL;
    if (fire && T > 32) return SNN_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(sum_g, 0, sizeof(float) * C, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(sum_gx, 0, sizeof(float) * C, st);
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    if (N == 0) return SNN_OK;
    if (!x || !grad) return SNN_ERR_NULL;
    const int es = io_size(dtype);
    if (!aligned(x, es) || !aligned(grad, es)) return SNN_ERR_ALIGN;
    const int Ti = fire ? static_cast<int>(T) : 1;
    const long long Ni = fire ? N : T * N;
    const int tmax = tmax_for(Ti);
    const int vec = pick_vec(vec_pref(dtype, tmax), Ni, es, {x, grad});
    snn::BnParams p{mean, weight, bias, nullptr, ivar, 0.f, static_cast<long long>(inner), static_cast<int>(C)};
    with_io(dtype, [&](auto tag) {
        using IO = decltype(tag);
        auto smem_for = [&](int VEC, int* nq) {
            const long long span = static_cast<long long>(kBlock) * VEC;
            const long long runs = (span + inner - 1) / inner + 1;    // channel runs a CTA can touch
            *nq = static_cast<int>(runs < C ? runs : C);             // more runs than channels: one slot per channel
            return 2 * sizeof(float) * static_cast<size_t>(*nq);
        };
        // runs of one neuron whose channels repeat with the CTA span: few fat CTAs, one flush each
        auto short_runs = [&](int VEC) {
            return inner == 1 && (static_cast<long long>(kBlock) * VEC) % C == 0 && Ni % VEC == 0 && C <= 4096;
        };
        auto fat_grid = [&](int VEC) {
            const long long slabs = (Ni + static_cast<long long>(kBlock) * VEC - 1) / (static_cast<long long>(kBlock) * VEC);
            int dev = 0, sms = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            const long long want = static_cast<long long>(sms) * 8;
            return static_cast<unsigned>(slabs < want ? slabs : want);
        };
        // long runs: a grid that is a multiple of C, every CTA stays on one channel (see the kernel)
        const long long runs = Ni / inner;                       // channel runs in the tensor: (T*)B*C
        auto long_runs = [&](int VEC) {
            return inner >= static_cast<long long>(kBlock) * VEC && inner % VEC == 0 && runs / C >= 1;
        };
        auto run_grid = [&]() {
            int dev = 0, sms = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            long long k = (static_cast<long long>(sms) * 8 + C - 1) / C;     // CTAs per channel
            const long long per_channel = runs / C;                          // visits available per channel
            if (k > per_channel) k = per_channel;
            if (k < 1) k = 1;
            return static_cast<unsigned>(k * C);
        };
        if (!fire) {
            with_vec4(vec, [&](auto v) {
                constexpr int VEC = decltype(v)::value;
                if (long_runs(VEC)) {
                    snn::bn_lif_bwd_sums_run_kernel<IO, VEC, 2, false><<<run_grid(), kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, runs, alpha,
                        thresh, beta, interval);
                    return;
                }
                if (short_runs(VEC)) {
                    snn::bn_lif_bwd_sums_cl_kernel<IO, VEC, 2, false><<<fat_grid(VEC), kBlock, 2 * sizeof(float) * C, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, alpha, thresh,
                        beta, interval);
                    return;
                }
                int nq; const size_t smem = smem_for(VEC, &nq);
                if (inner % (32 * VEC) == 0)
                    snn::bn_lif_bwd_sums_kernel<IO, VEC, 2, false, true><<<grid_for(Ni, VEC), kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, nq,
                        alpha, thresh, beta, interval);
                else
                    snn::bn_lif_bwd_sums_kernel<IO, VEC, 2, false, false><<<grid_for(Ni, VEC), kBlock, smem, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, nq,
                        alpha, thresh, beta, interval);
            });
            return;
        }
        with_tmax(tmax, [&](auto tm) {
            constexpr int TMAX = decltype(tm)::value;
            with_vec4(vec < max_vec<TMAX>() ? vec : max_vec<TMAX>(), [&](auto v) {
                constexpr int VEC = decltype(v)::value < max_vec<TMAX>() ? decltype(v)::value : max_vec<TMAX>();
                if (long_runs(VEC)) {
                    snn::bn_lif_bwd_sums_run_kernel<IO, VEC, TMAX, true><<<run_grid(), kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, runs, alpha,
                        thresh, beta, interval);
                    return;
                }
                if (short_runs(VEC)) {
                    snn::bn_lif_bwd_sums_cl_kernel<IO, VEC, TMAX, true><<<fat_grid(VEC), kBlock, 2 * sizeof(float) * C, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, alpha, thresh,
                        beta, interval);
                    return;
                }
                int nq; const size_t smem = smem_for(VEC, &nq);
                if (inner % (32 * VEC) == 0)
                    snn::bn_lif_bwd_sums_kernel<IO, VEC, TMAX, true, true><<<grid_for(Ni, VEC), kBlock, 0, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, nq,
                        alpha, thresh, beta, interval);
                else
                    snn::bn_lif_bwd_sums_kernel<IO, VEC, TMAX, true, false><<<grid_for(Ni, VEC), kBlock, smem, st>>>(
                        static_cast<const IO*>(x), static_cast<const IO*>(grad), sum_g, sum_gx, p, Ti, Ni, nq,
                        alpha, thresh, beta, interval);
            });
        });
    });
    return launch_status();
}

int snn_bn_channel_means(const float* sum_g, const float* sum_gx, const float* weight, float* gxhat,
                         float* gxhatx, int64_t C, double count, void* stream) {
    if (!sum_g || !sum_gx || !weight || !gxhat || !gxhatx) return SNN_ERR_NULL;
    if (C < 1 || C > INT32_MAX || !(count > 0)) return SNN_ERR_SHAPE;
    snn::bn_channel_means_kernel<<<static_cast<unsigned>((C + 127) / 128), 128, 0,
                                   static_cast<cudaStream_t>(stream)>>>(
        sum_g, sum_gx, weight, gxhat, gxhatx, static_cast<int>(C), static_cast<float>(1.0 / count));
    return launch_status();
}

int snn_bn_lif_bwd_input(const void* x, const void* grad, const float* weight, const float* bias,
                         const float* ivar, const float* mean, const float* gxhat,
                         const float* gxhatx, void* grad_x, int64_t T, int64_t N, int64_t C,
                         int64_t inner, int dtype, int fire, float alpha, float thresh, float beta,
                         float interval, void* stream) {
    int rc = check_geometry(T, N, C, inner, dtype);
    if (rc) return rc;
    if (!weight || !ivar || !mean || !gxhat || !gxhatx || (fire && !bias)) return SNN_ERR_NULL;
    if (fire && T > 32) return SNN_ERR_UNSUPPORTED;
    if (N == 0) return SNN_OK;
    if (!x || !grad || !grad_x) return SNN_ERR_NULL;
    const int es = io_size(dtype);
    if (!aligned(x, es) || !aligned(grad, es) || !aligned(grad_x, es)) return SNN_ERR_ALIGN;
    const int Ti = fire ? static_cast<int>(T) : 1;
    const long long Ni = fire ? N : T * N;
    const int tmax = tmax_for(Ti);
    const int vec = pick_vec(vec_pref(dtype, tmax), Ni, es, {x, grad, grad_x});
    snn::BnParams p{mean, weight, bias, nullptr, ivar, 0.f, static_cast<long long>(inner), static_cast<int>(C)};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    with_io(dtype, [&](auto tag) {
        using IO = decltype(tag);
        if (!fire) {
            with_vec4(vec, [&](auto v) {
                constexpr int VEC = decltype(v)::value;
                snn::bn_lif_bwd_input_kernel<IO, VEC, 2, false><<<grid_for(Ni, VEC), kBlock, 0, st>>>(
                    static_cast<const IO*>(x), static_cast<const IO*>(grad), gxhat, gxhatx,
                    static_cast<IO*>(grad_x), p, Ti, Ni, alpha, thresh, beta, interval);
            });
            return;
        }
        with_tmax(tmax, [&](auto tm) {
            constexpr int TMAX = decltype(tm)::value;
            with_vec4(vec < max_vec<TMAX>() ? vec : max_vec<TMAX>(), [&](auto v) {
                constexpr int VEC = decltype(v)::value < max_vec<TMAX>() ? decltype(v)::value : max_vec<TMAX>();
                snn::bn_lif_bwd_input_kernel<IO, VEC, TMAX, true><<<grid_for(Ni, VEC), kBlock, 0, st>>>(
                    static_cast<const IO*>(x), static_cast<const IO*>(grad), gxhat, gxhatx,
                    static_cast<IO*>(grad_x), p, Ti, Ni, alpha, thresh, beta, interval);
            });
        });
    });
    return launch_status();
}

}  // extern "C"
