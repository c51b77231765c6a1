// C ABI of the fused "LIF of a sum" kernels (lif_add_kernels.cuh); declarations: include/snn_b200.h.
#include "../../include/snn_b200.h"
#include "lif_add_kernels.cuh"

#include <cstdint>
#include <initializer_list>
#include <type_traits>

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int kBlock = 128;

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int elem_size(int dtype) {
    switch (dtype) {
        case SNN_F32: return 4;
        case SNN_BF16: case SNN_F16: return 2;
        default: return 0;
    }
}

// widest VEC <= want that divides N and keeps every pointer aligned to its vector
inline int pick_vec(int want, int64_t N, int es, std::initializer_list<const void*> ptrs) {
    for (int vec = want; vec > 1; vec >>= 1) {
        bool ok = N % vec == 0;
        for (const void* p : ptrs) ok = ok && aligned(p, static_cast<size_t>(es) * vec);
        if (ok) return vec;
    }
    return 1;
}

inline unsigned grid_for(int64_t N, int vec) {
    const int64_t threads = (N + vec - 1) / vec;
    return static_cast<unsigned>((threads + kBlock - 1) / kBlock);
}

template <typename F>
inline void with_io(int dtype, F&& f) {
    if (dtype == SNN_F32) f(float{});
    else if (dtype == SNN_BF16) f(__nv_bfloat16{});
    else f(__half{});
}
template <int MAXV, typename F>
inline void with_vec(int vec, F&& f) {
    if constexpr (MAXV >= 8) { if (vec >= 8) return f(std::integral_constant<int, 8>{}); }
    if constexpr (MAXV >= 4) { if (vec >= 4) return f(std::integral_constant<int, 4>{}); }
    if (vec >= 2) return f(std::integral_constant<int, 2>{});
    return f(std::integral_constant<int, 1>{});
}

inline int common_check(int64_t T, int64_t N, int dtype) {
    if (dtype == SNN_F64) return SNN_ERR_UNSUPPORTED;
    if (elem_size(dtype) == 0) return SNN_ERR_DTYPE;
    if (T < 1 || N < 0 || T > INT32_MAX) return SNN_ERR_SHAPE;
    if (static_cast<long double>(T) * static_cast<long double>(N) > 4.0e18L) return SNN_ERR_SHAPE;
    return SNN_OK;
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

}  // namespace

extern "C" {

int snn_lif_add_fwd(const void* a, const void* b, void* spike, int64_t T, int64_t N, int dtype, float alpha,
                    float thresh, void* stream) {
    int rc = common_check(T, N, dtype);
    if (rc) return rc;
    if (N == 0) return SNN_OK;
    if (!a || !b || !spike) return SNN_ERR_NULL;
    const int es = elem_size(dtype);
    if (!aligned(a, es) || !aligned(b, es) || !aligned(spike, es)) return SNN_ERR_ALIGN;
    const int vec = pick_vec(16 / es, N, es, {a, b, spike});
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    with_io(dtype, [&](auto tag) {
        using IO = decltype(tag);
        constexpr int kMaxVec = 16 / static_cast<int>(sizeof(IO));
        with_vec<kMaxVec>(vec, [&](auto v) {
            constexpr int VEC = decltype(v)::value;
            snn::lif_add_fwd_kernel<IO, VEC, 4><<<grid_for(N, VEC), kBlock, 0, st>>>(
                static_cast<const IO*>(a), static_cast<const IO*>(b), static_cast<IO*>(spike), static_cast<int>(T), N,
                alpha, thresh);
        });
    });
    return launch_status();
}

int snn_lif_add_bwd(const void* a, const void* b, const void* grad_spike, void* grad, int64_t T, int64_t N,
                    int dtype, float alpha, float thresh, float beta, float interval, void* stream) {
    int rc = common_check(T, N, dtype);
    if (rc) return rc;
    if (T > 16) return SNN_ERR_UNSUPPORTED;          // the time axis stays in registers
    if (N == 0) return SNN_OK;
    if (!a || !b || !grad_spike || !grad) return SNN_ERR_NULL;
    const int es = elem_size(dtype);
    if (!aligned(a, es) || !aligned(b, es) || !aligned(grad_spike, es) || !aligned(grad, es)) return SNN_ERR_ALIGN;
    // 8-byte accesses: 2 fp32 or 4 16-bit neurons per thread (three input tensors of up to 16 steps in registers)
    const int vec = pick_vec(8 / es, N, es, {a, b, grad_spike, grad});
    const int Ti = static_cast<int>(T);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    with_io(dtype, [&](auto tag) {
        using IO = decltype(tag);
        constexpr int kMaxVec = 8 / static_cast<int>(sizeof(IO));
        with_vec<kMaxVec>(vec, [&](auto v) {
            constexpr int VEC = decltype(v)::value;
            auto launch = [&](auto tm) {
                constexpr int TMAX = decltype(tm)::value;
                auto ap = static_cast<const IO*>(a); auto bp = static_cast<const IO*>(b);
                auto gp = static_cast<const IO*>(grad_spike); auto op = static_cast<IO*>(grad);
                if (Ti == TMAX)
                    snn::lif_add_bwd_kernel<IO, VEC, TMAX, true><<<grid_for(N, VEC), kBlock, 0, st>>>(
                        ap, bp, gp, op, Ti, N, alpha, thresh, beta, interval);
                else
                    snn::lif_add_bwd_kernel<IO, VEC, TMAX, false><<<grid_for(N, VEC), kBlock, 0, st>>>(
                        ap, bp, gp, op, Ti, N, alpha, thresh, beta, interval);
            };
            if (Ti <= 4) launch(std::integral_constant<int, 4>{});
            else if (Ti <= 8) launch(std::integral_constant<int, 8>{});
            else launch(std::integral_constant<int, 16>{});
        });
    });
    return launch_status();
}

}  // extern "C"
