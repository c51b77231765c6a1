// C ABI for the fused LIF + 2x2 average pool (declarations: include/snn_b200.h).
#include "../../include/snn_b200.h"
#include "lif_pool_kernels.cuh"

#include <type_traits>

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int kBlock = 256;

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int check(int64_t T, int64_t B, int64_t H, int64_t W, int64_t C, int dtype, int* es) {
    switch (dtype) {
        case SNN_F32: *es = 4; break;
        case SNN_BF16: case SNN_F16: *es = 2; break;
        case SNN_F64: return SNN_ERR_UNSUPPORTED;
        default: return SNN_ERR_DTYPE;
    }
    if (T < 1 || B < 0 || H < 2 || W < 2 || C < 1 || (H & 1) || (W & 1)) return SNN_ERR_SHAPE;
    if (T > 16) return SNN_ERR_UNSUPPORTED;            // time axis is held in registers
    if (B > INT32_MAX || H > INT32_MAX || W > INT32_MAX || C > INT32_MAX) return SNN_ERR_SHAPE;
    const long double total = static_cast<long double>(T) * B * H * W * C;
    if (total > 9.0e18L) return SNN_ERR_SHAPE;
    return SNN_OK;
}

inline int pick_vec(int64_t C, int es, std::initializer_list<const void*> ptrs) {
    for (int vec = 4; vec > 1; vec >>= 1) {
        if (C % vec) continue;
        bool ok = true;
        for (const void* p : ptrs) if (!aligned(p, static_cast<size_t>(es) * vec)) ok = false;
        if (ok) return vec;
    }
    return 1;
}

template <typename F>
inline void dispatch(int dtype, int vec, int T, F&& f) {
    auto with_t = [&](auto io, auto v) {
        if (T <= 4) f(io, v, std::integral_constant<int, 4>{});
        else if (T <= 8) f(io, v, std::integral_constant<int, 8>{});
        else f(io, v, std::integral_constant<int, 16>{});
    };
    auto with_v = [&](auto io) {
        if (vec >= 4) with_t(io, std::integral_constant<int, 4>{});
        else if (vec >= 2) with_t(io, std::integral_constant<int, 2>{});
        else with_t(io, std::integral_constant<int, 1>{});
    };
    if (dtype == SNN_F32) with_v(float{});
    else if (dtype == SNN_BF16) with_v(__nv_bfloat16{});
    else with_v(__half{});
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

}  // namespace

extern "C" {

int snn_lif_pool_fwd(const void* x, void* out, int64_t T, int64_t B, int64_t H, int64_t W, int64_t C,
                     int dtype, float alpha, float thresh, void* stream) {
    int es;
    int rc = check(T, B, H, W, C, dtype, &es);
    if (rc) return rc;
    if (B == 0) return SNN_OK;
    if (!x || !out) return SNN_ERR_NULL;
    if (!aligned(x, es) || !aligned(out, es)) return SNN_ERR_ALIGN;
    int vec = pick_vec(C, es, {x, out});
    if (T > 8 && dtype == SNN_F32 && vec > 2) vec = 2;      // 4 windows x 16 steps of loads stay in registers
    const long long threads = B * (H / 2) * (W / 2) * (C / vec);
    if ((threads + kBlock - 1) / kBlock > 0x7fffffffLL) return SNN_ERR_SHAPE;
    const unsigned grid = static_cast<unsigned>((threads + kBlock - 1) / kBlock);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dispatch(dtype, vec, static_cast<int>(T), [&](auto io, auto v, auto tm) {
        using IO = decltype(io);
        snn::lif_pool_fwd_kernel<IO, decltype(v)::value, decltype(tm)::value><<<grid, kBlock, 0, st>>>(
            static_cast<const IO*>(x), static_cast<IO*>(out), static_cast<int>(T), static_cast<int>(B),
            static_cast<int>(H), static_cast<int>(W), static_cast<int>(C), alpha, thresh);
    });
    return launch_status();
}

int snn_lif_pool_bwd(const void* x, const void* grad_out, void* grad_x, int64_t T, int64_t B, int64_t H,
                     int64_t W, int64_t C, int dtype, float alpha, float thresh, float beta,
                     float interval, void* stream) {
    int es;
    int rc = check(T, B, H, W, C, dtype, &es);
    if (rc) return rc;
    if (B == 0) return SNN_OK;
    if (!x || !grad_out || !grad_x) return SNN_ERR_NULL;
    if (!aligned(x, es) || !aligned(grad_out, es) || !aligned(grad_x, es)) return SNN_ERR_ALIGN;
    int vec = pick_vec(C, es, {x, grad_out, grad_x});
    // SNN_LIF_POOL_BWD_WINDOW=1: the one-thread-per-window kernel (kept for comparison)
    static const bool per_window = [] { const char* e = getenv("SNN_LIF_POOL_BWD_WINDOW"); return e && e[0] == '1'; }();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!per_window) {
        // one thread per full-resolution position: 128-thread CTAs, the LIF backward's register budget
        if (T > 8 && dtype == SNN_F32 && vec > 2) vec = 2;
        constexpr int kFlatBlock = 128;
        const long long threads = B * H * W * (C / vec);
        if ((threads + kFlatBlock - 1) / kFlatBlock > 0x7fffffffLL) return SNN_ERR_SHAPE;
        const unsigned grid = static_cast<unsigned>((threads + kFlatBlock - 1) / kFlatBlock);
        dispatch(dtype, vec, static_cast<int>(T), [&](auto io, auto v, auto tm) {
            using IO = decltype(io);
            snn::lif_pool_bwd_flat_kernel<IO, decltype(v)::value, decltype(tm)::value><<<grid, kFlatBlock, 0, st>>>(
                static_cast<const IO*>(x), static_cast<const IO*>(grad_out), static_cast<IO*>(grad_x),
                static_cast<int>(T), static_cast<int>(B), static_cast<int>(H), static_cast<int>(W),
                static_cast<int>(C), alpha, thresh, beta, interval);
        });
        return launch_status();
    }
    if (T > 8 && vec > 2) vec = 2;                          // 4 windows x 16 steps of loads + 16 steps of state in registers
    const long long threads = B * (H / 2) * (W / 2) * (C / vec);
    // 128-thread CTAs: at ~160 registers per thread three of them fit an SM, one 256-thread CTA would not
    constexpr int kBwdBlock = 128;
    if ((threads + kBwdBlock - 1) / kBwdBlock > 0x7fffffffLL) return SNN_ERR_SHAPE;
    const unsigned grid = static_cast<unsigned>((threads + kBwdBlock - 1) / kBwdBlock);
    dispatch(dtype, vec, static_cast<int>(T), [&](auto io, auto v, auto tm) {
        using IO = decltype(io);
        snn::lif_pool_bwd_kernel<IO, decltype(v)::value, decltype(tm)::value><<<grid, kBwdBlock, 0, st>>>(
            static_cast<const IO*>(x), static_cast<const IO*>(grad_out), static_cast<IO*>(grad_x),
            static_cast<int>(T), static_cast<int>(B), static_cast<int>(H), static_cast<int>(W),
            static_cast<int>(C), alpha, thresh, beta, interval);
    });
    return launch_status();
}

}  // extern "C"
