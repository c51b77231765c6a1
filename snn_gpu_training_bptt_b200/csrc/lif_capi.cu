// C ABI of libsnn_b200.so for the LIF fire path: argument validation, choice of vector
// width / time chunk, kernel launch. Declarations and the reference interfaces each entry
// point replaces: include/snn_b200.h.
#include "../../include/snn_b200.h"
#include "lif_kernels.cuh"

#include <stdlib.h>

#include <type_traits>

namespace {

constexpr int kBlock = 256;
constexpr int kRegT = 32;  // longest time axis the register-resident backward handles

thread_local int g_last_cuda_error = 0;

inline int dtype_size(int dtype) {
    switch (dtype) {
        case SNN_F32: return 4;
        case SNN_BF16: return 2;
        case SNN_F16: return 2;
        case SNN_F64: return 8;
        default: return 0;
    }
}
inline int state_size(int dtype) { return dtype == SNN_F64 ? 8 : 4; }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda_error = static_cast<int>(e);
        return SNN_ERR_CUDA;
    }
    return SNN_OK;
}

inline unsigned int grid_for(int64_t N, int vec, int block) {
    const int64_t threads = (N + vec - 1) / vec;
    return static_cast<unsigned int>((threads + block - 1) / block);
}

inline int common_shape_check(int64_t T, int64_t N, int dtype) {
    if (dtype_size(dtype) == 0) return SNN_ERR_DTYPE;
    if (T < 1 || N < 0) return SNN_ERR_SHAPE;
    if (T > INT32_MAX) return SNN_ERR_SHAPE;
    // element offsets are int64; thread count must fit the 1-D grid
    if (N > 0 && T > INT64_MAX / 16 / N) return SNN_ERR_SHAPE;
    if ((N + 127) / 128 > 0x7fffffffLL) return SNN_ERR_SHAPE;
    return SNN_OK;
}

// Largest power-of-two vector width <= pref such that every row start t*N stays aligned
// (N % vec == 0) and every listed pointer is aligned to vec * its element size (capped at
// 16 bytes, the widest single access).
struct PtrReq { const void* p; int elem; };
inline int pick_vec(int pref, int64_t N, const PtrReq* reqs, int nreq) {
    for (int vec = pref; vec > 1; vec >>= 1) {
        if (N % vec) continue;
        bool ok = true;
        for (int k = 0; k < nreq; ++k) {
            if (!reqs[k].p) continue;
            size_t a = static_cast<size_t>(reqs[k].elem) * vec;
            if (a > 16) a = 16;
            if (!aligned(reqs[k].p, a)) { ok = false; break; }
        }
        if (ok) return vec;
    }
    return 1;
}

// ---- launch configuration ------------------------------------------------------------------
// Chosen from timing sweeps on B200 at N = 2^25..2^26 (fp32 and bf16, T = 4..32): 8-byte
// accesses per thread with the time axis unrolled to the smallest instantiated bound >= T
// gave the highest bandwidth for fp32; 16-byte accesses and 128-thread CTAs for 16-bit I/O.
struct Tune { int vec; int block; };

inline Tune fwd_tune(int dtype) {
    switch (dtype) {
        case SNN_F32: return {2, 256};
        case SNN_F64: return {2, 256};
        default: return {8, 128};          // bf16 / fp16
    }
}
inline int fwd_tc(int dtype, int T) {
    if (dtype == SNN_BF16 || dtype == SNN_F16) return 4;
    return T <= 4 ? 4 : 8;
}
inline int bwd_tmax(int T) {
    const int steps[] = {2, 4, 6, 8, 12, 16, 24, 32};
    for (int s : steps) if (T <= s) return s;
    return 32;
}
inline Tune bwd_tune(int dtype, int tmax) {
    switch (dtype) {
        case SNN_F32: return {2, tmax >= 32 ? 128 : 256};
        case SNN_F64: return {tmax <= 16 ? 2 : 1, tmax >= 24 ? 128 : 256};
        default: {
            // 16-bit I/O: 16-byte accesses (8 neurons per thread) while the time axis is short, 8-byte
            // accesses from `wide_t` steps on. SNN_LIF_BWD_WIDE_T overrides the switch point (a tuning aid).
            static const int wide_t = [] { const char* e = getenv("SNN_LIF_BWD_WIDE_T"); return e ? atoi(e) : 6; }();
            return {tmax <= wide_t ? 8 : (tmax <= 16 ? 4 : 2), 128};
        }
    }
}

// Calls f(std::integral_constant<int, V>) for the largest instantiated V <= vec.
template <int MAXV, typename F>
inline void with_vec(int vec, F&& f) {
    if constexpr (MAXV >= 8) { if (vec >= 8) return f(std::integral_constant<int, 8>{}); }
    if constexpr (MAXV >= 4) { if (vec >= 4) return f(std::integral_constant<int, 4>{}); }
    if constexpr (MAXV >= 2) { if (vec >= 2) return f(std::integral_constant<int, 2>{}); }
    return f(std::integral_constant<int, 1>{});
}
template <typename F>
inline void with_dtype(int dtype, F&& f) {
    switch (dtype) {
        case SNN_F32: return f(float{});
        case SNN_BF16: return f(__nv_bfloat16{});
        case SNN_F16: return f(__half{});
        default: return f(double{});
    }
}

// ---- forward ------------------------------------------------------------------------------
int lif_fwd_impl(const void* x, void* spike, void* mem, void* bits, int64_t T, int64_t N,
                 int dtype, float alpha, float thresh, cudaStream_t st) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return rc;
    if (N == 0) return SNN_OK;                       // nothing to do; pointers may be NULL
    if (!x || (!spike && !mem && !bits)) return SNN_ERR_NULL;
    const int es = dtype_size(dtype), ss = state_size(dtype);
    int word_bytes = 0;
    if (bits) {
        if (T > 32) return SNN_ERR_UNSUPPORTED;
        word_bytes = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    }
    if (!aligned(x, es) || !aligned(spike, es) || !aligned(mem, ss) ||
        (bits && !aligned(bits, word_bytes)))
        return SNN_ERR_ALIGN;

    const Tune tune = fwd_tune(dtype);
    const PtrReq reqs[] = {{x, es}, {spike, es}, {mem, ss}, {bits, word_bytes ? word_bytes : 1}};
    const int vec = pick_vec(tune.vec, N, reqs, 4);
    const int tc = fwd_tc(dtype, static_cast<int>(T));
    const int Ti = static_cast<int>(T);
    with_dtype(dtype, [&](auto tag) {
        using IO = decltype(tag);
        using CT = typename snn::Elem<IO>::CT;
        constexpr int kMaxVec = 16 / static_cast<int>(sizeof(IO));
        with_vec<kMaxVec>(vec, [&](auto v) {
            constexpr int VEC = decltype(v)::value;
            const unsigned grid = grid_for(N, VEC, tune.block);
            auto xp = static_cast<const IO*>(x);
            auto sp = static_cast<IO*>(spike);
            auto mp = static_cast<CT*>(mem);
            if (tc == 4)
                snn::lif_fwd_kernel<IO, VEC, 4><<<grid, tune.block, 0, st>>>(xp, sp, mp, bits, word_bytes, Ti, N, alpha, thresh);
            else
                snn::lif_fwd_kernel<IO, VEC, 8><<<grid, tune.block, 0, st>>>(xp, sp, mp, bits, word_bytes, Ti, N, alpha, thresh);
        });
    });
    return check_launch();
}

// ---- backward -----------------------------------------------------------------------------
template <typename IO, int TMAX>
void launch_bwd_regs(int vec, int block, const void* x, const void* g, void* gx, int T, int64_t N,
                     float alpha, float thresh, float beta, float interval, cudaStream_t st) {
    // VEC * TMAX state words per thread stay in registers: cap the width for long time axes
    constexpr int kIoMax = 16 / static_cast<int>(sizeof(IO));
    // 16-bit I/O keeps 16-byte accesses (8 neurons) up to 16 steps: the inputs sit in registers as
    // packed pairs, so 8 x 16 fp32 membrane values + 2 x 64 packed words still fit (214 registers)
    constexpr int kWords = TMAX <= 8 ? 8 : (TMAX <= 16 ? (sizeof(IO) == 2 ? 8 : 4) : 2);
    constexpr int kRegMax = kWords * 4 / static_cast<int>(sizeof(typename snn::Elem<IO>::CT));
    constexpr int kMaxVec = kIoMax < kRegMax ? kIoMax : kRegMax;
    with_vec<kMaxVec>(vec, [&](auto v) {
        constexpr int VEC = decltype(v)::value;
        if (T == TMAX)
            snn::lif_bwd_kernel<IO, VEC, TMAX, true><<<grid_for(N, VEC, block), block, 0, st>>>(
                static_cast<const IO*>(x), static_cast<const IO*>(g), static_cast<IO*>(gx), T, N, alpha,
                thresh, beta, interval);
        else
            snn::lif_bwd_kernel<IO, VEC, TMAX, false><<<grid_for(N, VEC, block), block, 0, st>>>(
                static_cast<const IO*>(x), static_cast<const IO*>(g), static_cast<IO*>(gx), T, N, alpha,
                thresh, beta, interval);
    });
}

template <typename IO>
void launch_bwd_pick_t(int tmax, int vec, int block, const void* x, const void* g, void* gx, int T,
                       int64_t N, float alpha, float thresh, float beta, float interval,
                       cudaStream_t st) {
#define SNN_BWD_CASE(TM) \
    case TM: return launch_bwd_regs<IO, TM>(vec, block, x, g, gx, T, N, alpha, thresh, beta, interval, st);
    switch (tmax) {
        SNN_BWD_CASE(2) SNN_BWD_CASE(4) SNN_BWD_CASE(6) SNN_BWD_CASE(8)
        SNN_BWD_CASE(12) SNN_BWD_CASE(16) SNN_BWD_CASE(24)
        default: return launch_bwd_regs<IO, 32>(vec, block, x, g, gx, T, N, alpha, thresh, beta, interval, st);
    }
#undef SNN_BWD_CASE
}

int lif_bwd_impl(const void* x, const void* g, void* gx, int64_t T, int64_t N, int dtype,
                 float alpha, float thresh, float beta, float interval, void* workspace,
                 size_t workspace_bytes, cudaStream_t st) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return rc;
    const int es = dtype_size(dtype), ss = state_size(dtype);
    const int Ti = static_cast<int>(T);
    const bool long_t = T > kRegT;
    const size_t need = long_t ? static_cast<size_t>(T) * static_cast<size_t>(N) * ss : 0;
    if (long_t && need > 0 && (!workspace || workspace_bytes < need)) return SNN_ERR_WORKSPACE;
    if (N == 0) return SNN_OK;
    if (!x || !g || !gx) return SNN_ERR_NULL;
    if (!aligned(x, es) || !aligned(g, es) || !aligned(gx, es)) return SNN_ERR_ALIGN;

    if (!long_t) {
        const int tmax = bwd_tmax(Ti);
        const Tune tune = bwd_tune(dtype, tmax);
        const PtrReq reqs[] = {{x, es}, {g, es}, {gx, es}};
        const int vec = pick_vec(tune.vec, N, reqs, 3);
        with_dtype(dtype, [&](auto tag) {
            using IO = decltype(tag);
            launch_bwd_pick_t<IO>(tmax, vec, tune.block, x, g, gx, Ti, N, alpha, thresh, beta, interval, st);
        });
        return check_launch();
    }

    // long time axis: store u_t in the caller's scratch, then walk it in reverse
    if (!aligned(workspace, 256)) return SNN_ERR_ALIGN;
    rc = lif_fwd_impl(x, nullptr, workspace, nullptr, T, N, dtype, alpha, thresh, st);
    if (rc) return rc;
    const PtrReq reqs[] = {{workspace, ss}, {g, es}, {gx, es}};
    const int vec = pick_vec(es == 8 ? 2 : 4, N, reqs, 3);
    with_dtype(dtype, [&](auto tag) {
        using IO = decltype(tag);
        using CT = typename snn::Elem<IO>::CT;
        constexpr int kMaxVec = sizeof(IO) <= 4 ? 4 : 2;     // a chunk holds 8 steps of u and g
        with_vec<kMaxVec>(vec, [&](auto v) {
            constexpr int VEC = decltype(v)::value;
            snn::lif_bwd_mem_kernel<IO, VEC, 8><<<grid_for(N, VEC, kBlock), kBlock, 0, st>>>(
                static_cast<const CT*>(workspace), static_cast<const IO*>(g), static_cast<IO*>(gx), Ti,
                N, alpha, thresh, beta, interval);
        });
    });
    return check_launch();
}

// ---- unpack -------------------------------------------------------------------------------
template <typename IO, typename W>
void unpack_pick_vec(int vec, const void* bits, void* spike, int T, int64_t N, cudaStream_t st) {
    const W* b = static_cast<const W*>(bits);
    IO* s = static_cast<IO*>(spike);
    if constexpr (sizeof(IO) <= 4) {
        if (vec >= 4) {
            snn::spike_unpack_kernel<IO, 4, W><<<grid_for(N, 4, kBlock), kBlock, 0, st>>>(b, s, T, N);
            return;
        }
    }
    if (vec >= 2)
        snn::spike_unpack_kernel<IO, 2, W><<<grid_for(N, 2, kBlock), kBlock, 0, st>>>(b, s, T, N);
    else
        snn::spike_unpack_kernel<IO, 1, W><<<grid_for(N, 1, kBlock), kBlock, 0, st>>>(b, s, T, N);
}

template <typename IO>
void unpack_pick_word(int word_bytes, int vec, const void* bits, void* spike, int T, int64_t N,
                      cudaStream_t st) {
    if (word_bytes == 1) unpack_pick_vec<IO, unsigned char>(vec, bits, spike, T, N, st);
    else if (word_bytes == 2) unpack_pick_vec<IO, unsigned short>(vec, bits, spike, T, N, st);
    else unpack_pick_vec<IO, unsigned int>(vec, bits, spike, T, N, st);
}

}  // namespace

namespace snn_internal {
// lets other translation units of the library record the code snn_last_cuda_error() reports
void set_last_cuda_error(int e) { g_last_cuda_error = e; }
}  // namespace snn_internal

extern "C" {

int snn_version(void) { return 100; }

const char* snn_status_string(int status) {
    switch (status) {
        case SNN_OK: return "ok";
        case SNN_ERR_NULL: return "required pointer is NULL";
        case SNN_ERR_SHAPE: return "invalid T or N";
        case SNN_ERR_DTYPE: return "unknown dtype";
        case SNN_ERR_ALIGN: return "pointer not aligned to its element size";
        case SNN_ERR_UNSUPPORTED: return "request not supported";
        case SNN_ERR_WORKSPACE: return "workspace missing or too small";
        case SNN_ERR_CUDA: return "CUDA runtime error at launch";
        case SNN_ERR_TOO_LARGE: return "problem exceeds the built-in scratch array (SNN_STATIC_SCRATCH_BYTES)";
        default: return "unknown status";
    }
}

int snn_last_cuda_error(void) { return g_last_cuda_error; }

int snn_lif_fwd(const void* x, void* spike, void* mem, void* bits, int64_t T, int64_t N,
                int dtype, float alpha, float thresh, void* stream) {
    return lif_fwd_impl(x, spike, mem, bits, T, N, dtype, alpha, thresh,
                        static_cast<cudaStream_t>(stream));
}

int64_t snn_lif_bwd_workspace_bytes(int64_t T, int64_t N, int dtype) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return -static_cast<int64_t>(rc);
    if (T <= kRegT) return 0;
    return T * N * state_size(dtype);
}

int snn_lif_bwd(const void* x, const void* grad_spike, void* grad_x, int64_t T, int64_t N,
                int dtype, float alpha, float thresh, float beta, float interval,
                void* workspace, size_t workspace_bytes, void* stream) {
    return lif_bwd_impl(x, grad_spike, grad_x, T, N, dtype, alpha, thresh, beta, interval,
                        workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int snn_spike_unpack(const void* bits, void* spike, int64_t T, int64_t N, int dtype,
                     void* stream) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return rc;
    if (T > 32) return SNN_ERR_UNSUPPORTED;
    if (N == 0) return SNN_OK;
    if (!bits || !spike) return SNN_ERR_NULL;
    const int es = dtype_size(dtype);
    const int word_bytes = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    if (!aligned(spike, es) || !aligned(bits, word_bytes)) return SNN_ERR_ALIGN;
    if (N == 0) return SNN_OK;
    const PtrReq reqs[] = {{bits, word_bytes}, {spike, es}};
    const int vec = pick_vec(es == 8 ? 2 : 4, N, reqs, 2);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int Ti = static_cast<int>(T);
    switch (dtype) {
        case SNN_F32: unpack_pick_word<float>(word_bytes, vec, bits, spike, Ti, N, st); break;
        case SNN_BF16: unpack_pick_word<__nv_bfloat16>(word_bytes, vec, bits, spike, Ti, N, st); break;
        case SNN_F16: unpack_pick_word<__half>(word_bytes, vec, bits, spike, Ti, N, st); break;
        case SNN_F64: unpack_pick_word<double>(word_bytes, vec, bits, spike, Ti, N, st); break;
    }
    return check_launch();
}

int snn_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                        int64_t rows, int to_device, void* stream) {
    if (rows < 0) return SNN_ERR_SHAPE;
    if (rows == 0 || row_bytes == 0) return SNN_OK;
    if (!dst || !src) return SNN_ERR_NULL;
    if (dst_pitch < row_bytes || src_pitch < row_bytes) return SNN_ERR_SHAPE;
    cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, static_cast<size_t>(rows),
                                      to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                      static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

}  // extern "C"
