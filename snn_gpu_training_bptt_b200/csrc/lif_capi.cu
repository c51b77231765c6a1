// C ABI of libsnn_b200.so for the LIF fire path: argument validation, choice of vector
// width / time chunk, kernel launch. Declarations and the reference interfaces each entry
// point replaces: include/snn_b200.h.
#include "../../include/snn_b200.h"
#include "lif_kernels.cuh"

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

inline unsigned int grid_for(int64_t N, int vec) {
    const int64_t threads = (N + vec - 1) / vec;
    return static_cast<unsigned int>((threads + kBlock - 1) / kBlock);
}

inline int common_shape_check(int64_t T, int64_t N, int dtype) {
    if (dtype_size(dtype) == 0) return SNN_ERR_DTYPE;
    if (T < 1 || N < 0) return SNN_ERR_SHAPE;
    if (T > INT32_MAX) return SNN_ERR_SHAPE;
    // element offsets are int64; thread count must fit the 1-D grid
    if (N > 0 && T > INT64_MAX / 16 / N) return SNN_ERR_SHAPE;
    if ((N + kBlock - 1) / kBlock > 0x7fffffffLL) return SNN_ERR_SHAPE;
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

// ---- forward ------------------------------------------------------------------------------
template <typename IO, int VEC, int TC>
void launch_fwd(const void* x, void* spike, void* mem, void* bits, int word_bytes, int T,
                int64_t N, float alpha, float thresh, cudaStream_t st) {
    using CT = typename snn::Elem<IO>::CT;
    snn::lif_fwd_kernel<IO, VEC, TC><<<grid_for(N, VEC), kBlock, 0, st>>>(
        static_cast<const IO*>(x), static_cast<IO*>(spike), static_cast<CT*>(mem), bits,
        word_bytes, T, N, alpha, thresh);
}

template <typename IO, int VEC>
void fwd_pick_tc(const void* x, void* spike, void* mem, void* bits, int word_bytes, int T,
                 int64_t N, float alpha, float thresh, cudaStream_t st) {
    if (T <= 4) launch_fwd<IO, VEC, 4>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
    else launch_fwd<IO, VEC, 8>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
}

template <typename IO>
void fwd_pick_vec(int vec, const void* x, void* spike, void* mem, void* bits, int word_bytes,
                  int T, int64_t N, float alpha, float thresh, cudaStream_t st) {
    constexpr int kMax = 16 / static_cast<int>(sizeof(IO));
    if constexpr (kMax >= 8) {
        if (vec == 8) return fwd_pick_tc<IO, 8>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
    }
    if constexpr (kMax >= 4) {
        if (vec == 4) return fwd_pick_tc<IO, 4>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
    }
    if (vec == 2) return fwd_pick_tc<IO, 2>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
    return fwd_pick_tc<IO, 1>(x, spike, mem, bits, word_bytes, T, N, alpha, thresh, st);
}

int lif_fwd_impl(const void* x, void* spike, void* mem, void* bits, int64_t T, int64_t N,
                 int dtype, float alpha, float thresh, cudaStream_t st) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return rc;
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
    if (N == 0) return SNN_OK;

    const PtrReq reqs[] = {{x, es}, {spike, es}, {mem, ss}, {bits, word_bytes ? word_bytes : 1}};
    const int vec = pick_vec(16 / es, N, reqs, 4);
    const int Ti = static_cast<int>(T);
    switch (dtype) {
        case SNN_F32: fwd_pick_vec<float>(vec, x, spike, mem, bits, word_bytes, Ti, N, alpha, thresh, st); break;
        case SNN_BF16: fwd_pick_vec<__nv_bfloat16>(vec, x, spike, mem, bits, word_bytes, Ti, N, alpha, thresh, st); break;
        case SNN_F16: fwd_pick_vec<__half>(vec, x, spike, mem, bits, word_bytes, Ti, N, alpha, thresh, st); break;
        case SNN_F64: fwd_pick_vec<double>(vec, x, spike, mem, bits, word_bytes, Ti, N, alpha, thresh, st); break;
    }
    return check_launch();
}

// ---- backward -----------------------------------------------------------------------------
template <typename IO, int VEC, int TMAX>
void launch_bwd(const void* x, const void* g, void* gx, int T, int64_t N, float alpha,
                float thresh, float beta, float interval, cudaStream_t st) {
    snn::lif_bwd_kernel<IO, VEC, TMAX><<<grid_for(N, VEC), kBlock, 0, st>>>(
        static_cast<const IO*>(x), static_cast<const IO*>(g), static_cast<IO*>(gx), T, N, alpha,
        thresh, beta, interval);
}

// VEC * TMAX is held near 32 state words so x, g and u of all T steps fit in registers.
template <typename IO, int TMAX>
void bwd_pick_vec(int vec, const void* x, const void* g, void* gx, int T, int64_t N, float alpha,
                  float thresh, float beta, float interval, cudaStream_t st) {
    constexpr int kIoMax = 16 / static_cast<int>(sizeof(IO));
    constexpr int kRegMax = (32 / TMAX) < 1 ? 1 : (32 / TMAX);
    constexpr int kMax = kIoMax < kRegMax ? kIoMax : kRegMax;
    if constexpr (kMax >= 8) {
        if (vec >= 8) return launch_bwd<IO, 8, TMAX>(x, g, gx, T, N, alpha, thresh, beta, interval, st);
    }
    if constexpr (kMax >= 4) {
        if (vec >= 4) return launch_bwd<IO, 4, TMAX>(x, g, gx, T, N, alpha, thresh, beta, interval, st);
    }
    if constexpr (kMax >= 2) {
        if (vec >= 2) return launch_bwd<IO, 2, TMAX>(x, g, gx, T, N, alpha, thresh, beta, interval, st);
    }
    return launch_bwd<IO, 1, TMAX>(x, g, gx, T, N, alpha, thresh, beta, interval, st);
}

template <typename IO>
void bwd_pick_t(int vec, const void* x, const void* g, void* gx, int T, int64_t N, float alpha,
                float thresh, float beta, float interval, cudaStream_t st) {
    if (T <= 4) bwd_pick_vec<IO, 4>(vec, x, g, gx, T, N, alpha, thresh, beta, interval, st);
    else if (T <= 8) bwd_pick_vec<IO, 8>(vec, x, g, gx, T, N, alpha, thresh, beta, interval, st);
    else if (T <= 16) bwd_pick_vec<IO, 16>(vec, x, g, gx, T, N, alpha, thresh, beta, interval, st);
    else bwd_pick_vec<IO, 32>(vec, x, g, gx, T, N, alpha, thresh, beta, interval, st);
}

template <typename IO, int VEC>
void launch_bwd_mem(const void* mem, const void* g, void* gx, int T, int64_t N, float alpha,
                    float thresh, float beta, float interval, cudaStream_t st) {
    using CT = typename snn::Elem<IO>::CT;
    snn::lif_bwd_mem_kernel<IO, VEC, 8><<<grid_for(N, VEC), kBlock, 0, st>>>(
        static_cast<const CT*>(mem), static_cast<const IO*>(g), static_cast<IO*>(gx), T, N, alpha,
        thresh, beta, interval);
}

template <typename IO>
void bwd_mem_pick_vec(int vec, const void* mem, const void* g, void* gx, int T, int64_t N,
                      float alpha, float thresh, float beta, float interval, cudaStream_t st) {
    // 4 neurons per thread at most: a chunk holds 8 steps of u and g
    if constexpr (sizeof(IO) <= 4) {
        if (vec >= 4) return launch_bwd_mem<IO, 4>(mem, g, gx, T, N, alpha, thresh, beta, interval, st);
    }
    if (vec >= 2) return launch_bwd_mem<IO, 2>(mem, g, gx, T, N, alpha, thresh, beta, interval, st);
    return launch_bwd_mem<IO, 1>(mem, g, gx, T, N, alpha, thresh, beta, interval, st);
}

int lif_bwd_impl(const void* x, const void* g, void* gx, int64_t T, int64_t N, int dtype,
                 float alpha, float thresh, float beta, float interval, void* workspace,
                 size_t workspace_bytes, cudaStream_t st) {
    int rc = common_shape_check(T, N, dtype);
    if (rc) return rc;
    if (!x || !g || !gx) return SNN_ERR_NULL;
    const int es = dtype_size(dtype), ss = state_size(dtype);
    if (!aligned(x, es) || !aligned(g, es) || !aligned(gx, es)) return SNN_ERR_ALIGN;
    const int Ti = static_cast<int>(T);

    if (T <= kRegT) {
        if (N == 0) return SNN_OK;
        const PtrReq reqs[] = {{x, es}, {g, es}, {gx, es}};
        const int vec = pick_vec(16 / es, N, reqs, 3);
        switch (dtype) {
            case SNN_F32: bwd_pick_t<float>(vec, x, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
            case SNN_BF16: bwd_pick_t<__nv_bfloat16>(vec, x, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
            case SNN_F16: bwd_pick_t<__half>(vec, x, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
            case SNN_F64: bwd_pick_t<double>(vec, x, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
        }
        return check_launch();
    }

    // long time axis: store u_t in the caller's scratch, then walk it in reverse
    const size_t need = static_cast<size_t>(T) * static_cast<size_t>(N) * ss;
    if (need > 0 && (!workspace || workspace_bytes < need)) return SNN_ERR_WORKSPACE;
    if (workspace && !aligned(workspace, 256)) return SNN_ERR_ALIGN;
    if (N == 0) return SNN_OK;
    rc = lif_fwd_impl(x, nullptr, workspace, nullptr, T, N, dtype, alpha, thresh, st);
    if (rc) return rc;
    const PtrReq reqs[] = {{workspace, ss}, {g, es}, {gx, es}};
    const int vec = pick_vec(16 / es, N, reqs, 3);
    switch (dtype) {
        case SNN_F32: bwd_mem_pick_vec<float>(vec, workspace, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
        case SNN_BF16: bwd_mem_pick_vec<__nv_bfloat16>(vec, workspace, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
        case SNN_F16: bwd_mem_pick_vec<__half>(vec, workspace, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
        case SNN_F64: bwd_mem_pick_vec<double>(vec, workspace, g, gx, Ti, N, alpha, thresh, beta, interval, st); break;
    }
    return check_launch();
}

// ---- unpack -------------------------------------------------------------------------------
template <typename IO, typename W>
void unpack_pick_vec(int vec, const void* bits, void* spike, int T, int64_t N, cudaStream_t st) {
    const W* b = static_cast<const W*>(bits);
    IO* s = static_cast<IO*>(spike);
    if constexpr (sizeof(IO) <= 4) {
        if (vec >= 4) {
            snn::spike_unpack_kernel<IO, 4, W><<<grid_for(N, 4), kBlock, 0, st>>>(b, s, T, N);
            return;
        }
    }
    if (vec >= 2)
        snn::spike_unpack_kernel<IO, 2, W><<<grid_for(N, 2), kBlock, 0, st>>>(b, s, T, N);
    else
        snn::spike_unpack_kernel<IO, 1, W><<<grid_for(N, 1), kBlock, 0, st>>>(b, s, T, N);
}

template <typename IO>
void unpack_pick_word(int word_bytes, int vec, const void* bits, void* spike, int T, int64_t N,
                      cudaStream_t st) {
    if (word_bytes == 1) unpack_pick_vec<IO, unsigned char>(vec, bits, spike, T, N, st);
    else if (word_bytes == 2) unpack_pick_vec<IO, unsigned short>(vec, bits, spike, T, N, st);
    else unpack_pick_vec<IO, unsigned int>(vec, bits, spike, T, N, st);
}

}  // namespace

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
    if (!bits || !spike) return SNN_ERR_NULL;
    if (T > 32) return SNN_ERR_UNSUPPORTED;
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

}  // extern "C"
