// snn_lif_bwd_noalloc: the stored-membrane LIF backward with its scratch compiled into the
// library, for callers that cannot allocate device memory where the backward runs (a host whose
// own allocator owns the whole GPU, a latency-critical loop that cannot take cudaMalloc's device
// synchronisation, a plugin sandbox that only passes buffers). Declaration, limits and calling
// rules: include/snn_b200.h.
//
// The membrane tensor u[T, N] lives in g_membrane_scratch below: a file-scope device array of
// SNN_STATIC_SCRATCH_BYTES that every GPU holds from the moment this module is loaded until the
// process exits. In HOST code the identifier g_membrane_scratch is only a handle for the runtime,
// not a device address, so it is never passed to a kernel directly: the device address is
// obtained once per device with cudaGetSymbolAddress (with that device current) and cached.
// Nothing in this file calls cudaMalloc, cudaFree or any other allocating routine.
//
// The array is shared by every call on a GPU and keeps the previous call's contents. The forward
// pass launched here writes all T*N membrane values before the reverse pass reads them, so
// nothing has to start at zero; calls that may overlap on the GPU must be ordered by the caller.
#include "../../include/snn_b200.h"
#include "lif_kernels.cuh"

#include <atomic>
#include <mutex>

static __device__ __align__(256) unsigned char g_membrane_scratch[SNN_STATIC_SCRATCH_BYTES];

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int kBlock = 256;
constexpr int kMaxDevices = 64;

std::mutex g_setup_mutex;
std::atomic<void*> g_scratch_address[kMaxDevices] = {};

// Device address of g_membrane_scratch on the CURRENT device (looked up on the first call for
// that device, then cached; later calls read the cached pointer without taking the mutex).
// Returns nullptr and records the CUDA error on failure. A cudaDeviceReset() invalidates the
// cached address: a process that resets a device must not call this entry point on it again.
void* scratch_on_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && (dev < 0 || dev >= kMaxDevices)) e = cudaErrorInvalidDevice;
    if (e != cudaSuccess) {
        snn_internal::set_last_cuda_error(static_cast<int>(e));
        return nullptr;
    }
    void* ptr = g_scratch_address[dev].load(std::memory_order_acquire);
    if (ptr != nullptr) return ptr;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    ptr = g_scratch_address[dev].load(std::memory_order_relaxed);
    if (ptr == nullptr) {
        e = cudaGetSymbolAddress(&ptr, g_membrane_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            snn_internal::set_last_cuda_error(static_cast<int>(e));
            return nullptr;
        }
        g_scratch_address[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline unsigned grid_for(int64_t N, int vec) {
    const int64_t threads = (N + vec - 1) / vec;
    return static_cast<unsigned>((threads + kBlock - 1) / kBlock);
}

// u[T, N] into scratch, then the reverse walk; VEC neurons per thread.
template <typename IO, int VEC>
void launch_pair(const void* x, const void* g, void* gx, void* scratch, int T, int64_t N,
                 float alpha, float thresh, float beta, float interval, cudaStream_t st) {
    using CT = typename snn::Elem<IO>::CT;
    CT* mem = static_cast<CT*>(scratch);
    snn::lif_fwd_kernel<IO, VEC, 8><<<grid_for(N, VEC), kBlock, 0, st>>>(
        static_cast<const IO*>(x), nullptr, mem, nullptr, 0, T, N, alpha, thresh);
    snn::lif_bwd_mem_kernel<IO, VEC, 8><<<grid_for(N, VEC), kBlock, 0, st>>>(
        mem, static_cast<const IO*>(g), static_cast<IO*>(gx), T, N, alpha, thresh, beta, interval);
}

template <typename IO>
void launch_for_type(bool wide, const void* x, const void* g, void* gx, void* scratch, int T,
                     int64_t N, float alpha, float thresh, float beta, float interval,
                     cudaStream_t st) {
    if (wide) launch_pair<IO, 2>(x, g, gx, scratch, T, N, alpha, thresh, beta, interval, st);
    else launch_pair<IO, 1>(x, g, gx, scratch, T, N, alpha, thresh, beta, interval, st);
}

}  // namespace

extern "C" int snn_lif_bwd_noalloc(const void* x, const void* grad_spike, void* grad_x, int64_t T,
                                   int64_t N, int dtype, float alpha, float thresh, float beta,
                                   float interval, void* stream) {
    int es;
    switch (dtype) {
        case SNN_F32: es = 4; break;
        case SNN_BF16: case SNN_F16: es = 2; break;
        case SNN_F64: es = 8; break;
        default: return SNN_ERR_DTYPE;
    }
    const int ss = dtype == SNN_F64 ? 8 : 4;
    if (T < 1 || N < 0 || T > INT32_MAX) return SNN_ERR_SHAPE;
    if (N == 0) return SNN_OK;
    // size check first, in a form that cannot overflow: T*N*ss <= SNN_STATIC_SCRATCH_BYTES
    const int64_t max_steps = static_cast<int64_t>(SNN_STATIC_SCRATCH_BYTES) / ss;
    if (N > max_steps || T > max_steps / N) return SNN_ERR_TOO_LARGE;
    if (!x || !grad_spike || !grad_x) return SNN_ERR_NULL;
    if (!aligned(x, es) || !aligned(grad_spike, es) || !aligned(grad_x, es)) return SNN_ERR_ALIGN;

    void* scratch = scratch_on_current_device();
    if (scratch == nullptr) return SNN_ERR_CUDA;

    // two neurons per thread when every row start and pointer allows it, else one
    const bool wide = (N % 2 == 0) && aligned(x, 2 * es) && aligned(grad_spike, 2 * es) &&
                      aligned(grad_x, 2 * es);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int Ti = static_cast<int>(T);
    switch (dtype) {
        case SNN_F32: launch_for_type<float>(wide, x, grad_spike, grad_x, scratch, Ti, N, alpha, thresh, beta, interval, st); break;
        case SNN_BF16: launch_for_type<__nv_bfloat16>(wide, x, grad_spike, grad_x, scratch, Ti, N, alpha, thresh, beta, interval, st); break;
        case SNN_F16: launch_for_type<__half>(wide, x, grad_spike, grad_x, scratch, Ti, N, alpha, thresh, beta, interval, st); break;
        default: launch_for_type<double>(wide, x, grad_spike, grad_x, scratch, Ti, N, alpha, thresh, beta, interval, st); break;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snn_internal::set_last_cuda_error(static_cast<int>(e));
        return SNN_ERR_CUDA;
    }
    return SNN_OK;
}
