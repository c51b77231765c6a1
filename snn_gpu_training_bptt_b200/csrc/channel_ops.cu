// Per-channel bias add and per-channel gradient sum for the synaptic layers either side of the
// LIF kernels (declarations: include/snn_b200.h).
//
// The reference adds the convolution / linear bias inside its cuDNN / cuBLAS calls and forms
// the bias gradient with at::sum(grad, dims) (snnlib/cuda/snn_kernel_bp.cu:1127, :1401).
// With one library call over the merged T*B batch, the bias add and the bias-gradient
// reduction that torch would run as generic elementwise / reduce kernels on 16-bit
// channels-last tensors were 29 % of a training step of the VGG-style network; these two
// HBM-bound kernels replace them.
//
// Layout: element (o, c, i) at (o*C + c)*inner + i, i.e. channel = (n / inner) % C for flat
// index n: inner = 1 for channels-last images and [rows, C] matrices, inner = H*W for
// contiguous [N, C, H, W].
#include "../../include/snn_b200.h"
#include "lif_kernels.cuh"

#include <type_traits>

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int kBlock = 256;
constexpr int kIter = 8;      // vectors per thread in the sum kernel

// channel of flat index n; 32-bit arithmetic whenever the operands fit (64-bit division is
// emulated with ~100 instructions)
__device__ __forceinline__ int channel_index(long long n, long long inner, int C) {
    if (n <= 0xffffffffLL && inner <= 0xffffffffLL)
        return static_cast<int>((static_cast<unsigned int>(n) / static_cast<unsigned int>(inner)) % static_cast<unsigned int>(C));
    return static_cast<int>((n / inner) % C);
}

template <typename IO, int VEC>
__global__ void channel_bias_add_kernel(IO* __restrict__ y, const float* __restrict__ bias,
                                        long long total, long long inner, int C)
{
    const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
    if (i >= total) return;
    snn::Pack<IO, VEC> v = snn::ld_stream<IO, VEC>(y + i);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        const int c = channel_index(i + k, inner, C);
        v.v[k] = snn::Elem<IO>::store(snn::add_rn(snn::Elem<IO>::load(v.v[k]), bias[c]));
    }
    snn::st_stream<IO, VEC>(y + i, v);
}

// Fixed-pattern variants for inner == 1 (channels-last images, [rows, C] matrices) with C dividing
// kBlock * VEC: channel = n % C, so a thread that strides through the tensor in whole spans of
// kBlock * VEC elements meets the same VEC consecutive channels every time. The bias values (or the
// partial sums) of those channels stay in registers for the thread's whole walk; there is no
// division per element and, for the sum, one shared-memory reduction and C global atomics per CTA
// for the whole walk. The general kernels computed a division and a modulo per ELEMENT and were
// issue-bound at 2.1 TB/s (bias add) and 2.4 TB/s (sum) on the trainer's bf16 tensors, together
// 19 % of a training step. kUnroll vectors per thread are in flight at a time.
constexpr int kUnroll = 4;

template <typename IO, int VEC>
__global__ void __launch_bounds__(kBlock)
channel_bias_add_fixed_kernel(IO* __restrict__ y, const float* __restrict__ bias, long long total, int C)
{
    const int c0 = static_cast<int>((static_cast<long long>(threadIdx.x) * VEC) % C);
    float b[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) b[k] = bias[c0 + k];         // C % VEC == 0: no wrap inside a vector
    const long long span = static_cast<long long>(kBlock) * VEC;
    const long long stride = static_cast<long long>(gridDim.x) * span;
    long long i = static_cast<long long>(blockIdx.x) * span + static_cast<long long>(threadIdx.x) * VEC;
    for (; i + (kUnroll - 1) * stride < total; i += kUnroll * stride) {
        snn::Pack<IO, VEC> v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = snn::ld_stream<IO, VEC>(y + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int k = 0; k < VEC; ++k)
                v[u].v[k] = snn::Elem<IO>::store(snn::add_rn(snn::Elem<IO>::load(v[u].v[k]), b[k]));
            snn::st_stream<IO, VEC>(y + i + u * stride, v[u]);
        }
    }
    for (; i < total; i += stride) {
        snn::Pack<IO, VEC> v = snn::ld_stream<IO, VEC>(y + i);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v.v[k] = snn::Elem<IO>::store(snn::add_rn(snn::Elem<IO>::load(v.v[k]), b[k]));
        snn::st_stream<IO, VEC>(y + i, v);
    }
}

template <typename IO, int VEC>
__global__ void __launch_bounds__(kBlock)
channel_sum_fixed_kernel(const IO* __restrict__ g, float* __restrict__ out, long long total, int C)
{
    extern __shared__ float sacc[];
    for (int j = threadIdx.x; j < C; j += blockDim.x) sacc[j] = 0.f;
    __syncthreads();
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
    const long long span = static_cast<long long>(kBlock) * VEC;
    const long long stride = static_cast<long long>(gridDim.x) * span;
    long long i = static_cast<long long>(blockIdx.x) * span + static_cast<long long>(threadIdx.x) * VEC;
    for (; i + (kUnroll - 1) * stride < total; i += kUnroll * stride) {
        snn::Pack<IO, VEC> v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = snn::ld_stream<IO, VEC>(g + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int k = 0; k < VEC; ++k) acc[k] += snn::Elem<IO>::load(v[u].v[k]);
    }
    for (; i < total; i += stride) {
        const snn::Pack<IO, VEC> v = snn::ld_stream<IO, VEC>(g + i);
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] += snn::Elem<IO>::load(v.v[k]);
    }
    const int c0 = static_cast<int>((static_cast<long long>(threadIdx.x) * VEC) % C);
#pragma unroll
    for (int k = 0; k < VEC; ++k) atomicAdd(&sacc[c0 + k], acc[k]);
    __syncthreads();
    for (int j = threadIdx.x; j < C; j += blockDim.x) atomicAdd(&out[j], sacc[j]);
}

// out[c] += sum over all elements of channel c. Each CTA owns a contiguous span of
// kBlock*VEC*kIter elements and accumulates per channel in shared memory (one slot per channel;
// SMEM=false for very wide layers: straight to global atomics), then issues one global atomicAdd
// per channel it touched. When the channel pattern of a thread repeats from one of its vectors to
// the next (channels-last with C dividing kBlock*VEC) the thread first sums its kIter vectors
// in registers.
template <typename IO, int VEC, bool SMEM>
__global__ void channel_sum_kernel(const IO* __restrict__ g, float* __restrict__ out,
                                   long long total, long long inner, int C, int same_pattern)
{
    extern __shared__ float sacc[];
    float* acc_to = SMEM ? sacc : out;
    if (SMEM) {
        for (int j = threadIdx.x; j < C; j += blockDim.x) sacc[j] = 0.f;
        __syncthreads();
    }
    const long long span = static_cast<long long>(kBlock) * VEC * kIter;
    const long long blk0 = static_cast<long long>(blockIdx.x) * span;
    if (same_pattern) {
        float acc[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
#pragma unroll
        for (int it = 0; it < kIter; ++it) {
            const long long i = blk0 + (static_cast<long long>(it) * kBlock + threadIdx.x) * VEC;
            if (i < total) {
                const snn::Pack<IO, VEC> v = snn::ld_stream<IO, VEC>(g + i);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[k] += snn::Elem<IO>::load(v.v[k]);
            }
        }
        const long long i0 = blk0 + static_cast<long long>(threadIdx.x) * VEC;
#pragma unroll
        for (int k = 0; k < VEC; ++k) atomicAdd(&acc_to[channel_index(i0 + k, 1, C)], acc[k]);
    } else {
#pragma unroll
        for (int it = 0; it < kIter; ++it) {
            const long long i = blk0 + (static_cast<long long>(it) * kBlock + threadIdx.x) * VEC;
            if (i < total) {
                const snn::Pack<IO, VEC> v = snn::ld_stream<IO, VEC>(g + i);
                // consecutive elements usually share a channel: merge before the atomic
                int c_prev = channel_index(i, inner, C);
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const int c = channel_index(i + k, inner, C);
                    if (c != c_prev) {
                        atomicAdd(&acc_to[c_prev], acc);
                        acc = 0.f;
                        c_prev = c;
                    }
                    acc += snn::Elem<IO>::load(v.v[k]);
                }
                atomicAdd(&acc_to[c_prev], acc);
            }
        }
    }
    if (SMEM) {
        __syncthreads();
        for (int j = threadIdx.x; j < C; j += blockDim.x) {
            const float a = sacc[j];
            if (a != 0.f) atomicAdd(&out[j], a);
        }
    }
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int elem_size(int dtype) {
    switch (dtype) {
        case SNN_F32: return 4;
        case SNN_BF16: case SNN_F16: return 2;
        default: return 0;
    }
}

template <typename F>
inline void dispatch(int dtype, int vec, F&& f) {
    auto with_v = [&](auto io) {
        if (vec >= 8 && sizeof(io) == 2) f(io, std::integral_constant<int, 8>{});
        else if (vec >= 4) f(io, std::integral_constant<int, 4>{});
        else if (vec >= 2) f(io, std::integral_constant<int, 2>{});
        else f(io, std::integral_constant<int, 1>{});
    };
    if (dtype == SNN_F32) with_v(float{});
    else if (dtype == SNN_BF16) with_v(__nv_bfloat16{});
    else with_v(__half{});
}

inline int pick_vec(long long total, int es, const void* p) {
    for (int vec = 16 / es; vec > 1; vec >>= 1)
        if (total % vec == 0 && aligned(p, static_cast<size_t>(es) * vec)) return vec;
    return 1;
}

inline int geometry_ok(int64_t outer, int64_t C, int64_t inner, int dtype) {
    if (dtype == SNN_F64) return SNN_ERR_UNSUPPORTED;
    if (elem_size(dtype) == 0) return SNN_ERR_DTYPE;
    if (outer < 0 || C < 1 || inner < 1 || C > INT32_MAX) return SNN_ERR_SHAPE;
    const long double total = static_cast<long double>(outer) * C * inner;
    if (total > 4.0e18L) return SNN_ERR_SHAPE;
    return SNN_OK;
}

// channels repeat with the CTA span and never wrap inside a vector
inline bool fixed_pattern(int64_t inner, int64_t C, int vec, long long total) {
    return inner == 1 && C % vec == 0 && (static_cast<long long>(kBlock) * vec) % C == 0 && total % vec == 0;
}
// a few CTAs per SM, each walking the tensor in strides of the whole grid
inline unsigned fat_grid(long long total, int vec) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long span = static_cast<long long>(kBlock) * vec;
    const long long spans = (total + span - 1) / span;
    const long long want = static_cast<long long>(sms) * 8;
    return static_cast<unsigned>(spans < want ? spans : want);
}

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

}  // namespace

extern "C" {

int snn_channel_bias_add(void* y, const float* bias, int64_t outer, int64_t C, int64_t inner, int dtype,
                         void* stream) {
    int rc = geometry_ok(outer, C, inner, dtype);
    if (rc) return rc;
    const long long total = outer * C * inner;
    if (total == 0) return SNN_OK;
    if (!y || !bias) return SNN_ERR_NULL;
    const int es = elem_size(dtype);
    if (!aligned(y, es)) return SNN_ERR_ALIGN;
    const int vec = pick_vec(total, es, y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dispatch(dtype, vec, [&](auto io, auto v) {
        using IO = decltype(io);
        constexpr int VEC = decltype(v)::value;
        if (fixed_pattern(inner, C, VEC, total)) {
            channel_bias_add_fixed_kernel<IO, VEC><<<fat_grid(total, VEC), kBlock, 0, st>>>(
                static_cast<IO*>(y), bias, total, static_cast<int>(C));
            return;
        }
        const long long threads = (total + VEC - 1) / VEC;
        channel_bias_add_kernel<IO, VEC><<<static_cast<unsigned>((threads + kBlock - 1) / kBlock), kBlock, 0, st>>>(
            static_cast<IO*>(y), bias, total, inner, static_cast<int>(C));
    });
    return launch_status();
}

int snn_channel_sum(const void* grad, float* out, int64_t outer, int64_t C, int64_t inner, int dtype,
                    void* stream) {
    int rc = geometry_ok(outer, C, inner, dtype);
    if (rc) return rc;
    if (!out) return SNN_ERR_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(out, 0, sizeof(float) * C, st);
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    const long long total = outer * C * inner;
    if (total == 0) return SNN_OK;
    if (!grad) return SNN_ERR_NULL;
    const int es = elem_size(dtype);
    if (!aligned(grad, es)) return SNN_ERR_ALIGN;
    const int vec = pick_vec(total, es, grad);
    dispatch(dtype, vec, [&](auto io, auto v) {
        using IO = decltype(io);
        constexpr int VEC = decltype(v)::value;
        if (fixed_pattern(inner, C, VEC, total) && C <= 8192) {
            channel_sum_fixed_kernel<IO, VEC><<<fat_grid(total, VEC), kBlock, sizeof(float) * C, st>>>(
                static_cast<const IO*>(grad), out, total, static_cast<int>(C));
            return;
        }
        const long long span = static_cast<long long>(kBlock) * VEC * kIter;
        const long long blocks = (total + span - 1) / span;
        const int same = (inner == 1 && (static_cast<long long>(kBlock) * VEC) % C == 0) ? 1 : 0;
        if (C <= 8192)
            channel_sum_kernel<IO, VEC, true><<<static_cast<unsigned>(blocks), kBlock, sizeof(float) * C, st>>>(
                static_cast<const IO*>(grad), out, total, inner, static_cast<int>(C), same);
        else
            channel_sum_kernel<IO, VEC, false><<<static_cast<unsigned>(blocks), kBlock, 0, st>>>(
                static_cast<const IO*>(grad), out, total, inner, static_cast<int>(C), same);
    });
    return launch_status();
}

}  // extern "C"
