// Alternative LIF fwd/bwd kernel that stages its tiles through shared memory with
// cp.async.bulk (TMA 1-D bulk copies): persistent CTAs, a multi-stage input ring filled by one
// elected thread (mbarrier expect_tx / complete_tx), compute from shared memory, double-buffered
// bulk stores. Every wait is bounded: a barrier that does not flip within ~1 s sets *err and
// the CTA leaves its loop.
//
// NOT part of libsnn_b200.so. It is built only into the tuner (lif_tune.cu), where it measured
// 4-8 % slower on B200 than the register-resident vector-load kernels of lif_kernels.cuh
// (T=8, N=2^26: forward 6.34 vs 6.84 TB/s, backward 6.57 vs 7.00 TB/s), because those already
// keep >150 KB of loads in flight per SM without a shared-memory hop. Kept so the comparison
// can be re-run. Same arithmetic as lif_kernels.cuh (fp32, separately rounded operations).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace snn_tma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait: returns false if the barrier did not flip within the limit
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > 2000000000LL) return false;   // ~1 s at 2 GHz
    return true;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// TILE neurons per tile = 4 * THREADS. Requires N % 4 == 0 and 16-byte aligned bases.
// BWD=false: in = x, out = spike.   BWD=true: in = x and g, out = grad_x.
template <int T, int THREADS, int STAGES, bool BWD>
__global__ void __launch_bounds__(THREADS) lif_tma_kernel(const float* __restrict__ x,
                                                         const float* __restrict__ g,
                                                         float* __restrict__ out, int64_t N,
                                                         float alpha, float thresh, float beta,
                                                         float interval, int* __restrict__ err)
{
    constexpr int TILE = 4 * THREADS;
    constexpr int NIN = BWD ? 2 : 1;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float* s_in = reinterpret_cast<float*>(smem_raw);                       // [STAGES][NIN][T][TILE]
    float* s_out = s_in + static_cast<size_t>(STAGES) * NIN * T * TILE;    // [2][T][TILE]
    uint64_t* full = reinterpret_cast<uint64_t*>(s_out + 2 * T * TILE);   // [STAGES]

    const int64_t ntiles = (N + TILE - 1) / TILE;
    const int tid = threadIdx.x;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto issue = [&](int64_t tile, int stage) {
        const int64_t n0 = tile * TILE;
        const int64_t rem = N - n0;
        const uint32_t cols = rem >= TILE ? TILE : static_cast<uint32_t>(rem);
        const uint32_t bytes = cols * 4u;                    // multiple of 16 since N % 4 == 0
        mbar_expect_tx(&full[stage], bytes * T * NIN);
        float* base = s_in + static_cast<size_t>(stage) * NIN * T * TILE;
#pragma unroll
        for (int t = 0; t < T; ++t) {
            bulk_load(base + t * TILE, x + t * N + n0, bytes, &full[stage]);
            if (BWD) bulk_load(base + (T + t) * TILE, g + t * N + n0, bytes, &full[stage]);
        }
    };

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            const int64_t tile = blockIdx.x + static_cast<int64_t>(s) * gridDim.x;
            if (tile < ntiles) issue(tile, s);
        }
    }

    int it = 0;
    bool failed = false;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
        const int stage = it % STAGES;
        const uint32_t parity = (it / STAGES) & 1;
        if (!mbar_wait_bounded(&full[stage], parity)) { failed = true; }
        if (__syncthreads_or(failed)) { if (tid == 0) atomicExch(err, 1); break; }

        const int64_t n0 = tile * TILE;
        const int64_t rem = N - n0;
        const int cols = rem >= TILE ? TILE : static_cast<int>(rem);
        const float* base = s_in + static_cast<size_t>(stage) * NIN * T * TILE;
        float* obuf = s_out + static_cast<size_t>(it & 1) * T * TILE;
        const int c = tid * 4;
        if (c < cols) {
            float u[T][4];
            float uu[4] = {0, 0, 0, 0}, gate[4] = {1, 1, 1, 1};
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float4 xv = *reinterpret_cast<const float4*>(base + t * TILE + c);
                const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
                float sp[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    float leak = __fmul_rn(__fmul_rn(alpha, uu[v]), gate[v]);
                    uu[v] = __fadd_rn(leak, xa[v]);
                    const bool s = uu[v] > thresh;
                    gate[v] = s ? 0.f : 1.f;
                    sp[v] = s ? 1.f : 0.f;
                    u[t][v] = uu[v];
                }
                if (!BWD) *reinterpret_cast<float4*>(obuf + t * TILE + c) = make_float4(sp[0], sp[1], sp[2], sp[3]);
            }
            if (BWD) {
                float gu[4] = {0, 0, 0, 0};
#pragma unroll
                for (int t = T - 1; t >= 0; --t) {
                    const float4 gv = *reinterpret_cast<const float4*>(base + (T + t) * TILE + c);
                    const float ga4[4] = {gv.x, gv.y, gv.z, gv.w};
                    float o[4];
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const float ut = u[t][v];
                        const float ga = __fmul_rn(gu[v], alpha);
                        const bool inside = (__fsub_rn(ut, thresh) < interval) && (__fsub_rn(thresh, ut) < interval);
                        float gs = 0.f;
                        if (inside) gs = __fsub_rn(ga4[v], __fmul_rn(ga, ut));
                        const float keep = (ut <= thresh) ? 1.f : 0.f;
                        gu[v] = __fadd_rn(__fmul_rn(gs, beta), __fmul_rn(ga, keep));
                        o[v] = gu[v];
                    }
                    *reinterpret_cast<float4*>(obuf + t * TILE + c) = make_float4(o[0], o[1], o[2], o[3]);
                }
            }
        }
        fence_async_smem();           // make this thread's smem writes visible to the async proxy
        if (tid == 0) bulk_wait_read<0>();   // store issued one iteration ago has finished reading its buffer
        __syncthreads();
        if (tid == 0) {
            const uint32_t bytes = static_cast<uint32_t>(cols) * 4u;
#pragma unroll
            for (int t = 0; t < T; ++t) bulk_store(out + t * N + n0, obuf + t * TILE, bytes);
            bulk_commit();
            const int64_t next = tile + static_cast<int64_t>(STAGES) * gridDim.x;
            if (next < ntiles) issue(next, stage);
        }
    }
    if (tid == 0) bulk_wait_all<0>();
}

template <int T, int THREADS, int STAGES, bool BWD>
constexpr size_t lif_tma_smem() {
    return (static_cast<size_t>(STAGES) * (BWD ? 2 : 1) + 2) * T * 4 * THREADS * sizeof(float) + STAGES * 8;
}

}  // namespace snn_tma
