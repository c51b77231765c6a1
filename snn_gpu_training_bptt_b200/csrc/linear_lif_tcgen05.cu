// Fused synaptic linear + LIF forward on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   current[t, b, :] = x[t, b, :] @ W^T + bias          (bf16 operands, fp32 accumulation in TMEM)
//   spike[t, b, :]   = LIF over t of current[:, b, :]   (fp32 state, same arithmetic as lif_kernels.cuh)
//
// In the reference this is `Fc` followed by `Fire`: T separate cuBLAS calls with a copy each
// (fc_fp_cuda, snnlib/cuda/snn_kernel_fp.cu:332-357) and then fire_s_fp_kernel (:15-53) re-reading
// the currents from HBM. Here one kernel computes a 128 (output neurons) x 128 (T time steps x
// 128/T batch items) tile of currents in tensor memory and runs the recurrence on it in the
// epilogue, so spikes come straight out of the GEMM.
//
// GEMM orientation: D[m, n] = sum_k W[m, k] * X[n, k], M = output neurons, N = (t, b) pairs.
// The X tile is fetched by one 3-D TMA box {64 k, 128/T batch items, T steps} of the [T][B][K]
// tensor, which lands in shared memory as rows ordered (t major, b minor): accumulator column
// n = t*(128/T) + j. A TMEM lane is one output neuron, so the epilogue thread that owns the lane
// reads, for t = 0..T-1, the 128/T consecutive columns of that time step (tcgen05.ld 32x32b) and
// carries u / gate of its 128/T batch items in registers across the T loads.
//
// Two kernels share the pieces below: a one-tile-per-CTA version and, the default, a persistent
// version (further down) that overlaps the epilogue of one tile with the MMAs of the next and can
// use 128 x 256 tiles (2 x 128/T batch items per tile) to halve the W traffic per flop.
//
// Pipeline (192 threads): warp 4 = TMA producer (one lane), warp 5 = MMA issuer (one lane, also
// owns the TMEM allocation), warps 0-3 = epilogue (128 lanes of TMEM). STAGES shared-memory
// stages of {W tile 128x64, X tile 128x64} bf16 with 128-byte swizzle; full/empty mbarriers per
// stage; tcgen05.commit frees a stage when the MMAs that read it retire and finally signals the
// accumulator. Every mbarrier wait is bounded (~1 s): on expiry the thread records an error code
// in g_linear_lif_error, everybody falls through to the common exit, and TMEM is released.
// No cluster launch, no multicast: every CTA fetches its own tiles.
#include "../../include/snn_b200.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace snn_internal {
void set_last_cuda_error(int e);   // defined in lif_capi.cu
}

namespace {

constexpr int BM = 128;            // output neurons per CTA (= TMEM lanes)
constexpr int BN = 128;            // (t, b) pairs per CTA (= TMEM columns)
constexpr int BK = 64;             // K elements per stage: 64 bf16 = one 128-byte swizzled row
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;         // K per tcgen05.mma for 16-bit operands
constexpr int kThreads = 192;
constexpr uint32_t kStageBytesA = BM * BK * 2;
constexpr uint32_t kStageBytesB = BN * BK * 2;
constexpr uint32_t kTmemCols = 128;
constexpr long long kWaitCycles = 2000000000LL;       // ~1 s

__device__ int g_linear_lif_error = 0;

struct __align__(1024) SharedStorage {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BN * BK];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t accum_full;
    uint32_t tmem_base;
};

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
// false if the barrier did not reach the phase within the limit
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity))
        if (clock64() - t0 > kWaitCycles) return false;
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes (64 bf16) with the
// 128-byte swizzle: start address >> 4 in bits [0,14), leading byte offset (unused for swizzled
// K-major, encoded 1) in [16,30), stride byte offset = 1024 B between 8-row groups in [32,46),
// descriptor version 1 in [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* tile) {
    uint64_t d = static_cast<uint64_t>((smem_u32(tile) >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor, kind::f16: D fp32 (bits [4,6) = 1), A and B bf16 ([7,10) = [10,13) = 1),
// both K-major (bits 15, 16 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// T time steps, 128/T batch items per CTA tile.
template <int T>
__global__ void __launch_bounds__(kThreads, 1)
linear_lif_fwd_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const float* __restrict__ bias, __nv_bfloat16* __restrict__ current,
                      __nv_bfloat16* __restrict__ spike, int B, int K, int M, float alpha, float thresh)
{
    constexpr int BT = BN / T;                 // batch items per tile
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    SharedStorage& sm = *reinterpret_cast<SharedStorage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BM;
    const int b0 = blockIdx.y * BT;
    const int num_kb = K / BK;

    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        mbar_init(&sm.accum_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 5) {   // one whole warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = ((kb / STAGES) & 1) ^ 1;     // first pass: slots start empty
                if (!mbar_wait(&sm.empty[s], parity)) { atomicExch(&g_linear_lif_error, 1); break; }
                mbar_expect_tx(&sm.full[s], kStageBytesA + kStageBytesB);
                tma_load_2d(sm.a[s], &map_w, &sm.full[s], kb * BK, m0);
                tma_load_3d(sm.b[s], &map_x, &sm.full[s], kb * BK, b0, 0);
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = (kb / STAGES) & 1;
                if (!mbar_wait(&sm.full[s], parity)) { atomicExch(&g_linear_lif_error, 2); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_sw128(sm.a[s]);
                const uint64_t db = umma_desc_sw128(sm.b[s]);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // +32 bytes per K slice inside the swizzled 128-byte row: +2 in the (addr >> 4) field
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(&sm.empty[s]);        // stage reusable once these MMAs have read it
            }
            if (ok) umma_commit(&sm.accum_full);  // accumulator complete
        }
    } else {
        // ------------------------------ epilogue: LIF over the tile ---------------
        bool ok = mbar_wait(&sm.accum_full, 0);
        if (!ok) atomicExch(&g_linear_lif_error, 3);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int m = m0 + warp * 32 + lane;                     // this thread's output neuron
            const float bias_m = bias != nullptr ? bias[m] : 0.f;
            float u[BT], gate[BT];
#pragma unroll
            for (int j = 0; j < BT; ++j) { u[j] = 0.f; gate[j] = 1.f; }
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
            for (int t = 0; t < T; ++t) {
#pragma unroll
                for (int c = 0; c < BT; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(lane_base + t * BT + c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        // the current is rounded to bf16 first: it is what backward will re-read
                        const __nv_bfloat16 cur_h = __float2bfloat16_rn(__fadd_rn(__uint_as_float(r[j]), bias_m));
                        const float cur = __bfloat162float(cur_h);
                        const float leak = __fmul_rn(__fmul_rn(alpha, u[c + j]), gate[c + j]);
                        u[c + j] = __fadd_rn(leak, cur);
                        const bool s = u[c + j] > thresh;
                        gate[c + j] = s ? 0.f : 1.f;
                        const long long off = (static_cast<long long>(t) * B + b0 + c + j) * M + m;
                        if (current != nullptr) current[off] = cur_h;
                        spike[off] = __float2bfloat16_rn(s ? 1.f : 0.f);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Persistent variant: one CTA per SM walks a strided list of output tiles. Two accumulators in
// tensor memory (2 x WN columns) let the LIF epilogue of tile i run while the MMAs of tile i+1
// fill the other one; the epilogue writes its bf16 currents / spikes into a shared-memory tile
// laid out [t][b][m] and hands it to one 3-D TMA store per output instead of 2-byte stores.
//
// WN = accumulator columns per tile, 128 or 256. The mainloop is bound by what one SM can pull
// from L2 (measured ~58 B/clk against 128 B/clk needed to feed 128x128x64 MMAs at full rate);
// a 128 x 256 tile moves 48 KB per stage for twice the flops of a 128 x 128 tile's 32 KB, so
// the wide tile is used when it does not cost a wave of parallelism (see pick_wide()). The
// epilogue handles a wide tile as two 128-column chunks through the same staging buffers.
// ---------------------------------------------------------------------------------------------
template <int WN> struct PersistentCfg {
    static constexpr int kStages = WN == 128 ? 4 : 3;             // 4 x 32 KB or 3 x 48 KB in flight
    static constexpr uint32_t kTmemCols = 2 * WN;                 // two accumulators
    static constexpr uint32_t kStageBytesB = WN * BK * 2;
};

template <int WN>
struct __align__(1024) PersistentStorage {
    static constexpr int kStages = PersistentCfg<WN>::kStages;
    __nv_bfloat16 a[kStages][BM * BK];
    __nv_bfloat16 b[kStages][WN * BK];
    __nv_bfloat16 out_spike[128 * BM];     // one 128-column chunk: [n = t*(128/T) + j][m]
    __nv_bfloat16 out_current[128 * BM];
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    uint32_t epi_ok;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int T, int WN>
__global__ void __launch_bounds__(kThreads, 1)
linear_lif_fwd_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                 const __grid_constant__ CUtensorMap map_spike,
                                 const __grid_constant__ CUtensorMap map_current, int write_current,
                                 const float* __restrict__ bias, int B, int K, int M, float alpha, float thresh)
{
    constexpr int BT = WN / T;                  // batch items per tile
    constexpr int CB = 128 / T;                 // batch items per 128-column epilogue chunk
    constexpr int PSTAGES = PersistentCfg<WN>::kStages;
    constexpr uint32_t kTmemColsPersistent = PersistentCfg<WN>::kTmemCols;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    PersistentStorage<WN>& sm = *reinterpret_cast<PersistentStorage<WN>*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = K / BK;
    const int tiles_m = M / BM;
    const int num_tiles = tiles_m * (B / BT);

    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_spike) : "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemColsPersistent)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int it = 0;                                   // stage counter runs on across tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, b0 = (tile / tiles_m) * BT;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    const uint32_t parity = ((it / PSTAGES) & 1) ^ 1;
                    if (!mbar_wait(&sm.empty[s], parity)) { atomicExch(&g_linear_lif_error, 1); ok = false; break; }
                    mbar_expect_tx(&sm.full[s], kStageBytesA + PersistentCfg<WN>::kStageBytesB);
                    tma_load_2d(sm.a[s], &map_w, &sm.full[s], kb * BK, m0);
                    tma_load_3d(sm.b[s], &map_x, &sm.full[s], kb * BK, b0, 0);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(BM, WN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                const uint32_t acc_parity = ((local >> 1) & 1) ^ 1;      // first use of a buffer passes
                if (!mbar_wait(&sm.acc_empty[buf], acc_parity)) { atomicExch(&g_linear_lif_error, 4); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * WN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    const uint32_t parity = (it / PSTAGES) & 1;
                    if (!mbar_wait(&sm.full[s], parity)) { atomicExch(&g_linear_lif_error, 2); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc_sw128(sm.a[s]);
                    const uint64_t db = umma_desc_sw128(sm.b[s]);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&sm.empty[s]);
                }
                if (ok) umma_commit(&sm.acc_full[buf]);
            }
        }
    } else {
        // ------------------------------ epilogue warps 0-3 ------------------------
        const int row = warp * 32 + lane;                 // TMEM lane = output neuron inside the tile
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int m0 = (tile % tiles_m) * BM, b0 = (tile / tiles_m) * BT;
            const int buf = local & 1;
            const uint32_t acc_parity = (local >> 1) & 1;
            if (threadIdx.x == 0) {
                const bool ok0 = mbar_wait(&sm.acc_full[buf], acc_parity);
                if (!ok0) atomicExch(&g_linear_lif_error, 3);
                // the previous tile's TMA stores must have finished reading the staging tiles
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                sm.epi_ok = ok0 ? 1u : 0u;
            }
            epilogue_barrier();
            if (sm.epi_ok == 0u) break;
            mbar_wait(&sm.acc_full[buf], acc_parity);     // already complete: returns at once, orders this thread
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

            const float bias_m = bias != nullptr ? bias[m0 + row] : 0.f;
            const uint32_t lane_base = tmem_base + buf * WN + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
            for (int h = 0; h < WN / 128; ++h) {          // 128-column chunk = CB batch items x T steps
                if (h > 0) {
                    // the previous chunk's TMA stores must have finished reading the staging tiles
                    if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    epilogue_barrier();
                }
                float u[CB], gate[CB];
#pragma unroll
                for (int j = 0; j < CB; ++j) { u[j] = 0.f; gate[j] = 1.f; }
#pragma unroll
                for (int t = 0; t < T; ++t) {
#pragma unroll
                    for (int c = 0; c < CB; c += 16) {
                        uint32_t r[16];
                        tmem_ld16(lane_base + t * BT + h * CB + c, r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const __nv_bfloat16 cur_h =
                                __float2bfloat16_rn(__fadd_rn(__uint_as_float(r[j]), bias_m));
                            const float cur = __bfloat162float(cur_h);
                            const float leak = __fmul_rn(__fmul_rn(alpha, u[c + j]), gate[c + j]);
                            u[c + j] = __fadd_rn(leak, cur);
                            const bool s = u[c + j] > thresh;
                            gate[c + j] = s ? 0.f : 1.f;
                            const int n = t * CB + c + j;
                            sm.out_spike[n * BM + row] = __float2bfloat16_rn(s ? 1.f : 0.f);
                            sm.out_current[n * BM + row] = cur_h;
                        }
                    }
                }
                if (h == WN / 128 - 1) {
                    // accumulator drained: hand the TMEM buffer back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbar_arrive(&sm.acc_empty[buf]);
                }
                // staging tiles complete: one thread issues the bulk stores
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                epilogue_barrier();
                if (threadIdx.x == 0) {
                    tma_store_3d(&map_spike, sm.out_spike, m0, b0 + h * CB, 0);
                    if (write_current) tma_store_3d(&map_current, sm.out_current, m0, b0 + h * CB, 0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
        }
        if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemColsPersistent)
                     : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// swizzled = operand tiles read by the MMA (128-byte swizzle); plain = output tiles written by TMA stores
bool make_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
              const cuuint32_t* box, bool swizzled) {
    EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) return false;
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims,
               strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Encoding a tensor map costs a few microseconds of host time, comparable to the kernel itself for
// small layers, and a training loop calls with the same buffers step after step: keep the last
// few maps keyed by everything that went into them.
struct MapKey {
    const void* base; int rank; cuuint64_t dims[3]; cuuint32_t box[3]; bool swizzled;
    bool operator==(const MapKey& o) const {
        if (base != o.base || rank != o.rank || swizzled != o.swizzled) return false;
        for (int i = 0; i < 3; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        return true;
    }
};
bool cached_map(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                const cuuint32_t* box, bool swizzled = true) {
    constexpr int kSlots = 16;
    thread_local MapKey keys[kSlots];
    thread_local CUtensorMap maps[kSlots];
    thread_local int used = 0, next = 0;
    MapKey k{base, rank, {dims[0], dims[1], rank > 2 ? dims[2] : 1}, {box[0], box[1], rank > 2 ? box[2] : 1}, swizzled};
    for (int i = 0; i < used; ++i)
        if (keys[i] == k) { *out = maps[i]; return true; }
    if (!make_map(out, base, rank, dims, strides, box, swizzled)) return false;
    const int slot = used < kSlots ? used++ : (next++ % kSlots);
    keys[slot] = k;
    maps[slot] = *out;
    return true;
}

template <int T>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* current, void* spike, int B, int K,
           int M, float alpha, float thresh, cudaStream_t st) {
    const size_t smem = sizeof(SharedStorage) + 1024;
    auto kern = linear_lif_fwd_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    dim3 grid(M / BM, B / (BN / T));
    kern<<<grid, kThreads, smem, st>>>(mw, mx, bias, static_cast<__nv_bfloat16*>(current),
                                       static_cast<__nv_bfloat16*>(spike), B, K, M, alpha, thresh);
    e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

int sm_count() {
    thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        dev_cached = dev;
    }
    return sms;
}

template <int T, int WN>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& ms, const CUtensorMap& mc,
                      int write_current, const float* bias, int B, int K, int M, float alpha, float thresh,
                      cudaStream_t st) {
    static_assert(sizeof(PersistentStorage<WN>) + 1024 <= 227 * 1024, "shared memory budget");
    const size_t smem = sizeof(PersistentStorage<WN>) + 1024;
    auto kern = linear_lif_fwd_persistent_kernel<T, WN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const int sms = sm_count();
    if (e == cudaSuccess && sms <= 0) e = cudaErrorInvalidDevice;
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    const int tiles = (M / BM) * (B / (WN / T));
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, kThreads, smem, st>>>(mw, mx, ms, mc, write_current, bias, B, K, M, alpha, thresh);
    e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

// SNN_LINEAR_LIF_VARIANT: 1 = one-tile-per-CTA kernel (kept for comparison), 2 = persistent kernel
// with 128-column tiles, 3 = persistent kernel with 256-column tiles where the batch allows;
// default 0 = persistent kernel, tile width chosen by pick_wide().
int variant() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("SNN_LINEAR_LIF_VARIANT");
        v = (e != nullptr && e[0] >= '1' && e[0] <= '3') ? e[0] - '0' : 0;
    }
    return v;
}

// A 256-column tile does twice the work of a 128-column one in about 1.5x the time (48 KB
// instead of 2 x 32 KB through the SM's L2 port), but halves the tile count: compare the rounds
// of tiles each choice needs on this device.
bool pick_wide(int T, int B, int M) {
    if (B % (256 / T) != 0) return false;
    const int v = variant();
    if (v == 2) return false;
    if (v == 3) return true;
    const int sms = sm_count();
    if (sms <= 0) return false;
    const long long t128 = static_cast<long long>(M / BM) * (B / (128 / T));
    const long long t256 = t128 / 2;
    const long long cost128 = 2 * ((t128 + sms - 1) / sms);
    const long long cost256 = 3 * ((t256 + sms - 1) / sms);
    return cost256 < cost128;
}

}  // namespace

extern "C" {

int snn_linear_lif_fwd_supported(int64_t T, int64_t B, int64_t K, int64_t M, int dtype) {
    if (dtype != SNN_BF16) return 0;
    if (T != 4 && T != 8) return 0;          // 128/T batch items per tile, read 16 columns at a time
    if (B < 1 || B % (BN / T) != 0 || B > 65535 * (BN / T)) return 0;
    if (K < BK || K % BK != 0 || M < BM || M % BM != 0) return 0;
    if (K > INT32_MAX || M > INT32_MAX) return 0;
    return 1;
}

int snn_linear_lif_fwd(const void* x, const void* weight, const float* bias, void* current, void* spike,
                       int64_t T, int64_t B, int64_t K, int64_t M, int dtype, float alpha, float thresh,
                       void* stream) {
    if (dtype != SNN_BF16 && dtype != SNN_F32 && dtype != SNN_F16 && dtype != SNN_F64) return SNN_ERR_DTYPE;
    if (T < 1 || B < 1 || K < 1 || M < 1) return SNN_ERR_SHAPE;
    if (!snn_linear_lif_fwd_supported(T, B, K, M, dtype)) return SNN_ERR_UNSUPPORTED;
    if (!x || !weight || !spike) return SNN_ERR_NULL;
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; };
    if (!al(x, 16) || !al(weight, 16) || !al(spike, 2) || !al(current, 2) || !al(bias, 4)) return SNN_ERR_ALIGN;

    const bool one_tile = variant() == 1 || !al(spike, 16) || !al(current, 16);
    const bool wide = !one_tile && pick_wide(static_cast<int>(T), static_cast<int>(B), static_cast<int>(M));
    const cuuint32_t tile_n = wide ? 256 : 128;
    CUtensorMap mw, mx;
    const cuuint64_t wdims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
    const cuuint64_t wstr[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t wbox[2] = {BK, BM};
    const cuuint64_t xdims[3] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(B), static_cast<cuuint64_t>(T)};
    const cuuint64_t xstr[2] = {static_cast<cuuint64_t>(K) * 2, static_cast<cuuint64_t>(B) * K * 2};
    const cuuint32_t xbox[3] = {BK, tile_n / static_cast<cuuint32_t>(T), static_cast<cuuint32_t>(T)};
    if (!cached_map(&mw, weight, 2, wdims, wstr, wbox) || !cached_map(&mx, x, 3, xdims, xstr, xbox)) {
        snn_internal::set_last_cuda_error(static_cast<int>(cudaErrorInvalidValue));
        return SNN_ERR_CUDA;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int Bi = static_cast<int>(B), Ki = static_cast<int>(K), Mi = static_cast<int>(M);
    if (one_tile) {
        if (T == 4) return launch<4>(mw, mx, bias, current, spike, Bi, Ki, Mi, alpha, thresh, st);
        return launch<8>(mw, mx, bias, current, spike, Bi, Ki, Mi, alpha, thresh, st);
    }
    CUtensorMap ms, mc;
    const cuuint64_t odims[3] = {static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(B), static_cast<cuuint64_t>(T)};
    const cuuint64_t ostr[2] = {static_cast<cuuint64_t>(M) * 2, static_cast<cuuint64_t>(B) * M * 2};
    const cuuint32_t obox[3] = {BM, static_cast<cuuint32_t>(BN / T), static_cast<cuuint32_t>(T)};
    if (!cached_map(&ms, spike, 3, odims, ostr, obox, false) ||
        (current != nullptr && !cached_map(&mc, current, 3, odims, ostr, obox, false))) {
        snn_internal::set_last_cuda_error(static_cast<int>(cudaErrorInvalidValue));
        return SNN_ERR_CUDA;
    }
    if (current == nullptr) mc = ms;
    const int wc = current != nullptr ? 1 : 0;
    if (wide) {
        if (T == 4) return launch_persistent<4, 256>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, st);
        return launch_persistent<8, 256>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, st);
    }
    if (T == 4) return launch_persistent<4, 128>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, st);
    return launch_persistent<8, 128>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, st);
}

int snn_linear_lif_error(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_linear_lif_error, sizeof(int));
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return -1; }
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_linear_lif_error, &zero, sizeof(int));
    }
    return v;
}

}  // extern "C"
