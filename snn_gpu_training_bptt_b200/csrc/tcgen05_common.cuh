// Pieces shared by the tcgen05 kernels of this library (fused linear + LIF forward, and the
// backward GEMMs): mbarrier / TMA / tcgen05 PTX wrappers, shared-memory and instruction
// descriptors, bounded waits with a per-module error word, and the host-side tensor-map cache.
// sm_100a only. Every definition is header-local (static / inline); each translation unit that
// includes this file gets its own error word g_tc_error.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <type_traits>

namespace snn_tc {

// Bound of every mbarrier wait in SM cycles: ~1 s. The test-only build that checks the expiry path
// (tests/test_linear_lif_gpu.py) shortens it with -DSNN_TC_WAIT_CYCLES=...
#ifndef SNN_TC_WAIT_CYCLES
#define SNN_TC_WAIT_CYCLES 2000000000LL
#endif
constexpr long long kWaitCycles = SNN_TC_WAIT_CYCLES;
// Waits that depend on another role's progress (a free stage, a full or drained accumulator) get twice
// the limit of the waits for operands: when operands never arrive, the operand wait is the one that
// expires first and names the cause (dependent waits then stop early on seeing the error word).
constexpr long long kDependentWaitCycles = 2 * kWaitCycles;

// 0, or the code of the first bounded wait that expired in a kernel of this translation unit
static __device__ int g_tc_error = 0;

// Development aid, compiled out of the library: with -DSNN_TC_STAMPS a kernel records the SM's cycle
// counter at named points (slot) of each CTA into g_tc_stamps, which a test driver reads back.
#ifdef SNN_TC_STAMPS
static __device__ long long g_tc_stamps[512][64];
#define SNN_TC_STAMP(slot) do { if (blockIdx.x < 512) g_tc_stamps[blockIdx.x][slot] = clock64(); } while (0)
#else
#define SNN_TC_STAMP(slot) do { } while (0)
#endif

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
// Only the FIRST failure is kept (a producer that gives up makes the MMA issuer and the epilogue
// give up later: their codes would hide the cause).
__device__ __forceinline__ void record_error(int code) { atomicCAS(&g_tc_error, 0, code); }
// false if the barrier did not reach the phase within the limit, or if another role (of any CTA)
// has already recorded a failure: dependent waits then return at once instead of running out
// their own limit one after the other.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) return false;
        if ((spins & 63u) == 0u && *reinterpret_cast<volatile int*>(&g_tc_error) != 0) return false;
    }
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
// The same for an MN-major tile: the tile is stored as rows of the REDUCTION index, each row
// holding 64 consecutive M (or N) elements = 128 bytes, 128-byte swizzle (this is how a TMA box
// {64 elements, R rows} of a row-major [reduction][M or N] matrix lands). Eight such rows form
// one 1024-byte swizzle atom: stride byte offset (between 8-row groups along the reduction
// index) = 1024; a tile wider than 64 elements is made of several such boxes `lbo_bytes` apart:
// leading byte offset = distance between consecutive 64-element groups along M / N.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(const void* tile, uint32_t lbo_bytes) {
    uint64_t d = static_cast<uint64_t>((smem_u32(tile) >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor, kind::f16: D fp32 (bits [4,6) = 1), A and B bf16 ([7,10) = [10,13) = 1),
// both K-major (bits 15, 16 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
// Bit 15 / bit 16 = 1 selects an MN-major A / B operand.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, bool a_mn_major = false,
                                                       bool b_mn_major = false) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn_major ? (1u << 15) : 0u) | (b_mn_major ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void group_barrier(int g) {      // the 128 threads of epilogue group g
    asm volatile("bar.sync %0, 128;" ::"r"(1 + g) : "memory");
}

// tcgen05.ld of NCOL (2, 4, 8 or 16) consecutive columns of this warp's 32 lanes into r[0..NCOL)
template <int NCOL>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
    if constexpr (NCOL == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr));
    } else if constexpr (NCOL == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(taddr));
    } else if constexpr (NCOL == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                     : "r"(taddr));
    } else {
        static_assert(NCOL == 2, "2, 4, 8 or 16 columns");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr));
    }
}
// Waits for the loads issued so far. The 32 registers of a unit are passed through the statement
// so that no use of them can be scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// The linear + LIF kernels are 10-20 us each, so the ~2 us between one kernel's last CTA and the
// next kernel's first instruction is a tenth of a training step's time in this layer. Launched
// with launch_pdl() below, a kernel may begin (barrier set-up, tensor-memory allocation, tensor
// map prefetch) as soon as every CTA of the kernel before it has started and SM resources free
// up; pdl_wait() then holds it until that kernel has completed and its memory is visible. Every
// thread calls pdl_wait() before its first access to global memory. Both instructions are no-ops
// in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- CTA pairs (clusters of two, tcgen05 cta_group::2) ------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in the CTA of the given cluster rank
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier in another CTA of the cluster. CTA-scope release (the instruction's default):
// the barrier hands over tensor memory only, whose reads are ordered by tcgen05.wait::ld and
// tcgen05.fence::before_thread_sync on this side and tcgen05.fence::after_thread_sync on the
// waiting side; no data in shared or global memory is published through it. A cluster-scope
// release here measured ~2000 cycles per call in the thread that has a bulk store in flight.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far retire
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}

// ---- host side ---------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
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
// f32 = fp32 elements instead of bf16
inline bool make_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                     const cuuint32_t* box, bool swizzled, bool f32 = false) {
    EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) return false;
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    return enc(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), dims,
               strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzled ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Encoding a tensor map costs a few microseconds of host time, comparable to the kernel itself for
// small layers, and a training loop calls with the same buffers step after step: keep the last
// few maps keyed by everything that went into them.
struct MapKey {
    const void* base; int rank; cuuint64_t dims[3]; cuuint32_t box[3]; bool swizzled; bool f32; cuuint64_t stride0;
    bool operator==(const MapKey& o) const {
        if (base != o.base || rank != o.rank || swizzled != o.swizzled || f32 != o.f32 || stride0 != o.stride0)
            return false;
        for (int i = 0; i < 3; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        return true;
    }
};
inline bool cached_map(CUtensorMap* out, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                       const cuuint32_t* box, bool swizzled = true, bool f32 = false) {
    constexpr int kSlots = 32;
    thread_local MapKey keys[kSlots];
    thread_local CUtensorMap maps[kSlots];
    thread_local int used = 0, next = 0;
    MapKey k{base, rank, {dims[0], dims[1], rank > 2 ? dims[2] : 1}, {box[0], box[1], rank > 2 ? box[2] : 1},
             swizzled, f32, strides[0]};
    for (int i = 0; i < used; ++i)
        if (keys[i] == k) { *out = maps[i]; return true; }
    if (!make_map(out, base, rank, dims, strides, box, swizzled, f32)) return false;
    const int slot = used < kSlots ? used++ : (next++ % kSlots);
    keys[slot] = k;
    maps[slot] = *out;
    return true;
}

// SNN_LINEAR_LIF_PDL=0 turns programmatic dependent launch off (ordinary stream order).
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("SNN_LINEAR_LIF_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic-stream-serialization
// attribute (see pdl_wait above); also valid inside a stream capture.
template <typename... Params, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

inline int sm_count() {
    thread_local int dev_cached = -1, sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != dev_cached) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        dev_cached = dev;
    }
    return sms;
}

}  // namespace snn_tc
