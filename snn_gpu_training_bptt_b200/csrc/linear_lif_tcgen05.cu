// Fused synaptic linear + LIF forward on the 5th-generation tensor cores (tcgen05 / TMEM).
//
//   current[t, b, :] = x[t, b, :] @ W^T + bias          (bf16 operands, fp32 accumulation in TMEM)
//   spike[t, b, :]   = LIF over t of current[:, b, :]   (fp32 state, same arithmetic as lif_kernels.cuh)
//
// In the reference this is `Fc` followed by `Fire`: T separate cuBLAS calls with a copy each
// (fc_fp_cuda, snnlib/cuda/snn_kernel_fp.cu:332-357) and then fire_s_fp_kernel (:15-53) re-reading
// the currents from HBM. Here one kernel computes a tile of currents - 128 output neurons x
// (T time steps x a group of batch items) - in tensor memory and runs the recurrence on it in the
// epilogue, so spikes come straight out of the GEMM.
//
// GEMM orientation: D[m, n] = sum_k W[m, k] * X[n, k], M = output neurons, N = (t, b) pairs.
// The X tile is fetched by one 3-D TMA box {64 k, BT batch items, T steps} of the [T][B][K]
// tensor (BT = tile columns / T), which lands in shared memory as rows ordered (t major, b
// minor): accumulator column n = t*BT + j. A TMEM lane is one output neuron, so the epilogue
// thread that owns the lane reads the columns of its batch items step by step (tcgen05.ld
// 32x32b) and carries their u / gate in registers across the T steps.
//
// Three kernels share the pieces below:
//   * linear_lif_fwd_kernel            one 128 x 128 tile per CTA (the first version; fallback
//                                      for outputs that are not 16-byte aligned)
//   * linear_lif_fwd_persistent_kernel one CTA per SM walks a tile list; 128 x 128 or 128 x 256
//                                      tiles; two accumulators so the epilogue of one tile
//                                      overlaps the MMAs of the next; TMA-store epilogue
//   * linear_lif_fwd_pair_kernel       a cluster of two CTAs per 256 x 256 tile with
//                                      tcgen05.mma.cta_group::2; for layers with many tiles
// pick_kernel() on the host chooses among them per problem.
//
// Roles: warp 4 = TMA producer (one lane), warp 5 = MMA issuer (one lane, also owns the TMEM
// allocation), warps 0-3 = epilogue (the 128 lanes of TMEM); the persistent and pair kernels add
// a second epilogue group, warps 6-9. Shared-memory stages of {W tile, X tile} in bf16 with the
// 128-byte swizzle; full/empty mbarriers per stage; tcgen05.commit frees a stage when the MMAs
// that read it retire and finally signals the accumulator. Every mbarrier wait is bounded (~1 s):
// on expiry the thread records an error code in g_tc_error, everybody falls through to
// the common exit, and TMEM is released. No multicast loads anywhere: every CTA fetches its own
// operands.
#include "../../include/snn_b200.h"

#include "tcgen05_common.cuh"

namespace snn_internal {
void set_last_cuda_error(int e);      // defined in lif_capi.cu
int linear_lif_bwd_error(int reset);   // error word of the backward kernels, linear_lif_bwd_tcgen05.cu
}

namespace {

using namespace snn_tc;

// Test-only build (-DSNN_TC_WAIT_TEST, never part of libsnn_b200.so): the producer of the persistent
// kernel leaves out the loads of one K stage when told to, so that stage's operands never arrive,
// the MMA issuer's bounded wait runs out and the kernel must return with error code 2.
#ifdef SNN_TC_WAIT_TEST
__device__ int g_tc_test_skip_stage = -1;
#endif

constexpr int BM = 128;            // output neurons per CTA (= TMEM lanes)
constexpr int BN = 128;            // (t, b) pairs per CTA (= TMEM columns)
constexpr int BK = 64;             // K elements per stage: 64 bf16 = one 128-byte swizzled row
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;         // K per tcgen05.mma for 16-bit operands
constexpr int kThreads = 192;
constexpr uint32_t kStageBytesA = BM * BK * 2;
constexpr uint32_t kStageBytesB = BN * BK * 2;
constexpr uint32_t kTmemCols = 128;

struct __align__(1024) SharedStorage {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BN * BK];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t accum_full;
    uint32_t tmem_base;
};

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
                if (!mbar_wait(&sm.empty[s], parity, kDependentWaitCycles)) { record_error(1); break; }
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
                if (!mbar_wait(&sm.full[s], parity)) { record_error(2); ok = false; break; }
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
        bool ok = mbar_wait(&sm.accum_full, 0, kDependentWaitCycles);
        if (!ok) record_error(3);
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
// WN = accumulator columns per tile, 128 or 256. Measured with cycle-counter stamps at the MMA issuer: a K stage (four
// tcgen05.mma 128 x WN x 16) takes ~535 cycles for WN = 256, i.e. ~95 % of the tensor pipe's
// rate, and the same ~531 cycles for WN = 128 - half the flops. So the wide tile is used
// whenever it does not cost a round of parallelism (see pick_kernel()).
// ---------------------------------------------------------------------------------------------
// Threads of the persistent and pair kernels: warps 0-3 = epilogue group 0, warp 4 = TMA producer,
// warp 5 = MMA issuer / TMEM owner, warps 6-9 = epilogue group 1. A warp may only touch the TMEM
// lanes of its quarter (warp index mod 4), so the two groups split a tile by columns: it is cut
// into 32-column units (32/T batch items x T steps) and group g takes units g, g+2, ...
constexpr int kThreadsP = 320;
struct EpilogueStaging {                   // one 32-column unit: [n = t*(32/T) + j][m], 2 x 8 KB
    __nv_bfloat16 spike[32 * BM];
    __nv_bfloat16 current[32 * BM];
};

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
    EpilogueStaging epi[2][2];             // [epilogue group][double buffer]
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    uint32_t epi_ok[2];
};

// Packed fp32 pairs (sm_100): two lanes in one 64-bit register, each lane rounded on its own.
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// LIF epilogue of one accumulator tile for epilogue group g (thread = TMEM lane = output neuron
// `row` of the tile). The group walks its 32-column units (32/T batch items x all T steps = 32
// accumulator values per thread): the unit's TMEM loads are issued one unit ahead of the
// arithmetic; u / gate of the unit's batch items live in registers across its T steps; currents
// and spikes are staged [t][b][m] in one of the group's two staging buffers and written by one
// 3-D TMA store each, issued by the group's elected thread, so the store of one unit is read out
// of shared memory while the next unit is computed into the other buffer. `k` counts the units
// this group has staged since the kernel started (buffer = k & 1). `drained()` is called by every
// thread once its last TMEM read of the tile has completed. On entry the accumulator is full.
// T is the tile's step count (2, 4, 8 or 16); the tensor has t_real <= T steps: the steps beyond
// are zero-filled by the TMA loads, skipped here and clipped by the TMA stores (FULL = the tensor
// fills the tile, no step is checked).
template <int T, int WN, bool FULL, typename Drained>
__device__ __forceinline__ void lif_epilogue_tile(EpilogueStaging (&stage)[2], int& k, int g, bool elected,
                                                  uint32_t lane_base, int row, float bias_m, float alpha,
                                                  float thresh, int t_real, const CUtensorMap* map_spike,
                                                  const CUtensorMap* map_current, int write_current, int m0,
                                                  int b0, Drained&& drained)
{
    constexpr int BT = WN / T;                  // batch items per tile
    constexpr int SB = 32 / T;                  // batch items per unit
    constexpr int PER_GROUP = WN / 64;          // units per group and tile
    uint32_t r[2][32] = {};
#pragma unroll
    for (int t = 0; t < T; ++t) tmem_ld_cols<SB>(lane_base + t * BT + g * SB, &r[0][t * SB]);
#pragma unroll
    for (int i = 0; i < PER_GROUP; ++i) {
        const int q = g + 2 * i;                // unit index inside the tile
        tmem_ld_wait32(r[i & 1]);
        if (i + 1 < PER_GROUP) {
#pragma unroll
            for (int t = 0; t < T; ++t) tmem_ld_cols<SB>(lane_base + t * BT + (q + 2) * SB, &r[(i + 1) & 1][t * SB]);
        } else {
            // accumulator drained: hand the TMEM buffer back to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            drained();
        }
        // this buffer's previous store was waited for before the group barrier of the unit before
        EpilogueStaging& st = stage[k & 1];
        // The recurrence runs on PAIRS of batch items with the packed fp32 instructions of sm_100
        // (add.rn.f32x2 / mul.rn.f32x2: two independently rounded lanes per instruction, so the
        // results are bit-identical to the scalar __fadd_rn / __fmul_rn form) - the epilogue is
        // issue-bound, and this takes the arithmetic from ~11 to ~8.5 instructions per element.
        // The hard reset is a select on the previous spike instead of a multiplication by the
        // 0/1 gate: (alpha*u)*0 and 0 differ at most in the sign of a zero, which changes neither
        // u's comparisons nor any output of this kernel.
        static_assert(SB % 2 == 0, "batch items per unit come in pairs");
        uint64_t u2[SB / 2];
        bool fired[SB];
#pragma unroll
        for (int j = 0; j < SB / 2; ++j) u2[j] = 0ull;
#pragma unroll
        for (int j = 0; j < SB; ++j) fired[j] = false;
        const uint64_t bias2 = pack_f32x2(bias_m, bias_m), alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll
        for (int t = 0; t < T; ++t) {
            if (!FULL && t >= t_real) break;
#pragma unroll
            for (int jp = 0; jp < SB / 2; ++jp) {
                const int n = t * SB + 2 * jp;
                float c_lo, c_hi, a_lo, a_hi, u_lo, u_hi;
                unpack_f32x2(add_f32x2(pack_f32x2(__uint_as_float(r[i & 1][n]), __uint_as_float(r[i & 1][n + 1])), bias2),
                             c_lo, c_hi);
                // both currents rounded to bf16 by one instruction: it is what backward will re-read
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(c_lo, c_hi);
                const uint32_t bits = *reinterpret_cast<const uint32_t*>(&h2);
                const float cur_lo = __uint_as_float(bits << 16), cur_hi = __uint_as_float(bits & 0xffff0000u);
                unpack_f32x2(mul_f32x2(alpha2, u2[jp]), a_lo, a_hi);
                const float leak_lo = fired[2 * jp] ? 0.f : a_lo, leak_hi = fired[2 * jp + 1] ? 0.f : a_hi;
                u2[jp] = add_f32x2(pack_f32x2(leak_lo, leak_hi), pack_f32x2(cur_lo, cur_hi));
                unpack_f32x2(u2[jp], u_lo, u_hi);
                fired[2 * jp] = u_lo > thresh;
                fired[2 * jp + 1] = u_hi > thresh;
                unsigned short* sp = reinterpret_cast<unsigned short*>(st.spike);
                unsigned short* cp = reinterpret_cast<unsigned short*>(st.current);
                sp[n * BM + row] = fired[2 * jp] ? static_cast<unsigned short>(0x3F80) : static_cast<unsigned short>(0);
                sp[(n + 1) * BM + row] = fired[2 * jp + 1] ? static_cast<unsigned short>(0x3F80) : static_cast<unsigned short>(0);
                cp[n * BM + row] = static_cast<unsigned short>(bits & 0xffffu);
                cp[(n + 1) * BM + row] = static_cast<unsigned short>(bits >> 16);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the other buffer's store (issued a unit ago) must have been read before anyone passes
        // the barrier and starts the next unit in it
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        group_barrier(g);
        if (elected) {
            tma_store_3d(map_spike, st.spike, m0, b0 + q * SB, 0);
            if (write_current) tma_store_3d(map_current, st.current, m0, b0 + q * SB, 0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        ++k;
    }
}

template <int T, int WN>
__global__ void __launch_bounds__(kThreadsP, 1)
linear_lif_fwd_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                 const __grid_constant__ CUtensorMap map_spike,
                                 const __grid_constant__ CUtensorMap map_current, int write_current,
                                 const float* __restrict__ bias, int B, int K, int M, float alpha, float thresh,
                                 int t_real)
{
    constexpr int BT = WN / T;                  // batch items per tile
    constexpr int PSTAGES = PersistentCfg<WN>::kStages;
    constexpr uint32_t kTmemColsPersistent = PersistentCfg<WN>::kTmemCols;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    PersistentStorage<WN>& sm = *reinterpret_cast<PersistentStorage<WN>*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = K / BK;
    const int tiles_m = M / BM;
    const int num_tiles = tiles_m * (B / BT);

    pdl_launch_dependents();
    int preloaded = 0;                          // K stages the producer thread has already requested
    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 256); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        pdl_wait();                             // the loads below read what earlier kernels wrote
        // The first stages of the first tile need nothing but these barriers: request them now so
        // the TMEM allocation and the block-wide sync below overlap the first loads' latency.
        if (blockIdx.x < num_tiles) {
            const int m0 = (blockIdx.x % tiles_m) * BM, b0 = (blockIdx.x / tiles_m) * BT;
            preloaded = num_kb < PSTAGES ? num_kb : PSTAGES;
            for (int kb = 0; kb < preloaded; ++kb) {
                mbar_expect_tx(&sm.full[kb], kStageBytesA + PersistentCfg<WN>::kStageBytesB);
                tma_load_2d(sm.a[kb], &map_w, &sm.full[kb], kb * BK, m0);
                tma_load_3d(sm.b[kb], &map_x, &sm.full[kb], kb * BK, b0, 0);
            }
        }
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
    pdl_wait();

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int it = 0;                                   // stage counter runs on across tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, b0 = (tile / tiles_m) * BT;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    if (it < preloaded) continue;             // requested before the set-up sync
#ifdef SNN_TC_WAIT_TEST
                    if (it == g_tc_test_skip_stage) continue; // test build: these operands are never requested
#endif
                    const int s = it % PSTAGES;
                    const uint32_t parity = ((it / PSTAGES) & 1) ^ 1;
                    if (!mbar_wait(&sm.empty[s], parity, kDependentWaitCycles)) { record_error(1); ok = false; break; }
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
                if (!mbar_wait(&sm.acc_empty[buf], acc_parity, kDependentWaitCycles)) { record_error(4); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * WN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    const uint32_t parity = (it / PSTAGES) & 1;
                    if (!mbar_wait(&sm.full[s], parity)) { record_error(2); ok = false; break; }
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
        // ------------------------------ epilogue groups (warps 0-3, 6-9) ----------
        const int g = warp >= 6 ? 1 : 0;
        const int quarter = warp & 3;                     // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;              // TMEM lane = output neuron inside the tile
        const bool elected = lane == 0 && warp == (g ? 6 : 0);
        int local = 0, staged = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int m0 = (tile % tiles_m) * BM, b0 = (tile / tiles_m) * BT;
            const int buf = local & 1;
            const uint32_t acc_parity = (local >> 1) & 1;
            if (elected) {
                const bool ok0 = mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);
                if (!ok0) record_error(3);
                sm.epi_ok[g] = ok0 ? 1u : 0u;
            }
            group_barrier(g);
            if (sm.epi_ok[g] == 0u) break;
            mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);     // already complete: returns at once, orders this thread
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

            const float bias_m = bias != nullptr ? bias[m0 + row] : 0.f;
            const uint32_t lane_base = tmem_base + buf * WN + (static_cast<uint32_t>(quarter * 32) << 16);
            uint64_t* drained_bar = &sm.acc_empty[buf];
            auto drained = [drained_bar] { mbar_arrive(drained_bar); };
            if (t_real == T)
                lif_epilogue_tile<T, WN, true>(sm.epi[g], staged, g, elected, lane_base, row, bias_m, alpha, thresh,
                                               t_real, &map_spike, &map_current, write_current, m0, b0, drained);
            else
                lif_epilogue_tile<T, WN, false>(sm.epi[g], staged, g, elected, lane_base, row, bias_m, alpha, thresh,
                                                t_real, &map_spike, &map_current, write_current, m0, b0, drained);
        }
        // shared memory must outlive the reads of the last stores; the writes themselves complete
        // before the grid does
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemColsPersistent)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (the two SMs of a TPC) computes a 256 (output neurons)
// x 256 ((t, b) pairs) tile with tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of W
// and HALF of the X tile (time steps [rank*T/2, (rank+1)*T/2) of the tile's 256/T batch items =
// accumulator columns [rank*128, rank*128+128)); the pair's tensor cores read both halves, so a
// CTA pulls 32 KB per stage for the flops that cost the single-CTA kernels 48 KB (wide tile) or
// 64 KB (two narrow tiles). Each CTA's tensor memory receives its own 128 neurons x 256 columns,
// and its epilogue warps run the same LIF epilogue as above. While the operands fit in L2 and
// neighbouring CTAs run in step (config-3 size) the wide-tile mainloop is already tensor-bound
// and the pair kernel is no faster (K stage 547 cycles, plus ~1000 cycles of cluster set-up);
// with many tiles per CTA the wide kernel's stages stretch to 900-1300 cycles waiting for
// operands, and the pair's lower traffic pays: see pick_kernel().
//
// Roles per CTA as before; the MMA issuer runs in the leader (cluster rank 0) only. Both CTAs'
// TMA loads complete on the LEADER's full barrier (armed with the bytes of both); the leader's
// tcgen05.commit multicasts the stage-free / accumulator-full arrivals to both CTAs; epilogue
// threads of both CTAs arrive on the leader's accumulator-empty barriers. Two accumulators
// (2 x 256 columns = all of tensor memory), so the epilogue of one tile overlaps the MMAs of the
// pair's next tile. No multicast loads. All mbarrier waits are bounded as above; the cluster barriers at entry and
// exit are reached unconditionally by every thread of both CTAs.
// ---------------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 5;
constexpr uint32_t kPairTmemCols = 512;      // two accumulators of 256 columns: all of tensor memory
constexpr int PAIR_N = 256;

struct __align__(1024) PairStorage {
    __nv_bfloat16 a[PAIR_STAGES][BM * BK];
    __nv_bfloat16 b[PAIR_STAGES][(PAIR_N / 2) * BK];
    EpilogueStaging epi[2][2];
    uint64_t full[PAIR_STAGES];        // used in the leader
    uint64_t empty[PAIR_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];             // used in the leader: 2 CTAs x 256 epilogue threads arrive
    uint32_t tmem_base;
    uint32_t epi_ok[2];
};

template <int T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsP, 1)
linear_lif_fwd_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const __grid_constant__ CUtensorMap map_spike,
                           const __grid_constant__ CUtensorMap map_current, int write_current,
                           const float* __restrict__ bias, int B, int K, int M, float alpha, float thresh,
                           int t_real)
{
    constexpr int BT = PAIR_N / T;              // batch items per tile
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    PairStorage& sm = *reinterpret_cast<PairStorage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = K / BK;
    const int tiles_m = M / (2 * BM);
    pdl_launch_dependents();
    const int num_tiles = tiles_m * (B / BT);

    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 512); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_spike) : "memory");
    }
    if (warp == 5) {
        // one warp of each CTA of the pair takes part in the pair-wide allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kPairTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                         // the peer's barriers are initialised past this point
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;
    pdl_wait();

    if (warp == 4) {
        // ------------------------------ TMA producer (both CTAs) ------------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int m0 = (tile % tiles_m) * (2 * BM) + static_cast<int>(rank) * BM;
                const int b0 = (tile / tiles_m) * BT;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t parity = ((it / PAIR_STAGES) & 1) ^ 1;
                    if (!mbar_wait(&sm.empty[s], parity, kDependentWaitCycles)) { record_error(11); ok = false; break; }
                    const uint32_t full_leader = mapa_shared(smem_u32(&sm.full[s]), 0);
                    if (leader) mbar_expect_tx(&sm.full[s], 2 * (kStageBytesA + (PAIR_N / 2) * BK * 2));
                    tma_load_2d_pair(sm.a[s], &map_w, full_leader, kb * BK, m0);
                    tma_load_3d_pair(sm.b[s], &map_x, full_leader, kb * BK, b0, static_cast<int>(rank) * (T / 2));
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer (leader CTA only) --------------
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, PAIR_N);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const int buf = local & 1;
                const uint32_t acc_parity = ((local >> 1) & 1) ^ 1;      // first use of a buffer passes
                if (!mbar_wait(&sm.acc_empty[buf], acc_parity, kDependentWaitCycles)) { record_error(14); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * PAIR_N;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t parity = (it / PAIR_STAGES) & 1;
                    if (!mbar_wait(&sm.full[s], parity)) { record_error(12); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc_sw128(sm.a[s]);
                    const uint64_t db = umma_desc_sw128(sm.b[s]);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(&sm.empty[s]);
                }
                if (ok) umma_commit_pair(&sm.acc_full[buf]);
            }
        }
    } else {
        // ------------------------------ epilogue groups (both CTAs) ---------------
        const int g = warp >= 6 ? 1 : 0;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool elected = lane == 0 && warp == (g ? 6 : 0);
        const uint32_t acc_empty_leader0 = mapa_shared(smem_u32(&sm.acc_empty[0]), 0);
        const uint32_t acc_empty_leader1 = mapa_shared(smem_u32(&sm.acc_empty[1]), 0);
        int local = 0, staged = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
            const int m0 = (tile % tiles_m) * (2 * BM) + static_cast<int>(rank) * BM;
            const int b0 = (tile / tiles_m) * BT;
            const int buf = local & 1;
            const uint32_t acc_parity = (local >> 1) & 1;
            if (elected) {
                const bool ok0 = mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);
                if (!ok0) record_error(13);
                sm.epi_ok[g] = ok0 ? 1u : 0u;
            }
            group_barrier(g);
            if (sm.epi_ok[g] == 0u) break;
            mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);     // already complete: orders this thread
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

            const float bias_m = bias != nullptr ? bias[m0 + row] : 0.f;
            const uint32_t lane_base = tmem_base + buf * PAIR_N + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t acc_empty_leader = buf ? acc_empty_leader1 : acc_empty_leader0;
            auto drained = [acc_empty_leader] { mbar_arrive_cluster(acc_empty_leader); };
            if (t_real == T)
                lif_epilogue_tile<T, PAIR_N, true>(sm.epi[g], staged, g, elected, lane_base, row, bias_m, alpha, thresh,
                                                   t_real, &map_spike, &map_current, write_current, m0, b0, drained);
            else
                lif_epilogue_tile<T, PAIR_N, false>(sm.epi[g], staged, g, elected, lane_base, row, bias_m, alpha, thresh,
                                                    t_real, &map_spike, &map_current, write_current, m0, b0, drained);
        }
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                         // nobody touches the peer's memory or TMEM past this point
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPairTmemCols)
                     : "memory");
    }
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

template <int T, int WN>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& ms, const CUtensorMap& mc,
                      int write_current, const float* bias, int B, int K, int M, float alpha, float thresh,
                      int t_real, cudaStream_t st) {
    static_assert(sizeof(PersistentStorage<WN>) + 1024 <= 227 * 1024, "shared memory budget");
    const size_t smem = sizeof(PersistentStorage<WN>) + 1024;
    auto kern = linear_lif_fwd_persistent_kernel<T, WN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const int sms = sm_count();
    if (e == cudaSuccess && sms <= 0) e = cudaErrorInvalidDevice;
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    const int tiles = (M / BM) * (B / (WN / T));
    const int grid = tiles < sms ? tiles : sms;
    e = launch_pdl(kern, dim3(grid), dim3(kThreadsP), smem, st, mw, mx, ms, mc, write_current, bias, B, K, M, alpha,
                   thresh, t_real);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

template <int T>
int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& ms, const CUtensorMap& mc,
                int write_current, const float* bias, int B, int K, int M, float alpha, float thresh,
                int t_real, cudaStream_t st) {
    static_assert(sizeof(PairStorage) + 1024 <= 227 * 1024, "shared memory budget");
    const size_t smem = sizeof(PairStorage) + 1024;
    auto kern = linear_lif_fwd_pair_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    const int sms = sm_count();
    if (e == cudaSuccess && sms < 2) e = cudaErrorInvalidDevice;
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    const int tiles = (M / (2 * BM)) * (B / (PAIR_N / T));
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    e = launch_pdl(kern, dim3(2 * pairs), dim3(kThreadsP), smem, st, mw, mx, ms, mc, write_current, bias, B, K, M,
                   alpha, thresh, t_real);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

// SNN_LINEAR_LIF_VARIANT: 1 = one-tile-per-CTA kernel (kept for comparison), 2 = persistent kernel
// with 128-column tiles, 3 = persistent kernel with 256-column tiles where the batch allows,
// 4 = CTA-pair kernel where the shape allows; default 0 = chosen per problem by pick_kernel().
int variant() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("SNN_LINEAR_LIF_VARIANT");
        v = (e != nullptr && e[0] >= '1' && e[0] <= '4') ? e[0] - '0' : 0;
    }
    return v;
}

// Which persistent kernel: narrow (128 x 128 tiles), wide (128 x 256) or pair (256 x 256 per CTA
// pair). A wide tile costs about as much mainloop time as ONE narrow tile but halves the tile
// count, so compare the rounds of tiles each choice needs on this device. The pair kernel takes
// over once every CTA gets two or more wide tiles: its set-up cost is amortised and the operand
// traffic it saves is what the wide kernel then waits for.
// Step count of the tile that holds a tensor of T steps: the kernels are compiled for 2, 4, 8 and
// 16; other T (the reference's default is 6) run in the next larger tile with the missing steps
// zero-filled, at T / tile of the tensor-core efficiency.
int tile_steps(int64_t T) { return T <= 2 ? 2 : (T <= 4 ? 4 : (T <= 8 ? 8 : 16)); }
// the one-tile-per-CTA kernel exists for full tiles of 4 and 8 steps only
bool one_tile_kernel_covers(int64_t T) { return T == 4 || T == 8; }

template <typename F>
int with_tile_steps(int steps, F&& f) {
    switch (steps) {
        case 2: return f(std::integral_constant<int, 2>{});
        case 4: return f(std::integral_constant<int, 4>{});
        case 8: return f(std::integral_constant<int, 8>{});
        default: return f(std::integral_constant<int, 16>{});
    }
}

enum Kernel { kNarrow = 0, kWide = 1, kPair = 2 };
// T here is the tile's step count
Kernel plan_kernel(int T, int B, int M, int sms, int forced) {
    const bool wide_ok = B % (256 / T) == 0;
    const bool pair_ok = wide_ok && M % (2 * BM) == 0;
    if (forced == 2 || !wide_ok) return kNarrow;
    if (forced == 3) return kWide;
    if (forced == 4) return pair_ok ? kPair : kWide;
    if (sms <= 0) return kNarrow;
    const long long t128 = static_cast<long long>(M / BM) * (B / (128 / T));
    const long long t256 = t128 / 2;
    const long long rounds128 = (t128 + sms - 1) / sms;
    const long long rounds256 = (t256 + sms - 1) / sms;
    if (pair_ok && t256 >= 2LL * sms) return kPair;
    return 10 * rounds256 < 9 * rounds128 ? kWide : kNarrow;     // a wide round costs ~1.1 narrow rounds
}
Kernel pick_kernel(int tile_t, int B, int M) { return plan_kernel(tile_t, B, M, sm_count(), variant()); }

}  // namespace

extern "C" {

int snn_linear_lif_fwd_supported(int64_t T, int64_t B, int64_t K, int64_t M, int dtype) {
    if (dtype != SNN_BF16) return 0;
    if (T < 2 || T > 16) return 0;
    const int bt = BN / tile_steps(T);       // batch items per 128-column tile
    if (B < 1 || B % bt != 0 || B > 65535LL * bt) return 0;
    if (K < BK || K % BK != 0 || M < BM || M % BM != 0) return 0;
    if (K > INT32_MAX || M > INT32_MAX || B > INT32_MAX) return 0;
    return 1;
}

int snn_linear_lif_fwd_plan(int64_t T, int64_t B, int64_t K, int64_t M, int dtype, int sm_count) {
    if (!snn_linear_lif_fwd_supported(T, B, K, M, dtype) || sm_count < 1) return -1;
    return static_cast<int>(plan_kernel(tile_steps(T), static_cast<int>(B), static_cast<int>(M), sm_count, 0));
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

    const int Tt = tile_steps(T), Ti = static_cast<int>(T);
    const bool bulk_stores_ok = al(spike, 16) && al(current, 16);      // the persistent kernels store by TMA
    if (!bulk_stores_ok && !one_tile_kernel_covers(T)) return SNN_ERR_ALIGN;
    const bool one_tile = !bulk_stores_ok || (variant() == 1 && one_tile_kernel_covers(T));
    const Kernel kernel = one_tile ? kNarrow : pick_kernel(Tt, static_cast<int>(B), static_cast<int>(M));
    const cuuint32_t tile_n = kernel == kNarrow ? 128 : 256;
    // a pair member fetches half of the tile's time steps
    const cuuint32_t box_t = static_cast<cuuint32_t>(kernel == kPair ? Tt / 2 : Tt);
    CUtensorMap mw, mx;
    const cuuint64_t wdims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
    const cuuint64_t wstr[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t wbox[2] = {BK, BM};
    const cuuint64_t xdims[3] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(B), static_cast<cuuint64_t>(T)};
    const cuuint64_t xstr[2] = {static_cast<cuuint64_t>(K) * 2, static_cast<cuuint64_t>(B) * K * 2};
    const cuuint32_t xbox[3] = {BK, tile_n / static_cast<cuuint32_t>(Tt), box_t};
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
    const cuuint32_t obox[3] = {BM, static_cast<cuuint32_t>(32 / Tt), static_cast<cuuint32_t>(Tt)};   // one epilogue unit
    if (!cached_map(&ms, spike, 3, odims, ostr, obox, false) ||
        (current != nullptr && !cached_map(&mc, current, 3, odims, ostr, obox, false))) {
        snn_internal::set_last_cuda_error(static_cast<int>(cudaErrorInvalidValue));
        return SNN_ERR_CUDA;
    }
    if (current == nullptr) mc = ms;
    const int wc = current != nullptr ? 1 : 0;
    return with_tile_steps(Tt, [&](auto steps) {
        constexpr int S = decltype(steps)::value;
        if (kernel == kPair) return launch_pair<S>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, Ti, st);
        if (kernel == kWide) return launch_persistent<S, 256>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, Ti, st);
        return launch_persistent<S, 128>(mw, mx, ms, mc, wc, bias, Bi, Ki, Mi, alpha, thresh, Ti, st);
    });
}

#ifdef SNN_TC_WAIT_TEST
// test build only: K stage (counted over the CTA's whole tile list, >= 3) whose loads every producer skips; -1 = none
int snn_test_skip_stage(int stage) {
    return cudaMemcpyToSymbol(g_tc_test_skip_stage, &stage, sizeof(int)) == cudaSuccess ? SNN_OK : SNN_ERR_CUDA;
}
#endif

int snn_linear_lif_error(int reset) {
    // the forward and the backward kernels keep an error word each; report the forward's first
    const int bwd = snn_internal::linear_lif_bwd_error(reset);
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int));
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return -1; }
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    }
    return v != 0 ? v : bwd;
}

}  // extern "C"
