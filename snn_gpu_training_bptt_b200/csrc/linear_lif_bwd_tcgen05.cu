// Backward through time of the fused synaptic linear + LIF layer on the tcgen05 tensor cores.
//
//   dU[t, b, :]   = LIF reverse pass over t of (current, grad_spike)        (fp32 state, bf16 I/O)
//   grad_x[t,b,:] = dU[t, b, :] @ W                                         (bf16 operands, fp32 accumulation)
//   grad_W        = sum over (t, b) of dU[t, b, :]^T x[t, b, :]
//   grad_b        = sum over (t, b) of dU[t, b, :]
//
// In the reference this is fire_bp (snnlib/cuda/snn_kernel_bp.cu:141-168: membrane rebuild +
// fire_bp_kernel :95-139) followed by fc_bp_cuda (:1131-1173): per time step one at::mm for the
// input gradient and one for the weight gradient, accumulated over t, plus at::sum for the bias
// (fire_fc_bp_cuda :1065-1128 is the same pair in the other order). Here:
//
//   1. lif_du_kernel      one pass over current / grad_spike (both bf16, written by the forward
//                         kernel / the layer above): rebuilds u_t in registers, walks time in
//                         reverse, writes dU in bf16 (the GEMM operand) and per-block column sums
//                         of it (fp32 partials of grad_b, fixed summation order).
//   2. bwd_gemm_kernel    ONE persistent launch that walks the tiles of both gradient GEMMs:
//                         D[i, j] = sum_r A(i, r) * B(j, r), 128 x 256 tiles, 64 reduction indices
//                         per pipeline stage, two accumulators in tensor memory so the epilogue
//                         of a tile overlaps the MMAs of the next.
//                           grad_x: i = (t,b), j = k, r = m:  A = dU [TB][M]   (K-major),
//                                                             B = W  [M][K]    (MN-major)
//                           grad_W: i = m, j = k, r = (t,b):  A = dU [TB][M]   (MN-major),
//                                                             B = x  [TB][K]   (MN-major)
//                         MN-major operands are read by the tensor core straight from the
//                         row-major tensors (TMA boxes of 64 reduction rows x 64 elements, see
//                         umma_desc_sw128_mn): no transposed copy of W, x or dU is ever made.
//                         The epilogue converts the accumulator to the output type, stages
//                         128-byte rows in swizzled shared memory (16-byte stores, conflict-free)
//                         and writes them with 2-D TMA stores. The CTA that owns the first tile
//                         of a grad_W row block also adds up that block's bias partials.
//
// Roles per CTA as in the forward kernel: warp 4 = TMA producer (one lane), warp 5 = MMA issuer
// and TMEM owner, warps 0-3 and 6-9 = two epilogue groups that split a tile's columns. All
// mbarrier waits are bounded (~1 s) and report through an error word. Tiles that reach past the
// end of a tensor are handled by TMA itself (loads fill zeros, stores clip).
#include "../../include/snn_b200.h"
#include "lif_kernels.cuh"
#include "tcgen05_common.cuh"

namespace snn_internal {
void set_last_cuda_error(int e);     // defined in lif_capi.cu
int linear_lif_bwd_error(int reset);   // defined below; read by snn_linear_lif_error()
}

namespace {

using namespace snn_tc;

// ---------------------------------------------------------------------------------------------
// 1. dU = LIF reverse pass, bf16 in / bf16 out, plus column sums
// ---------------------------------------------------------------------------------------------
// Block = 128 output neurons (128/VEC threads of VEC consecutive neurons) x RB batch items; every
// thread keeps all T steps of its VEC neurons in registers (same arithmetic as lif_bwd_kernel:
// products and sums rounded one by one). partials[blockIdx.y][m] = sum over the block's batch
// items and all t of the bf16-rounded dU, i.e. exactly what the weight-gradient GEMM sees.
template <int TMAX, int VEC, bool EXACT>
__device__ __forceinline__ void lif_du_body(const __nv_bfloat16* __restrict__ cur,
                                            const __nv_bfloat16* __restrict__ gs,
                                            __nv_bfloat16* __restrict__ du, float* __restrict__ partials,
                                            int T, int B, int M, float alpha, float thresh, float beta,
                                            float interval)
{
    using namespace snn;
    using IO = __nv_bfloat16;
    constexpr int TX = 128 / VEC;          // threads along the neuron axis
    constexpr int RB = 256 / TX;           // batch items per block
    __shared__ float red[RB][128 + 4];

    pdl_launch_dependents();
    pdl_wait();                            // current / grad_spike come from the kernels before this one
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int m = blockIdx.x * 128 + tx * VEC;
    const int b = blockIdx.y * RB + ty;
    float colsum[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) colsum[v] = 0.f;

    if (b < B && m < M) {
        const long long N = static_cast<long long>(B) * M;
        const long long i = static_cast<long long>(b) * M + m;
        Pack<IO, VEC> xin[TMAX], gin[TMAX];
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) xin[t] = ld_stream<IO, VEC>(cur + static_cast<long long>(t) * N + i);
#pragma unroll
        for (int t = 0; t < TMAX; ++t)
            if (EXACT || t < T) gin[t] = ld_stream<IO, VEC>(gs + static_cast<long long>(t) * N + i);

        float u[TMAX][VEC];
        {
            float uu[VEC], gate[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) { uu[v] = 0.f; gate[v] = 1.f; }
#pragma unroll
            for (int t = 0; t < TMAX; ++t) {
                if (EXACT || t < T) {
#pragma unroll
                    for (int v = 0; v < VEC; ++v) {
                        const float leak = mul_rn(mul_rn(alpha, uu[v]), gate[v]);
                        uu[v] = add_rn(leak, Elem<IO>::load(xin[t].v[v]));
                        gate[v] = (uu[v] > thresh) ? 0.f : 1.f;
                        u[t][v] = uu[v];
                    }
                }
            }
        }
        float gu[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) gu[v] = 0.f;
#pragma unroll
        for (int t = TMAX - 1; t >= 0; --t) {
            if (EXACT || t < T) {
                Pack<IO, VEC> out;
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float ut = u[t][v];
                    const float ga = mul_rn(gu[v], alpha);
                    float g = 0.f;
                    if (inside_window(ut, thresh, interval)) g = sub_rn(Elem<IO>::load(gin[t].v[v]), mul_rn(ga, ut));
                    const float keep = (ut <= thresh) ? 1.f : 0.f;
                    gu[v] = add_rn(mul_rn(g, beta), mul_rn(ga, keep));
                    out.v[v] = Elem<IO>::store(gu[v]);
                    colsum[v] += Elem<IO>::load(out.v[v]);
                }
                st_stream<IO, VEC>(du + static_cast<long long>(t) * N + i, out);
            }
        }
    }
    if (partials == nullptr) return;
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[ty][tx * VEC + v] = colsum[v];
    __syncthreads();
    if (threadIdx.x < 128) {
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < RB; ++r) s += red[r][threadIdx.x];
        const int mm = blockIdx.x * 128 + threadIdx.x;
        if (mm < M) partials[static_cast<long long>(blockIdx.y) * M + mm] = s;
    }
}

template <int TMAX, int VEC>
__global__ void __launch_bounds__(256)
lif_du_kernel(const __nv_bfloat16* __restrict__ cur, const __nv_bfloat16* __restrict__ gs,
              __nv_bfloat16* __restrict__ du, float* __restrict__ partials, int T, int B, int M, float alpha,
              float thresh, float beta, float interval)
{
    if (T == TMAX) lif_du_body<TMAX, VEC, true>(cur, gs, du, partials, T, B, M, alpha, thresh, beta, interval);
    else lif_du_body<TMAX, VEC, false>(cur, gs, du, partials, T, B, M, alpha, thresh, beta, interval);
}

constexpr int du_vec(int tmax) { return tmax <= 8 ? 8 : 4; }
constexpr int du_rows_per_block(int tmax) { return 256 / (128 / du_vec(tmax)); }
int du_tmax(int64_t T) { return T <= 2 ? 2 : (T <= 4 ? 4 : (T <= 8 ? 8 : 16)); }

// ---------------------------------------------------------------------------------------------
// 2. the two gradient GEMMs as one persistent kernel
// ---------------------------------------------------------------------------------------------
constexpr int TI = 128;              // tile rows    (i = TMEM lanes)
constexpr int TJ = 256;              // tile columns (j = TMEM columns)
constexpr int BR = 64;               // reduction indices per pipeline stage
constexpr int UMMA_K = 16;
constexpr int GSTAGES = 3;
constexpr int kThreadsG = 320;
constexpr uint32_t kBoxBytes = 64 * 64 * 2;                 // one 64 x 64 bf16 box
constexpr uint32_t kStageA = TI * BR * 2;                   // 16 KB
constexpr uint32_t kStageB = TJ * BR * 2;                   // 32 KB
constexpr uint32_t kTmemColsG = 2 * TJ;                     // two accumulators = all of tensor memory
constexpr uint32_t kUnitBytes = TI * 128;                   // one staged output unit: 128 rows of 128 bytes

struct GemmProblem {
    CUtensorMap map_a;               // A operand (see a_mn)
    CUtensorMap map_b;               // B operand, always MN-major: box {64 j, 64 r, 4 groups of 64 j}
    CUtensorMap map_d;               // output [I][J], boxes {128 bytes of j, 128 i}, 128-byte swizzle
    int a_mn;                        // 1: A is MN-major, box {64 i, 64 r, 2 groups}; 0: K-major, box {64 r, 128 i}
    int out_f32;                     // output element type: 1 fp32 (32 columns per unit), 0 bf16 (64)
    int tiles_i, tiles_j, num_rb;    // tile grid and number of reduction stages
    int tile_begin;                  // first tile of this problem in the kernel's tile list
    int rows;                        // I
    const float* bias_partials;      // [partial_rows][rows] or null
    float* grad_bias;                // [rows] or null
    int partial_rows;
};
struct GemmParams {
    GemmProblem p[2];
    int count;
    int total_tiles;
};

struct __align__(1024) GemmStorage {
    __nv_bfloat16 a[GSTAGES][TI * BR];
    __nv_bfloat16 b[GSTAGES][TJ * BR];
    unsigned char out[2][2][kUnitBytes];         // [epilogue group][double buffer]
    uint64_t full[GSTAGES];
    uint64_t empty[GSTAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    uint32_t epi_ok[2];
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ uint32_t pack_bf16x2(uint32_t lo_bits, uint32_t hi_bits) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(lo_bits), __uint_as_float(hi_bits));
    return *reinterpret_cast<const uint32_t*>(&h);
}

// which problem a tile of the kernel's list belongs to
__device__ __forceinline__ int problem_of(const GemmParams& P, int tile) {
    return (P.count > 1 && tile >= P.p[1].tile_begin) ? 1 : 0;
}

// Epilogue of one accumulator for epilogue group g: the thread owns TMEM lane `row` = output row
// i0 + row. The tile's 256 columns are cut into units of 128 output bytes per row (32 fp32 or 64
// bf16 columns); group g takes units g, g + 2, ... Each unit is staged in one of the group's two
// buffers as rows of 128 bytes whose 16-byte chunks are XOR-swizzled with (row & 7) - the layout
// a 128-byte-swizzle tensor map expects - so the eight lanes that write chunk c of eight
// consecutive rows hit eight different bank groups.
// NBUF staging buffers per group: a TMA store takes ~1000 cycles to read its 16 KB out of shared
// memory, longer than a unit's arithmetic, so with NBUF buffers up to NBUF - 1 stores are in flight
// while the next unit is being staged.
template <bool F32, int NBUF, typename Drained>
__device__ __forceinline__ void gemm_epilogue_tile(unsigned char (&stage)[NBUF][kUnitBytes], int& k, int g, bool elected,
                                                   uint32_t lane_base, int row, const CUtensorMap* map_d, int i0,
                                                   int j0, Drained&& drained)
{
    constexpr int UC = F32 ? 32 : 64;           // columns per unit
    constexpr int PER_GROUP = TJ / UC / 2;
#pragma unroll 1
    for (int u = 0; u < PER_GROUP; ++u) {
        const int q = g + 2 * u;
        const bool stamp = elected && g == 0 && u < 2;
        if (stamp) SNN_TC_STAMP(56 + 4 * u);
        uint32_t r[UC / 32][32];
        tmem_ld32(lane_base + q * UC, r[0]);
        if (!F32) tmem_ld32(lane_base + q * UC + 32, r[UC / 32 - 1]);
        // the registers pass through the wait statement so that no use of them is scheduled ahead of it
        tmem_ld_wait32(r[0]);
        if (!F32) tmem_ld_wait32(r[UC / 32 - 1]);
        if (u + 1 == PER_GROUP) {
            if (stamp) SNN_TC_STAMP(6);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            drained();                          // last TMEM read of this tile done: give the buffer back
            if (stamp) SNN_TC_STAMP(7);
        }
        if (stamp) SNN_TC_STAMP(57 + 4 * u);
        unsigned char* st = stage[k % NBUF];
        uint4* rowp = reinterpret_cast<uint4*>(st + row * 128);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            uint4 v;
            if (F32) {
                v = make_uint4(r[0][4 * c], r[0][4 * c + 1], r[0][4 * c + 2], r[0][4 * c + 3]);
            } else {
                const uint32_t* h = r[c >> 2] + 8 * (c & 3);      // columns 8c .. 8c+7 of the unit
                v = make_uint4(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]), pack_bf16x2(h[4], h[5]),
                               pack_bf16x2(h[6], h[7]));
            }
            rowp[c ^ (row & 7)] = v;
        }
        if (stamp) SNN_TC_STAMP(58 + 4 * u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the next unit goes into the buffer whose store was issued NBUF - 1 units ago: that store
        // must have been read out of shared memory before anybody passes the barrier (the store
        // of this unit is not issued yet, so "all but the latest NBUF - 2" covers it)
        if (elected) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(NBUF - 2) : "memory");
        group_barrier(g);
        if (stamp) SNN_TC_STAMP(59 + 4 * u);
        if (elected) {
            tma_store_2d(map_d, st, j0 + q * UC, i0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            if (stamp && u == 0) SNN_TC_STAMP(48);
        }
        ++k;
    }
}

__global__ void __launch_bounds__(kThreadsG, 1)
bwd_gemm_kernel(const __grid_constant__ GemmParams P)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    GemmStorage& sm = *reinterpret_cast<GemmStorage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) SNN_TC_STAMP(0);
    pdl_launch_dependents();

    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < GSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 256); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int k = 0; k < P.count; ++k) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_b) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_d) : "memory");
        }
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemColsG)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;
    if (threadIdx.x == 0) SNN_TC_STAMP(1);
    pdl_wait();                                 // dU and the bias partials come from the kernel before this one
    if (threadIdx.x == 0) SNN_TC_STAMP(2);

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x) {
                const GemmProblem& pr = P.p[problem_of(P, tile)];
                const int local = tile - pr.tile_begin;
                const int i0 = (local % pr.tiles_i) * TI, j0 = (local / pr.tiles_i) * TJ;
                for (int rb = 0; rb < pr.num_rb; ++rb, ++it) {
                    const int s = it % GSTAGES;
                    const uint32_t parity = ((it / GSTAGES) & 1) ^ 1;      // first pass: slots start empty
                    if (!mbar_wait(&sm.empty[s], parity, kDependentWaitCycles)) { record_error(21); ok = false; break; }
                    mbar_expect_tx(&sm.full[s], kStageA + kStageB);
                    const int r0 = rb * BR;
                    unsigned char* a = reinterpret_cast<unsigned char*>(sm.a[s]);
                    unsigned char* b = reinterpret_cast<unsigned char*>(sm.b[s]);
                    // one TMA operation per operand: an MN-major tile is one 3-D box {64 elements, 64
                    // reduction rows, groups of 64 elements}, which lands as consecutive 8 KB boxes
                    if (pr.a_mn) tma_load_3d(a, &pr.map_a, &sm.full[s], 0, r0, i0 / 64);
                    else tma_load_2d(a, &pr.map_a, &sm.full[s], r0, i0);
                    tma_load_3d(b, &pr.map_b, &sm.full[s], 0, r0, j0 / 64);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < P.total_tiles && ok; tile += gridDim.x, ++local) {
                const GemmProblem& pr = P.p[problem_of(P, tile)];
                const bool a_mn = pr.a_mn != 0;
                const uint32_t idesc = umma_idesc_bf16(TI, TJ, a_mn, true);
                // per 16 reduction indices: a K-major tile advances 32 bytes inside its 128-byte rows,
                // an MN-major tile advances 16 rows of 128 bytes (descriptor address unit = 16 bytes)
                const uint32_t a_step = a_mn ? (16 * 128) >> 4 : 32 >> 4;
                constexpr uint32_t b_step = (16 * 128) >> 4;
                const int buf = local & 1;
                const uint32_t acc_parity = ((local >> 1) & 1) ^ 1;        // first use of a buffer passes
                if (!mbar_wait(&sm.acc_empty[buf], acc_parity, kDependentWaitCycles)) { record_error(24); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * TJ;
                for (int rb = 0; rb < pr.num_rb; ++rb, ++it) {
                    const int s = it % GSTAGES;
                    const uint32_t parity = (it / GSTAGES) & 1;
                    if (!mbar_wait(&sm.full[s], parity)) { record_error(22); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (it < 40) SNN_TC_STAMP(8 + it);
                    const uint64_t da = a_mn ? umma_desc_sw128_mn(sm.a[s], kBoxBytes) : umma_desc_sw128(sm.a[s]);
                    const uint64_t db = umma_desc_sw128_mn(sm.b[s], kBoxBytes);
#pragma unroll
                    for (int k = 0; k < BR / UMMA_K; ++k)
                        umma_bf16(tmem_acc, da + a_step * k, db + b_step * k, idesc, (rb | k) != 0 ? 1u : 0u);
                    umma_commit(&sm.empty[s]);        // stage reusable once these MMAs have read it
                }
                if (ok) umma_commit(&sm.acc_full[buf]);
                if (local < 2) SNN_TC_STAMP(3 + local);
            }
        }
    } else {
        // ------------------------------ epilogue groups (warps 0-3, 6-9) ----------
        const int g = warp >= 6 ? 1 : 0;
        const int quarter = warp & 3;                     // the TMEM lanes this warp may touch
        const int row = quarter * 32 + lane;
        const bool elected = lane == 0 && warp == (g ? 6 : 0);
        int local = 0, staged = 0;
        for (int tile = blockIdx.x; tile < P.total_tiles; tile += gridDim.x, ++local) {
            const GemmProblem& pr = P.p[problem_of(P, tile)];
            const int tl = tile - pr.tile_begin;
            const int i0 = (tl % pr.tiles_i) * TI, j0 = (tl / pr.tiles_i) * TJ;
            // bias gradient of this row block: fixed-order sum of the dU kernel's partials, done
            // by group 0 of the CTA that owns the block's first tile while the MMAs run
            if (g == 0 && j0 == 0 && pr.grad_bias != nullptr && i0 + row < pr.rows) {
                float s = 0.f;
                for (int pz = 0; pz < pr.partial_rows; ++pz)
                    s += pr.bias_partials[static_cast<long long>(pz) * pr.rows + i0 + row];
                pr.grad_bias[i0 + row] = s;
            }
            const int buf = local & 1;
            const uint32_t acc_parity = (local >> 1) & 1;
            if (elected) {
                const bool ok0 = mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);
                if (!ok0) record_error(23);
                sm.epi_ok[g] = ok0 ? 1u : 0u;
            }
            group_barrier(g);
            if (sm.epi_ok[g] == 0u) break;
            mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);     // already complete: returns at once, orders this thread
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (elected && g == 0 && local < 2) SNN_TC_STAMP(50 + 2 * local);

            const uint32_t lane_base = tmem_base + buf * TJ + (static_cast<uint32_t>(quarter * 32) << 16);
            uint64_t* drained_bar = &sm.acc_empty[buf];
            auto drained = [drained_bar] { mbar_arrive(drained_bar); };
            if (pr.out_f32)
                gemm_epilogue_tile<true, 2>(sm.out[g], staged, g, elected, lane_base, row, &pr.map_d, i0, j0, drained);
            else
                gemm_epilogue_tile<false, 2>(sm.out[g], staged, g, elected, lane_base, row, &pr.map_d, i0, j0, drained);
            if (elected && g == 0 && local < 2) SNN_TC_STAMP(51 + 2 * local);
        }
        // shared memory must outlive the reads of the last stores
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (elected && g == 0) SNN_TC_STAMP(5);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsG)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs (the two SMs of a TPC) computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and HALF of the B tile (128 of
// the 256 columns: two 64-column groups), so a CTA pulls 32 KB per stage for the flops that cost
// the single-CTA kernel 48 KB. Measured with cycle stamps at T=8, batch 256, 2048 -> 2048: the pair's
// K stage (four 256 x 256 x 16 MMAs) takes a steady 610-640 cycles whether or not operands are
// waited for - the tensor pipe's own rate for this instruction shape - while the single-CTA
// kernel's stages (590 cycles on a CTA's first tile) stretch to 700-1500 on its second tile, when
// the epilogue's stores compete for L2; with many tiles per CTA the pair is ~20 % faster. Each CTA's tensor
// memory receives its own 128 rows x 256 columns; both CTAs run the epilogue above on their rows.
// Barriers as in the forward pair kernel: both CTAs' TMA loads complete on the LEADER's full
// barrier (armed with the bytes of both), the leader's tcgen05.commit multicasts the stage-free /
// accumulator-full arrivals to both CTAs, the epilogue threads of both CTAs arrive on the leader's
// accumulator-empty barriers. No multicast loads. All waits bounded; the cluster barriers at entry
// and exit are reached unconditionally by every thread of both CTAs.
// ---------------------------------------------------------------------------------------------
constexpr int GPSTAGES = 5;                                  // 5 x 32 KB in flight (4 measured ~12 % slower on a CTA's second tile)
constexpr int kPairOutBufs = 2;                              // output staging buffers per epilogue group
constexpr int PTI = 2 * TI;                                  // tile rows of a pair
constexpr uint32_t kPairStageB = (TJ / 2) * BR * 2;          // 16 KB: this CTA's half of the B tile

struct __align__(1024) GemmPairStorage {
    __nv_bfloat16 a[GPSTAGES][TI * BR];
    __nv_bfloat16 b[GPSTAGES][(TJ / 2) * BR];
    unsigned char out[2][kPairOutBufs][kUnitBytes];
    uint64_t full[GPSTAGES];           // used in the leader
    uint64_t empty[GPSTAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];             // used in the leader: 2 CTAs x 256 epilogue threads arrive
    uint32_t tmem_base;
    uint32_t epi_ok[2];
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsG, 1)
bwd_gemm_pair_kernel(const __grid_constant__ GemmParams P)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    GemmPairStorage& sm = *reinterpret_cast<GemmPairStorage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    if (threadIdx.x == 0) SNN_TC_STAMP(0);
    pdl_launch_dependents();

    if (threadIdx.x == 4 * 32) {
        for (int s = 0; s < GPSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 512); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int k = 0; k < P.count; ++k) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_b) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&P.p[k].map_d) : "memory");
        }
    }
    if (warp == 5) {
        // one warp of each CTA of the pair takes part in the pair-wide allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemColsG)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                         // the peer's barriers are initialised past this point
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sm.tmem_base;
    if (threadIdx.x == 0) SNN_TC_STAMP(1);
    pdl_wait();                                 // dU and the bias partials come from the kernel before this one
    if (threadIdx.x == 0) SNN_TC_STAMP(2);

    if (warp == 4) {
        // ------------------------------ TMA producer (both CTAs) ------------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < P.total_tiles && ok; tile += num_pairs) {
                const GemmProblem& pr = P.p[problem_of(P, tile)];
                const int local = tile - pr.tile_begin;
                const int i0 = (local % pr.tiles_i) * PTI + static_cast<int>(rank) * TI;
                const int j0 = (local / pr.tiles_i) * TJ + static_cast<int>(rank) * (TJ / 2);
                for (int rb = 0; rb < pr.num_rb; ++rb, ++it) {
                    const int s = it % GPSTAGES;
                    const uint32_t parity = ((it / GPSTAGES) & 1) ^ 1;
                    if (!mbar_wait(&sm.empty[s], parity, kDependentWaitCycles)) { record_error(31); ok = false; break; }
                    const uint32_t full_leader = mapa_shared(smem_u32(&sm.full[s]), 0);
                    if (leader) mbar_expect_tx(&sm.full[s], 2 * (kStageA + kPairStageB));
                    const int r0 = rb * BR;
                    if (pr.a_mn) tma_load_3d_pair(sm.a[s], &pr.map_a, full_leader, 0, r0, i0 / 64);
                    else tma_load_2d_pair(sm.a[s], &pr.map_a, full_leader, r0, i0);
                    tma_load_3d_pair(sm.b[s], &pr.map_b, full_leader, 0, r0, j0 / 64);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer (leader CTA only) --------------
        if (lane == 0 && leader) {
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < P.total_tiles && ok; tile += num_pairs, ++local) {
                const GemmProblem& pr = P.p[problem_of(P, tile)];
                const bool a_mn = pr.a_mn != 0;
                const uint32_t idesc = umma_idesc_bf16(PTI, TJ, a_mn, true);
                const uint32_t a_step = a_mn ? (16 * 128) >> 4 : 32 >> 4;
                constexpr uint32_t b_step = (16 * 128) >> 4;
                const int buf = local & 1;
                const uint32_t acc_parity = ((local >> 1) & 1) ^ 1;
                if (!mbar_wait(&sm.acc_empty[buf], acc_parity, kDependentWaitCycles)) { record_error(34); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_acc = tmem_base + buf * TJ;
                for (int rb = 0; rb < pr.num_rb; ++rb, ++it) {
                    const int s = it % GPSTAGES;
                    const uint32_t parity = (it / GPSTAGES) & 1;
                    if (!mbar_wait(&sm.full[s], parity)) { record_error(32); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (it < 40) SNN_TC_STAMP(8 + it);
                    const uint64_t da = a_mn ? umma_desc_sw128_mn(sm.a[s], kBoxBytes) : umma_desc_sw128(sm.a[s]);
                    const uint64_t db = umma_desc_sw128_mn(sm.b[s], kBoxBytes);
#pragma unroll
                    for (int k = 0; k < BR / UMMA_K; ++k)
                        umma_bf16_pair(tmem_acc, da + a_step * k, db + b_step * k, idesc, (rb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(&sm.empty[s]);
                }
                if (ok) umma_commit_pair(&sm.acc_full[buf]);
                if (local < 2) SNN_TC_STAMP(3 + local);
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
        for (int tile = pair; tile < P.total_tiles; tile += num_pairs, ++local) {
            const GemmProblem& pr = P.p[problem_of(P, tile)];
            const int tl = tile - pr.tile_begin;
            const int i0 = (tl % pr.tiles_i) * PTI + static_cast<int>(rank) * TI;
            const int j0 = (tl / pr.tiles_i) * TJ;
            if (g == 0 && j0 == 0 && pr.grad_bias != nullptr && i0 + row < pr.rows) {
                float s = 0.f;
                for (int pz = 0; pz < pr.partial_rows; ++pz)
                    s += pr.bias_partials[static_cast<long long>(pz) * pr.rows + i0 + row];
                pr.grad_bias[i0 + row] = s;
            }
            const int buf = local & 1;
            const uint32_t acc_parity = (local >> 1) & 1;
            if (elected) {
                const bool ok0 = mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);
                if (!ok0) record_error(33);
                sm.epi_ok[g] = ok0 ? 1u : 0u;
            }
            group_barrier(g);
            if (sm.epi_ok[g] == 0u) break;
            mbar_wait(&sm.acc_full[buf], acc_parity, kDependentWaitCycles);     // already complete: orders this thread
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (elected && g == 0 && local < 2) SNN_TC_STAMP(50 + 2 * local);

            const uint32_t lane_base = tmem_base + buf * TJ + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t acc_empty_leader = buf ? acc_empty_leader1 : acc_empty_leader0;
            auto drained = [acc_empty_leader] { mbar_arrive_cluster(acc_empty_leader); };
            if (pr.out_f32)
                gemm_epilogue_tile<true, kPairOutBufs>(sm.out[g], staged, g, elected, lane_base, row, &pr.map_d, i0, j0, drained);
            else
                gemm_epilogue_tile<false, kPairOutBufs>(sm.out[g], staged, g, elected, lane_base, row, &pr.map_d, i0, j0, drained);
            if (elected && g == 0 && local < 2) SNN_TC_STAMP(51 + 2 * local);
        }
        if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (elected && g == 0) SNN_TC_STAMP(5);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                         // nobody touches the peer's memory or TMEM past this point
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsG)
                     : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
    size_t du_bytes, partial_bytes, total;
    int partial_rows;
};
Workspace workspace_layout(int64_t T, int64_t B, int64_t M) {
    Workspace w;
    const int rb = du_rows_per_block(du_tmax(T));
    w.partial_rows = static_cast<int>((B + rb - 1) / rb);
    w.du_bytes = align_up(static_cast<size_t>(T) * B * M * 2, 256);
    w.partial_bytes = align_up(static_cast<size_t>(w.partial_rows) * M * 4, 256);
    w.total = w.du_bytes + w.partial_bytes;
    return w;
}

template <int TMAX>
void launch_du(const void* cur, const void* gs, void* du, float* partials, int T, int B, int M, float alpha,
               float thresh, float beta, float interval, cudaStream_t st) {
    constexpr int VEC = du_vec(TMAX);
    constexpr int RB = du_rows_per_block(TMAX);
    dim3 grid((M + 127) / 128, (B + RB - 1) / RB);
    launch_pdl(lif_du_kernel<TMAX, VEC>, grid, dim3(256), 0, st, static_cast<const __nv_bfloat16*>(cur),
               static_cast<const __nv_bfloat16*>(gs), static_cast<__nv_bfloat16*>(du), partials, T, B, M, alpha, thresh,
               beta, interval);
}

bool map2d(CUtensorMap* out, const void* base, int64_t inner, int64_t outer, uint32_t box_inner, uint32_t box_outer,
           bool f32 = false) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * (f32 ? 4 : 2)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    return cached_map(out, base, 2, dims, strides, box, true, f32);
}

// A row-major [rows][cols] bf16 matrix seen as {64 columns, rows, cols / 64 column groups}: a box
// {64, 64, groups} fetches a 64-row slab of `groups` adjacent 64-column groups and lays it out in
// shared memory group after group, each group 64 rows of 128 bytes - the MN-major operand tile.
bool map_mn(CUtensorMap* out, const void* base, int64_t cols, int64_t rows, uint32_t groups) {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 64)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, 128};
    const cuuint32_t box[3] = {64, 64, groups};
    return cached_map(out, base, 3, dims, strides, box, true, false);
}

// SNN_LINEAR_LIF_BWD_VARIANT: 1 = single-CTA kernel (128 x 256 tiles), 2 = CTA-pair kernel
// (256 x 256 tiles per pair); default 0 = the pair kernel whenever both GEMMs have at least 256
// output rows (no half-empty pair tiles) and the device has SM pairs to run it.
int bwd_variant() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("SNN_LINEAR_LIF_BWD_VARIANT");
        v = (e != nullptr && e[0] >= '1' && e[0] <= '2') ? e[0] - '0' : 0;
    }
    return v;
}
bool use_pair_kernel(int64_t TB, int64_t M, int sms) {
    if (sms < 2) return false;
    if (bwd_variant() == 1) return false;
    if (bwd_variant() == 2) return true;
    return TB >= PTI && M >= PTI;
}

}  // namespace

namespace snn_internal {
int linear_lif_bwd_error(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, snn_tc::g_tc_error, sizeof(int));
    if (e != cudaSuccess) { set_last_cuda_error(static_cast<int>(e)); return -1; }
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(snn_tc::g_tc_error, &zero, sizeof(int));
    }
    return v;
}
}  // namespace snn_internal

extern "C" {

#ifdef SNN_TC_STAMPS
int snn_tc_stamps_read(long long* out, int ctas) {   // stamp builds only
    return cudaMemcpyFromSymbol(out, snn_tc::g_tc_stamps, sizeof(long long) * 64 * ctas) == cudaSuccess ? 0 : 7;
}
#endif

int snn_linear_lif_bwd_supported(int64_t T, int64_t B, int64_t K, int64_t M, int dtype) {
    if (dtype != SNN_BF16) return 0;
    if (T < 1 || T > 16 || B < 1) return 0;
    // TMA: row pitches are multiples of 16 bytes; boxes of 64 elements must fit the tensors
    if (K < 64 || K % 64 != 0 || M < 128 || M % 64 != 0) return 0;
    if (T * B < 128 || T * B > INT32_MAX || K > INT32_MAX || M > INT32_MAX) return 0;
    return 1;
}

int64_t snn_linear_lif_bwd_workspace_bytes(int64_t T, int64_t B, int64_t K, int64_t M, int dtype) {
    if (!snn_linear_lif_bwd_supported(T, B, K, M, dtype)) return -static_cast<int64_t>(SNN_ERR_UNSUPPORTED);
    return static_cast<int64_t>(workspace_layout(T, B, M).total);
}

int snn_linear_lif_bwd(const void* x, const void* weight, const void* current, const void* grad_spike,
                       void* grad_x, void* grad_weight, float* grad_bias, int64_t T, int64_t B, int64_t K,
                       int64_t M, int dtype, int grad_weight_dtype, float alpha, float thresh, float beta,
                       float interval, void* workspace, size_t workspace_bytes, void* stream) {
    if (dtype != SNN_BF16 && dtype != SNN_F32 && dtype != SNN_F16 && dtype != SNN_F64) return SNN_ERR_DTYPE;
    if (grad_weight_dtype != SNN_BF16 && grad_weight_dtype != SNN_F32) return SNN_ERR_DTYPE;
    if (T < 1 || B < 1 || K < 1 || M < 1) return SNN_ERR_SHAPE;
    if (!snn_linear_lif_bwd_supported(T, B, K, M, dtype)) return SNN_ERR_UNSUPPORTED;
    if (!current || !grad_spike) return SNN_ERR_NULL;
    if ((grad_x && !weight) || (grad_weight && !x)) return SNN_ERR_NULL;
    auto al = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; };
    if (!al(x, 16) || !al(weight, 16) || !al(current, 16) || !al(grad_spike, 16) || !al(grad_x, 16) ||
        !al(grad_weight, 16) || !al(grad_bias, 4))
        return SNN_ERR_ALIGN;
    const Workspace ws = workspace_layout(T, B, M);
    if (!workspace || workspace_bytes < ws.total || !al(workspace, 256)) return SNN_ERR_WORKSPACE;
    if (grad_bias != nullptr && grad_weight == nullptr) return SNN_ERR_NULL;   // the bias sum rides on the weight GEMM

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int Ti = static_cast<int>(T), Bi = static_cast<int>(B), Mi = static_cast<int>(M);
    void* du = workspace;
    float* partials = grad_bias != nullptr
        ? reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + ws.du_bytes) : nullptr;
    switch (du_tmax(T)) {
        case 2: launch_du<2>(current, grad_spike, du, partials, Ti, Bi, Mi, alpha, thresh, beta, interval, st); break;
        case 4: launch_du<4>(current, grad_spike, du, partials, Ti, Bi, Mi, alpha, thresh, beta, interval, st); break;
        case 8: launch_du<8>(current, grad_spike, du, partials, Ti, Bi, Mi, alpha, thresh, beta, interval, st); break;
        default: launch_du<16>(current, grad_spike, du, partials, Ti, Bi, Mi, alpha, thresh, beta, interval, st); break;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }

    const int64_t TB = T * B;
    const int sms = sm_count();
    if (sms <= 0) { snn_internal::set_last_cuda_error(static_cast<int>(cudaErrorInvalidDevice)); return SNN_ERR_CUDA; }
    const bool pair = use_pair_kernel(TB, M, sms);
    const int tile_rows = pair ? PTI : TI;
    const uint32_t b_groups = pair ? TJ / 2 / 64 : TJ / 64;     // a pair member fetches half of the tile's columns
    GemmParams P;
    P.count = 0;
    P.total_tiles = 0;
    bool maps_ok = true;
    auto add = [&](GemmProblem& pr, int64_t I, int64_t J, int64_t R) {
        pr.tiles_i = static_cast<int>((I + tile_rows - 1) / tile_rows);
        pr.tiles_j = static_cast<int>((J + TJ - 1) / TJ);
        pr.num_rb = static_cast<int>((R + BR - 1) / BR);
        pr.rows = static_cast<int>(I);
        pr.tile_begin = P.total_tiles;
        P.total_tiles += pr.tiles_i * pr.tiles_j;
        ++P.count;
    };
    // The weight-gradient tiles go first: the last round's epilogue is exposed, and the input
    // gradient writes half as many bytes per tile (bf16 against fp32).
    if (grad_weight != nullptr) {
        // grad_W[m, k] = sum_(t,b) dU[(t,b), m] x[(t,b), k]
        GemmProblem& pr = P.p[P.count];
        const bool f32 = grad_weight_dtype == SNN_F32;
        pr.a_mn = 1;
        pr.out_f32 = f32 ? 1 : 0;
        pr.bias_partials = partials; pr.grad_bias = grad_bias; pr.partial_rows = ws.partial_rows;
        maps_ok = maps_ok && map_mn(&pr.map_a, du, M, TB, TI / 64);          // {64 m, 64 (t,b), 2 groups of m}
        maps_ok = maps_ok && map_mn(&pr.map_b, x, K, TB, b_groups);          // {64 k, 64 (t,b), groups of k}
        maps_ok = maps_ok && map2d(&pr.map_d, grad_weight, K, M, f32 ? 32 : 64, TI, f32);
        add(pr, M, K, TB);
    }
    if (grad_x != nullptr) {
        // grad_x[(t,b), k] = sum_m dU[(t,b), m] W[m, k]
        GemmProblem& pr = P.p[P.count];
        pr.a_mn = 0;
        pr.out_f32 = 0;
        pr.bias_partials = nullptr; pr.grad_bias = nullptr; pr.partial_rows = 0;
        maps_ok = maps_ok && map2d(&pr.map_a, du, M, TB, 64, TI);            // {64 m, 128 (t,b)}
        maps_ok = maps_ok && map_mn(&pr.map_b, weight, K, M, b_groups);      // {64 k, 64 m, groups of k}
        maps_ok = maps_ok && map2d(&pr.map_d, grad_x, K, TB, 64, TI);        // {64 k = 128 bytes, 128 (t,b)}
        add(pr, TB, K, M);
    }
    if (!maps_ok) {
        snn_internal::set_last_cuda_error(static_cast<int>(cudaErrorInvalidValue));
        return SNN_ERR_CUDA;
    }
    if (P.count == 0) return SNN_OK;

    if (pair) {
        static_assert(sizeof(GemmPairStorage) + 1024 <= 227 * 1024, "shared memory budget");
        const size_t smem = sizeof(GemmPairStorage) + 1024;
        e = cudaFuncSetAttribute(bwd_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
        const int pairs = P.total_tiles < sms / 2 ? P.total_tiles : sms / 2;
        e = launch_pdl(bwd_gemm_pair_kernel, dim3(2 * pairs), dim3(kThreadsG), smem, st, P);
    } else {
        static_assert(sizeof(GemmStorage) + 1024 <= 227 * 1024, "shared memory budget");
        const size_t smem = sizeof(GemmStorage) + 1024;
        e = cudaFuncSetAttribute(bwd_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
        const int grid = P.total_tiles < sms ? P.total_tiles : sms;
        e = launch_pdl(bwd_gemm_kernel, dim3(grid), dim3(kThreadsG), smem, st, P);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { snn_internal::set_last_cuda_error(static_cast<int>(e)); return SNN_ERR_CUDA; }
    return SNN_OK;
}

}  // extern "C"
