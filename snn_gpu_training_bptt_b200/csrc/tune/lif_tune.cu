// Launch-configuration tuner for the LIF kernels (not part of libsnn_b200.so).
//
//   python -m snn_gpu_training_bptt_b200.build --tuner [--cache-policy 0|1|2]
//   snn_gpu_training_bptt_b200/csrc/tune/lif_tune T log2N reps [bulk=1]
//
// Times lif_fwd_kernel / lif_bwd_kernel of ../lif_kernels.cuh for fp32 and bf16 over vector
// widths, unroll bounds and block sizes (CUDA events, median and best of `reps`), beside a
// device-to-device cudaMemcpyAsync and, with bulk=1 at T=8, the cp.async.bulk staging variant
// of lif_bulk_variant.cuh. Every variant's output is compared with a scalar launch of the same
// kernel ("bad" = mismatching elements). The tables chosen in ../lif_capi.cu came from this.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include "../lif_kernels.cuh"
#include "lif_bulk_variant.cuh"

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); exit(1);} } while (0)
using bf16 = __nv_bfloat16;
static float *X, *G, *S, *GX, *REF_S, *REF_GX;
static bf16 *Xh, *Gh, *Sh, *GXh, *REF_Sh, *REF_GXh;
static int64_t N; static int T; static int reps; static int* d_err;

__global__ void fill_kernel(float* p, bf16* ph, int64_t n, uint32_t seed, float mean) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        uint64_t z = (uint64_t)i * 0x9E3779B97F4A7C15ull + seed;
        z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 27; z *= 0x94D049BB133111EBull; z ^= z >> 31;
        float a = ((z & 0xFFFF) + ((z >> 16) & 0xFFFF) + ((z >> 32) & 0xFFFF) + ((z >> 48) & 0xFFFF)) / 65536.0f - 2.0f;
        float v = mean + a * 1.7320508f;
        p[i] = v; ph[i] = __float2bfloat16_rn(v);
    }
}
template <typename E>
__global__ void diff_kernel(const E* a, const E* b, int64_t n, unsigned long long* cnt) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    unsigned long long c = 0;
    for (; i < n; i += stride) c += ((float)a[i] != (float)b[i]);
    if (c) atomicAdd(cnt, c);
}
template <typename E>
static unsigned long long ndiff(const E* a, const E* b) {
    static unsigned long long* d = nullptr;
    if (!d) CK(cudaMalloc(&d, 8));
    CK(cudaMemset(d, 0, 8));
    diff_kernel<E><<<1480, 256>>>(a, b, (int64_t)T * N, d);
    unsigned long long h; CK(cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost));
    return h;
}
template <typename E, typename F>
static void timeit(const char* name, double bytes, F launch, E* out, const E* ref) {
    CK(cudaMemset((void*)out, 0xFF, (size_t)T * N * sizeof(E)));
    launch();
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) { printf("%-52s SKIPPED (%s)\n", name, cudaGetErrorString(le)); return; }
    CK(cudaDeviceSynchronize());
    unsigned long long bad = ref ? ndiff<E>(out, ref) : 0;
    int herr = 0; CK(cudaMemcpy(&herr, d_err, 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < 3; ++i) launch();
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    std::vector<float> ms(reps);
    for (int i = 0; i < reps; ++i) {
        CK(cudaEventRecord(e0)); launch(); CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1));
        CK(cudaEventElapsedTime(&ms[i], e0, e1));
    }
    std::sort(ms.begin(), ms.end());
    float med = ms[reps / 2], best = ms[0];
    printf("%-52s med %8.4f ms %8.1f GB/s | best %8.1f GB/s | bad %llu err %d\n", name, med, bytes / med / 1e6, bytes / best / 1e6, bad, herr);
    fflush(stdout);
}
template <typename E> struct Buf;
template <> struct Buf<float> { static float* x() { return X; } static float* g() { return G; } static float* s() { return S; } static float* gx() { return GX; } static float* rs() { return REF_S; } static float* rgx() { return REF_GX; } static const char* nm() { return "f32"; } };
template <> struct Buf<bf16> { static bf16* x() { return Xh; } static bf16* g() { return Gh; } static bf16* s() { return Sh; } static bf16* gx() { return GXh; } static bf16* rs() { return REF_Sh; } static bf16* rgx() { return REF_GXh; } static const char* nm() { return "bf16"; } };

template <typename E, int VEC, int TC>
static void fwd_variant(int block) {
    char name[96]; snprintf(name, 96, "fwd %s VEC%d TC%d block%d", Buf<E>::nm(), VEC, TC, block);
    int64_t threads = N / VEC; unsigned grid = (unsigned)((threads + block - 1) / block);
    timeit<E>(name, 2.0 * sizeof(E) * T * N, [&] { snn::lif_fwd_kernel<E, VEC, TC><<<grid, block>>>(Buf<E>::x(), Buf<E>::s(), nullptr, nullptr, 0, T, N, 0.25f, 0.25f); }, Buf<E>::s(), Buf<E>::rs());
}
template <typename E, int VEC, int TMAX>
static void bwd_variant(int block) {
    if (T > TMAX) return;
    char name[96]; snprintf(name, 96, "bwd %s VEC%d TMAX%d block%d", Buf<E>::nm(), VEC, TMAX, block);
    int64_t threads = N / VEC; unsigned grid = (unsigned)((threads + block - 1) / block);
    timeit<E>(name, 3.0 * sizeof(E) * T * N, [&] { snn::lif_bwd_kernel<E, VEC, TMAX><<<grid, block>>>(Buf<E>::x(), Buf<E>::g(), Buf<E>::gx(), T, N, 0.25f, 0.25f, 1.0f, 0.5f); }, Buf<E>::gx(), Buf<E>::rgx());
}
template <int TT, int THREADS, int STAGES, bool BWD>
static void tma_variant(int cap) {
    if (T != TT) return;
    auto kern = snn_tma::lif_tma_kernel<TT, THREADS, STAGES, BWD>;
    size_t smem = snn_tma::lif_tma_smem<TT, THREADS, STAGES, BWD>();
    if (smem > 227 * 1024) return;
    CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0; CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, THREADS, smem));
    if (occ < 1) return;
    occ = std::min(occ, cap);
    int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    unsigned grid = sms * occ;
    char name[96]; snprintf(name, 96, "%s tma T%d thr%d stages%d ctas/sm%d smem%zuK", BWD ? "bwd" : "fwd", TT, THREADS, STAGES, occ, smem / 1024);
    timeit<float>(name, (BWD ? 12.0 : 8.0) * T * N, [&] { kern<<<grid, THREADS, smem>>>(X, G, BWD ? GX : S, N, 0.25f, 0.25f, 1.0f, 0.5f, d_err); }, BWD ? GX : S, BWD ? REF_GX : REF_S);
}
template <typename E, int TMAX>
static void ref_bwd() {
    snn::lif_bwd_kernel<E, 1, TMAX><<<(unsigned)((N + 255) / 256), 256>>>(Buf<E>::x(), Buf<E>::g(), Buf<E>::rgx(), T, N, 0.25f, 0.25f, 1.0f, 0.5f);
}

int main(int argc, char** argv) {
    T = argc > 1 ? atoi(argv[1]) : 8;
    int lg = argc > 2 ? atoi(argv[2]) : 26;
    reps = argc > 3 ? atoi(argv[3]) : 20;
    int do_tma = argc > 4 ? atoi(argv[4]) : 1;
    N = 1ll << lg;
    size_t bytes = (size_t)T * N * 4;
    for (float** p : {&X, &G, &S, &GX, &REF_S, &REF_GX}) CK(cudaMalloc(p, bytes));
    for (bf16** p : {&Xh, &Gh, &Sh, &GXh, &REF_Sh, &REF_GXh}) CK(cudaMalloc(p, bytes / 2));
    CK(cudaMalloc(&d_err, 4)); CK(cudaMemset(d_err, 0, 4));
    fill_kernel<<<2960, 256>>>(X, Xh, (int64_t)T * N, 1, 0.5f);
    fill_kernel<<<2960, 256>>>(G, Gh, (int64_t)T * N, 2, 0.0f);
    snn::lif_fwd_kernel<float, 1, 8><<<(unsigned)((N + 255) / 256), 256>>>(X, REF_S, nullptr, nullptr, 0, T, N, 0.25f, 0.25f);
    snn::lif_fwd_kernel<bf16, 1, 8><<<(unsigned)((N + 255) / 256), 256>>>(Xh, REF_Sh, nullptr, nullptr, 0, T, N, 0.25f, 0.25f);
    ref_bwd<float, 32>(); ref_bwd<bf16, 32>();
    CK(cudaDeviceSynchronize());
    printf("# T=%d N=2^%d reps=%d policy=%d\n", T, lg, reps, SNN_CACHE_POLICY);
    timeit<float>("memcpyD2D (1R+1W)", 2.0 * bytes, [&] { cudaMemcpyAsync(S, X, bytes, cudaMemcpyDeviceToDevice); }, S, nullptr);

    for (int block : {128, 256}) {
        fwd_variant<float, 4, 4>(block); fwd_variant<float, 4, 6>(block); fwd_variant<float, 4, 8>(block); fwd_variant<float, 4, 16>(block);
        fwd_variant<float, 2, 4>(block); fwd_variant<float, 2, 6>(block); fwd_variant<float, 2, 8>(block); fwd_variant<float, 2, 16>(block);
    }
    for (int block : {128, 256}) {
        bwd_variant<float, 4, 2>(block); bwd_variant<float, 4, 4>(block); bwd_variant<float, 2, 4>(block);
        bwd_variant<float, 4, 6>(block); bwd_variant<float, 2, 6>(block);
        bwd_variant<float, 4, 8>(block); bwd_variant<float, 2, 8>(block);
        bwd_variant<float, 4, 12>(block); bwd_variant<float, 2, 12>(block);
        bwd_variant<float, 4, 16>(block); bwd_variant<float, 2, 16>(block);
        bwd_variant<float, 2, 24>(block); bwd_variant<float, 1, 24>(block);
        bwd_variant<float, 2, 32>(block); bwd_variant<float, 1, 32>(block);
    }
    for (int block : {128, 256}) {
        fwd_variant<bf16, 8, 4>(block); fwd_variant<bf16, 8, 8>(block); fwd_variant<bf16, 8, 16>(block);
        fwd_variant<bf16, 4, 4>(block); fwd_variant<bf16, 4, 8>(block); fwd_variant<bf16, 4, 16>(block);
        bwd_variant<bf16, 8, 4>(block); bwd_variant<bf16, 4, 4>(block);
        bwd_variant<bf16, 8, 8>(block); bwd_variant<bf16, 4, 8>(block); bwd_variant<bf16, 2, 8>(block);
        bwd_variant<bf16, 8, 16>(block); bwd_variant<bf16, 4, 16>(block); bwd_variant<bf16, 2, 16>(block);
        bwd_variant<bf16, 4, 32>(block); bwd_variant<bf16, 2, 32>(block);
    }
    if (do_tma) {
        tma_variant<8, 256, 3, false>(8); tma_variant<8, 256, 2, false>(8); tma_variant<8, 128, 4, false>(8);
        tma_variant<8, 128, 3, false>(8); tma_variant<8, 128, 2, false>(8); tma_variant<8, 64, 4, false>(8);
        tma_variant<8, 256, 2, true>(8); tma_variant<8, 128, 3, true>(8); tma_variant<8, 128, 2, true>(8);
        tma_variant<8, 64, 4, true>(8); tma_variant<8, 64, 3, true>(8); tma_variant<8, 64, 2, true>(8);
    }
    return 0;
}
