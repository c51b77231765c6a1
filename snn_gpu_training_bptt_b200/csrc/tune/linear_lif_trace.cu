// Phase timeline of the fused linear + LIF kernels (developer tool, needs a B200 to run).
//
//   python -m snn_gpu_training_bptt_b200.build --trace
//   snn_gpu_training_bptt_b200/csrc/tune/linear_lif_trace [variant 2|3|4] [T B K M]
//
// Compiles ../linear_lif_tcgen05.cu with its cycle-counter stamps switched on, runs the chosen
// kernel variant (2 = 128x128 persistent tiles, 3 = 128x256 tiles, 4 = CTA pair) on a random
// problem (default: T=8, batch 256, 2048 -> 2048) and prints, for a few CTAs, how many cycles the
// set-up, the pipeline fill, each K stage, the epilogue and the last store took.
#define SNN_LINEAR_LIF_TRACE 1
#include "../linear_lif_tcgen05.cu"

#include <stdio.h>
#include <vector>

namespace snn_internal {
void set_last_cuda_error(int e) { fprintf(stderr, "cuda error %d\n", e); }
}

int main(int argc, char** argv) {
    const char* variant = argc > 1 ? argv[1] : "3";
    const int T = argc > 5 ? atoi(argv[2]) : 8, B = argc > 5 ? atoi(argv[3]) : 256;
    const int K = argc > 5 ? atoi(argv[4]) : 2048, M = argc > 5 ? atoi(argv[5]) : 2048;
    setenv("SNN_LINEAR_LIF_VARIANT", variant, 1);
    if (!snn_linear_lif_fwd_supported(T, B, K, M, SNN_BF16)) { fprintf(stderr, "unsupported shape\n"); return 2; }

    std::vector<__nv_bfloat16> hx((size_t)T * B * K), hw((size_t)M * K);
    unsigned st = 12345;
    for (auto& v : hx) { st = st * 1664525u + 1013904223u; v = __float2bfloat16(((st >> 16) % 5) == 0 ? 1.f : 0.f); }
    for (auto& v : hw) { st = st * 1664525u + 1013904223u; v = __float2bfloat16((((st >> 8) & 0xffff) / 65536.f - 0.5f) * 0.1f); }
    __nv_bfloat16 *x, *w, *cur, *spk;
    float* bias;
    cudaMalloc(&x, hx.size() * 2);
    cudaMalloc(&w, hw.size() * 2);
    cudaMalloc(&cur, (size_t)T * B * M * 2);
    cudaMalloc(&spk, (size_t)T * B * M * 2);
    cudaMalloc(&bias, M * 4);
    cudaMemset(bias, 0, M * 4);
    cudaMemcpy(x, hx.data(), hx.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(w, hw.data(), hw.size() * 2, cudaMemcpyHostToDevice);

    for (int i = 0; i < 20; ++i) {
        const int rc = snn_linear_lif_fwd(x, w, bias, cur, spk, T, B, K, M, SNN_BF16, 0.25f, 0.25f, nullptr);
        if (rc) { fprintf(stderr, "launch failed: status %d\n", rc); return 1; }
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaDeviceSynchronize();
    cudaEventRecord(e0);
    for (int i = 0; i < 50; ++i) snn_linear_lif_fwd(x, w, bias, cur, spk, T, B, K, M, SNN_BF16, 0.25f, 0.25f, nullptr);
    cudaEventRecord(e1);
    const cudaError_t e = cudaDeviceSynchronize();
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    printf("variant %s, T=%d B=%d K=%d M=%d: sync %d, kernel error word %d, %.2f us per launch (eager, back to back)\n",
           variant, T, B, K, M, (int)e, snn_linear_lif_error(0), ms * 1000 / 50);

    constexpr int kCtas = 148;
    static long long tr[kCtas][kTraceSlots];
    if (snn_linear_lif_trace_read(&tr[0][0], kCtas) != SNN_OK) return 1;
    const int stages = K / 64 < 40 ? K / 64 : 40;
    for (int b : {0, 1, 2, 64, 126}) {
        const long long t0 = tr[b][45];
        printf("cta %3d: set-up %lld | first operands +%lld | K-stage cadence", b, tr[b][46] - t0, tr[b][0] - tr[b][46]);
        for (int i = 1; i < stages; ++i) printf(" %lld", tr[b][i] - tr[b][i - 1]);
        const long long end = tr[b][44] > tr[b][54] ? tr[b][44] : tr[b][54];
        printf(" | accumulator seen at %lld | epilogue g0 %lld g1 %lld | last store read out %lld %lld | lifetime %lld\n",
               tr[b][42] - t0, tr[b][43] - tr[b][42], tr[b][53] - tr[b][52], tr[b][44] - tr[b][43],
               tr[b][54] - tr[b][53], end - t0);
    }
    printf("(a CTA that is not the leader of a pair issues no MMAs: its stage columns are meaningless;\n"
           " with several tiles per CTA the epilogue figure spans all of them)\n");
    return 0;
}
