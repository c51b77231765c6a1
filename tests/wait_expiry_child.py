"""Child process of test_bounded_wait_expires_and_is_reported: loads the test-only build of the
library (waits limited to ~10 ms, a hook that makes the persistent forward kernel's producer skip one
K stage), checks that the kernel returns with the MMA issuer's code, that clearing the error word
brings the kernel back, and prints one JSON line. Runs in its own process so that the CUDA context
of the test session never sees the deliberately starved launch."""
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    os.environ["SNN_LINEAR_LIF_VARIANT"] = "3"              # the single-CTA persistent kernel, never the pair
    from snn_gpu_training_bptt_b200 import build
    L = ctypes.CDLL(build.build_wait_test())
    vp, i64, f32, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int
    L.snn_linear_lif_fwd.argtypes = [vp] * 5 + [i64] * 4 + [ci, f32, f32, vp]
    torch.cuda.set_device(0)
    T, B, K, M = 8, 64, 512, 256                            # 8 K stages per tile: stage 5 exists on every CTA
    gen = torch.Generator().manual_seed(0)
    x = (torch.rand((T, B, K), generator=gen) < 0.2).to(torch.bfloat16).cuda()
    w = (torch.randn((M, K), generator=gen) * 0.05).to(torch.bfloat16).cuda()
    bias = torch.zeros(M).cuda()
    cur, spk = (torch.zeros((T, B, M), dtype=torch.bfloat16, device="cuda") for _ in range(2))
    P = lambda t: ctypes.c_void_p(t.data_ptr())

    def launch():
        rc = L.snn_linear_lif_fwd(P(x), P(w), P(bias), P(cur), P(spk), T, B, K, M, 1, 0.25, 0.25, None)
        torch.cuda.synchronize()
        return rc

    out = {"rc_good_before": launch(), "err_good_before": L.snn_linear_lif_error(1)}
    good = spk.clone()
    assert L.snn_test_skip_stage(5) == 0
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    out["rc_starved"] = L.snn_linear_lif_fwd(P(x), P(w), P(bias), P(cur), P(spk), T, B, K, M, 1, 0.25, 0.25, None)
    t1.record()
    torch.cuda.synchronize()                                # must return: every wait is bounded
    out["starved_ms"] = t0.elapsed_time(t1)
    out["err_starved"] = L.snn_linear_lif_error(0)          # read without clearing
    out["err_still_set"] = L.snn_linear_lif_error(1)        # read and clear
    out["err_after_clear"] = L.snn_linear_lif_error(0)
    assert L.snn_test_skip_stage(-1) == 0
    spk.zero_()
    out["rc_good_after"] = launch()
    out["err_good_after"] = L.snn_linear_lif_error(1)
    out["same_spikes_after"] = bool(torch.equal(spk, good))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
