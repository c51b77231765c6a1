"""GPU parity of the batch-norm family (BN folded into LIF, plain time-major BN, the sync-BN
split) against the CPU oracle and against vectors recorded from the reference's gold modules.

Forward is compared exactly with the oracle (same operation order): ivar, membrane potentials
and spikes bit-equal. Backward sums are accumulated with atomics in a different order than the
oracle's serial loops, so gradients are held to 1e-4 of the gradient's scale (the
gradient bar this library is built to); against the reference's gold modules the bars of tests/test_oracle_bn.py apply."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import lif_oracle as orc
from tests.helpers import CONSTS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
A, TH, BE, IV = CONSTS["alpha"], CONSTS["thresh"], CONSTS["beta"], CONSTS["interval"]
EPS = 1e-5


@pytest.fixture(scope="module")
def bn_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "bn_golden.npz"))


@pytest.fixture(scope="module")
def capi(built_lib):
    assert torch.cuda.is_available()
    from snn_gpu_training_bptt_b200 import _capi
    _capi.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    return _capi


def close(got, want, rtol=1e-4, what=""):
    got = got.detach().float().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    want = want.detach().float().cpu().numpy() if isinstance(want, torch.Tensor) else np.asarray(want)
    scale = float(np.abs(want).max()) or 1.0
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert err.max() <= rtol * scale + 1e-7, f"{what}: max err {err.max():.3e} vs scale {scale:.3e}"


def cu(a):
    return torch.as_tensor(np.ascontiguousarray(a)).cuda()


def make_case(shape, seed, C=None):
    gen = torch.Generator().manual_seed(seed)
    C = C or shape[2]
    x = torch.randn(shape, generator=gen) * 1.3 + 0.2
    g = torch.randn(shape, generator=gen)
    w = 0.5 + torch.rand(C, generator=gen)
    b = 0.3 * torch.randn(C, generator=gen)
    dims = (0, 1) if len(shape) == 3 else (0, 1, 3, 4)
    var, mean = torch.var_mean(x, dim=dims, unbiased=False)
    return x, g, w, b, var, mean


SHAPES = [(6, 2, 8), (6, 2, 8, 8, 8), (8, 3, 5, 7, 3), (4, 4, 16, 1, 1), (1, 2, 3, 2, 2), (12, 2, 6, 5, 5),
          (16, 2, 130), (20, 1, 4, 3, 3), (32, 2, 8, 2, 2), (8, 8, 64, 16, 16),
          # channel runs at least as long as a CTA's span (the one-channel-per-CTA sums kernel), one of
          # them not a multiple of the span, one with more CTAs per channel than batch items
          (8, 3, 5, 32, 32), (4, 2, 3, 24, 24), (6, 1, 4, 40, 40),
          # runs of one neuron with C dividing the CTA span (the fixed-channel sums kernel) and not
          (8, 64, 128), (6, 24, 48)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("fire", [True, False])
def test_forward_and_backward_against_oracle(capi, shape, fire):
    x, g, w, b, var, mean = make_case(shape, seed=sum(shape))
    ivar_ref, out_ref, u_ref = orc.c_bn_lif_fwd(x, w, b, var, mean, EPS, fire=fire)
    ivar, out, u = capi.bn_lif_fwd(x.cuda(), w.cuda(), b.cuda(), var.cuda(), mean.cuda(), EPS, A, TH,
                                   fire=fire, want_mem=True)
    assert np.array_equal(ivar.cpu().numpy(), ivar_ref)
    assert np.array_equal(out.cpu().numpy(), out_ref)
    if fire:
        assert np.array_equal(u.cpu().numpy(), u_ref)
    from snn_gpu_training_bptt_b200 import snnlib
    if fire:
        gx, gw, gb = snnlib.bn_fire_bp(x.cuda(), w.cuda(), b.cuda(), ivar, mean.cuda(), None, g.cuda(), A, TH, BE, IV)
    else:
        gx, gw, gb = snnlib.bn_bp(x.cuda(), w.cuda(), b.cuda(), ivar, mean.cuda(), None, g.cuda())
    gx_ref, gw_ref, gb_ref, _, _ = orc.c_bn_lif_bwd(x, g, w, b, ivar_ref, mean, fire=fire)
    close(gx, gx_ref, what="grad_x"); close(gw, gw_ref, what="grad_weight"); close(gb, gb_ref, what="grad_bias")


def test_backward_time_spike_rebuild(capi):
    x, g, w, b, var, mean = make_case((6, 2, 8, 8, 8), seed=3)
    ivar, _, _ = orc.c_bn_lif_fwd(x, w, b, var, mean, EPS)
    _, s_ref, _ = orc.c_bn_lif_fwd(x, w, b, None, mean, EPS, ivar=ivar)
    _, s, _ = capi.bn_lif_fwd(x.cuda(), w.cuda(), b.cuda(), None, mean.cuda(), 0.0, A, TH, ivar=cu(ivar))
    assert np.array_equal(s.cpu().numpy(), s_ref)


def test_channels_last_and_bf16(capi):
    """Same values whether images are contiguous or channels-last; bf16 I/O keeps fp32 state."""
    from snn_gpu_training_bptt_b200 import snnlib
    x, g, w, b, var, mean = make_case((4, 3, 16, 6, 6), seed=17)
    xd, gd = x.cuda(), g.cuda()
    P = [t.cuda() for t in (w, b, var, mean)]
    ivar, s, _ = capi.bn_lif_fwd(xd, P[0], P[1], P[2], P[3], EPS, A, TH)
    x_cl = xd.view(12, 16, 6, 6).contiguous(memory_format=torch.channels_last).view(4, 3, 16, 6, 6)
    g_cl = gd.view(12, 16, 6, 6).contiguous(memory_format=torch.channels_last).view(4, 3, 16, 6, 6)
    ivar2, s2, _ = capi.bn_lif_fwd(x_cl, P[0], P[1], P[2], P[3], EPS, A, TH)
    assert s2.stride() == x_cl.stride() and torch.equal(s2, s) and torch.equal(ivar2, ivar)
    ref = snnlib.bn_fire_bp(xd, P[0], P[1], ivar, P[3], None, gd, A, TH, BE, IV)
    got = snnlib.bn_fire_bp(x_cl, P[0], P[1], ivar, P[3], None, g_cl, A, TH, BE, IV)
    for a, c, n in zip(got, ref, ("gx", "gw", "gb")):
        close(a, c, 1e-5, n)
    # bf16: oracle in fp32 on the bf16-rounded inputs
    xb, gb16 = x.bfloat16(), g.bfloat16()
    var_b, mean_b = torch.var_mean(xb.float(), dim=(0, 1, 3, 4), unbiased=False)
    ivar_ref, s_ref, u_ref = orc.c_bn_lif_fwd(xb.float(), w, b, var_b, mean_b, EPS)
    ivar_b, s_b, u_b = capi.bn_lif_fwd(xb.cuda(), P[0], P[1], var_b.cuda(), mean_b.cuda(), EPS, A, TH, want_mem=True)
    assert s_b.dtype == torch.bfloat16 and np.array_equal(u_b.cpu().numpy(), u_ref)
    assert np.array_equal(s_b.float().cpu().numpy(), s_ref)
    gx_ref, gw_ref, gb_ref, _, _ = orc.c_bn_lif_bwd(xb.float(), gb16.float(), w, b, ivar_ref, mean_b)
    gx, gw, gbias = snnlib.bn_fire_bp(xb.cuda(), P[0], P[1], ivar_b, mean_b.cuda(), None, gb16.cuda(), A, TH, BE, IV)
    close(gx, gx_ref, 1e-2, "bf16 grad_x"); close(gw, gw_ref, 1e-4, "bf16 grad_w"); close(gbias, gb_ref, 1e-4, "bf16 grad_b")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(8, 2, 6, 32, 32), (16, 2, 4, 32, 48), (8, 32, 256)])
def test_sums_kernels_for_long_and_short_runs_in_16_bit(capi, dtype, shape):
    """The per-channel sums of the 16-bit backward on the layouts that take the fat-CTA kernels
    (long runs: 4 neurons per thread; [T, B, C]: fixed channels per thread) against the oracle run
    in fp32 on the rounded inputs."""
    from snn_gpu_training_bptt_b200 import snnlib
    x, g, w, b, _, _ = make_case(shape, seed=sum(shape) + 5)
    x16, g16 = x.to(dtype), g.to(dtype)
    dims = (0, 1) if len(shape) == 3 else (0, 1, 3, 4)
    var, mean = torch.var_mean(x16.float(), dim=dims, unbiased=False)
    ivar_ref, _, _ = orc.c_bn_lif_fwd(x16.float(), w, b, var, mean, EPS)
    gx_ref, gw_ref, gb_ref, _, _ = orc.c_bn_lif_bwd(x16.float(), g16.float(), w, b, ivar_ref, mean)
    ivar = torch.from_numpy(np.asarray(ivar_ref)).cuda()
    gx, gw, gb = snnlib.bn_fire_bp(x16.cuda(), w.cuda(), b.cuda(), ivar, mean.cuda(), None, g16.cuda(), A, TH, BE, IV)
    close(gw, gw_ref, 1e-4, "grad_w"); close(gb, gb_ref, 1e-4, "grad_b"); close(gx, gx_ref, 1e-2, "grad_x")


def test_sync_bn_split_matches_one_shot(capi):
    """dist1 on two half-batches + averaging (the all-reduce) + dist2 == the one-shot backward."""
    from snn_gpu_training_bptt_b200 import snnlib
    x, g, w, b, var, mean = make_case((6, 4, 8, 5, 5), seed=23)
    xd, gd = x.cuda(), g.cuda()
    P = [t.cuda() for t in (w, b, var, mean)]
    ivar = snnlib.bn_fire_s_fp(xd, P[0], P[1], P[2], P[3], EPS, A, TH)[0]
    gx, gw, gb = snnlib.bn_fire_bp(xd, P[0], P[1], ivar, P[3], (0, 1, 3, 4), gd, A, TH, BE, IV)
    parts = [snnlib.bn_fire_bp_dist1(xd[:, i:i + 2].contiguous(), P[0], P[1], ivar, P[3], (0, 1, 3, 4),
                                     gd[:, i:i + 2].contiguous(), A, TH, BE, IV) for i in (0, 2)]
    gxhat = (parts[0][0] + parts[1][0]) / 2
    gxhatx = (parts[0][1] + parts[1][1]) / 2
    close(parts[0][2] + parts[1][2], gw, 1e-5); close(parts[0][3] + parts[1][3], gb, 1e-5)
    gx_split = torch.cat([snnlib.bn_fire_bp_dist2(xd[:, i:i + 2].contiguous(), P[0], P[1], ivar, P[3],
                                                  gd[:, i:i + 2].contiguous(), gxhat, gxhatx, A, TH, BE, IV)
                          for i in (0, 2)], dim=1)
    close(gx_split, gx, 1e-5, "split grad_x")
    # plain BN split
    gxp, gwp, gbp = snnlib.bn_bp(xd, P[0], P[1], ivar, P[3], (0, 1, 3, 4), gd)
    pp = [snnlib.bn_bp_dist1(xd[:, i:i + 2].contiguous(), P[0], P[1], ivar, P[3], (0, 1, 3, 4), gd[:, i:i + 2].contiguous())
          for i in (0, 2)]
    gxp2 = torch.cat([snnlib.bn_bp_dist2(xd[:, i:i + 2].contiguous(), P[0], P[1], ivar, P[3], (0, 1, 3, 4),
                                         gd[:, i:i + 2].contiguous(), (pp[0][0] + pp[1][0]) / 2, (pp[0][1] + pp[1][1]) / 2)
                      for i in (0, 2)], dim=1)
    close(gxp2, gxp, 1e-5, "plain split grad_x")


# ---- modules against the reference's gold vectors ---------------------------------------------
def _set_bn(mod, g, k):
    mod.weight_bn.data.copy_(cu(g[k + "_w"]))
    mod.bias_bn.data.copy_(cu(g[k + "_b"]))


@pytest.mark.parametrize("kind", ["fc", "conv"])
def test_bn_and_bn_fire_modules_against_gold(capi, bn_golden, kind):
    from snn_gpu_training_bptt_b200 import snnlib_op as sop
    g = bn_golden
    dim = (0, 1) if kind == "fc" else (0, 1, 3, 4)
    k = f"bn_{kind}"
    mod = sop.Bn(8, dim).cuda()
    _set_bn(mod, g, k)
    x = cu(g[k + "_x"]).requires_grad_(True)
    y = mod(x)
    y.backward(cu(g[k + "_gy"]))
    close(y, g[k + "_y"], 1e-5, "bn y"); close(x.grad, g[k + "_gx"], what="bn gx")
    close(mod.weight_bn.grad, g[k + "_gw"], what="bn gw"); close(mod.bias_bn.grad, g[k + "_gb"], what="bn gb")
    # running statistics: momentum 0.1 with the unbiased correction, as nn.BatchNorm tracks them
    n = g[k + "_x"].size / 8
    close(mod.running_mean, 0.1 * g[k + "_mean"], 1e-5); close(mod.running_var, 0.9 + 0.1 * g[k + "_var"] * n / (n - 1), 1e-5)

    k = f"bnfire_{kind}"
    mod = sop.BnFire(8, dim).cuda()
    _set_bn(mod, g, k)
    x = cu(g[k + "_x"]).requires_grad_(True)
    s = mod(x)
    s.backward(cu(g[k + "_g"]))
    assert np.array_equal(s.detach().cpu().numpy(), g[k + "_s"])
    close(x.grad, g[k + "_gx"], what="bnfire gx"); close(mod.weight_bn.grad, g[k + "_gw"], what="bnfire gw")
    close(mod.bias_bn.grad, g[k + "_gb"], what="bnfire gb")
    # evaluation mode uses the running statistics
    mod.train_bn = False
    assert mod(x.detach()).shape == s.shape


@pytest.mark.parametrize("key", ["bnfirefc_fc", "bnfirefc_conv", "bnfireconv_conv"])
def test_fused_compositions_against_gold(capi, bn_golden, key):
    from snn_gpu_training_bptt_b200 import snnlib_op as sop
    g = bn_golden
    if key == "bnfirefc_fc":
        mod = sop.BnFireFc(8, 8, (0, 1)).cuda()
    elif key == "bnfirefc_conv":
        mod = sop.BnFireFc(512, 8, (0, 1, 3, 4), cin_bn=8).cuda()
    else:
        mod = sop.BnFireConv(8, 8).cuda()
    _set_bn(mod, g, key)
    wname, bname = ("weight_conv", "bias_conv") if key == "bnfireconv_conv" else ("weight_fc", "bias_fc")
    getattr(mod, wname).data.copy_(cu(g[key + "_lw"]))
    getattr(mod, bname).data.copy_(cu(g[key + "_lb"]))
    x = cu(g[key + "_x"]).requires_grad_(True)
    y = mod(x)
    y.backward(cu(g[key + "_gy"]))
    close(y, g[key + "_y"], 1e-4, "y"); close(x.grad, g[key + "_gx"], what="gx")
    close(mod.weight_bn.grad, g[key + "_gw"], what="gw_bn"); close(mod.bias_bn.grad, g[key + "_gb"], what="gb_bn")
    close(getattr(mod, wname).grad, g[key + "_glw"], what="gw_lin"); close(getattr(mod, bname).grad, g[key + "_glb"], what="gb_lin")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bn_modules_run_in_16_bit_with_fp32_statistics(capi, dtype):
    """Bn, BnFire, BnFireFc and BnFireConv on 16-bit activations (the trainer's precision): the
    statistics the modules compute are fp32 and equal an fp32 computation on the same values, the
    outputs equal the C ABI fed those statistics, the running statistics stay fp32, and backward
    produces finite gradients of the right types."""
    from snn_gpu_training_bptt_b200 import snnlib_op as sop
    gen = torch.Generator().manual_seed(17)
    x5 = (torch.randn((6, 4, 8, 6, 6), generator=gen) * 1.2 + 0.1).to(dtype).cuda()
    x3 = (torch.randn((6, 16, 8), generator=gen) * 1.2 + 0.1).to(dtype).cuda()
    for mod, x in ((sop.BnFire(8, (0, 1, 3, 4)), x5), (sop.Bn(8, (0, 1)), x3), (sop.BnFire(8, (0, 1)), x3),
                   (sop.BnFireConv(8, 16), x5), (sop.BnFireFc(8, 5, (0, 1)), x3)):
        mod = mod.cuda()
        var, mean = mod._statistics(x)
        assert var.dtype == mean.dtype == torch.float32
        v32, m32 = torch.var_mean(x.float(), dim=mod.dim_bn, unbiased=False)
        close(mean, m32, 1e-5, "mean"); close(var, v32, 1e-4, "var")
        xi = x.clone().requires_grad_(True)
        y = mod(xi)
        assert y.dtype == dtype and mod.running_var.dtype == torch.float32
        y.backward(torch.randn(y.shape, device="cuda").to(dtype))
        assert xi.grad.dtype == dtype and torch.isfinite(xi.grad.float()).all()
        assert mod.weight_bn.grad.dtype == torch.float32 and torch.isfinite(mod.weight_bn.grad).all()
        if isinstance(mod, sop.BnFire):
            # spikes equal the kernel's own output for the same fp32 statistics
            _, want, _ = capi.bn_lif_fwd(x, mod.weight_bn.detach(), mod.bias_bn.detach(), var, mean, mod.eps_bn, A, TH)
            assert torch.equal(y.detach(), want)


def test_bn_argument_errors(capi):
    x = torch.zeros(4, 2, 8, 3, 3, device="cuda")
    w = torch.ones(8, device="cuda")
    with pytest.raises(TypeError):
        capi.bn_lif_fwd(x, torch.ones(7, device="cuda"), w, w, w, EPS, A, TH)
    with pytest.raises(TypeError):
        capi.bn_lif_fwd(x.double(), w, w, w, w, EPS, A, TH)
    big_t = torch.zeros(40, 1, 8, device="cuda")
    with pytest.raises(capi.SnnError):
        capi.bn_lif_bwd_sums(big_t, big_t, w, w, w, w, A, TH, BE, IV)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_sync_bn_layers_over_nccl(tmp_path):
    """BnFireConvDist / BnFireFcDist / BnDist on 2 ranks (half batch each) == the single-GPU
    layers on the whole batch: outputs, input gradients, parameter gradients summed over ranks."""
    script = os.path.join(ROOT, "tests", "syncbn_nccl_child.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), script, str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    single = torch.load(str(tmp_path / "single.pt"))
    ranks = [torch.load(str(tmp_path / f"rank{r}.pt")) for r in range(2)]
    # bf16 activations through the sync-BN conv layer: fp32 statistics identical on both ranks, output
    # and input gradient near the fp32 run (bf16 rounding of activations and of the convolution)
    assert ranks[0]["bf16_running_var"].dtype == torch.float32
    assert torch.equal(ranks[0]["bf16_running_var"], ranks[1]["bf16_running_var"])
    y16 = torch.cat([ranks[0]["bf16_y_conv"], ranks[1]["bf16_y_conv"]], dim=1)
    assert torch.isfinite(y16).all()
    rel = float((y16 - single["y_conv"]).norm() / single["y_conv"].norm())
    assert rel < 0.2, rel
    for name in single:
        if name.startswith(("y_", "gx_")):
            both = torch.cat([ranks[0][name], ranks[1][name]], dim=1)
            close(both, single[name], 2e-4, name)
        else:   # parameter gradients: each rank holds its local sum
            close(ranks[0][name] + ranks[1][name], single[name], 2e-4, name)
