"""Fused synaptic linear + LIF forward (tcgen05 GEMM with the recurrence in its epilogue).

Parity: the LIF input currents against an fp32 GEMM of the same bf16 operands (bf16-rounded,
within one bf16 ulp: only the fp32 summation order differs); the spikes against the CPU oracle
run on the kernel's own currents (bit-exact); gradients of the FcFire op against the unfused
fc -> fire composition."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import lif_oracle as orc
from tests.helpers import CONSTS

pytestmark = pytest.mark.gpu
A, TH = CONSTS["alpha"], CONSTS["thresh"]


@pytest.fixture(scope="module")
def capi(built_lib):
    assert torch.cuda.is_available()
    from snn_gpu_training_bptt_b200 import _capi
    _capi.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    return _capi


def make(T, B, K, M, seed):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.rand((T, B, K), generator=gen) < 0.2).to(torch.bfloat16)
    bound = 1.0 / np.sqrt(K)
    w = ((torch.rand((M, K), generator=gen) * 2 - 1) * bound * 3).to(torch.bfloat16)
    b = (torch.rand(M, generator=gen) * 2 - 1) * bound
    return x.cuda(), w.cuda(), b.cuda()


# The last three shapes are large enough for the 256-column tiles (the second of them gives every
# CTA several wide tiles, the third is T=4 with 64 batch items per tile).
SHAPES = [(8, 16, 64, 128), (8, 32, 256, 256), (4, 32, 128, 128), (8, 48, 1024, 384), (4, 64, 512, 128),
          (8, 256, 2048, 2048), (8, 1024, 128, 2048), (4, 1024, 256, 2048),
          # step counts that do not fill a 2 / 4 / 8 / 16-step tile (6 is the reference's default), and 2 / 16
          (6, 64, 256, 256), (6, 256, 1024, 2048), (3, 64, 64, 128), (2, 128, 128, 128), (16, 64, 128, 256),
          (12, 32, 64, 256), (16, 512, 128, 2048), (5, 1024, 64, 2048)]


@pytest.mark.parametrize("shape", SHAPES)
def test_fused_forward_against_reference_gemm_and_oracle(capi, shape):
    T, B, K, M = shape
    x, w, b = make(T, B, K, M, seed=sum(shape))
    assert capi.linear_lif_supported(x, w)
    current, spike = capi.linear_lif_fwd(x, w, b, A, TH)
    torch.cuda.synchronize()
    assert capi.linear_lif_error() == 0
    ref = (x.float().view(T * B, K) @ w.float().t() + b).view(T, B, M)
    ref_h = ref.to(torch.bfloat16).float()
    cur = current.float()
    ulp = torch.maximum(ref.abs(), torch.tensor(2.0 ** -126, device=ref.device)) * 2.0 ** -7
    assert bool(((cur - ref_h).abs() <= ulp).all()), float((cur - ref_h).abs().max())
    assert float((cur != ref_h).float().mean()) < 2e-3          # rounding ties only
    s_ref, _ = orc.c_lif_fwd(cur.cpu().numpy())
    assert np.array_equal(spike.float().cpu().numpy(), s_ref)
    # and without the bias / without the current output
    _, spike2 = capi.linear_lif_fwd(x, w, None, A, TH, want_current=False)
    cur2 = (x.float().view(T * B, K) @ w.float().t()).view(T, B, M).to(torch.bfloat16)
    s_ref2, _ = orc.c_lif_fwd(cur2.float().cpu().numpy())
    assert float((spike2.float().cpu() != torch.from_numpy(s_ref2)).float().mean()) < 2e-3
    assert capi.linear_lif_error() == 0


@pytest.mark.parametrize("variant", ["1", "2", "3", "4"])
def test_each_kernel_variant_passes_the_forward_checks(capi, variant):
    """The library picks a kernel per problem; the environment switch forces the one-tile kernel (1),
    128-column persistent tiles (2), 256-column persistent tiles wherever the batch allows (3) or the
    CTA-pair kernel wherever the shape allows (4). It is read once per process, so each forced variant runs the forward test in a child process."""
    if os.environ.get("SNN_LINEAR_LIF_VARIANT"):
        pytest.skip("already inside a forced-variant run")
    env = dict(os.environ, SNN_LINEAR_LIF_VARIANT=variant)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
                          os.path.join("tests", "test_linear_lif_gpu.py"), "-k", "fused_forward"],
                         cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "%d passed" % len(SHAPES) in out.stdout, out.stdout[-500:]


def test_unsupported_problems_are_reported(capi):
    x, w, b = make(8, 16, 64, 128, seed=1)
    assert not capi.linear_lif_supported(x.float(), w)
    assert not capi.linear_lif_supported(x[:, :15], w)              # B not a multiple of 16
    assert capi.linear_lif_supported(x[:6], w)                      # T = 6 runs in an 8-step tile
    assert not capi.linear_lif_supported(x[:1], w)                  # T = 1
    x17 = torch.cat([x, x, x[:1]])                                  # T = 17
    assert not capi.linear_lif_supported(x17, w)
    with pytest.raises(ValueError):
        capi.linear_lif_fwd(x17, w, b, A, TH)
    L = capi.lib()
    assert L.snn_linear_lif_fwd_supported(8, 16, 64, 128, 1) == 1
    assert L.snn_linear_lif_fwd_supported(8, 16, 96, 128, 1) == 0
    assert L.snn_linear_lif_fwd_supported(8, 16, 64, 192, 1) == 0
    assert L.snn_linear_lif_fwd(None, None, None, None, None, 8, 16, 96, 128, 1, A, TH, None) == 5


@pytest.mark.parametrize("shape,dtype", [((8, 32, 256, 256), torch.bfloat16), ((6, 4, 40, 24), torch.float32),
                                         ((8, 16, 128, 128), torch.bfloat16), ((8, 256, 2048, 2048), torch.bfloat16)])
def test_fc_fire_op_forward_and_backward(capi, shape, dtype):
    """FcFire (fused where supported, library GEMM + LIF kernel otherwise): spikes equal the LIF of
    the op's own current; gradients equal LIF-backward of that current (CPU oracle) pushed through
    the two gradient GEMMs in fp32, within the 16-bit rounding of the GEMM outputs."""
    from snn_gpu_training_bptt_b200 import snnlib, snnlib_func as sf
    T, B, K, M = shape
    x, w, b = make(T, B, K, M, seed=7)
    x = x.to(dtype)
    w = w.float()
    gs = torch.randn((T, B, M), device="cuda").to(dtype)
    leaves = [t.clone().requires_grad_(True) for t in (x, w, b)]
    spikes = sf.fc_fire_func(*leaves)
    spikes.backward(gs)
    fused = capi.linear_lif_supported(x, w)
    assert fused == (dtype == torch.bfloat16)
    if fused:
        current = capi.linear_lif_fwd(x, w, b, A, TH)[0]
        assert capi.linear_lif_error() == 0
    else:
        current = snnlib.fc_fp(x, w, b)
    s_ref, _ = orc.c_lif_fwd(current.float().cpu().numpy())
    assert np.array_equal(spikes.detach().float().cpu().numpy(), s_ref)
    gcur = torch.from_numpy(orc.c_lif_bwd(current.float().cpu().numpy(), gs.float().cpu().numpy())).to(dtype).float().cuda()
    want = {"gx": (gcur.view(T * B, M) @ w).view(T, B, K), "gw": gcur.view(T * B, M).t() @ x.float().view(T * B, K),
            "gb": gcur.sum(dim=(0, 1))}
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-4
    for leaf, name in zip(leaves, ("gx", "gw", "gb")):
        scale = float(want[name].abs().max()) or 1.0
        err = float((leaf.grad.float() - want[name]).abs().max())
        assert err <= tol * scale, (name, err, scale)
