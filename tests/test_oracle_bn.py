"""The batch-norm half of the CPU oracle against golden vectors recorded from the reference's
gold modules (gold_op.Bn / BnFire / BnFireFc / BnFireConv in training mode).

The gold modules normalise with torch's batch-norm, the reference kernels (which the oracle
restates) with (x - mean) * (weight / sqrt(var + eps)) + bias, so agreement is to rounding,
not bitwise: membrane potentials within 1e-5 relative, spikes identical (the vectors were chosen
with no potential within 1e-4 of the threshold), gradients within 1e-4 relative of the
gradient's scale."""
import numpy as np
import pytest
import torch

from oracle import lif_oracle as orc

EPS = 1e-5


@pytest.fixture(scope="module")
def bn_golden():
    import os
    return np.load(os.path.join(os.path.dirname(__file__), "golden", "bn_golden.npz"))


def close(got, want, rtol=1e-4):
    scale = float(np.abs(want).max()) or 1.0
    err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    assert err.max() <= rtol * scale + 1e-7, f"max err {err.max():.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("kind", ["fc", "conv"])
def test_plain_bn(bn_golden, kind):
    g, k = bn_golden, f"bn_{kind}"
    ivar, y, _ = orc.c_bn_lif_fwd(g[k + "_x"], g[k + "_w"], g[k + "_b"], g[k + "_var"], g[k + "_mean"], EPS, fire=False)
    close(y, g[k + "_y"], 1e-5)
    close(ivar, 1.0 / np.sqrt(g[k + "_var"] + EPS), 1e-6)
    gx, gw, gb, _, _ = orc.c_bn_lif_bwd(g[k + "_x"], g[k + "_gy"], g[k + "_w"], g[k + "_b"], ivar, g[k + "_mean"], fire=False)
    close(gx, g[k + "_gx"]); close(gw, g[k + "_gw"]); close(gb, g[k + "_gb"])


@pytest.mark.parametrize("kind", ["fc", "conv"])
def test_bn_fire(bn_golden, kind):
    g, k = bn_golden, f"bnfire_{kind}"
    ivar, s, u = orc.c_bn_lif_fwd(g[k + "_x"], g[k + "_w"], g[k + "_b"], g[k + "_var"], g[k + "_mean"], EPS)
    assert np.array_equal(s, g[k + "_s"])
    close(u, g[k + "_u"], 1e-5)
    gx, gw, gb, _, _ = orc.c_bn_lif_bwd(g[k + "_x"], g[k + "_g"], g[k + "_w"], g[k + "_b"], ivar, g[k + "_mean"])
    close(gx, g[k + "_gx"]); close(gw, g[k + "_gw"]); close(gb, g[k + "_gb"])
    # the backward-time rebuild (w' = weight*ivar) gives the same spikes on these vectors
    _, s2, _ = orc.c_bn_lif_fwd(g[k + "_x"], g[k + "_w"], g[k + "_b"], None, g[k + "_mean"], EPS, ivar=ivar)
    assert np.array_equal(s2, s)


def test_sync_bn_split_is_consistent(bn_golden):
    """Feeding the means of the one-shot backward into the 'given means' form reproduces it, and
    means averaged over two half-batches (what the all-reduce produces) equal the full-batch ones."""
    g, k = bn_golden, "bnfire_conv"
    x, gr, w, b = g[k + "_x"], g[k + "_g"], g[k + "_w"], g[k + "_b"]
    ivar, _, _ = orc.c_bn_lif_fwd(x, w, b, g[k + "_var"], g[k + "_mean"], EPS)
    gx, gw, gb, gh, ghx = orc.c_bn_lif_bwd(x, gr, w, b, ivar, g[k + "_mean"])
    gx2, _, _, _, _ = orc.c_bn_lif_bwd(x, gr, w, b, ivar, g[k + "_mean"], means=(gh, ghx))
    assert np.array_equal(gx, gx2)
    halves = [orc.c_bn_lif_bwd(x[:, i:i + 1], gr[:, i:i + 1], w, b, ivar, g[k + "_mean"]) for i in (0, 1)]
    close((halves[0][3] + halves[1][3]) / 2, gh, 1e-5)
    close((halves[0][4] + halves[1][4]) / 2, ghx, 1e-5)
    close(halves[0][1] + halves[1][1], gw, 1e-5)
    gx_split = np.concatenate([orc.c_bn_lif_bwd(x[:, i:i + 1], gr[:, i:i + 1], w, b, ivar, g[k + "_mean"],
                                                means=(gh, ghx))[0] for i in (0, 1)], axis=1)
    close(gx_split, gx, 1e-6)
