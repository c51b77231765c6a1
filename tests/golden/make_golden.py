"""Generate the golden vectors under tests/golden/ from the REFERENCE's own gold ops.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py --ref /path/to/reference

It imports ``snnlib/example/gold_op.py`` of liangling76/snn_gpu_training_bptt (pure PyTorch,
CPU) and records, for seeded inputs, the membrane potentials, spikes and input gradients
that ``gold_fire`` (gold_op.py:34-44, surrogate gold_op.py:17-31) produces, plus the
fire->fc / fc compositions of ``gold_op.BnFireFc`` (gold_op.py:118-150). The reference
ships no stored vectors of its own: its test scripts (snnlib/example/test_fire.py,
test_fire_fc.py, test_fc.py) print differences against these very functions, so their
outputs are what pins parity. The committed ``*.npz`` files travel with the repository;
the reference itself is not needed to run the tests.
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def fire_case(gop, x, g):
    """gold_fire forward, then backward with upstream gradient g applied to the spikes."""
    gop.time_step = x.shape[0]
    xr = x.clone().requires_grad_(True)
    u, s = gop.gold_fire(xr)
    s.backward(g)
    return u.detach().numpy(), s.detach().numpy(), xr.grad.numpy()


def ce_head_case(gop, x, labels):
    """The reference test's own head (test_fire.py:24-46): time-mean -> CrossEntropy."""
    gop.time_step = x.shape[0]
    xr = x.clone().requires_grad_(True)
    u, s = gop.gold_fire(xr)
    out = s.view(s.shape[0], s.shape[1], -1).mean(dim=0)
    loss = torch.nn.CrossEntropyLoss()(out, labels)
    loss.backward()
    return u.detach().numpy(), s.detach().numpy(), xr.grad.numpy(), out.detach().numpy(), float(loss.detach())


def make_bn_golden(gop):
    """Batch-norm family: the reference's gold modules in training mode (batch statistics), as its
    test_bn.py / test_bn_fire.py / test_bn_fire_fc.py / test_bn_fire_conv.py use them. Seeds are
    advanced until no membrane potential lies within 1e-4 of the threshold, so the comparison
    does not hinge on how the normalisation happens to round."""
    gop.time_step = 6
    out = {}
    shapes = {"fc": (6, 2, 8), "conv": (6, 2, 8, 8, 8)}

    def stats(x, kind):
        dims = (0, 1) if kind == "fc" else (0, 1, 3, 4)
        var, mean = torch.var_mean(x, dim=dims, unbiased=False)
        return var.numpy(), mean.numpy()

    def randomise(bn, gen):
        w = 0.5 + torch.rand(bn.num_features, generator=gen)
        b = 0.3 * torch.randn(bn.num_features, generator=gen)
        bn.weight = torch.nn.Parameter(w.clone())
        bn.bias = torch.nn.Parameter(b.clone())
        return w.numpy(), b.numpy()

    for kind, shape in shapes.items():
        # plain BN
        gen = torch.Generator().manual_seed(31)
        mod = gop.Bn(8, kind)
        w, b = randomise(mod.bn, gen)
        x = torch.randn(shape, generator=gen)
        xr = x.clone().requires_grad_(True)
        y = mod(xr)
        gy = torch.randn(y.shape, generator=gen)
        y.backward(gy)
        k = f"bn_{kind}"
        out[f"{k}_x"], out[f"{k}_w"], out[f"{k}_b"], out[f"{k}_y"], out[f"{k}_gy"] = x.numpy(), w, b, y.detach().numpy(), gy.numpy()
        out[f"{k}_gx"], out[f"{k}_gw"], out[f"{k}_gb"] = xr.grad.numpy(), mod.bn.weight.grad.numpy(), mod.bn.bias.grad.numpy()
        out[f"{k}_var"], out[f"{k}_mean"] = stats(x, kind)

        # BN folded into LIF
        seed = 40
        while True:
            gen = torch.Generator().manual_seed(seed)
            mod = gop.BnFire(8, kind)
            w, b = randomise(mod.bn, gen)
            x = torch.randn(shape, generator=gen)
            xr = x.clone().requires_grad_(True)
            u, s = mod(xr)
            if float((u.detach() - gop.thresh).abs().min()) > 1e-4:
                break
            seed += 1
        g = torch.randn(s.shape, generator=gen)
        s.backward(g)
        k = f"bnfire_{kind}"
        out[f"{k}_x"], out[f"{k}_w"], out[f"{k}_b"], out[f"{k}_g"] = x.numpy(), w, b, g.numpy()
        out[f"{k}_u"], out[f"{k}_s"] = u.detach().numpy(), s.detach().numpy()
        out[f"{k}_gx"], out[f"{k}_gw"], out[f"{k}_gb"] = xr.grad.numpy(), mod.bn.weight.grad.numpy(), mod.bn.bias.grad.numpy()
        out[f"{k}_var"], out[f"{k}_mean"] = stats(x, kind)

        # BN + LIF + fc  /  BN + LIF + conv
        for comp in (("fc",) if kind == "fc" else ("fc", "conv")):
            seed = 60
            while True:
                torch.manual_seed(seed)
                gen = torch.Generator().manual_seed(seed)
                if comp == "fc":
                    # as test_bn_fire_fc.py does: BN over 8 channels, then the fc weight is
                    # replaced by one that matches the flattened input (8*8*8 = 512 for images)
                    mod = gop.BnFireFc(8, 8, bn_fire=True, bn_layer_type=kind)
                    if kind == "conv":
                        mod.fc.weight = torch.nn.Parameter(0.05 * torch.randn(8, 512))
                    lin_w, lin_b = mod.fc.weight, mod.fc.bias
                else:
                    mod = gop.BnFireConv(8, 8, bn_fire=True)
                    lin_w, lin_b = mod.conv.weight, mod.conv.bias
                w, b = randomise(mod.bn, gen)
                x = torch.randn(shape, generator=gen)
                with torch.no_grad():
                    u, _ = gop.gold_bn_fire(x, mod.bn)
                mod.bn.reset_running_stats()
                if float((u - gop.thresh).abs().min()) > 1e-4:
                    break
                seed += 1
            xr = x.clone().requires_grad_(True)
            y = mod(xr)
            gy = torch.randn(y.shape, generator=gen)
            y.backward(gy)
            k = f"bnfire{comp}_{kind}"
            out[f"{k}_x"], out[f"{k}_w"], out[f"{k}_b"] = x.numpy(), w, b
            out[f"{k}_lw"], out[f"{k}_lb"] = lin_w.detach().numpy().copy(), lin_b.detach().numpy().copy()
            out[f"{k}_y"], out[f"{k}_gy"], out[f"{k}_gx"] = y.detach().numpy(), gy.numpy(), xr.grad.numpy()
            out[f"{k}_gw"], out[f"{k}_gb"] = mod.bn.weight.grad.numpy(), mod.bn.bias.grad.numpy()
            out[f"{k}_glw"], out[f"{k}_glb"] = lin_w.grad.numpy(), lin_b.grad.numpy()
            out[f"{k}_var"], out[f"{k}_mean"] = stats(x, kind)
    np.savez_compressed(os.path.join(HERE, "bn_golden.npz"), **out)


def record_reference_model_layouts(ref_root):
    """Parameter names and shapes of the reference's own networks (snnlib/example/models.py),
    built from the reference's class definitions. Its modules import a compiled ``snnlib``; the
    constructors never call into it, so this repository's package is aliased under that name just
    to let the import succeed."""
    import importlib
    import json
    root = os.path.dirname(os.path.dirname(HERE))
    sys.path.insert(0, root)
    import snn_gpu_training_bptt_b200 as pkg
    from snn_gpu_training_bptt_b200 import snnlib as native
    saved = {k: sys.modules.get(k) for k in ("snnlib", "snnlib_func", "snnlib_op", "models")}
    for k in ("snnlib_func", "snnlib_op", "models"):
        sys.modules.pop(k, None)
    sys.modules["snnlib"] = native                # only the compiled module is substituted;
    ref_models = importlib.import_module("models")  # snnlib_func / snnlib_op / models are the reference's files
    assert ref_models.__file__.startswith(ref_root)
    layouts = {}
    for name in ("CIFAR_BN", "Alexnet_BN_DIST", "Resnet_DIST"):
        sd = getattr(ref_models, name)().state_dict()
        layouts[name] = {k: list(v.shape) for k, v in sd.items()}
    with open(os.path.join(HERE, "reference_model_layouts.json"), "w") as f:
        json.dump(layouts, f, indent=0, sort_keys=True)
    for k, v in saved.items():
        sys.modules.pop(k, None)
        if v is not None:
            sys.modules[k] = v


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of liangling76/snn_gpu_training_bptt")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "snnlib", "example"))
    import gold_op as gop  # the reference's module

    torch.set_num_threads(1)
    out = {}

    # ---- 1. shapes of the reference's own test fixtures (test_utils.py:5-27), T = 6 -------
    gen = torch.Generator().manual_seed(20240601)
    labels = torch.tensor([1, 0])
    for name, shape in (("ut_fc", (6, 2, 8)), ("ut_conv", (6, 2, 8, 8, 8))):
        x = torch.randn(shape, generator=gen)
        u, s, gx, head, loss = ce_head_case(gop, x, labels)
        out[f"{name}_x"], out[f"{name}_u"], out[f"{name}_s"] = x.numpy(), u, s
        out[f"{name}_gx_ce"], out[f"{name}_head"], out[f"{name}_loss"] = gx, head, np.float32(loss)
        g = torch.randn(shape, generator=gen)
        _, _, gx2 = fire_case(gop, x, g)
        out[f"{name}_g"], out[f"{name}_gx"] = g.numpy(), gx2

    # ---- 2. ragged neuron counts and several T, inputs N(0.5, 1), upstream N(0, 1) ---------
    for T, N in ((1, 37), (2, 130), (4, 1003), (6, 515), (8, 4099), (16, 1021), (20, 259), (33, 65)):
        gen = torch.Generator().manual_seed(1000 + T)
        x = 0.5 + torch.randn((T, 1, N), generator=gen)
        g = torch.randn((T, 1, N), generator=gen)
        u, s, gx = fire_case(gop, x, g)
        k = f"rag_T{T}_N{N}"
        out[f"{k}_x"], out[f"{k}_g"] = x.numpy(), g.numpy()
        out[f"{k}_u"], out[f"{k}_s"], out[f"{k}_gx"] = u, s, gx

    # ---- 3. hand-placed edge values: threshold, window edges, resets, zeros, large ---------
    th, iv = gop.thresh, gop.interval
    cols = [
        [th] * 8,                                     # u == thresh exactly: no spike (strict >)
        [np.nextafter(np.float32(th), np.float32(1))] * 8,   # one ulp above: spike every step
        [th + iv] * 8,                                # upper window edge (strict <): outside
        [th - iv] * 8,                                # lower window edge: outside
        [np.nextafter(np.float32(th + iv), np.float32(0))] * 8,
        [np.nextafter(np.float32(th - iv), np.float32(1))] * 8,
        [0.0] * 8,
        [-0.0] * 8,
        [1e30, -1e30, 1e-30, -1e-30, 3e38, -3e38, 1.0, -1.0],
        [0.2, 0.2, 0.2, 0.2, 0.2, 0.2, 0.2, 0.2],     # slow integration to a spike
        [1.0, 0.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0],     # spike then hard reset
        [-5.0, 1.5, -5.0, 1.5, -5.0, 1.5, -5.0, 1.5],
        [0.24999999, 0.25000003, 0.75, -0.25, 0.7499999, -0.2499999, 0.5, 0.1],
    ]
    x = torch.tensor(np.array(cols, dtype=np.float32).T.copy()).reshape(8, 1, len(cols))
    gen = torch.Generator().manual_seed(77)
    g = torch.randn(x.shape, generator=gen)
    u, s, gx = fire_case(gop, x, g)
    out["edge_x"], out["edge_g"], out["edge_u"], out["edge_s"], out["edge_gx"] = (
        x.numpy(), g.numpy(), u, s, gx)

    # ---- 4. fire->fc and plain fc compositions (test_fire_fc.py, test_fc.py), T = 6 -------
    gop.time_step = 6
    for name, shape, cin in (("fc", (6, 2, 8), 8), ("conv", (6, 2, 8, 8, 8), 512)):
        for fire in (True, False):
            torch.manual_seed(4242 + cin + int(fire))
            mod = gop.BnFireFc(cin, 8, fire=fire)
            w = torch.randn(8, cin)
            b = torch.randn(8)
            mod.fc.weight = torch.nn.Parameter(w.clone())
            mod.fc.bias = torch.nn.Parameter(b.clone())
            x = torch.randn(shape)
            xr = x.clone().requires_grad_(True)
            y = mod(xr)
            gy = torch.randn(y.shape)
            y.backward(gy)
            k = f"{'firefc' if fire else 'fc'}_{name}"
            out[f"{k}_x"], out[f"{k}_w"], out[f"{k}_b"] = x.numpy(), w.numpy(), b.numpy()
            out[f"{k}_y"], out[f"{k}_gy"] = y.detach().numpy(), gy.numpy()
            out[f"{k}_gx"] = xr.grad.numpy()
            out[f"{k}_gw"] = mod.fc.weight.grad.numpy()
            out[f"{k}_gb"] = mod.fc.bias.grad.numpy()

    np.savez_compressed(os.path.join(HERE, "lif_golden.npz"), **out)
    make_bn_golden(gop)
    record_reference_model_layouts(args.ref)

    # ---- 5. the full single-layer case: T=8, [32,128,16,16], seed 1234 ---------------------
    # Too large to store; keep digests of inputs and outputs plus a strided sample.
    torch.set_num_threads(os.cpu_count() or 1)
    gen = torch.Generator().manual_seed(1234)
    shape = (8, 32, 128, 16, 16)
    x = 0.5 + torch.randn(shape, generator=gen)
    g = torch.randn(shape, generator=gen)
    u, s, gx = fire_case(gop, x, g)
    stride = 4099
    big = {
        "shape": np.array(shape), "seed": np.array(1234), "stride": np.array(stride),
        "x_sha": np.array(sha(x.numpy())), "g_sha": np.array(sha(g.numpy())),
        "u_sha": np.array(sha(u)), "s_sha": np.array(sha(s)),
        "gx_sha": np.array(sha(gx + 0.0)),   # "+ 0.0" folds -0.0 into +0.0 before hashing
        "x_sample": x.numpy().reshape(-1)[::stride], "g_sample": g.numpy().reshape(-1)[::stride],
        "u_sample": u.reshape(-1)[::stride], "s_sample": s.reshape(-1)[::stride],
        "gx_sample": gx.reshape(-1)[::stride],
        "spike_rate": np.array(s.mean(dtype=np.float64)),
        "gx_abs_sum": np.array(np.abs(gx).sum(dtype=np.float64)),
    }
    np.savez_compressed(os.path.join(HERE, "lif_config1_digest.npz"), **big)
    print("wrote", sorted(os.listdir(HERE)))
    print("config-1 spike rate", float(big["spike_rate"]))


if __name__ == "__main__":
    main()
