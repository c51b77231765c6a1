"""Host-side logic of the layer modules / example networks that needs no GPU: parameter
names and shapes (state-dict compatibility with the reference), initialisation statistics,
checkpoint round trip, and the reference-name aliasing."""
import math
import sys

import torch

from snn_gpu_training_bptt_b200 import snnlib_op as sop
from snn_gpu_training_bptt_b200.example import models, train_synthetic


def test_layer_parameter_names_match_reference():
    assert list(sop.FireConv(4, 8).state_dict()) == ["weight_conv", "bias_conv"]
    assert list(sop.Conv(4, 8).state_dict()) == ["weight_conv", "bias_conv"]
    assert list(sop.FireFc(4, 8).state_dict()) == ["weight_fc", "bias_fc"]
    assert list(sop.Fc(4, 8).state_dict()) == ["weight_fc", "bias_fc"]
    bn_keys = ["weight_bn", "bias_bn", "running_var", "running_mean"]
    assert list(sop.BnFire(4, (0, 1)).state_dict()) == bn_keys
    assert list(sop.BnFireConv(4, 8).state_dict()) == bn_keys + ["weight_conv", "bias_conv"]
    assert list(sop.BnFireFc(16, 8, (0, 1, 3, 4), cin_bn=4).state_dict()) == bn_keys + ["weight_fc", "bias_fc"]
    assert sop.BnFireFc(16, 8, (0, 1, 3, 4), cin_bn=4).weight_bn.shape == (4,)
    assert list(sop.Fire().state_dict()) == []


def test_initialisation_follows_reference():
    torch.manual_seed(0)
    w = sop.Fc(400, 300).weight_fc
    assert abs(float(w.detach().std()) - 0.75 / math.sqrt(400)) < 2e-3 and abs(float(w.detach().mean())) < 1e-3
    c = sop.Conv(64, 32).weight_conv
    assert abs(float(c.detach().std()) - 0.75 / math.sqrt(64)) < 3e-3
    assert float(sop.Conv(64, 32).bias_conv.abs().max()) == 0.0
    bound = 1 / math.sqrt(64 * 9)                       # nn.Conv2d default for the fused layers
    assert float(sop.FireConv(64, 32).weight_conv.abs().max()) <= bound + 1e-6


def test_running_statistics_keep_identity_and_are_not_trained():
    m = sop.BnFireConv(4, 8)
    assert not m.running_var.requires_grad and not m.running_mean.requires_grad
    assert m.weight_bn.requires_grad
    assert [n for n, p in m.named_parameters() if p.requires_grad] == ["weight_bn", "bias_bn", "weight_conv", "bias_conv"]


def test_benchmark_networks_shapes():
    vgg = models.build("vgg", time_steps=8)
    n = sum(p.numel() for p in vgg.parameters())
    assert vgg.fc1.weight_fc.shape == (1024, 8192)
    assert 12_500_000 < n < 13_500_000                 # ~13 M parameters, fc1 is 8.4 M of them
    res = models.build("resnet19", time_steps=16)
    assert len(res.blocks) == 8 and res.fc2.out_features == 10


def test_checkpoint_round_trip(tmp_path):
    net = models.SpikingVGG(widths=(4, 8, 8), hidden=16)
    opt = torch.optim.SGD(net.parameters(), lr=0.01, momentum=0.9)
    for p in net.parameters():
        p.grad = torch.ones_like(p)
    opt.step()
    path = str(tmp_path / "ckpt.pth.tar")
    train_synthetic.save_checkpoint(path, net, opt, step=17)
    net2 = models.SpikingVGG(widths=(4, 8, 8), hidden=16)
    opt2 = torch.optim.SGD(net2.parameters(), lr=0.01, momentum=0.9)
    assert train_synthetic.load_checkpoint(path, net2, opt2) == 17
    for a, b in zip(net.parameters(), net2.parameters()):
        assert torch.equal(a, b)
    assert opt2.state_dict()["state"][0]["momentum_buffer"].shape == opt.state_dict()["state"][0]["momentum_buffer"].shape
    # a bare state dict, which is what the reference's scripts save, loads as well
    torch.save(net.state_dict(), path)
    assert train_synthetic.load_checkpoint(path, net2) == 0


def test_install_under_reference_names():
    import snn_gpu_training_bptt_b200 as pkg
    saved = {k: sys.modules.pop(k, None) for k in ("snnlib", "snnlib_func", "snnlib_op")}
    try:
        pkg.install_as_snnlib()
        import snnlib
        import snnlib_func
        import snnlib_op
        assert len(snnlib.__all__) == 24 and all(hasattr(snnlib, n) for n in snnlib.__all__)
        assert snnlib_func.time_step == 6 and snnlib_func.alpha == 0.25 and snnlib_func.thresh == 0.25
        assert snnlib_func.beta == 1.0 and snnlib_func.interval == 0.5
        for name in ("Fire", "Bn", "BnFire", "BnFireFc", "FireFc", "Fc", "BnFireConv", "FireConv", "Conv",
                     "BnDist", "BnFireFcDist", "BnFireConvDist"):
            assert hasattr(snnlib_op, name)
        for name in ("fire_func", "bn_func", "bn_fire_func", "bn_fire_fc_func", "fire_fc_func", "fc_func",
                     "bn_fire_conv_func", "fire_conv_func", "conv_func", "bn_dist_func",
                     "bn_fire_fc_dist_func", "bn_fire_conv_dist_func"):
            assert callable(getattr(snnlib_func, name))
    finally:
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v


def test_time_major_dense_detection():
    from snn_gpu_training_bptt_b200._capi import is_time_major_dense as dense
    x = torch.zeros(6, 4, 8, 5, 5)
    assert dense(x) and dense(x.permute(0, 2, 1, 3, 4))
    assert not dense(x[:, :, :, :, ::2]) and not dense(x[::2]) and not dense(x.transpose(0, 1))
    cl = torch.zeros(24, 8, 5, 5).to(memory_format=torch.channels_last).view(6, 4, 8, 5, 5)
    assert dense(cl) and torch.empty_like(cl).stride() == cl.stride()


def test_reference_networks_keep_their_state_dict_layout():
    """CIFAR_BN / Alexnet_BN_DIST / Resnet_DIST expose exactly the parameter names and shapes of
    the reference's classes (recorded from the reference's models.py by tests/golden/make_golden.py),
    so checkpoints interchange."""
    import json
    import os
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", "reference_model_layouts.json")) as f:
        layouts = json.load(f)
    for name, want in layouts.items():
        sd = getattr(models, name)().state_dict()
        assert {k: list(v.shape) for k, v in sd.items()} == want, name


def test_bucket_sgd_follows_torch_sgd_and_round_trips_its_state():
    """BucketSGD (per-bucket momentum SGD used by the trainer) against torch.optim.SGD on the same
    gradients, and its state dict through save / load."""
    from snn_gpu_training_bptt_b200.example.ddp import BucketSGD, DistributedDataParallel as DDP
    torch.manual_seed(3)
    make = lambda: torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.Tanh(), torch.nn.Linear(16, 16), torch.nn.Tanh(),
                                       torch.nn.Linear(16, 3))
    a, b = make(), make()
    b.load_state_dict(a.state_dict())
    ddp = DDP(a, bucket_mb=0.0005, defer_wait=True)
    assert len(ddp.buckets) > 2
    mine, ref = BucketSGD(ddp, lr=0.05, momentum=0.9), torch.optim.SGD(b.parameters(), lr=0.05, momentum=0.9)
    x, y = torch.randn(4, 5, 6), torch.randn(4, 5, 3)
    for step in range(4):
        mine.zero_grad(), ref.zero_grad()
        (a(x[step]) - y[step]).square().mean().backward()
        (b(x[step]) - y[step]).square().mean().backward()
        mine.step(), ref.step()
        if step == 1:
            saved = mine.state_dict()
            restored = BucketSGD(ddp, lr=0.0, momentum=0.0)
            restored.load_state_dict(saved)
            assert restored.groups[0][1].param_groups[0]["lr"] == 0.05
            mine = restored
    for p, q in zip(a.parameters(), b.parameters()):
        assert torch.allclose(p, q, rtol=1e-6, atol=1e-7)
