"""GPU tests of the layers either side of the LIF kernels and of the example trainer:
conv / fc wrappers against a time-stepped PyTorch composition, channels-last layouts, mixed
precision, and the data-parallel step (NCCL ranks as child processes when >= 2 GPUs)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import lif_oracle as orc
from tests.helpers import CONSTS, assert_grad_close

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", autouse=True)
def _strict_fp32(built_lib):
    assert torch.cuda.is_available()
    old = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = old


def _gold_fire_conv(x, w, b, fire):
    """Time-stepped composition as the reference's gold ops do it (gold_op.py:153-180)."""
    s = orc.torch_fire(x, **CONSTS)[1] if fire else x
    return torch.stack([F.conv2d(s[t], w, b, stride=1, padding=1) for t in range(x.shape[0])])


@pytest.mark.parametrize("fire", [False, True])
def test_conv_layers_against_time_stepped_composition(fire):
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    gen = torch.Generator().manual_seed(5)
    x = (0.3 + torch.randn((6, 2, 8, 8, 8), generator=gen)).cuda()
    w = (0.2 * torch.randn((8, 8, 3, 3), generator=gen)).cuda()
    b = torch.randn(8, generator=gen).cuda()
    gy = torch.randn((6, 2, 8, 8, 8), generator=gen).cuda()
    leaves = [t.clone().requires_grad_(True) for t in (x, w, b)]
    fn = sf.fire_conv_func if fire else sf.conv_func
    y = fn(leaves[0], leaves[1], leaves[2], (1, 1), (1, 1), True)
    y.backward(gy)
    ref = [t.clone().requires_grad_(True) for t in (x, w, b)]
    y_ref = _gold_fire_conv(ref[0], ref[1], ref[2], fire)
    y_ref.backward(gy)
    assert_grad_close(y.detach().cpu(), y_ref.detach().cpu(), rtol=1e-4, atol=1e-4, what="conv out")
    for got, want, name in zip(leaves, ref, ("grad_x", "grad_w", "grad_b")):
        assert_grad_close(got.grad.cpu(), want.grad.cpu(), rtol=1e-4, atol=2e-4, what=name)


def test_channels_last_activations_need_no_copy_and_match():
    """A channels-last [T*B, C, H, W] batch viewed as [T, B, C, H, W] goes through the LIF kernels
    as it is and gives the same values as the contiguous layout."""
    from snn_gpu_training_bptt_b200 import _capi, snnlib_func as sf
    gen = torch.Generator().manual_seed(9)
    x = (0.5 + torch.randn((4, 3, 16, 6, 6), generator=gen)).cuda()
    g = torch.randn(x.shape, generator=gen).cuda()
    x_cl = x.view(12, 16, 6, 6).contiguous(memory_format=torch.channels_last).view(4, 3, 16, 6, 6)
    g_cl = g.view(12, 16, 6, 6).contiguous(memory_format=torch.channels_last).view(4, 3, 16, 6, 6)
    assert not x_cl.is_contiguous() and _capi.is_time_major_dense(x_cl)
    a = x.clone().requires_grad_(True)
    b = x_cl.clone(memory_format=torch.preserve_format).requires_grad_(True)
    sa, sb = sf.fire_func(a), sf.fire_func(b)
    assert sb.stride() == x_cl.stride()
    sa.backward(g)
    sb.backward(g_cl)
    assert torch.equal(sa, sb) and torch.equal(a.grad, b.grad)
    # mismatched gradient layout is re-laid out, not misread
    c = x_cl.clone(memory_format=torch.preserve_format).requires_grad_(True)
    sf.fire_func(c).backward(g)
    assert torch.equal(c.grad, a.grad)


def test_small_vgg_fp32_against_autograd_composition():
    """The benchmark network (narrow) end to end in fp32 vs the same network written with plain
    PyTorch ops and the oracle's autograd LIF, both on the GPU."""
    from snn_gpu_training_bptt_b200.example import models
    torch.manual_seed(3)
    net = models.SpikingVGG(time_steps=4, widths=(8, 16, 16), hidden=32, image=16,
                            act_dtype=torch.float32).cuda()
    images = torch.rand(3, 3, 16, 16, device="cuda")
    labels = torch.tensor([1, 7, 3], device="cuda")
    loss = F.cross_entropy(net(images), labels)
    loss.backward()

    def fire(x):
        return orc.torch_fire(x, **CONSTS)[1]

    def conv(x, m):
        return torch.stack([F.conv2d(x[t], m.weight_conv, m.bias_conv, padding=1) for t in range(x.shape[0])])

    def pool(x):
        return torch.stack([F.avg_pool2d(x[t], 2) for t in range(x.shape[0])])

    grads = {n: p.grad.clone() for n, p in net.named_parameters()}
    net.zero_grad()
    x = torch.stack([images] * 4)
    x = pool(fire(conv(fire(conv(x, net.conv1_1)), net.conv1_2)))
    x = pool(fire(conv(fire(conv(x, net.conv2_1)), net.conv2_2)))
    x = pool(fire(conv(fire(conv(x, net.conv3_1)), net.conv3_2)))
    x = x.reshape(4, 3, -1)
    x = fire(F.linear(x, net.fc1.weight_fc, net.fc1.bias_fc))
    loss_ref = F.cross_entropy(net.fc2(x.mean(dim=0)), labels)
    loss_ref.backward()
    assert abs(float(loss.detach()) - float(loss_ref.detach())) < 1e-5
    for n, p in net.named_parameters():
        assert_grad_close(grads[n].cpu(), p.grad.cpu(), rtol=2e-3, atol=2e-5, what=n)


@pytest.mark.parametrize("model,T,B", [("vgg", 8, 8), ("resnet19", 4, 4)])
def test_training_steps_run_in_bf16(model, T, B, tmp_path):
    from snn_gpu_training_bptt_b200.example import train_synthetic
    ck = str(tmp_path / "ck.pth.tar")
    out = train_synthetic.run(model, time_steps=T, batch=B, steps=3, warmup=1, precision="bf16",
                              checkpoint=ck)
    assert np.isfinite(out["final_loss"]) and out["samples_per_s"] > 0
    assert os.path.exists(ck)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_nccl_data_parallel_matches_single_process(tmp_path):
    """2 NCCL ranks (child processes), each on half the batch: averaged gradients must equal the
    single-process gradients on the whole batch. NVLS is switched off for the children."""
    script = os.path.join(ROOT, "tests", "ddp_nccl_child.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), script, str(tmp_path)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    r0 = torch.load(str(tmp_path / "rank0.pt"))
    r1 = torch.load(str(tmp_path / "rank1.pt"))
    single = torch.load(str(tmp_path / "single.pt"))
    for name in single:
        assert torch.equal(r0[name], r1[name]), name
        assert_grad_close(r0[name], single[name], rtol=2e-3, atol=2e-5, what=name)


def test_reference_cifar_bn_network_trains_and_evaluates():
    """The reference's own CIFAR network (all layers BN-fused) through two SGD steps, then in
    evaluation mode with running statistics (train_test_cifar.py:52-92)."""
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    from snn_gpu_training_bptt_b200.example import models
    old_T = sf.time_step
    try:
        sf.time_step = 4
        torch.manual_seed(0)
        net = models.CIFAR_BN().cuda()
        opt = torch.optim.SGD(net.parameters(), lr=1e-2, momentum=0.9)
        images = torch.rand(4, 3, 32, 32, device="cuda")
        labels = torch.tensor([1, 2, 3, 4], device="cuda")
        net.set_bn(True)
        before = net.conv2_1.running_mean.clone()
        losses = []
        for _ in range(2):
            net.zero_grad()
            opt.zero_grad()
            loss = F.cross_entropy(net(images), labels)
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
        assert all(np.isfinite(v) for v in losses)
        assert not torch.equal(before, net.conv2_1.running_mean)
        assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in net.parameters() if p.requires_grad)
        net.set_bn(False)
        with torch.no_grad():
            out = net(images)
        assert out.shape == (4, 10) and torch.isfinite(out).all()
    finally:
        sf.time_step = old_T


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8, 2, 16, 8, 8), (6, 3, 5, 4, 6), (16, 1, 8, 4, 4), (4, 2, 130, 2, 2), (1, 1, 4, 2, 2)])
def test_fused_lif_pool_equals_lif_then_pool(dtype, shape):
    """FirePool == Fire followed by AvgPool2d(2) on every time step, forward and backward, bit for
    bit (pooled spikes are k/4, the pooled gradient is scaled by an exact 1/4); and in fp32 also
    equal to the CPU oracle's LIF composed with numpy pooling."""
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    T, B, C, H, W = shape
    gen = torch.Generator().manual_seed(sum(shape))
    x = (0.5 + torch.randn(shape, generator=gen)).to(dtype)
    g = torch.randn((T, B, C, H // 2, W // 2), generator=gen).to(dtype)
    a = x.cuda().requires_grad_(True)
    b = x.cuda().requires_grad_(True)
    ya = F.avg_pool2d(sf.fire_func(a).reshape(T * B, C, H, W), 2).view(T, B, C, H // 2, W // 2)
    yb = sf.fire_pool_func(b)
    assert yb.shape == ya.shape and torch.equal(ya, yb)
    ya.backward(g.cuda())
    yb.backward(g.cuda())
    assert torch.equal(a.grad, b.grad)
    if dtype == torch.float32:
        s_ref, _ = orc.c_lif_fwd(x.numpy())
        pooled = s_ref.reshape(T, B, C, H // 2, 2, W // 2, 2).mean(axis=(4, 6))
        assert np.array_equal(yb.detach().cpu().numpy(), pooled)
        g_full = np.repeat(np.repeat(g.numpy(), 2, axis=3), 2, axis=4) * np.float32(0.25)
        assert np.array_equal(b.grad.cpu().numpy(), orc.c_lif_bwd(x.numpy(), np.ascontiguousarray(g_full)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(8, 2, 16, 8, 8), (6, 3, 5, 3, 7), (16, 1, 8, 4, 4), (4, 2, 131), (1, 1, 3), (11, 4, 64, 2, 2)])
def test_fused_lif_of_a_sum_equals_add_then_lif(dtype, shape):
    """FireAdd(a, b) == Fire(a + b) bit for bit, spikes and both input gradients (odd sizes take the
    narrow-vector kernels, T not in {4, 8, 16} the guarded ones); in fp32 also equal to the CPU
    oracle applied to the rounded sum. One addend may arrive channels-last, the other contiguous."""
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    gen = torch.Generator().manual_seed(sum(shape) + 1)
    x = (0.3 + torch.randn(shape, generator=gen)).to(dtype)
    y = (0.2 + 0.7 * torch.randn(shape, generator=gen)).to(dtype)
    g = torch.randn(shape, generator=gen).to(dtype)
    a1, b1 = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    a2, b2 = x.cuda().requires_grad_(True), y.cuda().requires_grad_(True)
    b2_in = b2
    if len(shape) == 5:                       # same values, channels-last strides
        b2_in = b2.view(-1, *shape[2:]).contiguous(memory_format=torch.channels_last).view(shape)
    want = sf.fire_func(a1 + b1)
    got = sf.fire_add_func(a2, b2_in)
    assert torch.equal(want, got)
    want.backward(g.cuda())
    got.backward(g.cuda())
    assert torch.equal(a1.grad, a2.grad) and torch.equal(b1.grad, b2.grad)
    assert torch.equal(a2.grad, b2.grad)
    if dtype == torch.float32:
        total = (x + y).numpy()
        assert np.array_equal(got.detach().cpu().numpy(), orc.c_lif_fwd(total)[0])
        assert np.array_equal(a2.grad.cpu().numpy(), orc.c_lif_bwd(total, g.numpy()))


def test_lif_of_a_sum_fallback_and_errors():
    from snn_gpu_training_bptt_b200 import _capi, snnlib_func as sf
    x = torch.randn(20, 2, 33, device="cuda")            # 20 steps: add -> LIF composition
    y = torch.randn(20, 2, 33, device="cuda")
    assert torch.equal(sf.fire_add_func(x, y), sf.fire_func(x + y))
    with pytest.raises(ValueError):
        sf.fire_add_func(x[:4], y[:5])
    with pytest.raises(_capi.SnnError):
        _capi.lif_add_bwd(x, y, x, 0.3, 0.5, 1.0, 0.5)    # the native backward itself refuses T > 16
    only_a = x[:8].clone().requires_grad_(True)
    sf.fire_add_func(only_a, y[:8]).sum().backward()     # shortcut without gradient
    assert only_a.grad is not None


def test_fused_and_unfused_pool_networks_agree():
    from snn_gpu_training_bptt_b200.example import models
    images = torch.rand(2, 3, 16, 16, device="cuda")
    labels = torch.tensor([3, 5], device="cuda")
    grads = []
    for fused in (True, False):
        torch.manual_seed(4)
        net = models.SpikingVGG(time_steps=4, widths=(8, 16, 16), hidden=32, image=16,
                                act_dtype=torch.float32, fused_pool=fused).cuda()
        loss = F.cross_entropy(net(images), labels)
        loss.backward()
        grads.append((float(loss.detach()), {n: p.grad.clone() for n, p in net.named_parameters()}))
    assert abs(grads[0][0] - grads[1][0]) < 1e-6
    for n in grads[0][1]:
        assert_grad_close(grads[0][1][n].cpu(), grads[1][1][n].cpu(), rtol=1e-3, atol=1e-6, what=n)


def test_cuda_graph_training_matches_eager():
    """The captured training step replays to the same parameters as the eager loop."""
    from snn_gpu_training_bptt_b200.example import train_synthetic
    outs = [train_synthetic.run("vgg", time_steps=4, batch=4, steps=4, warmup=3, precision="bf16",
                                graph=flag, return_params=True, model_kwargs=dict(widths=(16, 32, 32), hidden=64))
            for flag in (False, True)]
    assert np.isfinite(outs[1]["final_loss"])
    assert abs(outs[0]["final_loss"] - outs[1]["final_loss"]) < 5e-2
    for a, b in zip(outs[0]["params"], outs[1]["params"]):
        assert torch.allclose(a, b, rtol=5e-2, atol=5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_channel_bias_add_and_sum_kernels(dtype):
    """snn_channel_bias_add / snn_channel_sum against torch on contiguous, channels-last and
    matrix layouts, narrow and very wide channel counts, ragged sizes."""
    from snn_gpu_training_bptt_b200 import _capi
    gen = torch.Generator().manual_seed(0)
    cases = [((512, 128, 8, 8), True), ((512, 128, 8, 8), False), ((37, 5, 3, 7), False), ((37, 6, 3, 7), True),
             ((2048, 1024), False), ((33, 9000), False), ((3, 7), False), ((64, 96, 4, 4), True),
             # large enough for the fixed-pattern kernels' unrolled walk (several strides of the whole grid) and its ragged tail
             ((520, 128, 16, 16), True), ((4097, 512), False)]
    for shape, channels_last in cases:
        y = torch.randn(shape, generator=gen).to(dtype).cuda()
        if channels_last:
            y = y.contiguous(memory_format=torch.channels_last)
        bias = torch.randn(shape[1], generator=gen).cuda()
        want = (y.float() + bias.view((1, -1) + (1,) * (len(shape) - 2))).to(dtype)
        got = _capi.channel_bias_add_(y.clone(memory_format=torch.preserve_format), bias)
        assert got.stride() == y.stride() and torch.equal(got, want), shape
        sums = _capi.channel_sum(y)
        ref = y.double().sum(dim=[d for d in range(len(shape)) if d != 1])
        scale = float(y.float().abs().sum(dim=[d for d in range(len(shape)) if d != 1]).max())
        assert float((sums.double() - ref).abs().max()) <= 2e-6 * scale + 1e-6, shape
