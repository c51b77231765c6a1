"""GPU parity of the CUDA LIF kernels (called through the C ABI) against the CPU oracle and
the golden vectors generated from the reference's gold_op.py.

Bars: membrane potentials and spikes bit-exact in fp32 (the stated bar is 1e-5 relative and
spike flips only where |u - thresh| < 1e-6; exact is stricter and is what the arithmetic
gives); gradients exact in value in fp32, which is inside the 1e-4 relative bar.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import lif_oracle as orc
from tests.helpers import CONSTS, assert_grad_close, config1_inputs, fire_cases, seeded_inputs, sha

pytestmark = pytest.mark.gpu

A, TH, BE, IV = CONSTS["alpha"], CONSTS["thresh"], CONSTS["beta"], CONSTS["interval"]


@pytest.fixture(scope="module")
def capi(built_lib):
    if not torch.cuda.is_available():
        pytest.fail("marked gpu but no CUDA device is visible")
    from snn_gpu_training_bptt_b200 import _capi
    _capi.lib()
    return _capi


def _gpu(a):
    return torch.as_tensor(a).cuda()


def _fwd_all(capi, x_dev, bits=True):
    T = x_dev.shape[0]
    s, u, b = capi.lif_fwd(x_dev, A, TH, want_spike=True, want_mem=True, want_bits=bits and T <= 32)
    return s, u, b


# ---------------------------------------------------------------------------------------------
# golden vectors from the reference
# ---------------------------------------------------------------------------------------------
def test_golden_cases_fp32(capi, golden):
    for name in fire_cases(golden):
        x, g = _gpu(golden[name + "_x"]), _gpu(golden[name + "_g"])
        s, u, _ = _fwd_all(capi, x)
        gx = capi.lif_bwd(x, g, A, TH, BE, IV)
        assert np.array_equal(u.cpu().numpy().view(np.uint32), golden[name + "_u"].view(np.uint32)), name
        assert np.array_equal(s.cpu().numpy(), golden[name + "_s"]), name
        assert np.array_equal(gx.cpu().numpy(), golden[name + "_gx"]), name
        assert_grad_close(gx.cpu().numpy(), golden[name + "_gx"], rtol=1e-4, what=name)


def test_reference_test_scenario_through_modules(capi, golden):
    """snnlib/example/test_fire.py: Fire module -> time-mean -> CrossEntropy -> backward."""
    from snn_gpu_training_bptt_b200 import snnlib_op as sop
    labels = torch.tensor([1, 0]).cuda()
    for name in ("ut_fc", "ut_conv"):
        x = _gpu(golden[name + "_x"]).requires_grad_(True)
        spikes = sop.Fire().cuda()(x)
        head = spikes.view(spikes.shape[0], spikes.shape[1], -1).mean(dim=0)
        loss = torch.nn.CrossEntropyLoss()(head, labels)
        loss.backward()
        assert np.array_equal(spikes.detach().cpu().numpy(), golden[name + "_s"])
        assert np.allclose(head.detach().cpu().numpy(), golden[name + "_head"], rtol=0, atol=1e-7)
        assert abs(float(loss.detach()) - float(golden[name + "_loss"])) < 1e-6
        assert_grad_close(x.grad.cpu().numpy(), golden[name + "_gx_ce"], rtol=1e-4, atol=1e-9, what=name)


def test_config1_full_case_digest(capi, config1_digest):
    """T=8, [32,128,16,16], seed 1234: digests recorded from the reference's gold op."""
    d = config1_digest
    x, g = config1_inputs()
    if sha(x.numpy()) != str(d["x_sha"]) or sha(g.numpy()) != str(d["g_sha"]):
        pytest.skip("this torch build draws different random numbers than the one that made the digests")
    xd, gd = x.cuda(), g.cuda()
    s, u, _ = _fwd_all(capi, xd, bits=False)
    gx = capi.lif_bwd(xd, gd, A, TH, BE, IV)
    assert sha(u.cpu().numpy()) == str(d["u_sha"])
    assert sha(s.cpu().numpy()) == str(d["s_sha"])
    assert sha(gx.cpu().numpy() + 0.0) == str(d["gx_sha"])


def test_config1_against_c_oracle(capi):
    x, g = config1_inputs()
    s_ref, u_ref = orc.c_lif_fwd(x.numpy())
    gx_ref = orc.c_lif_bwd(x.numpy(), g.numpy())
    s, u, _ = _fwd_all(capi, x.cuda(), bits=False)
    gx = capi.lif_bwd(x.cuda(), g.cuda(), A, TH, BE, IV)
    assert np.array_equal(u.cpu().numpy(), u_ref)
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(gx.cpu().numpy(), gx_ref)


# ---------------------------------------------------------------------------------------------
# shapes: every T regime (register-resident <= 32, scratch-backed beyond), ragged N,
# misaligned base pointers
# ---------------------------------------------------------------------------------------------
T_LIST = [1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16, 17, 24, 31, 32, 33, 40, 70]
N_LIST = [1, 2, 3, 5, 127, 1024, 4098, 100003]


@pytest.mark.parametrize("T", T_LIST)
def test_sweep_T_and_ragged_N_fp32(capi, T):
    for N in N_LIST:
        x, g = seeded_inputs(T, N, seed=7 * T + N)
        s_ref, u_ref = orc.c_lif_fwd(x.numpy())
        gx_ref = orc.c_lif_bwd(x.numpy(), g.numpy())
        s, u, b = _fwd_all(capi, x.cuda())
        gx = capi.lif_bwd(x.cuda(), g.cuda(), A, TH, BE, IV)
        assert np.array_equal(u.cpu().numpy(), u_ref), (T, N)
        assert np.array_equal(s.cpu().numpy(), s_ref), (T, N)
        assert np.array_equal(gx.cpu().numpy(), gx_ref), (T, N)
        if b is not None:
            want = orc.c_lif_bits(x.numpy())
            mask = (1 << (8 * b.element_size())) - 1      # words are stored in signed torch dtypes
            assert np.array_equal(b.cpu().numpy().reshape(-1).astype(np.int64) & mask,
                                  want.astype(np.int64)), (T, N)


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_misaligned_base_pointers(capi, offset):
    """Tensors that start 4/8/12 bytes past a 16-byte boundary take the narrower-vector path."""
    for T, N in ((8, 4096), (6, 1000), (16, 514), (40, 256)):
        x, g = seeded_inputs(T, N, seed=99 + offset)

        def shifted(t):
            buf = torch.empty(T * N + offset, device="cuda")
            view = buf[offset:].view(T, 1, N)
            view.copy_(t)
            return view

        xd, gd = shifted(x), shifted(g)
        assert xd.data_ptr() % 16 == 4 * offset
        s, u, _ = _fwd_all(capi, xd, bits=False)
        gx = capi.lif_bwd(xd, gd, A, TH, BE, IV)
        s_ref, u_ref = orc.c_lif_fwd(x.numpy())
        assert np.array_equal(s.cpu().numpy(), s_ref)
        assert np.array_equal(u.cpu().numpy(), u_ref)
        assert np.array_equal(gx.cpu().numpy(), orc.c_lif_bwd(x.numpy(), g.numpy()))


def test_empty_neuron_axis(capi):
    x = torch.empty(4, 2, 0, device="cuda")
    s, u, _ = capi.lif_fwd(x, A, TH, want_mem=True)
    assert s.shape == x.shape and u.shape == x.shape
    assert capi.lif_bwd(x, x, A, TH, BE, IV).shape == x.shape


def test_guard_bands_are_untouched(capi):
    """Outputs sit between sentinel-filled pads; nothing may be written outside [T*N)."""
    pad = 64
    for T, N in ((8, 1000), (8, 4096), (5, 333), (16, 2050), (36, 130)):
        x, g = seeded_inputs(T, N, seed=5)
        xd, gd = x.cuda(), g.cuda()
        bufs = [torch.full((T * N + 2 * pad,), -12345.0, device="cuda") for _ in range(3)]
        spike, mem, gx = (b[pad:pad + T * N] for b in bufs)
        L = capi.lib()
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert L.snn_lif_fwd(p(xd), p(spike), p(mem), None, T, N, 0, A, TH, st) == 0
        need = L.snn_lif_bwd_workspace_bytes(T, N, 0)
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
        assert L.snn_lif_bwd(p(xd), p(gd), p(gx), T, N, 0, A, TH, BE, IV, p(ws) if need else None, need, st) == 0
        torch.cuda.synchronize()
        for b in bufs:
            assert bool((b[:pad] == -12345.0).all()) and bool((b[-pad:] == -12345.0).all())
        assert np.array_equal(spike.cpu().numpy().reshape(T, 1, N), orc.c_lif_fwd(x.numpy())[0])
        assert np.array_equal(gx.cpu().numpy().reshape(T, 1, N), orc.c_lif_bwd(x.numpy(), g.numpy()))


# ---------------------------------------------------------------------------------------------
# other element types: bf16 / fp16 I/O with fp32 state, fp64
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_io_fp32_state(capi, dtype):
    """The oracle runs in fp32 on the (exactly representable) low-precision inputs; the kernel
    must give the same fp32 membrane, the same spikes, and the same gradient once the fp32
    oracle gradient is rounded to the I/O type."""
    for T, N in ((8, 4096), (4, 1000), (6, 1027), (16, 2048), (32, 520), (40, 264)):
        x, g = seeded_inputs(T, N, seed=11 + T, dtype=dtype)
        x32, g32 = x.float().numpy(), g.float().numpy()
        s_ref, u_ref = orc.c_lif_fwd(x32)
        gx_ref = torch.from_numpy(orc.c_lif_bwd(x32, g32)).to(dtype)
        s, u, _ = _fwd_all(capi, x.cuda(), bits=False)
        gx = capi.lif_bwd(x.cuda(), g.cuda(), A, TH, BE, IV)
        assert s.dtype == dtype and u.dtype == torch.float32 and gx.dtype == dtype
        assert np.array_equal(u.cpu().numpy(), u_ref), (T, N)
        assert np.array_equal(s.float().cpu().numpy(), s_ref), (T, N)
        assert torch.equal(gx.cpu().float(), gx_ref.float()), (T, N)


def test_fp64(capi):
    for T, N in ((8, 1000), (6, 4096), (16, 130), (33, 70)):
        x, g = seeded_inputs(T, N, seed=3, dtype=torch.float64)
        s_ref, u_ref = orc.c_lif_fwd(x.numpy())
        gx_ref = orc.c_lif_bwd(x.numpy(), g.numpy())
        s, u, _ = _fwd_all(capi, x.cuda(), bits=False)
        gx = capi.lif_bwd(x.cuda(), g.cuda(), A, TH, BE, IV)
        assert np.array_equal(u.cpu().numpy(), u_ref)
        assert np.array_equal(s.cpu().numpy(), s_ref)
        assert np.array_equal(gx.cpu().numpy(), gx_ref)


# ---------------------------------------------------------------------------------------------
# packed spikes
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T", [1, 6, 8, 9, 16, 17, 32])
def test_packed_spikes_round_trip(capi, T):
    for N in (4096, 1001):
        x, _ = seeded_inputs(T, N, seed=T)
        s, _, bits = capi.lif_fwd(x.cuda(), A, TH, want_spike=True, want_bits=True)
        assert bits.element_size() == (1 if T <= 8 else 2 if T <= 16 else 4)
        dense = capi.spike_unpack(bits, T, torch.float32)
        assert torch.equal(dense, s)
        assert torch.equal(capi.spike_unpack(bits, T, torch.bfloat16).float(), s)
        only_bits = capi.lif_fwd(x.cuda(), A, TH, want_spike=False, want_bits=True)[2]
        assert torch.equal(only_bits, bits)


# ---------------------------------------------------------------------------------------------
# API behaviour: streams, non-contiguous inputs, hyper-parameter globals, error paths
# ---------------------------------------------------------------------------------------------
def test_runs_on_the_current_stream(capi):
    x, g = seeded_inputs(8, 1 << 16, seed=1)
    xd, gd = x.cuda(), g.cuda()
    ref_s = capi.lif_fwd(xd, A, TH)[0]
    ref_g = capi.lif_bwd(xd, gd, A, TH, BE, IV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        s = capi.lif_fwd(xd, A, TH)[0]
        gx = capi.lif_bwd(xd, gd, A, TH, BE, IV)
    side.synchronize()
    assert torch.equal(s, ref_s) and torch.equal(gx, ref_g)


def test_non_contiguous_input_and_changed_constants(capi):
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    x, g = seeded_inputs(6, 2048, seed=21, batch=4)            # [6, 4, 512]
    xt = x.permute(0, 2, 1).contiguous().cuda().permute(0, 2, 1)  # same values, strided
    assert not xt.is_contiguous()
    xt.requires_grad_(True)
    old = (sf.alpha, sf.thresh, sf.beta, sf.interval)
    try:
        sf.alpha, sf.thresh, sf.beta, sf.interval = 0.5, 0.4, 0.7, 0.3
        s = sf.fire_func(xt)
        s.backward(g.cuda())
        kw = dict(alpha=0.5, thresh=0.4, beta=0.7, interval=0.3)
        s_ref, _ = orc.c_lif_fwd(x.numpy(), 0.5, 0.4)
        gx_ref = orc.c_lif_bwd(x.numpy(), g.numpy(), **kw)
    finally:
        sf.alpha, sf.thresh, sf.beta, sf.interval = old
    assert np.array_equal(s.detach().cpu().numpy(), s_ref)
    assert np.array_equal(xt.grad.cpu().numpy(), gx_ref)


def test_shape_and_dtype_errors(capi):
    x = torch.zeros(4, 2, 8, device="cuda")
    with pytest.raises(ValueError):
        capi.lif_bwd(x, torch.zeros(4, 2, 9, device="cuda"), A, TH, BE, IV)
    with pytest.raises(TypeError):
        capi.lif_bwd(x, x.double(), A, TH, BE, IV)
    with pytest.raises(TypeError):
        capi.lif_fwd(x.int(), A, TH)
    with pytest.raises(ValueError):
        capi.lif_fwd(torch.zeros(8, device="cuda"), A, TH)


# ---------------------------------------------------------------------------------------------
# synaptic linear compositions (fire -> fc, fc) against the reference's gold modules
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["firefc_fc", "firefc_conv", "fc_fc", "fc_conv"])
def test_fc_compositions_against_gold(capi, golden, kind):
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    torch.backends.cuda.matmul.allow_tf32 = False
    x = _gpu(golden[kind + "_x"]).requires_grad_(True)
    w = _gpu(golden[kind + "_w"]).requires_grad_(True)
    b = _gpu(golden[kind + "_b"]).requires_grad_(True)
    fn = sf.fire_fc_func if kind.startswith("firefc") else sf.fc_func
    y = fn(x, w, b)
    y.backward(_gpu(golden[kind + "_gy"]))
    assert_grad_close(y.detach().cpu().numpy(), golden[kind + "_y"], rtol=1e-4, atol=1e-4, what="y")
    assert_grad_close(x.grad.cpu().numpy(), golden[kind + "_gx"], rtol=1e-4, atol=1e-4, what="gx")
    assert_grad_close(w.grad.cpu().numpy(), golden[kind + "_gw"], rtol=1e-4, atol=1e-4, what="gw")
    assert_grad_close(b.grad.cpu().numpy(), golden[kind + "_gb"], rtol=1e-4, atol=1e-4, what="gb")


# ---------------------------------------------------------------------------------------------
# full benchmark size: properties that do not need a full-size oracle run
# ---------------------------------------------------------------------------------------------
def test_full_size_T8_N64M_properties(capi):
    """T=8, N=2^26 (2 GiB per tensor). Neurons are independent, so any slice of the result must
    equal the oracle run on that slice alone; packed spikes must agree with dense ones; the
    result must not depend on how the neuron axis is split across launches."""
    T, N = 8, 1 << 26
    gen = torch.Generator(device="cuda").manual_seed(2024)
    x = torch.randn((T, 1, N), device="cuda", generator=gen).add_(0.5)
    g = torch.randn((T, 1, N), device="cuda", generator=gen)
    s, _, bits = capi.lif_fwd(x, A, TH, want_spike=True, want_bits=True)
    gx = capi.lif_bwd(x, g, A, TH, BE, IV)
    torch.cuda.synchronize()
    rng = np.random.default_rng(0)
    starts = [0, N - 65536] + [int(v) for v in rng.integers(0, N - 65536, size=6)]
    for st in starts:
        sl = slice(st, st + 65536)
        xs, gs = x[:, :, sl].cpu().numpy(), g[:, :, sl].cpu().numpy()
        assert np.array_equal(s[:, :, sl].cpu().numpy(), orc.c_lif_fwd(xs)[0]), st
        assert np.array_equal(gx[:, :, sl].cpu().numpy(), orc.c_lif_bwd(xs, gs)), st
    # checksum of checksums: per-time-step spike counts from dense and packed forms
    dense_counts = s.view(T, N).sum(dim=1, dtype=torch.float64)
    for t in range(T):
        packed = ((bits.view(-1) >> t) & 1).sum(dtype=torch.int64)
        assert int(packed) == int(dense_counts[t])
    # split invariance: two half-size launches give the same bytes
    half = N // 2
    for lo in (0, half):
        xs = x[:, :, lo:lo + half].contiguous()
        gs = g[:, :, lo:lo + half].contiguous()
        assert torch.equal(capi.lif_fwd(xs, A, TH)[0], s[:, :, lo:lo + half])
        assert torch.equal(capi.lif_bwd(xs, gs, A, TH, BE, IV), gx[:, :, lo:lo + half])
        del xs, gs
    # gradient is linear in the upstream gradient through a fixed spike pattern: scaling g by a
    # power of two scales grad_x exactly
    gx2 = capi.lif_bwd(x, g * 2.0, A, TH, BE, IV)
    assert torch.equal(gx2, gx * 2.0)


@pytest.mark.parametrize("pitched", [True, False])
def test_host_buffer_pipeline_matches_the_oracle(capi, pitched):
    """HostLifPipeline (pinned host tensors in, pinned host tensors out; chunks of the neuron axis on
    several streams; one pitched copy per slab or T row copies) gives the oracle's spikes and
    gradients, including a ragged last chunk."""
    from snn_gpu_training_bptt_b200.host_pipeline import HostLifPipeline
    T, N = 8, 3 * 4096 + 1234
    x, g = seeded_inputs(T, N, seed=31)
    hx, hg = x.view(T, N).contiguous().pin_memory(), g.view(T, N).contiguous().pin_memory()
    hs, hgx = torch.empty((T, N)).pin_memory(), torch.empty((T, N)).pin_memory()
    pipe = HostLifPipeline(T, N, torch.float32, chunk=4096, lanes=3, pitched=pitched)
    for _ in range(2):                                   # the second run reuses the staging buffers
        hs.fill_(float("nan")), hgx.fill_(float("nan"))
        pipe.run(hx, hg, hs, hgx, **CONSTS)
    s_ref, _ = orc.c_lif_fwd(hx.numpy())
    assert np.array_equal(hs.numpy(), s_ref)
    assert (hgx.numpy() == orc.c_lif_bwd(hx.numpy(), hg.numpy())).all()
