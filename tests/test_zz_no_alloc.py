"""snn_lif_bwd_noalloc: the LIF backward for callers that must not allocate on the device.

Some hosts cannot call cudaMalloc where the backward pass runs (their own allocator owns the
whole GPU, or the call sits in a latency-critical loop, or a plugin sandbox only passes buffers
in and out). For them the library keeps the membrane scratch in an array compiled into it.
This file checks, through the C ABI, that the entry point gives exactly what snn_lif_bwd gives
and what the CPU oracle gives, on two calls in a row that reuse the shared array with different
problems, that it really leaves device memory alone, and that it refuses problems beyond the
array's size.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test. It also passes when run alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

A, TH, BE, IV = 0.25, 0.25, 1.0, 0.5


@pytest.fixture(scope="module")
def L(built_lib):
    assert torch.cuda.is_available()
    from snn_gpu_training_bptt_b200 import _capi
    return _capi.lib()


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _inputs(T, N, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    x = (0.5 + torch.randn((T, N), generator=gen)).to(dtype).cuda()
    g = torch.randn((T, N), generator=gen).to(dtype).cuda()
    return x, g


def _existing(L, x, g, code):
    """Result of the existing entry point (caller-provided scratch when T > 32)."""
    T, N = x.shape
    out = torch.empty_like(x)
    need = L.snn_lif_bwd_workspace_bytes(T, N, code)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
    rc = L.snn_lif_bwd(_p(x), _p(g), _p(out), T, N, code, A, TH, BE, IV, _p(ws) if need else None, need, _stream())
    assert rc == 0
    return out


def _oracle(x, g):
    """The CPU oracle's gradient, computed in the state type (fp32, or fp64 for fp64 tensors) on the
    exactly representable inputs and rounded to the tensors' element type, as the kernels do."""
    from oracle import lif_oracle as orc
    state = torch.float64 if x.dtype == torch.float64 else torch.float32
    want = orc.c_lif_bwd(x.cpu().to(state).numpy(), g.cpu().to(state).numpy(), A, TH, BE, IV)
    return torch.from_numpy(want).to(x.dtype)


def _noalloc(L, x, g, code):
    T, N = x.shape
    out = torch.full_like(x, float("nan"))
    rc = L.snn_lif_bwd_noalloc(_p(x), _p(g), _p(out), T, N, code, A, TH, BE, IV, _stream())
    assert rc == 0, L.snn_status_string(rc)
    return out


def test_two_calls_in_a_row_match_the_existing_entry_point(L):
    """A large long-T problem first, then a smaller, differently shaped one: the second call
    finds the first call's membrane values in the shared array and must not be affected."""
    cases = [(40, 100_000, 1, torch.float32, 0),     # T > 32: existing path uses caller scratch
             (8, 4099, 2, torch.float32, 0),         # T <= 32, odd N: existing path is register-resident
             (48, 2048, 3, torch.bfloat16, 1),
             (6, 65536, 4, torch.float64, 3)]
    for T, N, seed, dtype, code in cases:
        x, g = _inputs(T, N, seed, dtype)
        want = _existing(L, x, g, code)
        got = _noalloc(L, x, g, code)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (T, N, dtype)   # fp32 bar: exact (tolerance of the suite: 1e-4 rel)
        # and against the CPU oracle: equal in value (the oracle may emit -0.0 where the kernel emits +0.0)
        oracle = _oracle(x, g)
        assert bool((got.cpu() == oracle).all()), (T, N, dtype, "oracle")
    # same problem twice in a row gives the same bytes
    x, g = _inputs(40, 100_000, 1, torch.float32)
    assert torch.equal(_noalloc(L, x, g, 0), _noalloc(L, x, g, 0))


def test_device_memory_is_left_alone(L):
    x, g = _inputs(36, 50_000, 7, torch.float32)
    _noalloc(L, x, g, 0)                               # first call on the device: address look-up
    torch.cuda.synchronize()
    out = torch.empty_like(x)
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert L.snn_lif_bwd_noalloc(_p(x), _p(g), _p(out), 36, 50_000, 0, A, TH, BE, IV, _stream()) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_sizes_beyond_the_built_in_array_are_refused(L):
    from snn_gpu_training_bptt_b200 import _capi
    limit = _capi.STATIC_SCRATCH_BYTES // 4           # fp32 neuron-steps that fit
    x, g = _inputs(2, 8, 0, torch.float32)
    out = torch.empty_like(x)
    fake = ctypes.c_void_p(x.data_ptr())
    assert L.snn_lif_bwd_noalloc(fake, fake, _p(out), 64, limit // 64 + 1, 0, A, TH, BE, IV, None) == 8
    assert L.snn_lif_bwd_noalloc(fake, fake, _p(out), 1, limit + 1, 0, A, TH, BE, IV, None) == 8
    assert L.snn_lif_bwd_noalloc(fake, fake, _p(out), 8, limit // 8 // 2 + 1, 3, A, TH, BE, IV, None) == 8   # fp64 state
    assert b"built-in scratch" in L.snn_status_string(8)
    assert L.snn_lif_bwd_noalloc(None, fake, _p(out), 2, 8, 0, A, TH, BE, IV, None) == 1
    assert L.snn_lif_bwd_noalloc(fake, fake, _p(out), 0, 8, 0, A, TH, BE, IV, None) == 2
    # exactly at the limit is accepted
    T, N = 64, limit // 64
    xb, gb = _inputs(T, N, 5, torch.float32)
    got = _noalloc(L, xb, gb, 0)
    assert torch.equal(got, _existing(L, xb, gb, 0))
    assert bool((got.cpu() == _oracle(xb, gb)).all())


def test_python_wrapper_requires_preallocated_output(L):
    from snn_gpu_training_bptt_b200 import _capi
    x, g = _inputs(34, 1000, 9, torch.float32)
    out = torch.empty_like(x)
    assert _capi.lif_bwd_noalloc(x, g, out, A, TH, BE, IV) is out
    assert torch.equal(out, _existing(L, x, g, 0))
    with pytest.raises(_capi.SnnError):
        big = torch.empty((64, _capi.STATIC_SCRATCH_BYTES // 4 // 64 + 64), device="cuda")
        _capi.lif_bwd_noalloc(big, big, big, A, TH, BE, IV)
