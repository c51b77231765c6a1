"""The C-ABI boundary, checked without a GPU: the library loads, exports every symbol that
include/snn_b200.h declares, and validates arguments before it would launch anything."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "snn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(snn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path():
    names = _declared_symbols()
    for required in ("snn_lif_fwd", "snn_lif_bwd", "snn_lif_bwd_workspace_bytes", "snn_version"):
        assert required in names


def test_library_exports_every_declared_symbol(built_lib):
    handle = ctypes.CDLL(built_lib)
    for name in _declared_symbols():
        assert hasattr(handle, name), f"{name} declared in snn_b200.h but not exported"


def test_binding_table_matches_header(built_lib):
    from snn_gpu_training_bptt_b200 import _capi
    assert sorted(_capi.SIGNATURES) == _declared_symbols()
    assert _capi.lib().snn_version() >= 100


def test_argument_validation_needs_no_gpu(built_lib):
    """Every bad call returns its status before any CUDA call is made."""
    from snn_gpu_training_bptt_b200 import _capi
    L = _capi.lib()
    p = ctypes.c_void_p
    fake, odd = p(0x1000), p(0x1002)
    # forward
    assert L.snn_lif_fwd(None, fake, None, None, 8, 16, 0, 0.25, 0.25, None) == 1        # NULL x
    assert L.snn_lif_fwd(fake, None, None, None, 8, 16, 0, 0.25, 0.25, None) == 1        # no output
    assert L.snn_lif_fwd(fake, fake, None, None, 0, 16, 0, 0.25, 0.25, None) == 2        # T < 1
    assert L.snn_lif_fwd(fake, fake, None, None, 8, -1, 0, 0.25, 0.25, None) == 2        # N < 0
    assert L.snn_lif_fwd(fake, fake, None, None, 8, 16, 9, 0.25, 0.25, None) == 3        # dtype
    assert L.snn_lif_fwd(odd, fake, None, None, 8, 16, 0, 0.25, 0.25, None) == 4         # misaligned fp32
    assert L.snn_lif_fwd(fake, None, None, fake, 33, 16, 0, 0.25, 0.25, None) == 5       # bits beyond 32 steps
    assert L.snn_lif_fwd(fake, fake, None, None, 8, 0, 0, 0.25, 0.25, None) == 0         # empty: ok, nothing to do
    # backward
    assert L.snn_lif_bwd(fake, None, fake, 8, 16, 0, 0.25, 0.25, 1.0, 0.5, None, 0, None) == 1
    assert L.snn_lif_bwd(fake, fake, fake, 8, 16, 7, 0.25, 0.25, 1.0, 0.5, None, 0, None) == 3
    assert L.snn_lif_bwd(fake, fake, fake, 40, 16, 0, 0.25, 0.25, 1.0, 0.5, None, 0, None) == 6   # long T, no scratch
    assert L.snn_lif_bwd(fake, fake, fake, 40, 16, 0, 0.25, 0.25, 1.0, 0.5, fake, 100, None) == 6  # scratch too small
    assert L.snn_lif_bwd(fake, fake, fake, 8, 0, 0, 0.25, 0.25, 1.0, 0.5, None, 0, None) == 0
    # workspace query
    assert L.snn_lif_bwd_workspace_bytes(8, 1 << 26, 0) == 0
    assert L.snn_lif_bwd_workspace_bytes(32, 1000, 1) == 0
    assert L.snn_lif_bwd_workspace_bytes(33, 1000, 1) == 33 * 1000 * 4
    assert L.snn_lif_bwd_workspace_bytes(64, 10, 3) == 64 * 10 * 8
    assert L.snn_lif_bwd_workspace_bytes(0, 10, 0) == -2
    # LIF of a sum
    assert L.snn_lif_add_fwd(fake, None, fake, 8, 16, 0, 0.25, 0.25, None) == 1                  # NULL shortcut
    assert L.snn_lif_add_fwd(fake, fake, fake, 0, 16, 0, 0.25, 0.25, None) == 2
    assert L.snn_lif_add_fwd(fake, fake, fake, 8, 16, 3, 0.25, 0.25, None) == 5                  # no float64 form
    assert L.snn_lif_add_fwd(fake, odd, fake, 8, 16, 0, 0.25, 0.25, None) == 4
    assert L.snn_lif_add_fwd(fake, fake, fake, 8, 0, 0, 0.25, 0.25, None) == 0
    assert L.snn_lif_add_bwd(fake, fake, None, fake, 8, 16, 1, 0.25, 0.25, 1.0, 0.5, None) == 1
    assert L.snn_lif_add_bwd(fake, fake, fake, fake, 17, 16, 1, 0.25, 0.25, 1.0, 0.5, None) == 5  # T beyond the register form
    assert L.snn_lif_add_bwd(fake, fake, fake, fake, 8, 16, 9, 0.25, 0.25, 1.0, 0.5, None) == 3
    # unpack
    assert L.snn_spike_unpack(None, fake, 8, 16, 0, None) == 1
    assert L.snn_spike_unpack(fake, fake, 40, 16, 0, None) == 5
    assert L.snn_status_string(6).decode().startswith("workspace")


def test_linear_lif_kernel_plan(built_lib):
    """Kernel choice of the fused linear + LIF forward is host logic: no GPU needed. 0 = 128x128
    tiles, 1 = 128x256 tiles, 2 = CTA pair, -1 = unsupported."""
    from snn_gpu_training_bptt_b200 import _capi
    L = _capi.lib()
    BF16, F32 = 1, 0
    plan = lambda T, B, K, M, sms=148, dt=BF16: L.snn_linear_lif_fwd_plan(T, B, K, M, dt, sms)
    assert plan(8, 256, 2048, 2048) == 1             # the reference-sized layer: 128 wide tiles, one round
    assert plan(8, 1024, 2048, 2048) == 2            # 512 wide tiles on 148 SMs: the pair takes over
    assert plan(8, 4096, 2048, 2048) == 2
    assert plan(8, 512, 2048, 2048) == 1             # 256 wide tiles < 2 per SM: still single CTAs
    assert plan(8, 32, 256, 256) == 0                # everything fits in one round either way
    assert plan(8, 48, 1024, 384) == 0               # batch not a multiple of 32: no wide tiles
    assert plan(4, 64, 512, 128) == 0                # T=4 needs 64 batch items per wide tile; one round
    assert plan(4, 1024, 256, 2048) == 1
    assert plan(8, 2048, 128, 128 * 17) == 1         # odd number of 128-row tiles: no pair
    assert plan(8, 1024, 2048, 2048, sms=16) == 2    # fewer SMs: more tiles each
    assert plan(8, 256, 2048, 2048, sms=32) == 2
    assert plan(8, 256, 2048, 2048, dt=F32) == -1
    assert plan(6, 256, 2048, 2048) == 1             # 6 steps run in the 8-step tile
    assert plan(16, 512, 128, 2048) == 2
    assert plan(2, 128, 128, 128) == 0
    assert plan(3, 64, 64, 128) == 0
    assert plan(3, 48, 64, 128) == -1                # 4-step tile: batch must be a multiple of 32
    assert plan(1, 256, 2048, 2048) == -1
    assert plan(17, 256, 2048, 2048) == -1
    assert plan(8, 256, 2048, 2048, sms=0) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from snn_gpu_training_bptt_b200 import _capi
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", str(tmp_path / "libsnn_b200.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _capi.lib()


def test_cpu_tensors_are_rejected(built_lib):
    import torch
    from snn_gpu_training_bptt_b200 import snnlib
    x = torch.zeros(4, 2, 8)
    with pytest.raises(ValueError, match="CUDA"):
        snnlib.fire_s_fp(x, 0.25, 0.25)
    with pytest.raises(ValueError, match="CUDA"):
        snnlib.fire_bp(x, x, 0.25, 0.25, 1.0, 0.5)
    from snn_gpu_training_bptt_b200 import snnlib_func as sf
    with pytest.raises(ValueError, match="CUDA"):
        sf.fire_add_func(x, x)


def test_linear_lif_backward_host_logic(built_lib):
    """Support test and workspace size of the fused linear + LIF backward are host logic (no GPU):
    bf16 only, T <= 16, at least 128 (t, b) rows, K and M multiples of 64; the workspace holds dU
    (bf16 [T, B, M]) plus one fp32 row of bias partials per block of batch items, 256-byte aligned."""
    from snn_gpu_training_bptt_b200 import _capi
    L = _capi.lib()
    ok = lambda T, B, K, M, dt=1: L.snn_linear_lif_bwd_supported(T, B, K, M, dt)
    assert ok(8, 256, 2048, 2048) == 1 and ok(1, 128, 64, 128) == 1 and ok(16, 8, 64, 128) == 1
    assert ok(8, 256, 2048, 2048, dt=0) == 0          # fp32 operands
    assert ok(17, 256, 2048, 2048) == 0               # time axis beyond the register-resident reverse pass
    assert ok(8, 8, 2048, 2048) == 0                  # 64 (t, b) rows: less than one tile
    assert ok(8, 256, 2048 + 8, 2048) == 0 and ok(8, 256, 2048, 2048 + 32) == 0
    assert ok(8, 256, 32, 2048) == 0 and ok(8, 256, 2048, 64) == 0
    align = lambda v: (v + 255) // 256 * 256
    for T, B, K, M, rows_per_block in ((8, 256, 2048, 2048, 16), (4, 100, 64, 192, 16), (16, 40, 128, 128, 8), (12, 24, 64, 256, 8)):
        want = align(T * B * M * 2) + align(-(-B // rows_per_block) * M * 4)
        assert L.snn_linear_lif_bwd_workspace_bytes(T, B, K, M, 1) == want, (T, B, K, M)
    assert L.snn_linear_lif_bwd_workspace_bytes(8, 8, 2048, 2048, 1) < 0
    # argument checks that need no device: nothing is launched on a non-zero status
    assert L.snn_linear_lif_bwd(None, None, None, None, None, None, None, 8, 256, 2048, 2048, 0, 0,
                                0.25, 0.25, 1.0, 0.5, None, 0, None) == 5
    assert L.snn_linear_lif_bwd(None, None, None, None, None, None, None, 8, 256, 2048, 2048, 1, 2,
                                0.25, 0.25, 1.0, 0.5, None, 0, None) == 3      # grad_weight dtype f16
    assert L.snn_linear_lif_bwd(None, None, None, None, None, None, None, 8, 256, 2048, 2048, 1, 0,
                                0.25, 0.25, 1.0, 0.5, None, 0, None) == 1      # current / grad_spike missing
    assert L.snn_copy_rows_async(None, 16, None, 16, 16, 4, 1, None) == 1
    assert L.snn_copy_rows_async(None, 16, None, 16, 16, 0, 1, None) == 0       # nothing to copy
    assert L.snn_copy_rows_async(ctypes.c_void_p(256), 8, ctypes.c_void_p(512), 16, 16, 4, 1, None) == 2   # pitch < row
