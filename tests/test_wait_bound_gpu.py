"""The bounded device-side waits: a wait that can never be satisfied ends the kernel with
WSL_ERR_TIMEOUT in the status words, and the CUDA context stays usable.

The failure is made without faulting anything: a debug switch of the library makes the TMA
producer skip filling the ring, so the MMA warp's wait on the `full` barrier (a flag that
nothing sets) runs into its bound (shortened to 0.2 s here), records the status, raises the
CTA's abort flag, and every role falls through to the normal tear-down."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_status_is_reported_and_context_survives():
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    from weightshared_torchtitan_b200 import _lib, ops
    lib = _lib.lib()
    torch.cuda.synchronize()
    assert lib.wsl_reset_status() == 0
    g = torch.Generator().manual_seed(0)
    x = torch.randn(128, 64, generator=g).cuda().to(torch.bfloat16)
    W = torch.randn(64, 64, generator=g).cuda().to(torch.bfloat16)
    os.environ["WSL_DBG"] = "64"
    os.environ["WSL_WAIT_LIMIT_MS"] = "200"
    try:
        ops.linear_fwd(x, W)            # one tile, one CTA; returns after the bound
        torch.cuda.synchronize()        # no CUDA error: the kernel ended by itself
    finally:
        del os.environ["WSL_DBG"]
        del os.environ["WSL_WAIT_LIMIT_MS"]
    st, words = _lib.poll_status()
    assert st == _lib.WSL_ERR_TIMEOUT, (st, words)
    assert words[1] in (1, 2, 3) and words[2] == 0
    assert "bounded" in _lib.status_string(st)
    # the context is intact: reset the words and compute for real
    assert lib.wsl_reset_status() == 0
    y = ops.linear_fwd(x, W)
    torch.cuda.synchronize()
    ref = x.float() @ W.float().T
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
    assert _lib.poll_status()[0] == 0


def test_row_kernel_wait_runs_out_and_context_survives():
    """Same for the staged RMSNorm kernels: with their producer warp kept idle, the compute
    warps' wait on the `full` barrier of the first stage runs into its bound, the kernel records
    role 4 and ends; afterwards the same call computes correctly."""
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    if os.environ.get("WSL_ROW_STAGED") == "0":
        pytest.skip("the diagnostic switch sends these calls to the direct kernels, which have no waits")
    import torch.nn.functional as F
    from weightshared_torchtitan_b200 import _lib, ops
    lib = _lib.lib()
    torch.cuda.synchronize()
    assert lib.wsl_reset_status() == 0
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 1024, generator=g).cuda().to(torch.bfloat16)
    dy = torch.randn(256, 1024, generator=g).cuda().to(torch.bfloat16)
    w = torch.ones(1024, device="cuda")
    _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
    for call in (lambda: ops.rmsnorm_fwd(x, w, 1e-6),
                 lambda: ops.rmsnorm_bwd(dy, x, w, rstd, torch.zeros(1024, device="cuda"))):
        os.environ["WSL_DBG"] = "64"
        os.environ["WSL_WAIT_LIMIT_MS"] = "200"
        try:
            call()
            torch.cuda.synchronize()        # no CUDA error: the kernel ended by itself
        finally:
            del os.environ["WSL_DBG"]
            del os.environ["WSL_WAIT_LIMIT_MS"]
        st, words = _lib.poll_status()
        assert st == _lib.WSL_ERR_TIMEOUT, (st, words)
        assert words[1] == 4
        assert lib.wsl_reset_status() == 0
    y, _ = ops.rmsnorm_fwd(x, w, 1e-6)
    torch.cuda.synchronize()
    ref = F.rms_norm(x.float(), (1024,), w, 1e-6)
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
    assert _lib.poll_status()[0] == 0
