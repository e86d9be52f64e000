"""The bounded device-side waits: a wait that can never be satisfied ends the kernel with
WSL_ERR_TIMEOUT in the status words, and the CUDA context stays usable.

The failure is made without faulting anything: a test option of the library
(WSL_OPT_STALL_PRODUCER) makes the TMA producer skip filling the ring, so the MMA warp's wait
on the `full` barrier (a flag that nothing sets) runs into its bound (shortened to 0.2 s
here), records the status, raises the CTA's abort flag, and every role falls through to the
normal tear-down."""
import contextlib

import pytest
import torch

pytestmark = pytest.mark.gpu


@contextlib.contextmanager
def stalled_producer(limit_ms=200):
    from weightshared_torchtitan_b200 import _lib
    old = _lib.get_option(_lib.OPT_WAIT_LIMIT_MS)
    _lib.set_option(_lib.OPT_STALL_PRODUCER, 1)
    _lib.set_option(_lib.OPT_WAIT_LIMIT_MS, limit_ms)
    try:
        yield
    finally:
        _lib.set_option(_lib.OPT_STALL_PRODUCER, 0)
        _lib.set_option(_lib.OPT_WAIT_LIMIT_MS, old)


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
    with stalled_producer():
        ops.linear_fwd(x, W)            # one tile, one CTA; returns after the bound
        torch.cuda.synchronize()        # no CUDA error: the kernel ended by itself
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
    import torch.nn.functional as F
    from weightshared_torchtitan_b200 import _lib, ops
    if _lib.get_option(_lib.OPT_ROW_STAGED) == 0:
        pytest.skip("the option sends these calls to the direct kernels, which have no waits")
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
        with stalled_producer():
            call()
            torch.cuda.synchronize()        # no CUDA error: the kernel ended by itself
        st, words = _lib.poll_status()
        assert st == _lib.WSL_ERR_TIMEOUT, (st, words)
        assert words[1] == 4
        assert lib.wsl_reset_status() == 0
    y, _ = ops.rmsnorm_fwd(x, w, 1e-6)
    torch.cuda.synchronize()
    ref = F.rms_norm(x.float(), (1024,), w, 1e-6)
    assert ((y.float() - ref).abs().max() / ref.abs().max()).item() < 1e-2
    assert _lib.poll_status()[0] == 0
