"""The allocation-free weight-gradient entry point against the regular one.

Collected last on purpose (file name): if it fails under `-x`, every other test has run.

Who needs it: hosts that cannot allocate device memory around the call (all memory handed
out at start-up, a callback context, a language binding that only owns the tensors it was
given) and so cannot pass the split-K workspace that wsl_lora_linear_bwd_dw wants. The
variant keeps the partial sums in a fixed 64 MiB array inside the library. This test calls
it twice in a row through the C ABI -- the second call runs on top of the first call's
leftovers in the shared array -- and compares with the regular entry point given a
workspace from the framework's allocator.
"""
import pytest
import torch

from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


def test_noalloc_bwd_dw_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    from weightshared_torchtitan_b200 import _lib, ops
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems that both split the token contraction, so the second call
    # finds partial sums of another shape in the array
    for seed, (M, N, K, r) in enumerate([(8192, 256, 512, 16), (6144, 384, 256, 32)]):
        assert lib.wsl_bwd_dw_workspace_bytes(M, N, K, r, 1, 1, 1) > 0
        x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(40 + seed, M, N, K, r)]
        T = ops.lora_prepass(x, A, 2.0)
        U = ops.lora_bwd_prepass(dY, B, 2.0)
        ref = [torch.ones(N, K, device="cuda"), torch.ones(r, K, device="cuda"), torch.ones(N, r, device="cuda")]
        ops.lora_linear_bwd_dw(dY, U, x, T, *ref)
        for attempt in range(2):
            got = [torch.ones(N, K, device="cuda"), torch.ones(r, K, device="cuda"), torch.ones(N, r, device="cuda")]
            st = lib.wsl_lora_linear_bwd_dw_noalloc(dY.data_ptr(), N, U.data_ptr(), r, x.data_ptr(), K,
                                                    T.data_ptr(), r, got[0].data_ptr(), got[1].data_ptr(),
                                                    got[2].data_ptr(), M, N, K, r, stream)
            assert st == 0, _lib.status_string(st)
            torch.cuda.synchronize()
            for g, w, name in zip(got, ref, ("dW", "dA", "dB")):
                # same kernels and, at these sizes, the same split: tolerance of the fp32
                # parity tests (1e-5 max-relative)
                assert O.max_rel_err(g, w) < 1e-5, (seed, attempt, name, O.max_rel_err(g, w))
    # beyond the fixed array: a clear error, nothing launched
    big = torch.zeros(1, device="cuda")
    st = lib.wsl_lora_linear_bwd_dw_noalloc(big.data_ptr(), 4096, None, 0, big.data_ptr(), 4096, None, 0,
                                            big.data_ptr(), None, None, 128, 4096, 4096, 0, stream)
    assert st == _lib.WSL_ERR_TOO_LARGE
    st, words = _lib.poll_status()
    assert st == 0, words
