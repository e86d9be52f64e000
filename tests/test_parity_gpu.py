"""GPU parity tests: the CUDA path, called through the C ABI, against the oracle and the
golden fixtures on the same seeded inputs.

Tolerances (per-tensor max|a-b| / max|b|, the metric of the baseline):
  bf16 inputs, fp32 accumulation : 1e-2
  fp32 mode                      : 1e-5
  embedding gather               : bit-exact
"""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
TOL_F32 = 1e-5


@pytest.fixture(scope="module")
def wsl():
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    from weightshared_torchtitan_b200 import _lib, ops
    _lib.lib()
    torch.backends.cuda.matmul.allow_tf32 = False
    yield ops
    torch.cuda.synchronize()
    st, words = _lib.poll_status()
    assert st == 0, f"device status {st} {words}"


def _t(a):
    return torch.from_numpy(np.asarray(a))


def rel(a, b):
    return O.max_rel_err(a, b)


def run_projection(ops, x, W, A, B, dY, s=2.0):
    """The five kernels of one projection; returns y, dX, dW, dA, dB (fp32 grads, from zero)."""
    T = ops.lora_prepass(x, A, s)
    y = ops.lora_linear_fwd(x, W, T, B)
    U = ops.lora_bwd_prepass(dY, B, s)
    dX = ops.lora_linear_bwd_dx([dY], [U], [W], [A])
    dW = torch.zeros(W.shape, device=x.device)
    dA = torch.zeros(A.shape, device=x.device)
    dB = torch.zeros(B.shape, device=x.device)
    ops.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB)
    return y, dX, dW, dA, dB


def oracle_projection(x, W, A, B, dY):
    return O.lora_linear_fwd_bwd(x.float().cpu(), W.float().cpu(), A.float().cpu(), B.float().cpu(),
                                 dY.float().cpu())


# ------------------------------------------------------------------ golden fixtures
@pytest.mark.parametrize("mode", ["f32", "bf16"])
def test_golden_small(wsl, golden_dir, mode):
    g = np.load(os.path.join(golden_dir, "lora_small.npz"))
    dt = torch.float32 if mode == "f32" else torch.bfloat16
    ins = [_t(g[k]).cuda().to(dt) for k in ("x", "W", "A", "B", "dY")]
    outs = run_projection(wsl, *ins)
    if mode == "f32":
        want = [_t(g[k]) for k in ("y", "dX", "dW", "dA", "dB")]
        tol = TOL_F32
    else:   # compare against the oracle evaluated on the bf16-rounded inputs
        want = oracle_projection(*ins)
        tol = TOL_BF16
    for got, w, name in zip(outs, want, ("y", "dX", "dW", "dA", "dB")):
        assert rel(got, w) < tol, (name, rel(got, w))


def test_golden_config0_fp32(wsl, golden_dir):
    """Baseline configuration 0 in fp32 mode: four layers share W and accumulate into ONE dW."""
    g = np.load(os.path.join(golden_dir, "lora_cfg0.npz"))
    inp = O.config0_inputs()
    W = inp["W"].cuda()
    dW = torch.zeros_like(W)
    for l in range(4):
        x, A, B, dY = (inp[k][l].cuda() for k in ("xs", "As", "Bs", "dYs"))
        T = wsl.lora_prepass(x, A, 2.0)
        y = wsl.lora_linear_fwd(x, W, T, B)
        U = wsl.lora_bwd_prepass(dY, B, 2.0)
        dX = wsl.lora_linear_bwd_dx([dY], [U], [W], [A])
        dA = torch.zeros_like(A)
        dB = torch.zeros_like(B)
        wsl.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB)
        assert rel(y[::97, ::89], _t(g[f"y{l}_s"])) < TOL_F32
        assert rel(dX[::97, ::89], _t(g[f"dX{l}_s"])) < TOL_F32
        assert rel(dA[:, ::7], _t(g[f"dA{l}"])) < TOL_F32
        assert rel(dB[::7], _t(g[f"dB{l}"])) < TOL_F32
        for t, key in ((y, f"y{l}_c"), (dX, f"dX{l}_c")):
            c = g[key]
            assert abs(t.double().abs().sum().item() - c[1]) <= 1e-5 * c[1], key
    assert rel(dW[::31, ::29], _t(g["dW_s"])) < TOL_F32
    c = g["dW_c"]
    assert abs(dW.double().abs().sum().item() - c[1]) <= 1e-5 * c[1]


def test_config0_bf16_against_oracle(wsl):
    inp = O.config0_inputs()
    bf = torch.bfloat16
    W = inp["W"].cuda().to(bf)
    dW = torch.zeros(W.shape, device="cuda")
    xs = [t.cuda().to(bf) for t in inp["xs"]]
    As = [t.cuda().to(bf) for t in inp["As"]]
    Bs = [t.cuda().to(bf) for t in inp["Bs"]]
    dYs = [t.cuda().to(bf) for t in inp["dYs"]]
    ys_o, dXs_o, dW_o, dAs_o, dBs_o = O.shared_w_layers_fwd_bwd(
        [t.float().cpu() for t in xs], W.float().cpu(), [t.float().cpu() for t in As],
        [t.float().cpu() for t in Bs], [t.float().cpu() for t in dYs])
    for l in range(4):
        T = wsl.lora_prepass(xs[l], As[l], 2.0)
        y = wsl.lora_linear_fwd(xs[l], W, T, Bs[l])
        U = wsl.lora_bwd_prepass(dYs[l], Bs[l], 2.0)
        dX = wsl.lora_linear_bwd_dx([dYs[l]], [U], [W], [As[l]])
        dA = torch.zeros(As[l].shape, device="cuda")
        dB = torch.zeros(Bs[l].shape, device="cuda")
        wsl.lora_linear_bwd_dw(dYs[l], U, xs[l], T, dW, dA, dB)
        for got, want, name in ((y, ys_o[l], "y"), (dX, dXs_o[l], "dX"), (dA, dAs_o[l], "dA"), (dB, dBs_o[l], "dB")):
            assert rel(got, want) < TOL_BF16, (l, name, rel(got, want))
    assert rel(dW, dW_o) < TOL_BF16


# ----------------------------------------------------------------- shapes and edges
SHAPES = [
    # M, N, K, r     (ragged M, narrow and wide N, every rank of the sweep, single row)
    (1, 64, 64, 8),
    (127, 1024, 1024, 16),
    (200, 328, 264, 8),
    (333, 3072, 1024, 16),
    (512, 1024, 3072, 32),
    (640, 2048, 2048, 64),
    (300, 2560, 1024, 128),
    (1000, 1024, 512, 48),
]


@pytest.mark.parametrize("M,N,K,r", SHAPES)
def test_projection_bf16_shapes(wsl, M, N, K, r):
    ins = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(100 + M + r, M, N, K, r)]
    outs = run_projection(wsl, *ins)
    want = oracle_projection(*ins)
    for got, w, name in zip(outs, want, ("y", "dX", "dW", "dA", "dB")):
        assert rel(got, w) < TOL_BF16, (name, rel(got, w))


@pytest.mark.parametrize("M,N,K,r", [(1, 64, 64, 8), (200, 328, 264, 8), (257, 520, 136, 20)])
def test_projection_fp32_shapes(wsl, M, N, K, r):
    ins = [t.cuda() for t in O.projection_inputs(7 + M, M, N, K, r)]
    outs = run_projection(wsl, *ins)
    want = oracle_projection(*ins)
    for got, w, name in zip(outs, want, ("y", "dX", "dW", "dA", "dB")):
        assert rel(got, w) < TOL_F32, (name, rel(got, w))


def test_grouped_dx_sums_projections(wsl):
    """q|k|v: one dX kernel contracts over all three projections (fp32 accumulate, one rounding)."""
    M, K, r = 384, 1024, 16
    g = torch.Generator().manual_seed(11)
    bf = torch.bfloat16
    Ns = (2048, 1024, 1024)
    dYs = [torch.randn(M, n, generator=g).cuda().to(bf) for n in Ns]
    Ws = [(torch.randn(n, K, generator=g) * 0.02).cuda().to(bf) for n in Ns]
    Us = [torch.randn(M, r, generator=g).cuda().to(bf) for _ in Ns]
    As = [(torch.randn(r, K, generator=g) * 0.03).cuda().to(bf) for _ in Ns]
    dX = wsl.lora_linear_bwd_dx(dYs, Us, Ws, As)
    want = sum(d.float().cpu() @ w.float().cpu() + u.float().cpu() @ a.float().cpu()
               for d, w, u, a in zip(dYs, Ws, Us, As))
    assert rel(dX, want) < TOL_BF16


def test_zero_B_and_scale_linearity(wsl):
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(5, 256, 512, 256, 16)]
    y0, _, _, dA0, _ = run_projection(wsl, x, W, A, torch.zeros_like(B), dY)
    assert torch.equal(y0, wsl.linear_fwd(x, W))       # B = 0: exactly the base projection
    assert dA0.abs().max().item() == 0.0               # and A receives no gradient
    # the adapter term is linear in s (s = 2 and s = 4 are exact scalings in bf16)
    T2, T4 = wsl.lora_prepass(x, A, 2.0), wsl.lora_prepass(x, A, 4.0)
    assert torch.equal(T4.float(), 2.0 * T2.float())


def test_rank_padding_invariance(wsl):
    """Zero-padding the adapter from r=8 to r=16 must not change any result."""
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(9, 256, 384, 320, 8)]
    A2 = torch.cat([A, torch.zeros_like(A)], 0)
    B2 = torch.cat([B, torch.zeros_like(B)], 1).contiguous()
    y, dX, dW, dA, dB = run_projection(wsl, x, W, A, B, dY)
    y2, dX2, dW2, dA2, dB2 = run_projection(wsl, x, W, A2, B2, dY)
    assert torch.equal(y, y2) and torch.equal(dX, dX2) and torch.equal(dW, dW2)
    assert torch.equal(dA, dA2[:8]) and dA2[8:].abs().max().item() == 0.0
    assert torch.equal(dB, dB2[:, :8]) and dB2[:, 8:].abs().max().item() == 0.0


def test_guard_bands_and_repeatability(wsl):
    """Outputs live inside larger sentinel-filled buffers: nothing outside the result may be
    written, and two runs on the same inputs must agree bit for bit."""
    M, N, K, r = 200, 328, 264, 8
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(21, M, N, K, r)]
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    pad = 16

    def guarded(rows, cols, dtype, fill):
        buf = torch.full((rows + 2 * pad, cols + 2 * pad), fill, device="cuda", dtype=dtype)
        return buf, buf[pad:pad + rows, pad:pad + cols]

    results = []
    for _ in range(2):
        Tb, T = guarded(M, r, torch.bfloat16, 7.0)
        yb, y = guarded(M, N, torch.bfloat16, 7.0)
        dWb, dW = guarded(N, K, torch.float32, 0.0)
        st = lib.wsl_lora_prepass(x.data_ptr(), K, A.data_ptr(), T.data_ptr(), Tb.stride(0), M, K, r, 2.0, 0, stream)
        assert st == 0
        st = lib.wsl_lora_linear_fwd(x.data_ptr(), K, W.data_ptr(), T.data_ptr(), Tb.stride(0), B.data_ptr(),
                                     y.data_ptr(), yb.stride(0), M, N, K, r, 0, stream)
        assert st == 0
        torch.cuda.synchronize()
        for buf, inner_rows, inner_cols in ((Tb, M, r), (yb, M, N)):
            mask = torch.ones_like(buf, dtype=torch.bool)
            mask[pad:pad + inner_rows, pad:pad + inner_cols] = False
            assert (buf[mask].float() == 7.0).all()
        results.append((T.clone(), y.clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    # dW accumulates deterministically: two identical accumulations give identical buffers
    U = wsl.lora_bwd_prepass(dY, B, 2.0)
    T = results[0][0].contiguous()
    outs = []
    for _ in range(2):
        dW = torch.zeros(N, K, device="cuda")
        dA = torch.zeros(r, K, device="cuda")
        dB = torch.zeros(N, r, device="cuda")
        wsl.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB)
        outs.append((dW, dA, dB))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_argument_errors_return_codes(wsl):
    """Bad arguments come back as status codes before any launch."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    x = torch.zeros(128, 72, device="cuda", dtype=torch.bfloat16)
    W = torch.zeros(64, 72, device="cuda", dtype=torch.bfloat16)
    y = torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)
    s = torch.cuda.current_stream().cuda_stream
    assert lib.wsl_linear_fwd(None, 72, W.data_ptr(), y.data_ptr(), 64, 128, 64, 72, 0, 0, s) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_linear_fwd(x.data_ptr(), 72, W.data_ptr(), y.data_ptr(), 64, 0, 64, 72, 0, 0, s) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_linear_fwd(x.data_ptr(), 72, W.data_ptr(), y.data_ptr(), 64, 128, 64, 72, 0, 5, s) == _lib.WSL_ERR_BAD_ARG
    # pitch not a multiple of 8 elements / pointer not 16-byte aligned
    assert lib.wsl_linear_fwd(x.data_ptr(), 73, W.data_ptr(), y.data_ptr(), 64, 128, 64, 72, 0, 0, s) == _lib.WSL_ERR_ALIGN
    assert lib.wsl_linear_fwd(x.data_ptr() + 2, 72, W.data_ptr(), y.data_ptr(), 64, 127, 64, 72, 0, 0, s) == _lib.WSL_ERR_ALIGN
    assert "alignment" in _lib.status_string(_lib.WSL_ERR_ALIGN)


# ---------------------------------------------------------------- embedding
def test_embedding_gather_is_bit_exact(wsl):
    g = torch.Generator().manual_seed(3)
    V, r_e = 151936, 256
    E = torch.randn(V, r_e, generator=g).cuda().to(torch.bfloat16)
    tok = torch.randint(0, V, (4, 1000), generator=g).cuda()
    G = wsl.embed_gather(tok, E)
    assert torch.equal(G, E[tok.reshape(-1)])
    # repeated and boundary ids
    tok2 = torch.tensor([0, V - 1, 5, 5, 5, V - 1], device="cuda")
    assert torch.equal(wsl.embed_gather(tok2, E), E[tok2])


@pytest.mark.parametrize("mode", ["f32", "bf16"])
def test_factorized_embedding_fwd_bwd(wsl, mode):
    from weightshared_torchtitan_b200.modules import factorized_embedding
    g = torch.Generator().manual_seed(4)
    V, r_e, d, M = 2048, 64, 192, 600
    dt = torch.float32 if mode == "f32" else torch.bfloat16
    tol = TOL_F32 if mode == "f32" else TOL_BF16
    E = torch.randn(V, r_e, generator=g).to(dt)
    P = (torch.randn(d, r_e, generator=g) * 0.05).to(dt)
    tok = torch.randint(0, 300, (M,), generator=g)      # many collisions
    dH = torch.randn(M, d, generator=g).to(dt)
    Eo, Po = E.float().clone().requires_grad_(True), P.float().clone().requires_grad_(True)
    ho = O.factorized_embedding(tok, Eo, Po)
    ho.backward(dH.float())
    Ec, Pc = E.detach().cuda().requires_grad_(True), P.detach().cuda().requires_grad_(True)
    h = factorized_embedding(tok.cuda(), Ec, Pc)
    h.backward(dH.cuda())
    assert rel(h, ho) < tol
    assert rel(Pc.grad, Po.grad) < tol
    assert rel(Ec.grad, Eo.grad) < tol


# ------------------------------------------------ baseline sizes, size-independent checks
def test_headline_shape_sampled_rows_and_linearity(wsl):
    """Configuration 4 MLP gate shape (M=16384, N=12288, K=4096, r=64): rows of y and dX and
    columns of dW against the oracle on a sample, plus linearity of the in-place dW."""
    M, N, K, r = 16384, 12288, 4096, 64
    g = torch.Generator(device="cuda").manual_seed(1238)
    bf = torch.bfloat16
    x = torch.randn(M, K, device="cuda", generator=g).to(bf)
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(bf)
    A = ((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf)
    B = (torch.randn(N, r, device="cuda", generator=g) * 0.02).to(bf)
    dY = torch.randn(M, N, device="cuda", generator=g).to(bf)
    T = wsl.lora_prepass(x, A, 2.0)
    y = wsl.lora_linear_fwd(x, W, T, B)
    U = wsl.lora_bwd_prepass(dY, B, 2.0)
    dX = wsl.lora_linear_bwd_dx([dY], [U], [W], [A])
    rows = torch.arange(0, M, 257, device="cuda")[:48]
    xr, dYr = x[rows].float().cpu(), dY[rows].float().cpu()
    Wc, Ac, Bc = W.float().cpu(), A.float().cpu(), B.float().cpu()
    y_o = O.lora_linear(xr, Wc, Ac, Bc)
    assert rel(y[rows], y_o) < TOL_BF16
    dX_o = dYr @ Wc + 2.0 * (dYr @ Bc) @ Ac
    assert rel(dX[rows], dX_o) < TOL_BF16
    dW = torch.zeros(N, K, device="cuda")
    dA = torch.zeros(r, K, device="cuda")
    dB = torch.zeros(N, r, device="cuda")
    wsl.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB)
    cols = torch.arange(0, N, 509, device="cuda")[:24]
    dW_o = dY[:, cols].float().T @ x.float()            # fp32 on the device for the big contraction
    assert rel(dW[cols], dW_o) < TOL_BF16
    assert rel(dB[cols], dY[:, cols].float().T @ T.float()) < TOL_BF16
    assert rel(dA, U.float().T @ x.float()) < TOL_BF16
    # accumulating the same contribution twice doubles the buffer exactly (in-place +=)
    before = dW.clone()
    wsl.lora_linear_bwd_dw(dY, U, x, T, dW, None, None)
    assert rel(dW, 2.0 * before) < 1e-6


def test_split_contraction_for_small_weight_grads(wsl):
    """Long token count, small weight: the dW kernel splits the token contraction across CTAs
    through a workspace and reduces in a fixed order. Result must match the oracle, must not
    depend on the run, and must agree with the unsplit kernel to fp32 rounding."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    M, N, K, r = 8192, 256, 512, 16
    assert lib.wsl_bwd_dw_workspace_bytes(M, N, K, r, 1, 1, 1) > 0     # this shape does split
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(31, M, N, K, r)]
    T = wsl.lora_prepass(x, A, 2.0)
    U = wsl.lora_bwd_prepass(dY, B, 2.0)
    runs = []
    for _ in range(2):
        dW = torch.ones(N, K, device="cuda")
        dA = torch.ones(r, K, device="cuda")
        dB = torch.ones(N, r, device="cuda")
        wsl.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB)
        runs.append((dW, dA, dB))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    s = torch.cuda.current_stream().cuda_stream
    dW0 = torch.ones(N, K, device="cuda")
    dA0 = torch.ones(r, K, device="cuda")
    dB0 = torch.ones(N, r, device="cuda")
    st = lib.wsl_lora_linear_bwd_dw(dY.data_ptr(), N, U.data_ptr(), r, x.data_ptr(), K, T.data_ptr(), r,
                                    dW0.data_ptr(), dA0.data_ptr(), dB0.data_ptr(), M, N, K, r, None, 0, 0, s)
    assert st == 0
    want = (1 + dY.float().T @ x.float(), 1 + U.float().T @ x.float(), 1 + dY.float().T @ T.float())
    for got, unsplit, w in zip(runs[0], (dW0, dA0, dB0), want):
        assert rel(got, w) < 1e-4 and rel(unsplit, w) < 1e-4


def test_split_tail_of_a_large_weight_gradient(wsl):
    """Large tile grid whose last wave is only partly full (242 tile pairs on 74 CTA pairs):
    the launch cuts only the tiles of that wave into split-K units. The workspace is then a
    fraction of the output; results match the oracle, are bit-reproducible, agree with the
    launch without a tail to fp32 rounding, and the grouped launch's bf16 copy G comes out of
    the folded sums. Ragged N so that the tail holds a partial tile. Launches that carry the
    narrow rank-r regions as well take no tail."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    M, N, K, r = 8192, 5632 - 24, 2816, 16
    ws = lib.wsl_bwd_dw_workspace_bytes(M, N, K, 0, 1, 0, 0)
    assert 0 < ws < N * K * 4                                   # a tail, not a split of everything
    assert lib.wsl_bwd_dw_workspace_bytes(M, N, K, r, 1, 1, 1) == 0
    g = torch.Generator().manual_seed(77)
    x = (torch.randn(M, K, generator=g) * 0.5).cuda().to(torch.bfloat16)
    dY = (torch.randn(M, N, generator=g) * 0.5).cuda().to(torch.bfloat16)
    want_dW = dY.float().T @ x.float()

    def run():
        dW = torch.ones(N, K, device="cuda")
        wsl.lora_linear_bwd_dw(dY, None, x, None, dW, None, None)
        return dW

    a, b = run(), run()
    assert torch.equal(a, b)
    _lib.set_option(_lib.OPT_SPLIT_TAIL, 0)
    try:
        assert lib.wsl_bwd_dw_workspace_bytes(M, N, K, 0, 1, 0, 0) == 0
        plain = run()
    finally:
        _lib.set_option(_lib.OPT_SPLIT_TAIL, 1)
    assert rel(a, 1 + want_dW) < 1e-4 and rel(plain, 1 + want_dW) < 1e-4 and rel(a, plain) < 1e-5
    assert not torch.equal(a, plain)                            # the tail did sum in another order
    # grouped launch with the bf16 copy: two projections reading the same x
    Ns = (3072, N - 3072)
    ll = ctypes.c_longlong * 2
    assert 0 < lib.wsl_bwd_dw_group_workspace_bytes(2, ll(*Ns), ll(0, 0), M, K) < N * K * 4
    dYs = [dY[:, :Ns[0]].contiguous(), dY[:, Ns[0]:].contiguous()]
    dWs = [torch.ones(n, K, device="cuda") for n in Ns]
    Gs = wsl.bwd_dw_layer_group(dYs, x, dWs)
    off = 0
    for n, dWp, G in zip(Ns, dWs, Gs):
        w = want_dW[off:off + n]
        assert rel(dWp, 1 + w) < 1e-4
        assert rel(G.float(), w) < TOL_BF16
        assert torch.equal(G, (dWp - 1).to(torch.bfloat16)) or rel(G.float(), dWp - 1) < 4e-3
        off += n
    # a weight too short for CTA pairs (N < 512): 192 single-CTA tiles on 148 SMs, same treatment
    M2, N2, K2 = 8192, 448, 12288
    ws2 = lib.wsl_bwd_dw_workspace_bytes(M2, N2, K2, 0, 1, 0, 0)
    assert 0 < ws2 and ws2 % (N2 * K2 * 4) != 0 and ws2 % (128 * 256 * 4) == 0
    x2 = (torch.randn(M2, K2, generator=g) * 0.5).cuda().to(torch.bfloat16)
    dY2 = (torch.randn(M2, N2, generator=g) * 0.5).cuda().to(torch.bfloat16)
    dW2 = torch.ones(N2, K2, device="cuda")
    wsl.lora_linear_bwd_dw(dY2, None, x2, None, dW2, None, None)
    assert rel(dW2, 1 + dY2.float().T @ x2.float()) < 1e-4


def test_fused_embedding_gathers_exact_rows(wsl):
    """The TMA-gather GEMM (wsl_embed_fwd) with P = [I ; 0]: h[:, :r_e] must be E_small[tokens]
    bit for bit (indices exact), ragged token count, repeated ids, full vocabulary size."""
    g = torch.Generator().manual_seed(8)
    V, r_e, d, M = 151936, 256, 512, 1000
    E = torch.randn(V, r_e, generator=g).cuda().to(torch.bfloat16)
    tok = torch.randint(0, V, (M,), generator=g).cuda()
    tok[:6] = torch.tensor([0, V - 1, 7, 7, 7, V - 1], device="cuda")
    P = torch.zeros(d, r_e, device="cuda", dtype=torch.bfloat16)
    P[:r_e] = torch.eye(r_e, device="cuda", dtype=torch.bfloat16)
    h = wsl.embed_fwd(tok, E, P)
    assert torch.equal(h[:, :r_e], E[tok])
    assert h[:, r_e:].abs().max().item() == 0.0
    # same product through the stand-alone gather + GEMM
    P2 = (torch.randn(d, r_e, generator=g) * 0.05).cuda().to(torch.bfloat16)
    ref = wsl.linear_fwd(wsl.embed_gather(tok, E), P2)
    assert rel(wsl.embed_fwd(tok, E, P2), ref) < 1e-6
    # projection gradient with the gather in the contraction
    dH = torch.randn(M, d, generator=g).cuda().to(torch.bfloat16)
    dP = torch.zeros(d, r_e, device="cuda")
    wsl.embed_bwd_dproj(tok, dH, E, dP)
    assert rel(dP, dH.float().T @ E[tok].float()) < 1e-4


def test_random_shapes_against_oracle(wsl):
    """Seeded random shapes (multiples of 8, ragged against every tile size) for the whole
    projection fwd+bwd in bf16; covers both the 1-CTA and the CTA-pair variants."""
    import random
    rnd = random.Random(20260101)
    for case in range(10):
        M = rnd.choice([8, 72, 136, 520, 776, 1288, 2056])
        N = 8 * rnd.randint(2, 160)
        K = 8 * rnd.randint(2, 160)
        r = rnd.choice([8, 16, 24, 32, 64])
        ins = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(500 + case, M, N, K, r)]
        outs = run_projection(wsl, *ins)
        want = oracle_projection(*ins)
        for got, w, name in zip(outs, want, ("y", "dX", "dW", "dA", "dB")):
            assert rel(got, w) < TOL_BF16, (case, (M, N, K, r), name, rel(got, w))


def test_dx_mixed_segments(wsl):
    """dX over projections with and without an adapter (r = 0 for one of them) and different
    widths: the segment list is built per projection."""
    g = torch.Generator().manual_seed(77)
    bf = torch.bfloat16
    M, K = 640, 512
    Ns, rs = (768, 256, 1024), (16, 0, 32)
    dYs = [torch.randn(M, n, generator=g).cuda().to(bf) for n in Ns]
    Ws = [(torch.randn(n, K, generator=g) * 0.03).cuda().to(bf) for n in Ns]
    Us = [torch.randn(M, r, generator=g).cuda().to(bf) if r else None for r in rs]
    As = [(torch.randn(r, K, generator=g) * 0.05).cuda().to(bf) if r else None for r in rs]
    dX = wsl.lora_linear_bwd_dx(dYs, Us, Ws, As)
    want = sum(d.float().cpu() @ w.float().cpu() for d, w in zip(dYs, Ws))
    want = want + sum(u.float().cpu() @ a.float().cpu() for u, a in zip(Us, As) if u is not None)
    assert rel(dX, want) < TOL_BF16


def test_grouped_weight_gradients_match_single_launches(wsl):
    """q|k|v in one dW launch (9 regions) against three single-projection launches."""
    g = torch.Generator().manual_seed(91)
    bf = torch.bfloat16
    M, K, r = 4096, 512, 16
    Ns = (1024, 256, 256)
    x = torch.randn(M, K, generator=g).cuda().to(bf)
    dYs = [torch.randn(M, n, generator=g).cuda().to(bf) for n in Ns]
    Us = [torch.randn(M, r, generator=g).cuda().to(bf) for _ in Ns]
    T_cat = torch.randn(M, 3 * r, generator=g).cuda().to(bf)
    Ts = [T_cat[:, i * r:(i + 1) * r] for i in range(3)]
    one = [[torch.ones(n, K, device="cuda"), torch.ones(r, K, device="cuda"), torch.ones(n, r, device="cuda")] for n in Ns]
    grp = [[torch.ones(n, K, device="cuda"), torch.ones(r, K, device="cuda"), torch.ones(n, r, device="cuda")] for n in Ns]
    for p in range(3):
        wsl.lora_linear_bwd_dw(dYs[p], Us[p], x, Ts[p], *one[p])
    wsl.lora_linear_bwd_dw_group(dYs, Us, x, Ts, [t[0] for t in grp], [t[1] for t in grp], [t[2] for t in grp])
    for p in range(3):
        want = (1 + dYs[p].float().T @ x.float(), 1 + Us[p].float().T @ x.float(), 1 + dYs[p].float().T @ Ts[p].float())
        for a, b, w in zip(one[p], grp[p], want):
            assert rel(b, w) < 1e-4 and rel(a, b) < 1e-5


def test_grouped_forward_matches_single_launches(wsl):
    """q|k|v forward in one launch (3 regions x 2 segments) is bit-identical to three
    single-projection launches."""
    g = torch.Generator().manual_seed(92)
    bf = torch.bfloat16
    M, K, r = 1000, 512, 16
    Ns = (1024, 256, 264)
    x = torch.randn(M, K, generator=g).cuda().to(bf)
    Ws = [(torch.randn(n, K, generator=g) * 0.03).cuda().to(bf) for n in Ns]
    Bs = [(torch.randn(n, r, generator=g) * 0.1).cuda().to(bf) for n in Ns]
    A_cat = (torch.randn(3 * r, K, generator=g) * 0.05).cuda().to(bf)
    T_cat = wsl.lora_prepass(x, A_cat, 2.0)
    Ts = [T_cat[:, i * r:(i + 1) * r] for i in range(3)]
    ys = wsl.lora_linear_fwd_group(x, Ws, Ts, Bs)
    for p in range(3):
        assert torch.equal(ys[p], wsl.lora_linear_fwd(x, Ws[p], Ts[p], Bs[p]))
        ref = x.float() @ Ws[p].float().T + Ts[p].float() @ Bs[p].float().T
        assert rel(ys[p], ref) < TOL_BF16


# ------------------------------------------- backward through the layer's own weight gradient
def test_merge_weight(wsl):
    """W_eff = bf16(W + s B A) against the same sum in fp32 (one rounding either way: at most
    one bf16 ulp apart)."""
    g = torch.Generator().manual_seed(101)
    bf = torch.bfloat16
    # the last shape is large enough for the 4-rows-per-thread variant, with a ragged row count
    for N, K, r in [(1024, 1024, 16), (264, 520, 8), (3072, 1024, 64), (4102, 2560, 16)]:
        W = (torch.randn(N, K, generator=g) * 0.03).cuda().to(bf)
        A = (torch.randn(r, K, generator=g) * 0.05).cuda().to(bf)
        B = (torch.randn(N, r, generator=g) * 0.1).cuda().to(bf)
        got = wsl.lora_merge_weight([W], [A], [B], 2.0)[0]
        want = W.float() + 2.0 * (B.float() @ A.float())
        assert got.dtype == bf and got.shape == W.shape
        # 1e-6: elements where W and s B A nearly cancel see the fp32 summation order
        assert bool(((got.float() - want).abs() <= want.abs() * 2.0 ** -7 + 1e-6).all())
    # q|k|v in one launch, different widths and ranks
    Ns, rs, K = (1024, 256, 262), (8, 8, 8), 512
    Ws = [(torch.randn(n, K, generator=g) * 0.03).cuda().to(bf) for n in Ns]
    As = [(torch.randn(r, K, generator=g) * 0.05).cuda().to(bf) for r in rs]
    Bs = [(torch.randn(n, r, generator=g) * 0.1).cuda().to(bf) for n, r in zip(Ns, rs)]
    outs = wsl.lora_merge_weight(Ws, As, Bs, 2.0)
    for p in range(3):
        assert torch.equal(outs[p], wsl.lora_merge_weight([Ws[p]], [As[p]], [Bs[p]], 2.0)[0])
        want = Ws[p].float() + 2.0 * (Bs[p].float() @ As[p].float())
        assert rel(outs[p], want) < 4e-3


@pytest.mark.parametrize("M,K,Ns", [(8192, 512, (1024, 256, 256)),      # split contraction
                                    (1024, 2048, (2048, 2048)),         # whole tiles, staged epilogue
                                    (1000, 520, (264,))])               # ragged edges
def test_layer_weight_gradient_with_copy(wsl, M, K, Ns):
    """dW += dY^T x in place and, from the same launch, the bf16 matrix dY^T x of this call
    alone."""
    g = torch.Generator().manual_seed(M + K)
    bf = torch.bfloat16
    x = torch.randn(M, K, generator=g).cuda().to(bf)
    dYs = [torch.randn(M, n, generator=g).cuda().to(bf) for n in Ns]
    dWs = [torch.full((n, K), 3.0, device="cuda") for n in Ns]
    dWls = wsl.bwd_dw_layer_group(dYs, x, dWs)
    for p, n in enumerate(Ns):
        want = dYs[p].float().T @ x.float()
        assert rel(dWs[p] - 3.0, want) < 1e-4
        assert dWls[p].dtype == bf and dWls[p].shape == (n, K)
        assert rel(dWls[p], want) < TOL_BF16
        # the copy is the fp32 addend rounded once
        assert rel(dWls[p].float(), (dWs[p] - 3.0).to(bf).float()) < 1e-2


@pytest.mark.parametrize("Ns", [(1024, 256, 256), (512, 512), (264,)])
def test_adapter_gradients_from_layer_gradient(wsl, Ns):
    """dA = s B^T G and dB = s G A^T with G = dY^T x against the oracle's autograd."""
    g = torch.Generator().manual_seed(sum(Ns))
    bf = torch.bfloat16
    M, K, r, s = 2048, 520, 16, 2.0
    x = (torch.randn(M, K, generator=g)).to(bf)
    dWs, dAs, dBs, want = [], [], [], []
    dYs, As, Bs = [], [], []
    for n in Ns:
        W = (torch.randn(n, K, generator=g) * 0.03).to(bf)
        A = (torch.randn(r, K, generator=g) * 0.05).to(bf)
        B = (torch.randn(n, r, generator=g) * 0.1).to(bf)
        dY = (torch.randn(M, n, generator=g) * 0.1).to(bf)
        want.append(oracle_projection(x, W, A, B, dY))
        dYs.append(dY.cuda()); As.append(A.cuda()); Bs.append(B.cuda())
        dWs.append(torch.zeros(n, K, device="cuda"))
        dAs.append(torch.full((r, K), 1.0, device="cuda"))
        dBs.append(torch.full((n, r), 1.0, device="cuda"))
    dWls = wsl.bwd_dw_layer_group(dYs, x.cuda(), dWs)
    wsl.lora_adapter_grads_from_dw(dWls, As, Bs, dAs, dBs, s)
    for p in range(len(Ns)):
        _, _, dW_o, dA_o, dB_o = want[p]
        assert rel(dWs[p], dW_o) < TOL_BF16
        assert rel(dAs[p] - 1.0, dA_o) < TOL_BF16
        assert rel(dBs[p] - 1.0, dB_o) < TOL_BF16


@pytest.mark.parametrize("P", [1, 3])
def test_autograd_function_both_backward_formulations(wsl, P):
    """LoRALinearGroupFunction with in-place sinks: the backward through the layer's weight
    gradient and the direct one (U = s dY B) both match the oracle."""
    from weightshared_torchtitan_b200 import functional as Fn
    g = torch.Generator().manual_seed(7 + P)
    bf = torch.bfloat16
    M, K, r, s = 1536, 512, 16, 2.0
    Ns = (1024, 256, 256)[:P]
    x = torch.randn(M, K, generator=g).to(bf)
    Ws = [(torch.randn(n, K, generator=g) * 0.03).to(bf) for n in Ns]
    As = [(torch.randn(r, K, generator=g) * 0.05).to(bf) for n in Ns]
    Bs = [(torch.randn(n, r, generator=g) * 0.1).to(bf) for n in Ns]
    dYs = [(torch.randn(M, n, generator=g) * 0.1).to(bf) for n in Ns]
    want = [oracle_projection(x, Ws[p], As[p], Bs[p], dYs[p]) for p in range(P)]
    dX_want = sum(w[1] for w in want)
    saved = Fn.DERIVED_ADAPTER_GRADS
    try:
        for derived in (True, False):
            Fn.DERIVED_ADAPTER_GRADS = derived
            xc = x.cuda().requires_grad_(True)
            sinks = [(torch.zeros(n, K, device="cuda"), torch.zeros(r, K, device="cuda"),
                      torch.zeros(n, r, device="cuda")) for n in Ns]
            ys = Fn.lora_linear_group(xc, [w.cuda() for w in Ws], [a.cuda() for a in As],
                                      [b.cuda() for b in Bs], s, sinks)
            torch.autograd.backward(list(ys), [d.cuda() for d in dYs])
            assert rel(xc.grad, dX_want) < TOL_BF16
            for p in range(P):
                assert rel(ys[p], want[p][0]) < TOL_BF16
                for got, ref in zip(sinks[p], want[p][2:]):
                    assert rel(got, ref) < TOL_BF16
    finally:
        Fn.DERIVED_ADAPTER_GRADS = saved


def test_adapter_gradients_of_a_whole_layer_in_one_call(wsl):
    """The seven projections of a decoder layer (three different input widths, four output
    widths) in ONE adapter-gradient call: regions with shorter contractions than the launch's
    read as zeros beyond their end."""
    g = torch.Generator().manual_seed(2024)
    bf = torch.bfloat16
    r, s = 16, 2.0
    shapes = [(512, 256), (256, 256), (256, 256), (256, 512), (768, 256), (768, 256), (256, 768)]   # (N, K)
    Gs = [torch.randn(n, k, generator=g).cuda().to(bf) for n, k in shapes]
    As = [(torch.randn(r, k, generator=g) * 0.05).cuda().to(bf) for n, k in shapes]
    Bs = [(torch.randn(n, r, generator=g) * 0.1).cuda().to(bf) for n, k in shapes]
    dAs = [torch.full((r, k), 0.5, device="cuda") for n, k in shapes]
    dBs = [torch.full((n, r), 0.5, device="cuda") for n, k in shapes]
    wsl.lora_adapter_grads_from_dw(Gs, As, Bs, dAs, dBs, s)
    for p in range(len(shapes)):
        assert rel(dAs[p] - 0.5, s * Bs[p].float().T @ Gs[p].float()) < 1e-4
        assert rel(dBs[p] - 0.5, s * Gs[p].float() @ As[p].float().T) < 1e-4


def test_adapter_gradient_batch_with_a_group_on_the_direct_formulation(wsl):
    """One group goes through its weight gradient, the other computes dA/dB directly: the
    second still reports to the batch, which therefore runs as soon as both are done (inside
    the backward pass, not from the end-of-pass callback)."""
    from weightshared_torchtitan_b200 import functional as Fn
    g = torch.Generator().manual_seed(77)
    bf = torch.bfloat16
    M, K, r, s = 1024, 512, 16, 2.0
    x = torch.randn(M, K, generator=g).to(bf)
    xc = x.cuda().requires_grad_(True)
    batch = Fn.AdapterGradBatch(2)
    saved = Fn.DERIVED_ADAPTER_GRADS
    outs, dYs_all, all_sinks, want = [], [], [], []
    try:
        for n, derived in ((768, True), (256, False)):
            Fn.DERIVED_ADAPTER_GRADS = derived
            W = (torch.randn(n, K, generator=g) * 0.03).to(bf)
            A = (torch.randn(r, K, generator=g) * 0.05).to(bf)
            B = (torch.randn(n, r, generator=g) * 0.1).to(bf)
            dY = (torch.randn(M, n, generator=g) * 0.1).to(bf)
            want.append(oracle_projection(x, W, A, B, dY))
            sinks = [(torch.zeros(n, K, device="cuda"), torch.zeros(r, K, device="cuda"),
                      torch.zeros(n, r, device="cuda"))]
            outs += list(Fn.lora_linear_group(xc, [W.cuda()], [A.cuda()], [B.cuda()], s, sinks, (), batch))
            dYs_all.append(dY.cuda())
            all_sinks += sinks
    finally:
        Fn.DERIVED_ADAPTER_GRADS = saved
    flushed_inside = []
    real_flush = batch.flush
    batch.flush = lambda: (flushed_inside.append(len(batch.pending)), real_flush())[1]
    torch.autograd.backward(outs, dYs_all)
    assert flushed_inside and flushed_inside[0] == 1 and not batch.pending
    assert rel(xc.grad, sum(w[1] for w in want)) < TOL_BF16
    for sk, w in zip(all_sinks, want):
        for got, ref in zip(sk, w[2:]):
            assert rel(got, ref) < TOL_BF16


@pytest.mark.parametrize("expected", [2, 3])
def test_adapter_gradient_batch_across_groups(wsl, expected):
    """Two projection groups share an AdapterGradBatch: with expected = 2 it runs when the
    second group reports, with expected = 3 (one group never reports) at the end of the
    backward pass. Either way the gradients match the oracle."""
    from weightshared_torchtitan_b200 import functional as Fn
    g = torch.Generator().manual_seed(55 + expected)
    bf = torch.bfloat16
    M, K, r, s = 1024, 512, 16, 2.0
    groups = [(1024, 256), (768,)]
    x = torch.randn(M, K, generator=g).to(bf)
    batch = Fn.AdapterGradBatch(expected)
    xc = x.cuda().requires_grad_(True)
    outs, all_sinks, want, dYs_all = [], [], [], []
    saved = Fn.DERIVED_ADAPTER_GRADS
    Fn.DERIVED_ADAPTER_GRADS = True   # small shapes: force the formulation under test
    launches = []
    real = wsl.lora_adapter_grads_from_dw
    for Ns in groups:
        Ws = [(torch.randn(n, K, generator=g) * 0.03).to(bf) for n in Ns]
        As = [(torch.randn(r, K, generator=g) * 0.05).to(bf) for n in Ns]
        Bs = [(torch.randn(n, r, generator=g) * 0.1).to(bf) for n in Ns]
        dYs = [(torch.randn(M, n, generator=g) * 0.1).to(bf) for n in Ns]
        want += [oracle_projection(x, Ws[p], As[p], Bs[p], dYs[p]) for p in range(len(Ns))]
        sinks = [(torch.zeros(n, K, device="cuda"), torch.zeros(r, K, device="cuda"),
                  torch.zeros(n, r, device="cuda")) for n in Ns]
        ys = Fn.lora_linear_group(xc, [w.cuda() for w in Ws], [a.cuda() for a in As],
                                  [b.cuda() for b in Bs], s, sinks, (), batch)
        outs += list(ys)
        dYs_all += [d.cuda() for d in dYs]
        all_sinks += sinks
    Fn.DERIVED_ADAPTER_GRADS = saved

    def counting(dWls, *a, **k):
        launches.append(len(dWls))
        return real(dWls, *a, **k)

    wsl.lora_adapter_grads_from_dw = counting
    try:
        torch.autograd.backward(outs, dYs_all)
    finally:
        wsl.lora_adapter_grads_from_dw = real
    assert launches == [3]          # all three projections of the two groups in ONE call
    assert not batch.pending
    assert rel(xc.grad, sum(w[1] for w in want)) < TOL_BF16
    for sk, w in zip(all_sinks, want):
        for got, ref in zip(sk, w[2:]):
            assert rel(got, ref) < TOL_BF16


def test_empty_batch_launches_nothing(wsl):
    """Zero tokens: outputs of the right shape, zero gradients, no kernel launch, sinks untouched."""
    from weightshared_torchtitan_b200 import _lib
    from weightshared_torchtitan_b200 import functional as Fn
    bf = torch.bfloat16
    K, r = 64, 8
    Ns = (128, 64)
    x = torch.zeros(0, K, device="cuda", dtype=bf, requires_grad=True)
    Ws = [torch.randn(n, K, device="cuda").to(bf) for n in Ns]
    As = [torch.randn(r, K, device="cuda").to(bf) for n in Ns]
    Bs = [torch.randn(n, r, device="cuda").to(bf) for n in Ns]
    sinks = [(torch.ones(n, K, device="cuda"), torch.ones(r, K, device="cuda"), torch.ones(n, r, device="cuda"))
             for n in Ns]
    before = _lib.launch_count()
    ys = Fn.lora_linear_group(x, Ws, As, Bs, 2.0, sinks)
    assert [tuple(y.shape) for y in ys] == [(0, n) for n in Ns]
    torch.autograd.backward(list(ys), [torch.zeros_like(y) for y in ys])
    assert x.grad.shape == (0, K)
    w = torch.ones(K, device="cuda", requires_grad=True)
    n = Fn.rmsnorm(x.detach().requires_grad_(True), w, 1e-6)
    n.sum().backward()
    assert n.shape == (0, K) and float(w.grad.abs().sum()) == 0.0
    g = Fn.swiglu(x.detach().requires_grad_(True), x.detach())
    g.sum().backward()
    assert _lib.launch_count() == before
    for t in sinks:
        for buf in t:
            assert float((buf - 1.0).abs().sum()) == 0.0


# ------------------------------------ projection shapes of baseline configurations 2, 3 and 4
@pytest.mark.parametrize("M,N,K,r", [
    (2048, 6144, 2048, 32),     # configuration 2: gate/up
    (2048, 2048, 6144, 32),     # configuration 2: down
    (2048, 9728, 2560, 64),     # configuration 3: gate/up
    (2048, 2560, 9728, 64),     # configuration 3: down
    (2048, 4096, 2560, 64),     # configuration 3: q
    (2048, 1024, 4096, 64),     # configuration 4: k/v
])
def test_projection_shapes_of_the_baseline_configurations(wsl, M, N, K, r):
    """The five kernels at the true N, K, r of configurations 2-4 (2048 token rows) against the
    CPU oracle evaluated on the same bf16-rounded inputs."""
    ins = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(60 + r, M, N, K, r)]
    outs = run_projection(wsl, *ins)
    want = oracle_projection(*ins)
    for got, w, name in zip(outs, want, ("y", "dX", "dW", "dA", "dB")):
        assert rel(got, w) < TOL_BF16, (name, rel(got, w))


def test_headline_down_shape_sampled_rows_against_oracle(wsl):
    """Configuration 4 MLP down shape (M=16384, N=4096, K=12288, r=64: 192 k-blocks forward, another
    split plan than the gate shape): sampled rows of y and dX, sampled output rows of dW, dB and all
    of dA against the CPU oracle's arithmetic on the same bf16 values (fp64 on the host for the
    16384-token contractions of the sampled rows)."""
    M, N, K, r = 16384, 4096, 12288, 64
    g = torch.Generator(device="cuda").manual_seed(1239)
    bf = torch.bfloat16
    x = torch.randn(M, K, device="cuda", generator=g).to(bf)
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(bf)
    A = ((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf)
    B = (torch.randn(N, r, device="cuda", generator=g) * 0.02).to(bf)
    dY = torch.randn(M, N, device="cuda", generator=g).to(bf)
    y, dX, dW, dA, dB = run_projection(wsl, x, W, A, B, dY)
    rows = torch.arange(0, M, 331, device="cuda")[:48]
    xr, dYr = x[rows].float().cpu(), dY[rows].float().cpu()
    Wc, Ac, Bc = W.float().cpu(), A.float().cpu(), B.float().cpu()
    assert rel(y[rows], O.lora_linear(xr, Wc, Ac, Bc)) < TOL_BF16
    assert rel(dX[rows], dYr @ Wc + 2.0 * (dYr @ Bc) @ Ac) < TOL_BF16
    # weight gradients of sampled output rows: the oracle's formulas dW = dY^T x, dB = s dY^T (x A^T),
    # dA = s (dY B)^T x on the host in fp64
    cols = torch.arange(0, N, 173, device="cuda")[:24]
    xd, dYd = x.double().cpu(), dY[:, cols].double().cpu()
    assert rel(dW[cols], dYd.T @ xd) < TOL_BF16
    Td = 2.0 * (xd @ A.double().cpu().T)
    assert rel(dB[cols], dYd.T @ Td) < TOL_BF16
    Ud = 2.0 * (dY.double().cpu() @ B.double().cpu())
    assert rel(dA, Ud.T @ xd) < TOL_BF16


def test_merged_weight_route_with_a_small_adapter(wsl):
    """Backward through the merged weight W_eff = bf16(W + s B A) when the adapter is tiny
    (B scaled by 1e-3, the regime right after the reference's zero initialisation of B): the
    adapter's share of dX falls below W's bf16 resolution there, which the tolerance on dX (a
    per-tensor maximum) absorbs; dA, which is carried by that share alone in the direct
    formulation, must still come out right because it is computed from G = dY^T x and B."""
    M, N, K, r = 4096, 512, 1024, 16
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(71, M, N, K, r)]
    B = (B.float() * 1e-3).to(torch.bfloat16)
    want = oracle_projection(x, W, A, B, dY)
    W_eff = wsl.lora_merge_weight([W], [A], [B], 2.0)[0]
    dX = wsl.lora_linear_bwd_dx([dY], [None], [W_eff], [None])
    dW = torch.zeros(N, K, device="cuda")
    dA = torch.zeros(r, K, device="cuda")
    dB = torch.zeros(N, r, device="cuda")
    G = wsl.bwd_dw_layer_group([dY], x, [dW])
    wsl.lora_adapter_grads_from_dw(G, [A], [B], [dA], [dB], 2.0)
    for got, w, name in zip((dX, dW, dA, dB), want[1:], ("dX", "dW", "dA", "dB")):
        assert rel(got, w) < TOL_BF16, (name, rel(got, w))


# ------------------------------------------------- gate|up GEMM with the SwiGLU epilogue
@pytest.mark.parametrize("M,N,K,r", [(1024, 256, 512, 16), (640, 384, 328, 8), (2048, 3072, 1024, 16),
                                     (1000, 1280, 2560, 64), (512, 128, 64, 0)])
def test_gate_up_swiglu_one_launch_matches_the_separate_kernels(wsl, M, N, K, r):
    """wsl_lora_swiglu_fwd against wsl_lora_linear_fwd_group + wsl_swiglu_fwd: g, u and
    h = silu(g) * u must be the same bits (the fused epilogue rounds g and u to bf16 before the
    activation, as a pass over the stored matrices would), and h must agree with the oracle's
    F.silu(w1 x) * w3 x within the bf16 tolerance. Ragged M and K, ranks 0 to 64."""
    assert wsl.lora_swiglu_supported(M, N, K, r)
    g_ = torch.Generator().manual_seed(90 + r)
    bf = torch.bfloat16
    x = torch.randn(M, K, generator=g_).cuda().to(bf)
    Wg = (torch.randn(N, K, generator=g_) * 0.05).cuda().to(bf)
    Wu = (torch.randn(N, K, generator=g_) * 0.05).cuda().to(bf)
    if r:
        Ag = ((torch.rand(r, K, generator=g_) * 2 - 1) / K ** 0.5).cuda().to(bf)
        Au = ((torch.rand(r, K, generator=g_) * 2 - 1) / K ** 0.5).cuda().to(bf)
        Bg = (torch.randn(N, r, generator=g_) * 0.05).cuda().to(bf)
        Bu = (torch.randn(N, r, generator=g_) * 0.05).cuda().to(bf)
        T_cat = wsl.lora_prepass(x, torch.cat((Ag, Au)), 2.0)
        g1, u1, h1 = wsl.lora_swiglu_fwd(x, Wg, Wu, T_cat, Bg, Bu)
        g0, u0 = wsl.lora_linear_fwd_group(x, [Wg, Wu], [T_cat[:, :r], T_cat[:, r:]], [Bg, Bu])
        want_g = O.lora_linear(x.float().cpu(), Wg.float().cpu(), Ag.float().cpu(), Bg.float().cpu())
        want_u = O.lora_linear(x.float().cpu(), Wu.float().cpu(), Au.float().cpu(), Bu.float().cpu())
    else:
        g1, u1, h1 = wsl.lora_swiglu_fwd(x, Wg, Wu, None, None, None)
        g0, u0 = wsl.linear_fwd(x, Wg), wsl.linear_fwd(x, Wu)
        want_g, want_u = x.float().cpu() @ Wg.float().cpu().T, x.float().cpu() @ Wu.float().cpu().T
    h0 = wsl.swiglu_fwd(g0, u0)
    assert torch.equal(g1, g0) and torch.equal(u1, u0)
    assert torch.equal(h1, h0)
    assert rel(g1, want_g) < TOL_BF16 and rel(u1, want_u) < TOL_BF16
    assert rel(h1, torch.nn.functional.silu(want_g) * want_u) < TOL_BF16


def test_gate_up_swiglu_function_gradients_match_the_unfused_composition(wsl):
    """The autograd Function of the fused MLP front half against lora_linear_group + swiglu:
    same output bits and the same in-place gradients, for both backward formulations."""
    from weightshared_torchtitan_b200 import functional as Fn
    M, N, K, r = 2048, 768, 512, 16
    gen = torch.Generator().manual_seed(123)
    bf = torch.bfloat16
    x0 = torch.randn(M, K, generator=gen).cuda().to(bf)
    Ws = [(torch.randn(N, K, generator=gen) * 0.05).cuda().to(bf) for _ in range(2)]
    As = [((torch.rand(r, K, generator=gen) * 2 - 1) / K ** 0.5).cuda().to(bf) for _ in range(2)]
    Bs = [(torch.randn(N, r, generator=gen) * 0.05).cuda().to(bf) for _ in range(2)]
    dh = torch.randn(M, N, generator=gen).cuda().to(bf)
    saved = Fn.DERIVED_ADAPTER_GRADS
    try:
        for flag in (False, True):
            Fn.DERIVED_ADAPTER_GRADS = flag
            res = []
            for fused in (True, False):
                x = x0.clone().requires_grad_(True)
                sinks = [(torch.zeros(N, K, device="cuda"), torch.zeros(r, K, device="cuda"),
                          torch.zeros(N, r, device="cuda")) for _ in range(2)]
                if fused:
                    h = Fn.lora_gate_up_swiglu(x, Ws, As, Bs, 2.0, sinks)
                else:
                    gate, up = Fn.lora_linear_group(x, Ws, As, Bs, 2.0, sinks)
                    h = Fn.swiglu(gate, up)
                h.backward(dh)
                res.append((h.detach(), x.grad, sinks))
            (h1, dx1, s1), (h0, dx0, s0) = res
            assert torch.equal(h1, h0) and torch.equal(dx1, dx0)
            for a, b in zip(s1, s0):
                for ta, tb in zip(a, b):
                    assert torch.equal(ta, tb)
    finally:
        Fn.DERIVED_ADAPTER_GRADS = saved


def test_first_library_call_of_a_fresh_thread(wsl):
    """A thread whose very first CUDA-related action is one of this library's GEMM launches (an
    autograd worker starting a backward pass with cached allocations) has no driver context bound
    yet; encoding a tensor map there must bind it instead of failing."""
    import threading
    x, W, A, B, dY = [t.cuda().to(torch.bfloat16) for t in O.projection_inputs(5, 640, 256, 192, 16)]
    want = wsl.linear_fwd(x, W)
    x2 = x.clone()          # new address: its tensor map is not in the library's cache yet
    torch.cuda.synchronize()
    out = {}

    def work():
        try:
            out["y"] = wsl.linear_fwd(x2, W)
            torch.cuda.synchronize()
        except Exception as e:      # noqa: BLE001
            out["err"] = e

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "err" not in out, out.get("err")
    assert torch.equal(out["y"], want)


def test_mlp_function_matches_the_unfused_composition(wsl):
    """The whole-MLP autograd node (activation in the gate|up epilogue, its backward in the
    epilogue of the down projection's input-gradient GEMM) against lora_gate_up_swiglu +
    lora_linear_group + the stand-alone SwiGLU backward kernel: same output bits, same dX bits and
    the same in-place gradients, for both backward formulations; and y against the oracle."""
    from weightshared_torchtitan_b200 import functional as Fn
    M, N, K, r = 1536, 768, 512, 16           # N = inner width of the MLP, K = model width
    gen = torch.Generator().manual_seed(321)
    bf = torch.bfloat16
    x0 = torch.randn(M, K, generator=gen).cuda().to(bf)
    Ws = [(torch.randn(N, K, generator=gen) * 0.05).cuda().to(bf) for _ in range(2)]
    Ws.append((torch.randn(K, N, generator=gen) * 0.05).cuda().to(bf))
    As = [((torch.rand(r, K, generator=gen) * 2 - 1) / K ** 0.5).cuda().to(bf) for _ in range(2)]
    As.append(((torch.rand(r, N, generator=gen) * 2 - 1) / N ** 0.5).cuda().to(bf))
    Bs = [(torch.randn(N, r, generator=gen) * 0.05).cuda().to(bf) for _ in range(2)]
    Bs.append((torch.randn(K, r, generator=gen) * 0.05).cuda().to(bf))
    dy = torch.randn(M, K, generator=gen).cuda().to(bf)
    assert wsl.swiglu_bwd_in_dx_supported(M, K, N, r) and wsl.lora_swiglu_supported(M, N, K, r)

    def sinks():
        return [(torch.zeros(W.shape, device="cuda"), torch.zeros(A.shape, device="cuda"),
                 torch.zeros(B.shape, device="cuda")) for W, A, B in zip(Ws, As, Bs)]

    saved, saved_fuse = Fn.DERIVED_ADAPTER_GRADS, Fn.FUSE_SWIGLU_BWD
    try:
        for flag in (False, True):
            Fn.DERIVED_ADAPTER_GRADS = flag
            Fn.FUSE_SWIGLU_BWD = True          # the epilogue form, whatever "auto" would pick at this width
            res = []
            for fused in (True, False):
                x = x0.clone().requires_grad_(True)
                sk = sinks()
                if fused:
                    y = Fn.lora_mlp(x, Ws, As, Bs, 2.0, sk)
                else:
                    act = Fn.lora_gate_up_swiglu(x, Ws[:2], As[:2], Bs[:2], 2.0, sk[:2])
                    y = Fn.lora_linear_group(act, [Ws[2]], [As[2]], [Bs[2]], 2.0, sk[2:])[0]
                y.backward(dy)
                res.append((y.detach(), x.grad, sk))
            (y1, dx1, s1), (y0, dx0, s0) = res
            assert torch.equal(y1, y0) and torch.equal(dx1, dx0)
            for a, b in zip(s1, s0):
                for ta, tb in zip(a, b):
                    assert torch.equal(ta, tb)
    finally:
        Fn.DERIVED_ADAPTER_GRADS, Fn.FUSE_SWIGLU_BWD = saved, saved_fuse
    xc = x0.float().cpu()
    gate = O.lora_linear(xc, Ws[0].float().cpu(), As[0].float().cpu(), Bs[0].float().cpu())
    up = O.lora_linear(xc, Ws[1].float().cpu(), As[1].float().cpu(), Bs[1].float().cpu())
    want = O.lora_linear(torch.nn.functional.silu(gate) * up, Ws[2].float().cpu(), As[2].float().cpu(),
                         Bs[2].float().cpu())
    assert rel(y1, want) < 2 * TOL_BF16       # two roundings of the hidden activation on the way


@pytest.mark.parametrize("M,N,K,r", [(1024, 256, 512, 16), (777, 328, 1280, 64), (2048, 1024, 3072, 0)])
def test_dx_with_swiglu_backward_epilogue_matches_two_kernels(wsl, M, N, K, r):
    """wsl_lora_linear_bwd_dx_swiglu against wsl_lora_linear_bwd_dx + wsl_swiglu_bwd, bit for bit;
    ragged M, contraction not a multiple of the k-block, with and without the rank-r segment."""
    assert wsl.swiglu_bwd_in_dx_supported(M, N, K, r)
    gen = torch.Generator().manual_seed(55 + r)
    bf = torch.bfloat16
    dY = torch.randn(M, N, generator=gen).cuda().to(bf)
    W = (torch.randn(N, K, generator=gen) * 0.05).cuda().to(bf)
    g = torch.randn(M, K, generator=gen).cuda().to(bf)
    u = torch.randn(M, K, generator=gen).cuda().to(bf)
    if r:
        U = torch.randn(M, r, generator=gen).cuda().to(bf)
        A = (torch.randn(r, K, generator=gen) * 0.05).cuda().to(bf)
        dg1, du1 = wsl.lora_linear_bwd_dx_swiglu(dY, U, W, A, g, u)
        dh = wsl.lora_linear_bwd_dx([dY], [U], [W], [A])
    else:
        dg1, du1 = wsl.lora_linear_bwd_dx_swiglu(dY, None, W, None, g, u)
        dh = wsl.lora_linear_bwd_dx([dY], [None], [W], [None])
    dg0, du0 = wsl.swiglu_bwd(dh, g, u)
    assert torch.equal(dg1, dg0) and torch.equal(du1, du0)
