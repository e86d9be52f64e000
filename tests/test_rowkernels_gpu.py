"""GPU parity of the row kernels either side of the projections (softmax cross-entropy,
SwiGLU, RMSNorm with fused rotary embedding) against the oracle's eager PyTorch
formulas. Tolerances: 1e-2 for bf16 storage; in fp32 1e-5 for cross-entropy and SwiGLU and
3e-5 for the norm kernels (their scale gradient is summed with fp32 atomics in no fixed
order, and the rotary tables come from the device's cos/sin)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import lora_oracle as O

pytestmark = pytest.mark.gpu


def rel(a, b):
    return O.max_rel_err(a, b)


def leaf(t, device="cpu", dtype=None):
    """A fresh leaf tensor (never an alias of its source) that requires grad."""
    t = t.detach().to(device=device, dtype=dtype if dtype is not None else t.dtype, copy=True)
    return t.requires_grad_(True)


@pytest.fixture(scope="module", autouse=True)
def _dev():
    if not torch.cuda.is_available():
        pytest.fail("gpu tests need a CUDA device")
    yield
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype,V,tol", [(torch.float32, 1003, 1e-5), (torch.float32, 4096, 1e-5),
                                          (torch.bfloat16, 151936, 1e-2), (torch.bfloat16, 1003, 1e-2)])
def test_cross_entropy_forward_and_gradient(dtype, V, tol):
    from weightshared_torchtitan_b200 import ops
    g = torch.Generator().manual_seed(V)
    rows = 37
    ld = (V + 7) // 8 * 8
    buf = torch.zeros(rows, ld)
    buf[:, :V] = torch.randn(rows, V, generator=g) * 3
    labels = torch.randint(0, V, (rows,), generator=g)
    labels[5] = -100                      # ignored row, as F.cross_entropy's ignore_index
    logits = buf.to(dtype).cuda()
    ref_in = leaf(logits[:, :V], "cpu", torch.float32)
    ref = F.cross_entropy(ref_in, labels, reduction="none", ignore_index=-100)
    scale = 1.0 / 36
    (ref.sum() * scale).backward()
    view = logits[:, :V]
    row_loss = ops.ce_fwd_bwd(view, labels.cuda(), scale)
    assert rel(row_loss, ref.detach()) < max(tol, 1e-5)
    assert row_loss[5].item() == 0.0 and view[5].abs().max().item() == 0.0
    assert rel(view, ref_in.grad) < tol
    if ld > V:
        assert logits[:, V:].abs().max().item() == 0.0     # pitch padding untouched


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_swiglu(dtype, tol):
    from weightshared_torchtitan_b200.functional import swiglu
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(300, 3072, generator=g) * 2).to(dtype)
    b = torch.randn(300, 3072, generator=g).to(dtype)
    d = torch.randn(300, 3072, generator=g).to(dtype)
    ar, br = leaf(a, dtype=torch.float32), leaf(b, dtype=torch.float32)
    (F.silu(ar) * br).backward(d.float())
    ac, bc = leaf(a, "cuda"), leaf(b, "cuda")
    out = swiglu(ac, bc)
    out.backward(d.cuda())
    assert rel(out, F.silu(ar) * br) < tol
    assert rel(ac.grad, ar.grad) < tol and rel(bc.grad, br.grad) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("D", [16, 64, 128, 1024, 2048, 2560, 4096])
def test_rmsnorm(dtype, tol, D):
    from weightshared_torchtitan_b200 import ops
    from weightshared_torchtitan_b200.functional import rmsnorm
    if dtype == torch.float32 and D > 1024:
        assert not ops.rmsnorm_supported(D, dtype)
        return
    assert ops.rmsnorm_supported(D, dtype)
    g = torch.Generator().manual_seed(D)
    rows = 333
    x = torch.randn(rows, D, generator=g).to(dtype)
    w = 1.0 + 0.2 * torch.randn(D, generator=g)
    dy = torch.randn(rows, D, generator=g).to(dtype)
    xr, wr = leaf(x, dtype=torch.float32), leaf(w)
    yr = F.rms_norm(xr, (D,), wr, 1e-6)
    yr.backward(dy.float())
    xc, wc = leaf(x, "cuda"), leaf(w, "cuda")
    y = rmsnorm(xc, wc, 1e-6)
    y.backward(dy.cuda())
    assert rel(y, yr) < tol and rel(xc.grad, xr.grad) < tol
    assert rel(wc.grad, wr.grad) < tol
    # in-place sink: gradient of the scale accumulates into a caller buffer
    sink = torch.ones(D, device="cuda")
    xc2 = leaf(x, "cuda")
    rmsnorm(xc2, wc.detach(), 1e-6, None, sink).backward(dy.cuda())
    assert rel(sink - 1.0, wr.grad) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("D,heads", [(128, 16), (128, 8), (16, 4), (64, 2)])
def test_head_norm_with_rotary(dtype, tol, D, heads):
    """q/k head RMSNorm followed by the rotary embedding, against the oracle's formulas
    (rms_norm, then apply_rope on [b, s, h, d])."""
    from weightshared_torchtitan_b200.decoder import rope_tables
    from weightshared_torchtitan_b200.functional import rmsnorm
    g = torch.Generator().manual_seed(D + heads)
    b, s = 2, 37
    x = torch.randn(b, s, heads, D, generator=g).to(dtype)
    w = 1.0 + 0.2 * torch.randn(D, generator=g)
    dy = torch.randn(b, s, heads, D, generator=g).to(dtype)
    cache = O.rope_cache(D, s, 1_000_000.0)
    xr, wr = leaf(x, dtype=torch.float32), leaf(w)
    n = F.rms_norm(xr, (D,), wr, 1e-6)
    yr, _ = O.apply_rope(n, n, cache)
    yr.backward(dy.float())
    cos, sin = rope_tables(D, s, 1_000_000.0, "cuda")
    xc, wc = leaf(x, "cuda"), leaf(w, "cuda")
    y = rmsnorm(xc, wc, 1e-6, (cos.contiguous(), sin.contiguous(), heads, s))
    y.backward(dy.cuda())
    assert rel(y, yr) < tol and rel(xc.grad, xr.grad) < tol
    assert rel(wc.grad, wr.grad) < tol


@pytest.mark.parametrize("D,rows,heads", [(128, 100_003, 0), (128, 80_000, 16), (1024, 9_477, 0),
                                          (2048, 5_000, 0), (256, 40_001, 0), (2560, 4_003, 0),
                                          (4096, 3_001, 0)])
def test_rmsnorm_backward_over_many_tiles(D, rows, heads):
    """Row counts at which every CTA of the staged backward walks its ring of shared-memory
    stages several times (so the barrier phases flip) and the last tile is ragged."""
    from weightshared_torchtitan_b200.decoder import rope_tables
    from weightshared_torchtitan_b200.functional import rmsnorm
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, D, generator=g).to(torch.bfloat16)
    w = 1.0 + 0.2 * torch.randn(D, generator=g)
    dy = torch.randn(rows, D, generator=g).to(torch.bfloat16)
    xr, wr = leaf(x, "cuda", dtype=torch.float32), leaf(w, "cuda")
    n = F.rms_norm(xr, (D,), wr, 1e-6)
    rope = None
    if heads:
        s = rows // heads // 2
        cache = O.rope_cache(D, s, 1_000_000.0).cuda()
        n, _ = O.apply_rope(n.view(2, s, heads, D), n.view(2, s, heads, D), cache)
        n = n.reshape(rows, D)
        cos, sin = rope_tables(D, s, 1_000_000.0, "cuda")
        rope = (cos.contiguous(), sin.contiguous(), heads, s)
    n.backward(dy.cuda().float())
    xc, wc = leaf(x, "cuda"), leaf(w, "cuda")
    y = rmsnorm(xc, wc, 1e-6, rope)
    y.backward(dy.cuda())
    assert rel(y, n) < 1e-2 and rel(xc.grad, xr.grad) < 1e-2
    assert rel(wc.grad, wr.grad) < 1e-2


def test_rmsnorm_strided_rows_take_the_direct_kernel():
    """Rows with a pitch larger than their width cannot be bulk-copied as dense tiles; the
    entry points accept them and must give the same result as dense rows."""
    from weightshared_torchtitan_b200 import ops
    g = torch.Generator().manual_seed(5)
    rows, D = 777, 1024
    xw = torch.randn(rows, D + 64, generator=g).to(torch.bfloat16).cuda()
    dyw = torch.randn(rows, D + 64, generator=g).to(torch.bfloat16).cuda()
    w = (1.0 + 0.2 * torch.randn(D, generator=g)).cuda()
    x_s, dy_s = xw[:, :D], dyw[:, :D]
    y_s, rstd_s = ops.rmsnorm_fwd(x_s, w, 1e-6)
    y_d, rstd_d = ops.rmsnorm_fwd(x_s.contiguous(), w, 1e-6)
    assert rel(y_s, y_d) < 1e-2 and rel(rstd_s, rstd_d) < 1e-6
    dw_s, dw_d = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    dx_s = ops.rmsnorm_bwd(dy_s, x_s, w, rstd_s, dw_s)
    dx_d = ops.rmsnorm_bwd(dy_s.contiguous(), x_s.contiguous(), w, rstd_d, dw_d)
    # two kernels, two summation orders: equal up to the bf16 rounding of y and dx
    assert rel(dx_s, dx_d) < 1e-2
    assert rel(dw_s, dw_d) < 1e-4


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("D,rows", [(1024, 333), (2048, 5_003), (256, 40_001), (64, 77), (2560, 3_001),
                                    (4096, 2_005)])
def test_residual_add_folded_into_the_norm(dtype, tol, D, rows):
    """h = x + res and y = RMSNorm(h) in one kernel; the backward adds the gradient of the
    residual stream to the norm's dx. Against the same three steps in fp32 PyTorch; h must be
    exactly the sum rounded once."""
    from weightshared_torchtitan_b200 import ops
    from weightshared_torchtitan_b200.functional import add_rmsnorm
    if not ops.rmsnorm_supported(D, dtype):
        pytest.skip("width not covered in this dtype")
    g = torch.Generator().manual_seed(D + rows)
    x = torch.randn(rows, D, generator=g).to(dtype)
    res = torch.randn(rows, D, generator=g).to(dtype)
    w = 1.0 + 0.2 * torch.randn(D, generator=g)
    dh = torch.randn(rows, D, generator=g).to(dtype)
    dy = torch.randn(rows, D, generator=g).to(dtype)
    xr, rr, wr = leaf(x, "cuda", dtype=torch.float32), leaf(res, "cuda", dtype=torch.float32), leaf(w, "cuda")
    hr = (xr + rr).to(dtype).float()          # the rounding an add kernel applies
    hr_exact = xr + rr
    yr = F.rms_norm(hr_exact, (D,), wr, 1e-6)
    torch.autograd.backward([hr_exact, yr], [dh.cuda().float(), dy.cuda().float()])
    xc, rc, wc = leaf(x, "cuda"), leaf(res, "cuda"), leaf(w, "cuda")
    h, y = add_rmsnorm(xc, rc, wc, 1e-6)
    torch.autograd.backward([h, y], [dh.cuda(), dy.cuda()])
    assert torch.equal(h.float(), hr)
    assert rel(y, yr) < tol
    assert rel(xc.grad, xr.grad) < tol and torch.equal(xc.grad, rc.grad)
    assert rel(wc.grad, wr.grad) < tol
    # only y used downstream: the residual-stream gradient is absent
    xc2, rc2 = leaf(x, "cuda"), leaf(res, "cuda")
    sink = torch.zeros(D, device="cuda")
    _, y2 = add_rmsnorm(xc2, rc2, wc.detach(), 1e-6, sink)
    y2.backward(dy.cuda())
    xr2, rr2 = leaf(x, "cuda", dtype=torch.float32), leaf(res, "cuda", dtype=torch.float32)
    F.rms_norm(xr2 + rr2, (D,), wr.detach(), 1e-6).backward(dy.cuda().float())
    assert rel(xc2.grad, xr2.grad) < tol


@pytest.mark.parametrize("max_norm", [None, 1.0, 1e9])
def test_flat_adamw_step_matches_torch(max_norm):
    """Clip + AdamW + bf16 copy in one pass over flat arenas against clip_grad_norm_ and
    torch.optim.AdamW on the same numbers, three steps."""
    from weightshared_torchtitan_b200 import ops
    g = torch.Generator().manual_seed(17)
    n = 4 * 70_001
    p0 = torch.randn(n, generator=g)
    lr, b1, b2, eps, wd = 3e-3, 0.9, 0.95, 1e-8, 0.1
    pr = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([pr], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd)
    p = p0.clone().cuda()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    copy = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        grad = torch.randn(n, generator=g) * (0.5 if step != 2 else 1e-3)
        pr.grad = grad.clone()
        if max_norm is not None:
            want_norm = torch.nn.utils.clip_grad_norm_([pr], max_norm)
        opt.step()
        gc = grad.cuda()
        partials = ops.grad_sumsq_partials(gc) if max_norm is not None else None
        ops.adamw_flat_step(p, gc, m, v, copy, lr, b1, b2, eps, wd, step, partials, max_norm)
        if max_norm is not None:
            assert abs(partials.sum().sqrt().item() - want_norm.item()) < 1e-5 * want_norm.item()
        assert torch.equal(gc.cpu(), grad)                      # gradients are left as they were
        assert rel(p, pr.detach()) < 2e-6
        assert torch.equal(copy, p.to(torch.bfloat16))
