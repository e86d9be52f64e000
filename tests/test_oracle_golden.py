"""The oracle restatement against the golden fixtures produced by the REFERENCE's own
modules (tests/golden/make_golden.py). CPU only, fp32; tolerance 2e-5 max-relative covers
differences between BLAS builds (the values were produced by the same torch arithmetic)."""
import os

import numpy as np
import pytest
import torch

from oracle import lora_oracle as O

TOL = 2e-5


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _rel(a, b):
    return O.max_rel_err(a, b)


def test_small_projection_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "lora_small.npz"))
    y, dX, dW, dA, dB = O.lora_linear_fwd_bwd(_t(g["x"]), _t(g["W"]), _t(g["A"]), _t(g["B"]), _t(g["dY"]))
    for got, key in ((y, "y"), (dX, "dX"), (dW, "dW"), (dA, "dA"), (dB, "dB")):
        assert _rel(got, _t(g[key])) < TOL, key


def test_small_inputs_regenerate_from_seed(golden_dir):
    g = np.load(os.path.join(golden_dir, "lora_small.npz"))
    x, W, A, B, dY = O.projection_inputs(seed=77, M=96, N=72, K=80, r=8)
    for got, key in ((x, "x"), (W, "W"), (A, "A"), (B, "B"), (dY, "dY")):
        assert torch.equal(got, _t(g[key])), key


def test_broadcast_add_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "broadcast_add.npz"))
    for name in ("g1", "g2"):
        out = O.broadcast_add(_t(g[f"{name}_base"]), _t(g[f"{name}_delta"]), dim=-1, g=int(g[f"{name}_g"]))
        assert torch.equal(out, _t(g[f"{name}_out"])), name


def test_config0_matches_reference(golden_dir):
    """Baseline configuration 0: M=2048, K=N=1024, r=16, four layers sharing one W."""
    g = np.load(os.path.join(golden_dir, "lora_cfg0.npz"))
    inp = O.config0_inputs()
    assert torch.equal(inp["W"][::61, ::67], _t(g["in_W"]))
    assert torch.equal(inp["xs"][0][::127, ::61], _t(g["in_x0"]))
    assert torch.equal(inp["As"][3][::3, ::67], _t(g["in_A3"]))
    assert torch.equal(inp["Bs"][2][::61, ::3], _t(g["in_B2"]))
    assert torch.equal(inp["dYs"][1][::127, ::61], _t(g["in_dY1"]))
    ys, dXs, dW, dAs, dBs = O.shared_w_layers_fwd_bwd(inp["xs"], inp["W"], inp["As"], inp["Bs"], inp["dYs"])
    assert _rel(dW[::31, ::29], _t(g["dW_s"])) < TOL

    def chk(t, key):
        c = g[key]
        d = t.double()
        got = np.array([d.sum().item(), d.abs().sum().item(), (d * d).sum().item()])
        assert abs(got[1] - c[1]) <= 1e-5 * abs(c[1]), key
        assert abs(got[2] - c[2]) <= 1e-5 * abs(c[2]), key
        assert abs(got[0] - c[0]) <= 1e-5 * abs(c[1]), key

    chk(dW, "dW_c")
    for l in range(4):
        assert _rel(ys[l][::97, ::89], _t(g[f"y{l}_s"])) < TOL
        assert _rel(dXs[l][::97, ::89], _t(g[f"dX{l}_s"])) < TOL
        assert _rel(dAs[l][:, ::7], _t(g[f"dA{l}"])) < TOL
        assert _rel(dBs[l][::7], _t(g[f"dB{l}"])) < TOL
        chk(ys[l], f"y{l}_c")
        chk(dXs[l], f"dX{l}_c")
        chk(dAs[l], f"dA{l}_c")
        chk(dBs[l], f"dB{l}_c")


def test_shared_dw_is_sum_of_layer_contributions():
    inp = O.config0_inputs(M=128, K=64, N=48, r=8, L=3)
    _, _, dW, _, _ = O.shared_w_layers_fwd_bwd(inp["xs"], inp["W"], inp["As"], inp["Bs"], inp["dYs"])
    want = sum(dY.double().T @ x.double() for dY, x in zip(inp["dYs"], inp["xs"]))
    assert _rel(dW, want) < 1e-6


def test_identities():
    x, W, A, B, dY = O.projection_inputs(seed=3, M=40, N=24, K=32, r=8)
    y0, _, _, dA0, _ = O.lora_linear_fwd_bwd(x, W, A, torch.zeros_like(B), dY)
    assert _rel(y0, x @ W.T) < 1e-6           # B = 0: the adapter vanishes
    assert dA0.abs().max() == 0               # and A gets no gradient
    y, *_ = O.lora_linear_fwd_bwd(x, W, A, B, dY)
    assert _rel(y, x @ W.T + 2.0 * (x @ A.T) @ B.T) < 1e-6


def _tiny_args():
    return O.DecoderArgs(dim=64, hidden_dim=160, n_layers=4, n_unique=2, n_heads=4, n_kv_heads=2,
                         head_dim=16, rank=8, vocab_size=512, embed_rank=32, max_seq_len=24)


def tiny_decoder_params():
    a = _tiny_args()
    p = O.init_decoder_params(a, seed=4321)
    g = torch.Generator().manual_seed(99)
    for k in list(p):
        if k.endswith("norm"):
            p[k] = 1.0 + 0.1 * torch.randn(p[k].shape, generator=g)
    return a, p


def test_tiny_decoder_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "decoder_tiny.npz"))
    a, p = tiny_decoder_params()
    p = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    tokens, labels = _t(g["tokens"]), _t(g["labels"])
    logits = O.decoder_forward(a, p, tokens)
    assert _rel(logits[:, ::5, ::37], _t(g["logits_s"])) < TOL
    loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1).float(), labels.flatten(0, 1))
    assert abs(loss.item() - float(g["loss"])) < 1e-5 * abs(float(g["loss"]))
    loss.backward()
    for key in g.files:
        if not key.startswith("g."):
            continue
        name = key[2:]
        if name == "embed.E_small_rows":
            got = p["embed.E_small"].grad[tokens.flatten()[:8]]
        elif name == "output_s":
            got = p["output"].grad[::17, ::3]
        else:
            got = p[name].grad
        assert _rel(got, _t(g[key])) < 5e-5, key
