"""CPU tests: the C-ABI library loads and exports every symbol include/wsl.h declares (no
compute without a GPU), host-side logic (modules' structure, converter, arena, cache), and
the product's refusal to run without its CUDA library or on CPU tensors."""
import json
import os
import re
import types

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "wsl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wsl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    declared = _header_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(declared)
    assert lib.wsl_version() > 0
    assert _lib.status_string(0) == "ok"
    for code in range(-7, 0):
        assert _lib.status_string(code) != "unknown status"


def test_argument_validation_needs_no_device():
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    assert lib.wsl_linear_fwd(None, 8, None, None, 8, 1, 8, 8, 0, 0, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_lora_prepass(None, 8, None, None, 8, 0, 8, 8, 2.0, 0, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_lora_linear_bwd_dw_noalloc(None, 0, None, 0, None, 0, None, 0, None, None, None,
                                              1, 1, 1, 0, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_bwd_dw_workspace_bytes(32768, 1024, 1024, 16, 1, 1, 1) > 0
    assert lib.wsl_bwd_dw_workspace_bytes(16384, 12288, 4096, 64, 1, 1, 1) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback():
    from weightshared_torchtitan_b200 import _lib, ops
    from weightshared_torchtitan_b200.modules import LoRAModule
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.linear_fwd(torch.zeros(8, 8), torch.zeros(8, 8))
    with pytest.raises(RuntimeError):
        LoRAModule(16, 16, rank=8)(torch.zeros(2, 16))
    x = torch.zeros(1)
    st = _lib.lib().wsl_linear_fwd(x.data_ptr(), 8, x.data_ptr(), x.data_ptr(), 8, 8, 8, 8, 0, 0, None)
    assert st == _lib.WSL_ERR_DEVICE


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from weightshared_torchtitan_b200 import _lib
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libwsl.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "weightshared_torchtitan_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(root, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "lora_oracle" not in src, f


def test_lora_module_structure_matches_reference_naming():
    from weightshared_torchtitan_b200.modules import LoRAModule, SharedLoRALinear
    base = nn.Linear(32, 48, bias=False)
    a, b = LoRAModule(32, 48, rank=8), LoRAModule(32, 48, rank=8)
    m1, m2 = SharedLoRALinear(base, a), SharedLoRALinear(base, b)
    assert m1.base is m2.base
    assert sorted(n for n, _ in m1.named_parameters()) == ["base.weight", "offset.w_a.weight", "offset.w_b.weight"]
    assert a.alpha / a.rank == 2.0
    with pytest.raises(ValueError):
        SharedLoRALinear(nn.Linear(32, 24, bias=False), a)      # head-sharing widths stay eager
    holder = nn.ModuleList([m1, m2])
    assert sum(p.numel() for p in holder.parameters()) == 32 * 48 + 2 * (8 * 32 + 48 * 8)   # W counted once


def test_broadcast_add_product_equals_oracle_on_cpu():
    from oracle import lora_oracle as O
    from weightshared_torchtitan_b200.modules import broadcast_add
    g = torch.Generator().manual_seed(2)
    for gg, H, D in ((1, 4, 8), (2, 8, 4), (4, 4, 16), (2, 2, 8)):
        base = torch.randn(2, 7, gg * D, generator=g)
        delta = torch.randn(2, 7, H * D, generator=g)
        assert torch.equal(broadcast_add(base, delta, dim=-1, g=gg), O.broadcast_add(base, delta, dim=-1, g=gg))


def test_copy_cache_refreshes_on_update():
    from weightshared_torchtitan_b200.modules import CopyCache
    c = CopyCache()
    p = nn.Parameter(torch.ones(4, 4))
    a = c.get(torch.bfloat16, p)
    assert c.get(torch.bfloat16, p) is a
    with torch.no_grad():
        p.add_(1.0)
    b = c.get(torch.bfloat16, p)
    assert b is not a and float(b[0, 0]) == 2.0
    q = nn.Parameter(torch.zeros(2, 4))
    cat = c.get(torch.bfloat16, p, q)
    assert cat.shape == (6, 4)
    assert c.get(torch.float32, p).data_ptr() == p.data_ptr()
    # a fused optimizer moves the parameter without touching its version counter: the global
    # post-step hook drops the copy all the same
    before = c.get(torch.bfloat16, p)
    p.grad = torch.ones_like(p)
    v = p._version
    torch.optim.AdamW([p], lr=0.5, fused=True).step()
    assert p._version == v
    after = c.get(torch.bfloat16, p)
    assert after is not before and torch.equal(after, p.detach().to(torch.bfloat16))


def test_fused_optimizers_leave_version_counters_alone_so_the_cache_must_be_told():
    """Why the cache is bound to the arena (or cleared by the post-optimizer hook): a copy
    keyed on the version counter alone would go stale under a fused optimizer."""
    from weightshared_torchtitan_b200.dp import GradArena
    from weightshared_torchtitan_b200.modules import CopyCache
    m = nn.Sequential(nn.Linear(8, 16, bias=False), nn.Linear(16, 4, bias=False))
    w0 = m[0].weight.detach().clone()
    arena = GradArena(m)
    flat = arena.flatten_parameters()
    assert torch.equal(m[0].weight.detach(), w0) and m[0].weight.data_ptr() == flat.data_ptr()
    assert m[1].weight.data_ptr() == flat.data_ptr() + 4 * arena.offsets[1]
    cache = CopyCache()
    cache.bind(arena)
    c = cache.get(torch.bfloat16, m[0].weight)
    assert c.shape == (16, 8) and torch.equal(c, w0.to(torch.bfloat16))
    P = nn.Parameter(flat)
    P.grad = arena.buffer
    arena.buffer.fill_(1.0)
    v0 = m[0].weight._version
    torch.optim.AdamW([P], lr=0.1, fused=True).step()
    assert not torch.equal(m[0].weight.detach(), w0)            # the master moved ...
    assert m[0].weight._version == v0                            # ... and no counter noticed
    assert torch.equal(cache.get(torch.bfloat16, m[0].weight), w0.to(torch.bfloat16))
    arena.refresh_compute_copies()
    assert torch.equal(cache.get(torch.bfloat16, m[0].weight), m[0].weight.detach().to(torch.bfloat16))
    assert cache.get(torch.bfloat16, m[0].weight).data_ptr() == c.data_ptr()   # same view, new values


class _TinyAttn(nn.Module):
    def __init__(self):
        super().__init__()
        self.wq, self.wk, self.wv, self.wo = (nn.Linear(16, 16, bias=False) for _ in range(4))


class _TinyFfn(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1, self.w2, self.w3 = nn.Linear(16, 32, bias=False), nn.Linear(32, 16, bias=False), nn.Linear(16, 32, bias=False)


class _TinyBlock(nn.Module):
    def __init__(self):
        super().__init__()
        self.attention, self.feed_forward = _TinyAttn(), _TinyFfn()


class _TinyModel(nn.Module):
    def __init__(self, n):
        super().__init__()
        self.tok_embeddings = nn.Embedding(64, 16)
        self.layers = nn.ModuleDict({str(i): _TinyBlock() for i in range(n)})


def test_converter_shares_bases_cyclically():
    from weightshared_torchtitan_b200 import converter as C
    from weightshared_torchtitan_b200.modules import FactorizedEmbedding, SharedLoRALinear
    job = types.SimpleNamespace(model=types.SimpleNamespace(converters=["shared_lora"]),
                                shared_lora=types.SimpleNamespace(n_unique=2, rank=8, embed_rank=8))
    model = _TinyModel(6)
    conv = C.build_model_converters(job, None)
    conv.convert(model)
    L = [model.layers[str(i)] for i in range(6)]
    for l in range(6):
        for n in ("wq", "wk", "wv", "wo"):
            m = getattr(L[l].attention, n)
            assert isinstance(m, SharedLoRALinear)
            assert m.base is getattr(L[l % 2].attention, n).base
            assert m.offset is not getattr(L[(l + 2) % 6].attention, n).offset
        assert L[l].feed_forward.w2.base is L[l % 2].feed_forward.w2.base
    assert isinstance(model.tok_embeddings, FactorizedEmbedding)
    names = [n for n, _ in model.named_parameters()]
    assert "layers.0.attention.wq.base.weight" in names and "layers.3.attention.wq.offset.w_a.weight" in names
    assert not any(n.startswith("layers.2.") and ".base." in n for n in names)      # shared: listed once
    n_base = sum(1 for n in names if n.endswith(".base.weight"))
    assert n_base == 2 * 7                                   # 6 layers, 2 unique blocks, 7 projections
    conv.post_optimizer_hook(model)
    with pytest.raises(AssertionError):
        C.register_model_converter(C.SharedLoRAConverter, "shared_lora")


def test_grad_arena_layout_and_clip():
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    from weightshared_torchtitan_b200.dp import GradArena, shard_tokens
    m = WeightSharedDecoder(DecoderConfig(dim=32, hidden_dim=64, n_layers=4, n_unique=2, n_heads=2, n_kv_heads=1,
                                          head_dim=16, rank=8, vocab_size=64, embed_rank=16, max_seq_len=8))
    a = GradArena(m)
    # laid out in the order the gradients become final: head, (final norm, last layer), ...,
    # (layer 1, shared block 1), (layer 0, shared block 0), embedding
    assert [r for r, _, _ in a.ready_bounds] == [0, 1, 2, 3, 4, 5]
    assert a.ready_bounds[0][1] == 0 and a.ready_bounds[-1][2] == a.buffer.numel()
    for (_, b0, e0), (_, b1, _) in zip(a.ready_bounds, a.ready_bounds[1:]):
        assert e0 == b1
    rank_of = dict(zip(a.names, (m.grad_ready_rank(n) for n in a.names)))
    assert rank_of["output.weight"] == 0 and rank_of["norm.weight"] == 1
    assert rank_of["layers.3.w2_offset.w_b.weight"] == 1 and rank_of["layers.0.attention_norm.weight"] == 4
    assert rank_of["blocks.1.wq.weight"] == 3 and rank_of["blocks.0.w2.weight"] == 4
    assert rank_of["tok_embeddings.embed.weight"] == 5
    for p, off in zip(a.params, a.offsets):
        assert off % 64 == 0 and p.grad.data_ptr() == a.buffer.data_ptr() + 4 * off
    assert len(a.params) == len(list(m.parameters()))       # shared weights appear once
    a.buffer.fill_(1.0)
    n = a.clip_(1.0)
    assert abs(n.item() - a.buffer.numel() ** 0.5) < 1e-2
    assert abs(a.grad_norm().item() - 1.0) < 1e-3
    a.zero()
    a.check_attached()
    m.zero_grad(set_to_none=True)
    with pytest.raises(RuntimeError):
        a.check_attached()
    assert shard_tokens(16, 3, 4) == (12, 16)
    with pytest.raises(ValueError):
        shard_tokens(10, 0, 4)


def test_flops_formula():
    from weightshared_torchtitan_b200.decoder import CONFIGS, flops_per_token, proj_shapes
    c = CONFIGS["qwen3-8b-ws"]
    f = flops_per_token(c, 8192)
    per_layer = sum(6 * o * i + 6 * c.rank * (o + i) for o, i in proj_shapes(c).values())
    assert f["linear"] == per_layer * 36
    # the 8B-shape projections cost 19.44 TF per layer at M = 16384 (fwd + bwd, adapters included)
    assert abs(per_layer * 16384 / 1e12 - 19.44) < 0.05


def test_row_kernel_entry_points_validate_arguments():
    """Null pointers and impossible sizes come back as status codes from every entry point
    added around the projections (no device needed: validation precedes any CUDA call or
    reports the missing device)."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    bad = {_lib.WSL_ERR_BAD_ARG, _lib.WSL_ERR_DEVICE}
    assert lib.wsl_ce_fwd_bwd(None, 8, None, None, 1, 8, 1.0, None, 0, None) in bad
    assert lib.wsl_ce_fwd_bwd(None, 8, None, None, 1, 8, 1.0, None, 9, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_swiglu_fwd(None, None, None, 8, 0, None) in bad
    assert lib.wsl_swiglu_bwd(None, None, None, None, None, 8, 0, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_rmsnorm_fwd(None, 8, None, None, 8, None, 1, 8, 1e-6, None, None, 0, 0, 0, None) in bad
    assert lib.wsl_rmsnorm_bwd(None, 8, None, 8, None, None, None, 8, None, 1, 8, None, None, 0, 0, 3, None) \
        == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_embed_fwd(None, None, None, None, 8, 1, 8, 8, 8, None) == _lib.WSL_ERR_BAD_ARG
    assert lib.wsl_embed_bwd_dproj(None, None, 8, None, None, 1, 8, 8, 8, None, 0, None) == _lib.WSL_ERR_BAD_ARG


def test_rmsnorm_supported_widths():
    from weightshared_torchtitan_b200 import ops
    bf, f32 = torch.bfloat16, torch.float32
    assert all(ops.rmsnorm_supported(d, bf) for d in (16, 64, 128, 256, 512, 1024, 2048))
    assert ops.rmsnorm_supported(2560, bf) and ops.rmsnorm_supported(4096, bf)      # hidden sizes of the 4B / 8B shapes
    assert not ops.rmsnorm_supported(5120, bf) and not ops.rmsnorm_supported(2560, f32)
    assert ops.rmsnorm_supported(128, bf, rope=True) and not ops.rmsnorm_supported(512, bf, rope=True)
    assert ops.rmsnorm_supported(1024, f32) and not ops.rmsnorm_supported(2048, f32)


class _QAttn(nn.Module):
    def __init__(self, dim, heads, kv, hd):
        super().__init__()
        self.wq = nn.Linear(dim, heads * hd, bias=False)
        self.wk = nn.Linear(dim, kv * hd, bias=False)
        self.wv = nn.Linear(dim, kv * hd, bias=False)
        self.wo = nn.Linear(heads * hd, dim, bias=False)
        self.q_norm, self.k_norm = nn.RMSNorm(hd), nn.RMSNorm(hd)


class _QFfn(nn.Module):
    def __init__(self, dim, hidden):
        super().__init__()
        self.w1, self.w2, self.w3 = (nn.Linear(dim, hidden, bias=False), nn.Linear(hidden, dim, bias=False),
                                     nn.Linear(dim, hidden, bias=False))


class _QBlock(nn.Module):
    def __init__(self, dim, hidden, heads, kv, hd):
        super().__init__()
        self.attention, self.feed_forward = _QAttn(dim, heads, kv, hd), _QFfn(dim, hidden)
        self.attention_norm, self.ffn_norm = nn.RMSNorm(dim), nn.RMSNorm(dim)


class _QModel(nn.Module):
    """Module tree with the attribute names of the reference's Qwen3Model."""

    def __init__(self, vocab, dim, hidden, n_layers, heads, kv, hd):
        super().__init__()
        self.tok_embeddings = nn.Embedding(vocab, dim)
        self.layers = nn.ModuleDict({str(i): _QBlock(dim, hidden, heads, kv, hd) for i in range(n_layers)})
        self.norm = nn.RMSNorm(dim)
        self.output = nn.Linear(dim, vocab, bias=False)


def test_state_dict_round_trip_with_the_converted_reference_layout():
    """The decoder's parameters under the converted reference model's names load strictly into
    such a model (same keys, same shapes, shared bases aliased the same way), come back
    unchanged, and de-duplicate to one tensor per unique block."""
    from weightshared_torchtitan_b200 import converter as C
    from weightshared_torchtitan_b200 import state_dict_adapter as A
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    c = DecoderConfig(dim=64, hidden_dim=160, n_layers=4, n_unique=2, n_heads=4, n_kv_heads=2, head_dim=16,
                      rank=8, vocab_size=512, embed_rank=32, max_seq_len=24, loss_chunk=32)
    torch.manual_seed(0)
    dec = WeightSharedDecoder(c)
    for p in dec.parameters():
        nn.init.normal_(p, 0.0, 0.1)
    ref = _QModel(512, 64, 160, 4, 4, 2, 16)
    job = types.SimpleNamespace(model=types.SimpleNamespace(converters=["shared_lora"]),
                                shared_lora=types.SimpleNamespace(n_unique=2, rank=8, embed_rank=32))
    C.build_model_converters(job, None).convert(ref)
    sd = A.to_reference(dec)
    assert set(sd) == set(ref.state_dict())
    ref.load_state_dict(sd, strict=True)
    assert sd["layers.0.attention.wq.base.weight"] is sd["layers.2.attention.wq.base.weight"]
    assert ref.layers["0"].attention.wq.base is ref.layers["2"].attention.wq.base
    unique, aliases = A.deduplicate(sd)
    assert len(aliases) == 7 * (4 - 2) and len(unique) + len(aliases) == len(sd)
    assert set(A.expand(unique, aliases)) == set(sd)
    dec2 = WeightSharedDecoder(c)
    A.from_reference(dec2, ref.state_dict())
    for (k, a), (_, b) in zip(dec.named_parameters(), dec2.named_parameters()):
        assert torch.equal(a, b), k
    bad = {k: v.clone() for k, v in ref.state_dict().items()}
    bad["layers.2.attention.wq.base.weight"] += 1.0
    with pytest.raises(ValueError):
        A.from_reference(WeightSharedDecoder(c), bad)


def test_route_table_covers_the_baseline_configurations():
    """Every projection group (q|k|v, o, gate|up, down) of baseline configurations 1-4 at its own
    token count has a measured entry in functional.ROUTE_TABLE (so the step never decides by the
    fallback rule there), the entries reproduce through derived_route_pays, and the fallback rule
    separates the table's clear cases."""
    from weightshared_torchtitan_b200 import functional as Fn
    from weightshared_torchtitan_b200.decoder import CONFIGS, proj_shapes
    tokens = {"qwen3-0.6b-ws": 8 * 4096, "qwen3-1.7b-ws": 8 * 4096, "qwen3-4b-ws": 4 * 8192, "qwen3-8b-ws": 2 * 8192}
    seen = set()
    for name, c in CONFIGS.items():
        shp = proj_shapes(c)
        for names in (("wq", "wk", "wv"), ("wo",), ("w1", "w3"), ("w2",)):
            key = (tokens[name], shp[names[0]][1], tuple(shp[n][0] for n in names), c.rank)
            assert key in Fn.ROUTE_TABLE, (name, names, key)
            assert Fn.derived_route_pays(*key) is Fn.ROUTE_TABLE[key]
            seen.add(key)
    # plus the isolated-op headline shape (one gate projection of configuration 4 on its own)
    headline = (16384, 4096, (12288,), 64)
    assert seen | {headline} == set(Fn.ROUTE_TABLE)
    # outside the table: many tokens per input width -> through the layer gradient, few -> direct
    assert Fn.derived_route_pays(65536, 1024, (1024,), 16) is True
    assert Fn.derived_route_pays(4096, 4096, (4096,), 64) is False


def test_runtime_options_round_trip():
    """wsl_set_option / wsl_get_option need no device: values come back, out-of-range values and
    unknown keys are refused, and the defaults are the documented ones."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    assert _lib.get_option(_lib.OPT_RESERVED_SMS) == 0 and _lib.get_option(_lib.OPT_GRID_WAVES) == 0
    assert _lib.get_option(_lib.OPT_STALL_PRODUCER) == 0 and _lib.get_option(_lib.OPT_MERGE_SIMT) == 0
    assert _lib.get_option(_lib.OPT_SPLIT_TAIL) == 1 and _lib.get_option(_lib.OPT_DEPENDENT_LAUNCH) == 1
    old = _lib.get_option(_lib.OPT_WAIT_LIMIT_MS)
    assert old == 2000 or "WSL_WAIT_LIMIT_MS" in __import__("os").environ
    try:
        _lib.set_option(_lib.OPT_WAIT_LIMIT_MS, 250)
        assert _lib.get_option(_lib.OPT_WAIT_LIMIT_MS) == 250
        _lib.set_option(_lib.OPT_RESERVED_SMS, 16)
        assert _lib.get_option(_lib.OPT_RESERVED_SMS) == 16
        _lib.set_option(_lib.OPT_GRID_WAVES, 2)
        assert _lib.get_option(_lib.OPT_GRID_WAVES) == 2
        assert lib.wsl_set_option(_lib.OPT_WAIT_LIMIT_MS, 0) == _lib.WSL_ERR_BAD_ARG
        assert lib.wsl_set_option(_lib.OPT_RESERVED_SMS, 1000) == _lib.WSL_ERR_BAD_ARG
        assert lib.wsl_set_option(_lib.OPT_GRID_WAVES, 9) == _lib.WSL_ERR_BAD_ARG
        assert lib.wsl_set_option(99, 1) == _lib.WSL_ERR_BAD_ARG
    finally:
        _lib.set_option(_lib.OPT_WAIT_LIMIT_MS, old)
        _lib.set_option(_lib.OPT_RESERVED_SMS, 0)
        _lib.set_option(_lib.OPT_GRID_WAVES, 0)


def test_split_plan_of_weight_gradient_launches():
    """The workspace a weight-gradient launch asks for tells its split plan (host code, no device):
    nothing for a grid that fills its waves, the whole output times S for a small grid, and a few
    tile blocks (S x T x 256 KiB) for a large grid with a partly filled last wave; launches that
    carry the narrow rank-r regions, and contractions too short to pay, take no tail."""
    from weightshared_torchtitan_b200 import _lib
    lib = _lib.lib()
    blk = 256 * 256 * 4
    assert _lib.get_option(_lib.OPT_SPLIT_TAIL) == 1
    # configuration 4: q|k|v 384 tile pairs = 5.19 waves -> a tail; gate|up 1536 = 20.76 waves -> none
    ws = lib.wsl_bwd_dw_workspace_bytes(16384, 6144, 4096, 0, 1, 0, 0)
    assert 0 < ws < 6144 * 4096 * 4 // 4 and ws % blk == 0
    assert lib.wsl_bwd_dw_workspace_bytes(16384, 24576, 4096, 0, 1, 0, 0) == 0
    assert lib.wsl_bwd_dw_workspace_bytes(16384, 6144, 4096, 64, 1, 1, 1) == 0       # with dB, dA regions
    assert lib.wsl_bwd_dw_workspace_bytes(2048, 6144, 4096, 0, 1, 0, 0) == 0         # 32 k-blocks per tile
    # a small grid splits every tile: S x the whole output
    small = lib.wsl_bwd_dw_workspace_bytes(32768, 256, 512, 0, 1, 0, 0)
    assert small >= 2 * 256 * 512 * 4 and small % (256 * 512 * 4) == 0
    _lib.set_option(_lib.OPT_SPLIT_TAIL, 0)
    try:
        assert lib.wsl_bwd_dw_workspace_bytes(16384, 6144, 4096, 0, 1, 0, 0) == 0
        assert lib.wsl_bwd_dw_workspace_bytes(32768, 256, 512, 0, 1, 0, 0) == small
    finally:
        _lib.set_option(_lib.OPT_SPLIT_TAIL, 1)


def test_checkpoint_round_trip_in_the_reference_folder_layout(tmp_path):
    """step-N folders with model.safetensors (every shared base weight once, alias table), an index
    whose weight_map lists every reference key, and the optimizer state of a TrainStep; the files
    are plain safetensors (cross-read with the safetensors package when it is installed)."""
    from weightshared_torchtitan_b200 import checkpoint as C
    from weightshared_torchtitan_b200 import state_dict_adapter as SDA
    from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder
    from weightshared_torchtitan_b200.train_step import TrainStep
    cfg = DecoderConfig(dim=32, hidden_dim=64, n_layers=4, n_unique=2, n_heads=2, n_kv_heads=1, head_dim=16, rank=8,
                        vocab_size=64, embed_rank=16, max_seq_len=8)
    torch.manual_seed(0)
    m = WeightSharedDecoder(cfg)
    st = TrainStep(m, lr=1e-3)                    # CPU: torch AdamW over the flat arena
    st.arena.buffer.normal_()                     # stand-in gradients, then one optimizer step for non-trivial state
    st.optimizer.step()
    st.steps = 7
    folder = str(tmp_path / "checkpoint")
    assert C.latest_step(folder) == -1
    out = C.save_checkpoint(folder, 7, m, st)
    C.save_checkpoint(folder, 3, m)
    assert C.latest_step(folder) == 7 and out.endswith("step-7")
    index = json.load(open(os.path.join(out, "model.safetensors.index.json")))
    full = SDA.to_reference(m)
    assert sorted(index["weight_map"]) == sorted(full)
    tensors, meta = C.read_safetensors(os.path.join(out, "model.safetensors"))
    aliases = json.loads(meta["aliases"])
    assert len(tensors) == len(list(m.parameters())) and len(tensors) + len(aliases) == len(full)
    assert aliases["layers.2.attention.wq.base.weight"] == "layers.0.attention.wq.base.weight"
    try:
        from safetensors.torch import load_file
        other = load_file(os.path.join(out, "model.safetensors"))
        assert sorted(other) == sorted(tensors) and all(torch.equal(other[k], tensors[k]) for k in tensors)
    except ImportError:
        pass
    torch.manual_seed(1)
    m2 = WeightSharedDecoder(cfg)
    st2 = TrainStep(m2, lr=5e-4)
    assert C.load_checkpoint(folder, m2, st2) == 7
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2)
    assert st2.steps == 7 and st2.lr == 1e-3
    sd1, sd2 = st.state_dict(), st2.state_dict()
    moments = [k for k in sd1 if k.startswith("exp_avg")]
    assert len(moments) == 2 * len(list(m.parameters())) and sd1["exp_avg.output.weight"].abs().max() > 0
    assert all(torch.equal(sd1[k], sd2[k]) for k in moments)
    assert all(float(s["step"]) == 7.0 for s in st2.optimizer.state.values())
    with pytest.raises(FileNotFoundError):
        C.load_checkpoint(str(tmp_path / "nothing"), m2)
