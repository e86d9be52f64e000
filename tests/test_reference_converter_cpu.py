"""The converter on the reference's REAL Qwen3Model (meta device), when the reference checkout
is present: parameter names and sharing must be exactly what state_dict_adapter maps to, the
converter and the ``qwen3_shared_lora`` TrainSpec must sit in the trainer's own registries, and
the ``shared_lora`` section must merge into the reference's JobConfig through its
custom_args_module mechanism.

Runs in a child process (importing torchtitan takes seconds and must see the reference
checkout, not another torchtitan that may be installed, first on sys.path). Skipped where the
checkout does not exist."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: WSL_REFERENCE_CHECKOUT, else a directory `reference` beside this repository
REFERENCE = os.environ.get("WSL_REFERENCE_CHECKOUT", os.path.join(os.path.dirname(ROOT), "reference"))

CHILD = r"""
import json, sys
import torch
import torchtitan                                   # the checkout: loaded BEFORE the converter
from torchtitan.experiments.qwen3.model.args import Qwen3ModelArgs
from torchtitan.experiments.qwen3.model.model import Qwen3Model
from torchtitan.protocols import model_converter as mc
from torchtitan.config.manager import ConfigManager
from weightshared_torchtitan_b200 import converter as C
from weightshared_torchtitan_b200 import train_spec as TS
from torchtitan.protocols.train_spec import get_train_spec
from weightshared_torchtitan_b200 import state_dict_adapter as SDA
from weightshared_torchtitan_b200.decoder import DecoderConfig, WeightSharedDecoder

out = {}
out["registered"] = mc._registry_model_converter_cls.get("shared_lora") is C.SharedLoRAConverter
# the job-config section arrives through the reference's own extension mechanism
cfg = ConfigManager().parse_args([
    "--experimental.custom_args_module", "weightshared_torchtitan_b200.job_config_ext",
    "--model.converters", "shared_lora", "--shared_lora.n_unique", "2", "--shared_lora.rank", "8",
    "--shared_lora.embed_rank", "32"])
out["cfg"] = [cfg.shared_lora.n_unique, cfg.shared_lora.rank, cfg.shared_lora.embed_rank,
              cfg.shared_lora.grad_in_place, list(cfg.model.converters)]
args = Qwen3ModelArgs(dim=64, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=512, head_dim=16,
                      hidden_dim=160, max_seq_len=32)
with torch.device("meta"):
    model = Qwen3Model(args)
mc.build_model_converters(cfg, None).convert(model)
names = [n for n, _ in model.named_parameters()]
ours = WeightSharedDecoder(DecoderConfig(dim=64, hidden_dim=160, n_layers=4, n_unique=2, n_heads=4,
                                         n_kv_heads=2, head_dim=16, rank=8, vocab_size=512, embed_rank=32,
                                         max_seq_len=32))
want = SDA.to_reference(ours)
uniq, aliases = SDA.deduplicate(want)
full = dict(model.state_dict(keep_vars=True))          # shared tensors listed under every user
out["same_keys"] = sorted(full) == sorted(want)
out["missing"] = sorted(set(want) - set(full))[:5]
out["unexpected"] = sorted(set(full) - set(want))[:5]
out["same_shapes"] = all(tuple(full[k].shape) == tuple(want[k].shape) for k in want if k in full)
out["named_parameters_are_the_unique_ones"] = sorted(names) == sorted(uniq)
L = model.layers
out["shared_objects"] = all(L[str(l)].attention.wq.base is L[str(l % 2)].attention.wq.base and
                            L[str(l)].feed_forward.w2.base is L[str(l % 2)].feed_forward.w2.base for l in range(4))
out["adapters_distinct"] = len({id(L[str(l)].attention.wq.offset) for l in range(4)}) == 4
# the TrainSpec the trainer would pick with --model.name qwen3_shared_lora
spec = get_train_spec(TS.SPEC_NAME)
out["spec"] = [spec.name, spec.model_cls is Qwen3Model, sorted(spec.model_args)[:2], spec.parallelize_fn is TS.parallelize_shared_lora]
class _PD:                                   # single process: nothing to wrap
    dp_replicate_enabled = tp_enabled = cp_enabled = pp_enabled = dp_shard_enabled = ep_enabled = False
out["parallelize_identity"] = spec.parallelize_fn(model, _PD(), cfg) is model
class _TP(_PD):
    tp_enabled = True
try:
    spec.parallelize_fn(model, _TP(), cfg)
    out["refuses_tp"] = False
except NotImplementedError:
    out["refuses_tp"] = True
print("RESULT " + json.dumps(out))
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "torchtitan")),
                    reason="reference checkout not present on this machine")
def test_converter_on_the_reference_qwen3_model():
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([REFERENCE, ROOT, env.get("PYTHONPATH", "")])
    res = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [ln for ln in res.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    assert out["registered"]
    assert out["cfg"] == [2, 8, 32, False, ["shared_lora"]]
    assert out["same_keys"], (out["missing"], out["unexpected"])
    assert out["same_shapes"]
    assert out["named_parameters_are_the_unique_ones"]
    assert out["shared_objects"] and out["adapters_distinct"]
    assert out["spec"] == ["qwen3_shared_lora", True, ["0.6B", "1.7B"], True]
    assert out["parallelize_identity"] and out["refuses_tp"]
