"""Checkpoints of the weight-shared decoder in the layout the reference trainer uses.

The reference's CheckpointManager (torchtitan/components/checkpoint.py:324-423) writes one
folder per step, ``<folder>/step-<N>/``, and, for the Hugging Face form (``to_hf``: a state-dict
adapter + HuggingFaceStorageWriter), safetensors files with a ``model.safetensors.index.json``
whose ``weight_map`` names the file of every key. This module writes that form for this
package's decoder:

    <folder>/step-<N>/model.safetensors              every tensor ONCE, under the FQNs of a reference
                                                     Qwen3Model after SharedLoRAConverter
    <folder>/step-<N>/model.safetensors.index.json   weight_map for every key, shared ones included,
                                                     and the alias table (a base weight shared by
                                                     several layers is stored once)
    <folder>/step-<N>/optimizer.safetensors          the fused step's AdamW moments per parameter
                                                     + step count (TrainStep.state_dict)

The safetensors container is written and read here directly (8-byte little-endian header
length, JSON header {name: {dtype, shape, data_offsets}, "__metadata__": {str: str}}, raw
little-endian tensor bytes), so nothing but torch is needed; files are readable by the
``safetensors`` package and the other way round.
"""
from __future__ import annotations

import json
import os
import re
import struct
from typing import Dict, Optional, Tuple

import torch

from . import state_dict_adapter as SDA

_DTYPES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int64: "I64",
           torch.float64: "F64", torch.int32: "I32", torch.uint8: "U8"}
_FROM = {v: k for k, v in _DTYPES.items()}


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    """One safetensors file; tensors are copied to the host one at a time."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for k in order:
        t = tensors[k]
        n = t.numel() * t.element_size()
        header[k] = {"dtype": _DTYPES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for k in order:
            t = tensors[k].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def read_safetensors(path: str) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    meta = header.pop("__metadata__", {})
    out = {}
    for k, h in header.items():
        a, b = h["data_offsets"]
        raw = torch.frombuffer(bytearray(data[a:b]), dtype=torch.uint8) if b > a else torch.empty(0, dtype=torch.uint8)
        out[k] = raw.view(_FROM[h["dtype"]]).reshape(h["shape"])
    return out, meta


def step_folder(folder: str, step: int) -> str:
    return os.path.join(folder, f"step-{step}")


def latest_step(folder: str) -> int:
    """Largest N with a complete ``step-N`` folder, or -1 (the reference's folder convention)."""
    best = -1
    if os.path.isdir(folder):
        for name in os.listdir(folder):
            m = re.fullmatch(r"step-(\d+)", name)
            if m and os.path.isfile(os.path.join(folder, name, "model.safetensors.index.json")):
                best = max(best, int(m.group(1)))
    return best


def save_checkpoint(folder: str, step: int, model, train_step=None) -> str:
    """Writes ``<folder>/step-<step>/``; returns that path."""
    out = step_folder(folder, step)
    os.makedirs(out, exist_ok=True)
    full = SDA.to_reference(model)
    unique, aliases = SDA.deduplicate(full)
    write_safetensors(os.path.join(out, "model.safetensors"), unique,
                      {"format": "pt", "aliases": json.dumps(aliases, sort_keys=True)})
    if train_step is not None:
        sd = train_step.state_dict()
        tensors = {k: v for k, v in sd.items() if torch.is_tensor(v)}
        write_safetensors(os.path.join(out, "optimizer.safetensors"), tensors,
                          {"steps": str(sd["steps"]), "lr": json.dumps(sd.get("lr"))})
    # the index goes last: its presence marks the folder complete
    total = sum(t.numel() * t.element_size() for t in unique.values())
    index = {"metadata": {"total_size": total, "aliases": aliases},
             "weight_map": {k: "model.safetensors" for k in sorted(full)}}
    tmp = os.path.join(out, "model.safetensors.index.json.tmp")
    with open(tmp, "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
    os.replace(tmp, os.path.join(out, "model.safetensors.index.json"))
    return out


def load_checkpoint(folder: str, model, train_step=None, step: int = -1) -> int:
    """Loads ``step`` (default: the latest complete one) into the model (and the step's optimizer
    state, when a TrainStep is given and the file exists). Returns the step loaded; raises
    FileNotFoundError when there is none."""
    if step < 0:
        step = latest_step(folder)
    src = step_folder(folder, step)
    if step < 0 or not os.path.isfile(os.path.join(src, "model.safetensors.index.json")):
        raise FileNotFoundError(f"no complete checkpoint under {folder}")
    unique, meta = read_safetensors(os.path.join(src, "model.safetensors"))
    SDA.from_reference(model, SDA.expand(unique, json.loads(meta.get("aliases", "{}"))))
    opt = os.path.join(src, "optimizer.safetensors")
    if train_step is not None and os.path.isfile(opt):
        tensors, ometa = read_safetensors(opt)
        sd: Dict[str, object] = dict(tensors)
        sd["steps"] = int(ometa["steps"])
        sd["lr"] = json.loads(ometa.get("lr", "null"))
        train_step.load_state_dict(sd)
    return step
