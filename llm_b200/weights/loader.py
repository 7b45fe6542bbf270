"""Weights by tensor name, from model.safetensors (or the files of a model.safetensors.index.json)
or from a seed.

The reference binds tensors by the names its modules register
(runtime/LLM.h:75-89,101-190) and looks each up with `infos.at(name)`: a missing
tensor is an out_of_range, extra tensors are ignored and neither dtype nor shape is
checked.  Here everything that does not fit is collected and reported in one error:
missing tensors, unexpected tensors, wrong shapes.  Matrices are kept in the compute
dtype (bfloat16 or float32), small gain vectors in float32, integer tables in int32.
"""
from __future__ import annotations

import hashlib
import json
import os
import warnings
from typing import Dict, List

import torch

from ..parts.base import ParamInfo
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

WEIGHTS_FILE = "model.safetensors"
CONFIG_FILE = "config.json"


class WeightError(ValueError):
    """The checkpoint does not hold what the model expects."""

    def __init__(self, path: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{path} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def _target_dtype(info: ParamInfo, compute_dtype: torch.dtype) -> torch.dtype:
    if info.kind == "matrix":
        return compute_dtype
    if info.kind == "gain":
        return torch.float32
    if info.kind == "int_table":
        return torch.int32
    raise ValueError(f"unknown parameter kind '{info.kind}'")


INDEX_FILE = "model.safetensors.index.json"


class _Checkpoint:
    """The tensors of a model folder: model.safetensors, or the files that
    model.safetensors.index.json names ({"weight_map": {tensor name: file name}}), seen as one."""

    def __init__(self, model_dir: str):
        single = os.path.join(model_dir, WEIGHTS_FILE)
        index = os.path.join(model_dir, INDEX_FILE)
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.isfile(single):
            self.path = single
            self.files[WEIGHTS_FILE] = SafetensorsFile(single)
            self.where = {n: WEIGHTS_FILE for n in self.files[WEIGHTS_FILE].entries}
        elif os.path.isfile(index):
            self.path = index
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise SafetensorsError(f"{index}: not an index with a 'weight_map': {e}") from e
            for fname in sorted(set(weight_map.values())):
                part = os.path.join(model_dir, str(fname))
                if os.path.dirname(str(fname)) or not os.path.isfile(part):
                    raise SafetensorsError(f"{index}: names the file '{fname}', which is not in the model folder")
                self.files[fname] = SafetensorsFile(part)
            for name, fname in weight_map.items():
                if name not in self.files[fname].entries:
                    raise SafetensorsError(f"{index}: says '{name}' is in {fname}, which does not hold it")
                self.where[name] = fname
            # tensors that a file holds but the index does not name are unexpected like any other
            for fname, f in self.files.items():
                for n in f.entries:
                    self.where.setdefault(n, fname)
        else:
            raise SafetensorsError(f"{single}: no {WEIGHTS_FILE} (and no {INDEX_FILE}) in the model folder")

    def entry(self, name: str):
        return self.files[self.where[name]].entries[name]

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def _harmless_extra(name: str, ck: "_Checkpoint", expected: Dict[str, ParamInfo]) -> bool:
    """Tensors that checkpoints of this family often carry although no part binds them: the
    rotary inverse-frequency buffers (the tables are rebuilt from rope_theta), and an lm_head.weight
    beside tied embeddings when it has the embedding's shape.  Everything else that is not
    expected stays an error."""
    if name.endswith("rotary_emb.inv_freq"):
        return True
    if name == "lm_head.weight" and "model.embed_tokens.weight" in expected:
        return tuple(ck.entry(name).shape) == tuple(expected["model.embed_tokens.weight"].shape)
    return False


def load_tensors(model_dir: str, expected: Dict[str, ParamInfo], compute_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Read, validate, convert and move every expected tensor."""
    ck = _Checkpoint(model_dir)
    path = ck.path
    missing = sorted(n for n in expected if n not in ck.where)
    unexpected = sorted(n for n in ck.where if n not in expected and not _harmless_extra(n, ck, expected))
    wrong = []
    for name, info in expected.items():
        if name not in ck.where:
            continue
        e = ck.entry(name)
        if tuple(e.shape) != tuple(info.shape):
            wrong.append(f"{name}: file has {list(e.shape)}, model expects {list(info.shape)}")
        elif info.kind == "int_table" and e.dtype.is_floating_point:
            wrong.append(f"{name}: file has {e.dtype}, model expects an integer table")
        elif info.kind != "int_table" and not e.dtype.is_floating_point:
            wrong.append(f"{name}: file has {e.dtype}, model expects floating point")
    if missing or unexpected or wrong:
        ck.close()
        raise WeightError(path, missing, unexpected, wrong)
    out = {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)     # read-only mapping: tensors are copied, never written
        for name, info in expected.items():
            t = ck.tensor(name)
            out[name] = t.to(device=device, dtype=_target_dtype(info, compute_dtype)).contiguous()
    ck.close()
    return out


def adopt_tensors(given: Dict[str, torch.Tensor], expected: Dict[str, ParamInfo], compute_dtype: torch.dtype,
                  device: torch.device) -> Dict[str, torch.Tensor]:
    """Tensors that are already in memory, checked and converted like a file's."""
    missing = sorted(n for n in expected if n not in given)
    unexpected = sorted(n for n in given if n not in expected)
    wrong = [f"{n}: given {list(given[n].shape)}, model expects {list(i.shape)}" for n, i in expected.items()
             if n in given and tuple(given[n].shape) != tuple(i.shape)]
    if missing or unexpected or wrong:
        raise WeightError("the given tensors", missing, unexpected, wrong)
    return {n: given[n].to(device=device, dtype=_target_dtype(i, compute_dtype)).contiguous() for n, i in expected.items()}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") >> 1


def random_tensor(name: str, info: ParamInfo, seed: int) -> torch.Tensor:
    """The seeded value of one tensor in float32: a function of (seed, name, shape) only."""
    if info.kind == "int_table":
        return torch.zeros(info.shape, dtype=torch.int32)
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, name))
    x = torch.randn(info.shape, generator=g, dtype=torch.float32)
    if info.init == "normal":
        return x * 0.02
    if info.init == "ones_normal":
        return 1.0 + x * 0.01
    if info.init == "zeros":
        return torch.zeros(info.shape, dtype=torch.float32)
    raise ValueError(f"unknown init rule '{info.init}'")


def random_tensors_on_device(expected: Dict[str, ParamInfo], seed: int, compute_dtype: torch.dtype,
                             device: torch.device, stored_dtype: str = "bfloat16",
                             on_device: bool = False) -> Dict[str, torch.Tensor]:
    """What load_tensors would return for the folder that write_random_model(seed,
    stored_dtype) writes, without the folder.  on_device: the values come from the device's own
    generator instead (seeded per tensor the same way, same distributions, other numbers): models
    of billions of weights are drawn in a second instead of minutes."""
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[stored_dtype]
    out = {}
    for name, info in expected.items():
        if on_device and info.kind != "int_table" and info.init in ("normal", "ones_normal"):
            g = torch.Generator(device=device)
            g.manual_seed(_tensor_seed(seed, name))
            t = torch.randn(info.shape, generator=g, dtype=torch.float32, device=device)
            t = t * 0.02 if info.init == "normal" else 1.0 + t * 0.01
            if info.kind == "matrix":
                t = t.to(store)
            out[name] = t.to(dtype=_target_dtype(info, compute_dtype)).contiguous()
            continue
        t = random_tensor(name, info, seed)
        if info.kind == "matrix":
            t = t.to(store)
        out[name] = t.to(device=device, dtype=_target_dtype(info, compute_dtype)).contiguous()
    return out


def expected_tensors(config_dict: dict) -> Dict[str, ParamInfo]:
    """Names and shapes a model of this config.json expects, found by building its parts
    without a device."""
    from ..engine.model import collect_parameters
    return collect_parameters(config_dict)


def write_random_model(model_dir: str, config_dict: dict, seed: int, dtype: str = "bfloat16") -> str:
    """Write config.json and model.safetensors with seeded random weights: matrices and
    embeddings N(0, 0.02), norm gains 1 + N(0, 0.01).  `dtype` is the stored dtype of the
    matrices ("bfloat16" or "float32"); gains are stored in float32."""
    store = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    expected = expected_tensors(config_dict)
    os.makedirs(model_dir, exist_ok=True)
    tensors = {}
    for name, info in expected.items():
        t = random_tensor(name, info, seed)
        if info.kind == "matrix":
            t = t.to(store)
        tensors[name] = t
    cfg = dict(config_dict)
    cfg.setdefault("torch_dtype", dtype)
    with open(os.path.join(model_dir, CONFIG_FILE), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    write_safetensors(os.path.join(model_dir, WEIGHTS_FILE), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
