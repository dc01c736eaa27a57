"""Weights by tensor name from a model folder, checked against what the model's parts ask for.

integrallis/models looks every tensor up by name and fails on the first one that is absent
("Tensor not found: <name>", backend-java/.../gguf/GgufFile.java:38-48) or has the wrong length
(backend-java/.../llama/LlamaWeights.java:197-211).  Here all faults of a folder are collected
and reported in one error: missing tensors, unexpected tensors, wrong shapes.
"""

from __future__ import annotations

import fnmatch
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Mapping, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightsError(ValueError):
    """The tensors of a model folder do not match the model."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class ParamRequest:
    """A tensor a part needs.  kind: "matrix" (used by matrix products, random init N(0, std)),
    "gain" (a norm's weight, random init 1 + N(0, gain_std)), "bias" (random init N(0, std))."""

    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"


def _open_files(folder: Path) -> Tuple[List[SafetensorsFile], Dict[str, SafetensorsFile]]:
    index_path = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    files: List[SafetensorsFile] = []
    by_name: Dict[str, SafetensorsFile] = {}
    if single.is_file():
        paths = [single]
    elif index_path.is_file():
        weight_map = json.loads(index_path.read_text()).get("weight_map", {})
        paths = sorted({folder / shard for shard in weight_map.values()})
        for p in paths:
            if not p.is_file():
                raise WeightsError(f"{index_path}: names the shard {p.name}, which is not in the folder")
    else:
        raise FileNotFoundError(f"{folder}: a model folder needs model.safetensors (or model.safetensors.index.json)")
    try:
        for p in paths:
            f = SafetensorsFile(p)
            files.append(f)
            for name in f.names():
                if name in by_name:
                    raise WeightsError(f"tensor {name!r} is stored in both {by_name[name].path.name} and {p.name}")
                by_name[name] = f
    except (SafetensorsError, WeightsError):
        for f in files:
            f.close()
        raise
    return files, by_name


def check_names_and_shapes(requests: Mapping[str, ParamRequest], found: Mapping[str, Tuple[int, ...]], where: str):
    missing = sorted(n for n in requests if n not in found)
    unexpected = sorted(n for n in found if n not in requests)
    wrong = sorted(
        (n, tuple(requests[n].shape), tuple(found[n])) for n in requests if n in found and tuple(found[n]) != tuple(requests[n].shape)
    )
    if not (missing or unexpected or wrong):
        return
    lines = [f"{where}: the tensors do not match the model"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
            f"{n} is {list(got)}, the model needs {list(need)}" for n, need, got in wrong))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def load_tensors(folder, requests: Mapping[str, ParamRequest], ignored: Sequence[str] = (),
                 duplicates: Mapping[str, str] = {}) -> Dict[str, torch.Tensor]:
    """Host tensors for every requested name.  bfloat16 stays bfloat16, a tensor stored in 32-bit
    stays 32-bit, integer tables become int32.  A stored tensor that nobody asked for is an error,
    listed with the missing ones and the wrong shapes, unless its name matches one of the `ignored`
    patterns (buffers the model recomputes), or `duplicates` names the requested tensor it must
    repeat bit for bit (then it is dropped; if it differs, that is the error)."""
    folder = Path(folder)
    files, by_name = _open_files(folder)
    try:
        found = {n: f.shape(n) for n, f in by_name.items()
                 if n in requests or not any(fnmatch.fnmatchcase(n, pattern) for pattern in ignored)}
        repeated = [n for n in found if n not in requests and duplicates.get(n) in found]
        for name in repeated:
            del found[name]
        check_names_and_shapes(requests, found, str(folder))
        tensors = {name: by_name[name].tensor(name) for name in requests}
        for name in repeated:
            original = duplicates[name]
            copy = by_name[name].tensor(name)
            if copy.shape != tensors[original].shape or copy.dtype != tensors[original].dtype or not torch.equal(copy, tensors[original]):
                raise WeightsError(
                    f"{folder}: {name} is stored although the model takes it from {original}, and the two differ "
                    "(the configuration says they are tied)", unexpected=[name])
        return tensors
    finally:
        for f in files:
            f.close()
