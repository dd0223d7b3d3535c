"""Weights by tensor name. The model's `ModelSpec` says which checkpoint tensors it needs and their shapes; this
loader reads them and reports everything that is wrong in ONE error: missing tensors, unexpected tensors, wrong
shapes (the reference raises separate errors: src/etalii_dllm/transformer.py:270-273, 291-293;
src/etalii_dllm/importing/importer.py:544).

Storage dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 is widened to
float32 (exact), integer tables become int32. What a part then computes in is the part's business.
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..parts.registry import part_factory
from ..parts.spec import ModelSpec, ParamSpec
from .safetensors_io import SafetensorsError, SafetensorsFile, checkpoint_files


class WeightError(ValueError):
    """The checkpoint does not fit the model; `missing`, `unexpected` and `wrong_shape` say how."""

    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        self.other = list(other)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name} is {list(have)}, expected {list(want)}" for name, have, want in self.wrong_shape))
        lines += [f"  {text}" for text in self.other]
        super().__init__("\n".join(lines))


def expected_tensors(spec: ModelSpec) -> dict[str, ParamSpec]:
    """Checkpoint name -> shape and init rule, from every part's own declaration. A name used by two parts (a tied
    head) must be declared with one shape."""
    out: dict[str, ParamSpec] = {}
    for path, role, part_spec in spec.part_specs():
        declared = part_factory(role, part_spec.kind).parameters(**dict(part_spec.params))
        for local, param in declared.items():
            name = part_spec.names.get(local)
            if name is None:
                raise ValueError(f"{path} ({part_spec.kind}) has no checkpoint name for its tensor {local!r}")
            if name in out and tuple(out[name].shape) != tuple(param.shape):
                raise ValueError(f"tensor {name!r} is declared with shapes {out[name].shape} and {param.shape}")
            out.setdefault(name, param)
    return out


def _keep(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.dtype == torch.float16:
        return tensor.float()
    if tensor.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return tensor.to(torch.int32)
    return tensor


def load_weights(folder: str, spec: ModelSpec) -> dict[str, torch.Tensor]:
    """Reads the tensors `spec` needs from `folder`'s safetensors file(s); raises `WeightError` listing every
    mismatch at once."""
    expected = expected_tensors(spec)
    files = [SafetensorsFile(path) for path in checkpoint_files(folder)]
    try:
        where: dict[str, SafetensorsFile] = {}
        other = []
        for handle in files:
            for name in handle.names():
                if name in where:
                    other.append(f"tensor {name} is in more than one file")  # safetensors.py:167-168
                where[name] = handle
        missing = [name for name in expected if name not in where]
        unexpected, wrong = [], []
        for name, handle in where.items():
            if name in expected:
                if tuple(handle.shape(name)) != tuple(expected[name].shape):
                    wrong.append((name, handle.shape(name), expected[name].shape))
                elif handle.dtype(name) == torch.float64:
                    other.append(f"tensor {name} is stored as F64, which is not supported")
            elif name in spec.equal_if_present or name.endswith(tuple(spec.ignored_suffixes) or ("\0",)):
                continue
            else:
                unexpected.append(name)
        if missing or unexpected or wrong or other:
            raise WeightError(missing, unexpected, wrong, other)
        tensors = {name: _keep(where[name].tensor(name)) for name in expected}
        for name, twin in spec.equal_if_present.items():
            if name in where and twin in tensors:
                extra = _keep(where[name].tensor(name))
                if extra.shape != tensors[twin].shape or not torch.equal(extra.float(), tensors[twin].float()):
                    # a tied model whose stored head differs from its embedding (importer.py:1279-1283)
                    raise WeightError([], [], [], [f"{name} is stored but differs from {twin}, which the model uses"])
        return tensors
    finally:
        for handle in files:
            handle.close()


__all__ = ["WeightError", "SafetensorsError", "expected_tensors", "load_weights"]
