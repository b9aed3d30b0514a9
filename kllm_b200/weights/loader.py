"""Binding the tensors of a model folder to what the model's parts expect.

The model lists its tensors (name, shape, how to store).  The loader reads each
by name and keeps it in the model's dtype: bfloat16 for serving, float32 for the
32-bit path; a tensor that a part declares as 32-bit (norm gains) stays float32 and
integer tables become int32.  Files may hold F32, BF16 or F16 (the reference takes
F32 only, engine/engine.go:140-141).  Everything that is wrong with the set of
tensors is reported in ONE ``WeightError`` that lists the missing names, the
unexpected names, the wrong shapes and the wrong dtypes (the reference stops at the
first missing name or element count, backend/model.cu:510-519).

Tensors that the model does not ask for are not a fault by themselves: the reference
uploads whatever a file holds and uses what it needs (backend/model.cu:747-765; its
converter drops the rest offline, tools/convert_hf.py:86-93), and older checkpoints
carry tables such as ``rotary_emb.inv_freq``.  They are left unread, counted, and
named in a ``UserWarning``; the error for a folder with real faults names them too,
since a misspelt tensor shows up as one missing and one unexpected name.
``strict=True`` makes them a fault of their own.
"""
from __future__ import annotations

import warnings
from typing import Dict, Iterable, List, Tuple

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import ModelFiles

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    def __init__(self, model_dir: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], wrong_dtype: List[Tuple[str, str]]):
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        self.wrong_dtype = wrong_dtype
        lines = [f"weights in {model_dir} do not fit the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong_shape))
        if wrong_dtype:
            lines.append(f"  wrong dtype ({len(wrong_dtype)}): " + ", ".join(
                f"{n} is {got}" for n, got in wrong_dtype))
        super().__init__("\n".join(lines))


def stored_dtype(spec: TensorSpec, model_dtype: torch.dtype) -> torch.dtype:
    if spec.store == "compute":
        return model_dtype
    if spec.store == "float32":
        return torch.float32
    if spec.store == "int32":
        return torch.int32
    raise ValueError(f"tensor {spec.name}: unknown store {spec.store!r}")


def check_names(files: ModelFiles, specs: Iterable[TensorSpec], model_dir: str, strict: bool = False) -> List[str]:
    """Raise ONE ``WeightError`` for everything that is wrong; return the names the model
    does not ask for (an error of their own only when ``strict``)."""
    specs = list(specs)
    by_name = {s.name: s for s in specs}
    have = set(files.names())
    missing = sorted(s.name for s in specs if s.name not in have and not s.optional)
    unexpected = sorted(have - set(by_name))
    wrong_shape, wrong_dtype = [], []
    for name in sorted(have & set(by_name)):
        e = files.entry(name)
        if tuple(e.shape) != tuple(by_name[name].shape):
            wrong_shape.append((name, tuple(e.shape), tuple(by_name[name].shape)))
        ok = _INTS if by_name[name].store == "int32" else _FLOATS
        if e.dtype not in ok:
            wrong_dtype.append((name, str(e.dtype)))
    if missing or wrong_shape or wrong_dtype or (strict and unexpected):
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_dtype)
    return unexpected


def load_weights(model_dir: str, specs: Iterable[TensorSpec], model_dtype: torch.dtype,
                 device, strict: bool = False) -> Dict[str, torch.Tensor]:
    """name -> tensor on ``device`` for every expected tensor that the files hold.
    Tensors that no part asked for stay unread; a warning counts and names them
    (``strict``: they are an error)."""
    specs = list(specs)
    out: Dict[str, torch.Tensor] = {}
    with ModelFiles(model_dir) as files:
        extra = check_names(files, specs, model_dir, strict)
        if extra:
            shown = ", ".join(extra[:8]) + (", ..." if len(extra) > 8 else "")
            warnings.warn(f"{model_dir}: {len(extra)} tensor(s) that the model does not use were ignored: {shown}",
                          stacklevel=2)
        have = set(files.names())
        for s in specs:
            if s.name not in have:
                continue
            t = files.read(s.name, copy=False)
            # copy=True: the result must not alias the file mapping, which closes below
            out[s.name] = t.to(device=device, dtype=stored_dtype(s, model_dtype), copy=True).contiguous()
            del t
    return out
