"""Random-weights mode: write a model folder (config.json, model.safetensors) from
a configuration and a seed.

Matrices are N(0, std) and norm gains N(1, gain_std), as the reference's tiny-model
generator draws them (tools/make_test_model.py:59-80: std 0.02, gains 1 + 0.01 N).
Each tensor has a random stream of its own, keyed by (seed, tensor name), so the
values do not depend on the order of creation or on which other tensors exist.
The file is streamed, one tensor in memory at a time.

``random_tensors`` fills the same tensors in place of a folder, on the device the
model lives on: measurements of models with billions of parameters need not write and
read tens of gigabytes first.  Its streams are keyed the same way but drawn by the
device's generator, so its numbers are not the file's numbers.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Union

import torch

from ..config.base import ModelConfig, build_model_spec, parse_config
from ..parts.model import DecoderModel
from .loader import stored_dtype
from .safetensors_io import write_safetensors


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(spec, seed: int, std: float, gain_std: float, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, spec.name))
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    if spec.store == "int32":
        raise ValueError(f"random-weights mode cannot fill the integer table {spec.name}")
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    if spec.init == "gain":
        t = 1.0 + gain_std * t
    elif spec.init == "normal":
        t = std * t
    else:
        raise ValueError(f"tensor {spec.name}: unknown init {spec.init!r}")
    return t.to(dtype)


def random_tensors(specs, seed: int, dtype: torch.dtype, device, std: float = 0.02,
                   gain_std: float = 0.0) -> dict:
    """name -> random tensor on ``device`` for every tensor of ``specs`` that is not
    optional, stored as the loader would store it (``dtype`` for matrices, float32 for
    tensors that stay 32-bit)."""
    return {s.name: random_tensor(s, seed, std, gain_std, stored_dtype(s, dtype), device)
            for s in specs if not s.optional}


def write_random_model(out_dir: str, config: Union[ModelConfig, dict], seed: int,
                       dtype: torch.dtype = torch.float32, std: float = 0.02,
                       gain_std: float = 0.0) -> str:
    """Create ``out_dir`` with config.json and model.safetensors; returns out_dir.

    ``dtype`` is the dtype of the matrices in the file; tensors that the model keeps
    in 32-bit (norm gains) are written as F32.
    """
    import kllm_b200.models  # noqa: F401  (registers the architectures)
    if isinstance(config, dict):
        config = parse_config(config)
    spec = build_model_spec(config)
    model = DecoderModel(spec, dtype, "cpu")
    specs = [s for s in model.tensor_specs() if not s.optional]
    os.makedirs(out_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16",
                          torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    by_name = {s.name: s for s in specs}
    listing = [(s.name, tuple(s.shape), stored_dtype(s, dtype)) for s in specs]
    write_safetensors(os.path.join(out_dir, "model.safetensors"), listing,
                      lambda n: random_tensor(by_name[n], seed, std, gain_std,
                                              stored_dtype(by_name[n], dtype)))
    return out_dir
