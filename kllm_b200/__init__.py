"""kllm_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

    import kllm_b200
    out = kllm_b200.generate("path/to/model", [1, 17, 42, 100, 7], steps=16)

``Engine`` is the long-lived form: it loads a model folder (config.json and
safetensors) once and serves ``generate`` calls, single steps and a scheduler.
"""
from __future__ import annotations

from typing import List, Sequence, Union

__version__ = "0.1.0"


def __getattr__(name):
    # torch and the engine are imported on first use, so that tools that only need
    # the configuration or the cache manager start quickly
    if name in ("Engine", "Options", "Scheduler", "StepEntry"):
        from . import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)


def generate(model: str, ids: Union[Sequence[int], Sequence[Sequence[int]]], steps: int = 16,
             max_seq: int = 256, device: int = 0, temperature: float = 0.0, seed: int = 0,
             dtype: str = "bfloat16", **options) -> Union[List[int], List[List[int]]]:
    """Generate up to ``steps`` tokens after the prompt ``ids`` (token ids; a list
    of prompts is batched).  Arguments mirror the reference's ``generate`` command
    (cmd/generate/main.go:15-20): ``model`` folder, ``device`` index, ``ids``,
    ``steps`` = most new tokens, ``max_seq`` = cache capacity in tokens per request.
    Greedy unless ``temperature`` > 0."""
    from .engine import Engine, Options
    eng = Engine(model, Options(device=device, max_seq=max_seq, dtype=dtype, **options))
    try:
        return eng.generate(ids, max_new_tokens=steps, temperature=temperature, seed=seed)
    finally:
        eng.close()
