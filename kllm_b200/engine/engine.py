"""``Engine``: a model folder turned into something that generates tokens.

Build-up as in the reference (engine/engine.go:48-97): read and type the
configuration, pick the model by its architecture name, build it from parts, bind
the weights by name, size the cache.  ``Options`` keeps the reference's knobs and
defaults (engine/engine.go:16-33): ``max_seq`` 256, ``block_size`` 16, ``num_blocks``
4 * max_seq / block_size; ``cache_bytes`` sizes the pools from a memory budget and
the model's layers instead; the per-step token budget and the batch limit are knobs
of their own here (the reference reuses max_seq for the first and fixes the second
in its scheduler, engine/scheduler.go:43-46).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Union

import torch

from .. import kernels
from .. import models  # noqa: F401  (registers the architectures)
from ..cache.manager import CacheManager, RequestCache
from ..config.base import ModelConfig, build_model_spec, load_config, parse_config
from ..parts.model import DecoderModel
from ..sampling.sampler import Sampler
from ..weights.loader import load_weights
from ..weights.random_init import random_tensors
from .step import StepEntry, StepRunner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32}


@dataclass
class Options:
    device: int = 0
    max_seq: int = 256            # most tokens one request may hold
    block_size: int = 16          # tokens per cache page
    num_blocks: int = 0           # pages per cache group; 0: from cache_bytes, else 4 * max_seq / block_size
    cache_bytes: int = 0          # device memory for the paged cache; sizes the pools when num_blocks is 0
    max_step_tokens: int = 0      # token budget of one step; 0: max_seq
    max_batch: int = 8            # most requests in one step
    dtype: str = "bfloat16"       # "bfloat16" (serving) or "float32" (true 32-bit)
    cuda_graphs: bool = True      # replay decode steps as CUDA graphs

    def fill(self) -> "Options":
        o = Options(**self.__dict__)
        if o.max_seq <= 0:
            o.max_seq = 256
        if o.block_size <= 0:
            o.block_size = 16
        if o.num_blocks <= 0:
            # with a byte budget the count follows from the model's layers (Engine.__init__)
            o.num_blocks = 0 if o.cache_bytes > 0 else max(1, 4 * o.max_seq // o.block_size)
        if o.max_step_tokens <= 0:
            o.max_step_tokens = o.max_seq
        if o.max_batch <= 0:
            o.max_batch = 8
        if o.dtype not in _DTYPES:
            raise ValueError(f"dtype {o.dtype!r}: choose bfloat16 or float32")
        return o


class Sequence_:
    """One generation stream, in the manner of the reference's ``Sequence``
    (engine/engine.go:148-188): ``forward(tokens)`` runs it alone and returns the
    logits of its last token; ``release()`` gives its pages back."""

    def __init__(self, engine: "Engine"):
        self.engine = engine
        self.cache: RequestCache = engine.cache.open()

    def __len__(self) -> int:
        return self.cache.length

    def forward(self, tokens: Sequence[int]) -> torch.Tensor:
        """The caller's own tensor: a replayed decode step writes its logits into a buffer
        that the next step overwrites."""
        logits = self.engine.runner.run([StepEntry(self.cache, list(tokens), [len(tokens) - 1])])
        return logits[0].clone()

    def release(self) -> None:
        if not self.cache.closed:
            self.engine.cache.close(self.cache)


class Engine:
    def __init__(self, model_dir: Optional[str], options: Optional[Options] = None, *,
                 config: Union[None, dict, ModelConfig] = None, random_seed: int = 0, **kw):
        """``model_dir``: a folder with config.json and safetensors.  With ``model_dir``
        None and a ``config`` (the dict of a config.json, or a typed configuration) the
        model gets random weights drawn on the device from ``random_seed`` (N(0, 0.02)
        matrices, gains 1): for measurements at sizes whose files would take longer to
        write than to measure."""
        opts = (options or Options(**kw)).fill()
        self.options = opts
        if not torch.cuda.is_available():
            raise RuntimeError("kllm_b200 runs on a CUDA device (sm_100a); none is visible and there "
                               "is no CPU path")
        self.device = torch.device("cuda", opts.device)
        torch.cuda.set_device(self.device)
        torch.backends.cuda.matmul.allow_tf32 = False   # float32 stays true 32-bit
        torch.backends.cudnn.allow_tf32 = False
        self.dtype = _DTYPES[opts.dtype]
        if model_dir is not None:
            self.config: ModelConfig = load_config(model_dir)
        elif config is not None:
            self.config = parse_config(config) if isinstance(config, dict) else config
        else:
            raise ValueError("Engine needs a model folder or a configuration")
        self.spec = build_model_spec(self.config)
        with torch.no_grad():
            self.model = DecoderModel(self.spec, self.dtype, self.device)
            if model_dir is not None:
                tensors = load_weights(model_dir, self.model.tensor_specs(), self.dtype, self.device)
            else:
                tensors = random_tensors(self.model.tensor_specs(), random_seed, self.dtype, self.device)
            self.model.bind(tensors)
            del tensors
            if opts.num_blocks <= 0:
                opts.num_blocks = CacheManager.pages_within(self.model.cache_needs(), opts.block_size,
                                                            self.dtype, opts.cache_bytes)
            self.cache = CacheManager(self.model.cache_needs(), opts.block_size, opts.num_blocks,
                                      max_requests=opts.max_batch, dtype=self.dtype, device=self.device)
        self.runner = StepRunner(self.model, self.cache, opts.max_step_tokens, opts.max_batch, opts.max_seq,
                                 use_graphs=opts.cuda_graphs)
        self.sampler = Sampler(self.device)
        self.eos_token_ids = tuple(self.spec.eos_token_ids)

    @property
    def max_seq(self) -> int:
        return self.runner.max_seq

    def new_sequence(self) -> Sequence_:
        return Sequence_(self)

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """One batch through the model; see ``StepRunner.run``.  The result is the
        caller's own tensor (a replayed decode step writes into a buffer that the next
        step overwrites; the scheduler, which samples at once, reads that buffer)."""
        logits = self.runner.run(entries)
        return None if logits is None else logits.clone()

    @torch.no_grad()
    def generate(self, prompt: Union[Sequence[int], Sequence[Sequence[int]]], max_new_tokens: int = 16,
                 temperature: float = 0.0, seed: int = 0) -> Union[List[int], List[List[int]]]:
        """Token ids in, generated token ids out (host lists).  One prompt gives one
        list; a list of prompts is run through the continuous-batching scheduler and
        gives a list per prompt.  Generation stops at an EOS id of the configuration
        (the EOS token is emitted) or after ``max_new_tokens``
        (reference engine/engine.go:192-213)."""
        from .scheduler import Scheduler
        single = len(prompt) > 0 and not isinstance(prompt[0], (list, tuple))
        prompts = [list(prompt)] if single else [list(p) for p in prompt]
        sched = Scheduler(self)
        reqs = [sched.submit(p, max_new_tokens, temperature=temperature, seed=seed) for p in prompts]
        sched.run()
        for r in reqs:
            if r.error:
                raise RuntimeError(f"request {r.rid}: {r.error}")
        outs = [list(r.generated) for r in reqs]
        return outs[0] if single else outs

    def close(self) -> None:
        for r in list(self.cache.live.values()):
            self.cache.close(r)
        self.runner.release_graphs()
        kernels.check_status(self.device)

    @staticmethod
    def launches() -> int:
        return kernels.launches
