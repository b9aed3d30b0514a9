"""Choosing the next token: greedy and temperature sampling.

Greedy is the reference's only rule: the first index of the maximum
(engine/engine.go:216-224).  Temperature sampling draws from softmax(z / T)
(described, not built, in the reference: docs/theory/02-autoregressive-decoding.md
:122-124).  The uniform number of a draw comes from a counter-based generator
keyed by (seed, request id, index of the generated token), so what a request
samples does not depend on what else is in the batch or on how steps were cut.
The selection itself runs on the device (``csrc/sampling.cu``).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .. import kernels

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x &= _MASK
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK
    x ^= x >> 31
    return x


def uniform_for(seed: int, request_id: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits, exact in float32."""
    x = _mix((seed & _MASK) + 0x9E3779B97F4A7C15)
    x = _mix(x ^ ((request_id & _MASK) * 0xD6E8FEB86659FD93 & _MASK))
    x = _mix(x ^ ((index & _MASK) * 0xCA5A826395121157 & _MASK))
    return (x >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float],
               keys: Sequence[Tuple[int, int, int]], last_token=None, slots=None, host_out=None) -> torch.Tensor:
        """int32 [rows] on the device.  Row r is greedy when temperatures[r] <= 0,
        else drawn with the uniform number of keys[r] = (seed, request id, index).
        ``last_token`` / ``slots``: see ``kernels.sample`` (the choice also goes to the
        request slot's entry, for a next step that is launched before this one is read;
        ``host_out``: pinned host memory that the kernel also writes the choices to)."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        if all(t <= 0 for t in temperatures):
            kernels.sample(out, logits, None, None, last_token, slots, host_out)
            return out
        host = torch.empty((2, rows), dtype=torch.float32, pin_memory=logits.is_cuda)
        for r in range(rows):
            host[0, r] = float(temperatures[r])
            host[1, r] = uniform_for(*keys[r]) if temperatures[r] > 0 else 0.0
        dev = host.to(logits.device, non_blocking=True)
        kernels.sample(out, logits, dev[0], dev[1], last_token, slots, host_out)
        return out

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        kernels.sample(out, logits, None, None)
        return out
