"""Choosing the next token: greedy, or a draw at a temperature.

Greedy is the reference's rule (`src/core_kernels/argmax.cu:19-67`): the largest
logit, the lowest index on a tie, NaN never wins; a row with no finite winner is
an error (`src/core_kernels/bindings_device.cpp:183-196`). Temperature sampling
is this library's addition: one draw from softmax(logits / T), made with the
Gumbel-max rule from noise keyed by (seed, request, step), so that a request's
tokens depend neither on the batch it is in nor on the order of batches.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self):
        if not (self.temperature >= 0.0) or self.temperature == float("inf"):
            raise ValueError(f"temperature must be a number >= 0, got {self.temperature}")
        if self.seed < 0:
            raise ValueError(f"seed must not be negative, got {self.seed}")


def choose(logits: torch.Tensor, params: SamplingParams, requests=None, steps=None) -> torch.Tensor:
    """Token ids (int32, on the device) for rows of fp32 logits. `requests[i]` and
    `steps[i]` say whose row i is and how many tokens that request has drawn."""
    if params.temperature == 0.0:
        return ops.choose(logits)
    device = logits.device
    request = torch.as_tensor(list(requests), dtype=torch.int32).to(device, non_blocking=True)
    step = torch.as_tensor(list(steps), dtype=torch.int32).to(device, non_blocking=True)
    return ops.choose(logits, params.temperature, params.seed, request, step)


def check_chosen(tokens, vocab: int) -> None:
    """Refuse an id past the vocabulary: the row had no finite logit."""
    bad = [i for i, t in enumerate(tokens) if not 0 <= int(t) < vocab]
    if bad:
        raise RuntimeError(f"no finite logit in row(s) {bad}: the model produced NaN or "
                           "infinities only")
