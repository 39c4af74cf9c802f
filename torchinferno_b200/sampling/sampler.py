"""Next-token choice: greedy and temperature sampling, per request.

The reference samples with ``argmax`` when ``temperature <= 0`` and otherwise
draws from ``softmax(logits.float() / temperature)`` with ``torch.multinomial``
(src/torchinferno/runtime/sampling.py:7-11); its tensor-parallel model draws the
same distribution in Gumbel-max form
(src/torchinferno/models/llama3/tensor_parallel.py:9946-9996).  Per-request
temperatures override the engine default (src/torchinferno/runtime/serving.py:413).
top_p other than 1, top-k and penalties are not offered there
(src/torchinferno/server/openai_protocol.py:34-38) nor here.

Here the Gumbel-max form runs in one kernel with counter-based noise keyed by
(request seed, position of the token being drawn, vocabulary index): given the
same logits, a request's token does not depend on what else is in the batch,
nor on how its prompt was cut.  (In bfloat16 the logits themselves may differ in
their last bits with the number of rows of a step, because products of few and
of many rows run different kernels; in float32 they do not.)

The engine keeps every live request's seed and temperature in its record on the
device (``CacheManager.request_records``); :meth:`Sampler.sample_records` reads
them there by slot and leaves the drawn token in the record, so a sampled step
copies nothing from the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from torchinferno_b200.kernels import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")


class Sampler:
    def __init__(self, device: torch.device) -> None:
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], positions: Sequence[int]) -> torch.Tensor:
        """Token ids (int32, on the device) for fp32 ``logits`` [n, vocab].

        ``positions[i]`` is the position in its sequence of the token being drawn for row i.
        """
        n = logits.shape[0]
        if len(params) != n or len(positions) != n:
            raise ValueError("one SamplingParams and one position per logits row are needed")
        out = torch.empty(n, dtype=torch.int32, device=self.device)
        if n == 0:
            return out
        if all(p.temperature <= 0 for p in params):
            return ops.sample(logits, out)
        temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(self.device)
        seeds = torch.tensor([_as_int64(p.seed) for p in params], dtype=torch.int64).to(self.device)
        pos = torch.tensor(list(positions), dtype=torch.int32).to(self.device)
        return ops.sample(logits, out, temperature, seeds, pos)


    def sample_records(self, logits: torch.Tensor, records: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
        """Token ids (int32, on the device) for fp32 ``logits`` [n, vocab] whose row i belongs to the request in
        slot ``slots[i]``: temperature, seed and the position of the token being drawn (the request's length)
        come from ``records``; the token is also written there as the request's next input."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=self.device)
        if logits.shape[0] == 0:
            return out
        return ops.sample_records(logits, out, records, slots)



def _as_int64(seed: int) -> int:
    seed &= 0xFFFFFFFFFFFFFFFF
    return seed - (1 << 64) if seed >= (1 << 63) else seed
