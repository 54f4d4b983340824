"""The sampler of a batch: logits on the device in, one token per row out.

Order of operations as in the reference's ``TokenSampler``
(crates/synaptix-models/llm/common/src/generate.rs:124-145,304-340): repetition penalty,
presence/frequency penalty, temperature, top-k, top-p, min-p, then argmax (temperature
<= 0) or a multinomial draw.  The reference copies each row of logits to the host and
samples there; here the whole batch is sampled by kernels and only the tokens come back.

Random numbers: the reference has one Philox4x32-10 stream per request and draws one 32-bit
word per token.  Here row ``r`` of a call draws word number ``step`` of the stream
(seed, counter = (step // 4, request index, 0, 0)), so a request's tokens do not depend on
which other requests share its batch, and request 0 reproduces the reference's stream.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import sampling as K
from .params import SamplingParams


class Sampler:
    def __init__(self, params: SamplingParams, device):
        params.validate()
        self.params = params
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, request_index: Sequence[int], step: Sequence[int],
               contexts: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """``logits`` float32 ``[rows, vocab]`` on the device (modified in place when
        penalties are on); ``request_index[r]`` and ``step[r]`` pick row ``r``'s random word;
        ``contexts[r]`` is the row's context (prompt and tokens so far) for the penalties.
        Returns int32 ``[rows]`` on the device."""
        p = self.params
        R = logits.shape[0]
        if p.penalties_on:
            if contexts is None:
                raise ValueError("penalties need each row's context")
            n = max(1, max(len(c) for c in contexts))
            hist = torch.zeros((R, n), dtype=torch.int32)
            lens = torch.zeros(R, dtype=torch.int32)
            for r, c in enumerate(contexts):
                if len(c):
                    hist[r, :len(c)] = torch.as_tensor(list(c), dtype=torch.int32)
                lens[r] = len(c)
            K.apply_penalties(logits, hist.to(self.device), lens.to(self.device), p.repeat_last_n,
                              p.repetition_penalty, p.presence_penalty, p.frequency_penalty)
        if p.greedy:
            return K.argmax_rows(logits)
        meta = torch.tensor([list(request_index), list(step)], dtype=torch.int32).to(self.device)
        return K.sample_rows(logits, p.temperature, p.top_k, p.top_p, p.min_p, p.seed, meta[0], meta[1])

    def sample_to_host(self, logits, request_index, step, contexts=None) -> List[int]:
        return self.sample(logits, request_index, step, contexts).tolist()
