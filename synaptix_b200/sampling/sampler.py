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


def sample_on_device(params: SamplingParams, logits: torch.Tensor, request: torch.Tensor, rng_step: torch.Tensor,
                     history: Optional[torch.Tensor] = None, hist_len: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` (float32 ``[rows, vocab]``, modified in place when penalties
    are on), everything on the device: ``request[r]`` and ``rng_step[r]`` (int32) pick row ``r``'s
    random word, ``history[r, :hist_len[r]]`` is its context for the penalties.  Returns int32
    ``[rows]`` (``out`` if given).  Nothing here looks at a value on the host, so a decode step
    can record it into its CUDA graph."""
    p = params
    if p.penalties_on:
        if history is None or hist_len is None:
            raise ValueError("penalties need each row's context")
        K.apply_penalties(logits, history, hist_len, p.repeat_last_n, p.repetition_penalty, p.presence_penalty,
                          p.frequency_penalty)
    if p.greedy:
        return K.argmax_rows(logits, out=out)
    return K.sample_rows(logits, p.temperature, p.top_k, p.top_p, p.min_p, p.seed, request, rng_step, out=out)


class Sampler:
    """The sampler for logits that come back from a step on the host's schedule (the prompt step
    of a batch): it brings each row's request index, step and context to the device and calls
    ``sample_on_device``.  Decode sessions keep those on the device and call it themselves."""

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
        hist = lens = None
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
            hist, lens = hist.to(self.device), lens.to(self.device)
        meta = torch.tensor([list(request_index), list(step)], dtype=torch.int32).to(self.device)
        return sample_on_device(p, logits, meta[0], meta[1], hist, lens)

    def sample_to_host(self, logits, request_index, step, contexts=None) -> List[int]:
        return self.sample(logits, request_index, step, contexts).tolist()
