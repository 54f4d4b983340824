"""The Python entry point: load a model once, generate for lists of token ids.

The reference's facade is ``load_llm(...) -> Llm`` with ``generate_streaming`` and
``GenerationOptions`` (crates/synaptix/src/facade/llm.rs:297-310,933-1006); option
names and defaults are those of its ``GenerationConfig``
(crates/synaptix-models/llm/common/src/generate.rs:16-57).  Prompts are token ids:
tokenizers are outside this library.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

from .engine.generate import GenerationOptions, GenerationStats, run_generation
from .engine.step import Engine
from .models import load_model
from .sampling import Sampler, SamplingParams


class LLM:
    """A loaded model with its cache.

    ``max_tokens`` sizes the cache: the most tokens live sequences hold at any time, each
    sequence's count rounded up to a multiple of 64.  ``max_seq`` (the reference's name for
    the per-sequence capacity) is a shorthand: with ``max_batch`` it gives
    ``max_tokens = max_batch * max_seq``.
    """

    def __init__(self, model_dir: str, compute_dtype="bf16", device: str = "cuda:0",
                 max_tokens: Optional[int] = None, max_seq: Optional[int] = None, max_batch: int = 8,
                 graph: bool = True, source=None, nvtx: bool = False):
        self._setup(load_model(model_dir, dtype=compute_dtype, device=device, source=source),
                    max_tokens, max_seq, max_batch, graph, nvtx)

    @classmethod
    def from_model(cls, model, max_tokens: Optional[int] = None, max_seq: Optional[int] = None,
                   max_batch: int = 8, graph: bool = True, nvtx: bool = False) -> "LLM":
        """An ``LLM`` around a model that already has its weights bound (``DecoderModel.load``)."""
        self = cls.__new__(cls)
        self._setup(model, max_tokens, max_seq, max_batch, graph, nvtx)
        return self

    def _setup(self, model, max_tokens, max_seq, max_batch, graph, nvtx=False) -> None:
        self.model = model
        cfg = self.model.config
        if max_tokens is None:
            per_seq = max_seq or getattr(cfg, "max_position_embeddings", None) or 4096
            max_tokens = max_batch * per_seq
        self.engine = Engine(self.model, max_tokens=max_tokens, use_graphs=graph, nvtx=nvtx)
        self.last_stats: Optional[GenerationStats] = None

    @property
    def config(self):
        return self.model.config

    @property
    def vocab_size(self) -> int:
        return self.model.vocab_size

    @property
    def device(self):
        return self.engine.device

    @property
    def kv_bytes_per_token(self) -> int:
        """Bytes of cache a token takes over all layers (as the reference's ``Llm::kv_bytes_per_token``)."""
        return self.engine.cache.kv_bytes_per_token

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 64, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                 repeat_last_n: int = 0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                 seed: int = 0, eos_token_id: Optional[int] = None, eos_token_ids: Optional[Sequence[int]] = None,
                 max_batch_size: Optional[int] = None, prefill_batch: int = 0,
                 on_token: Optional[Callable[[int, int], Optional[bool]]] = None,
                 return_details: bool = False):
        """Generate for each prompt (a list of token ids); returns the new tokens of each.

        Stop tokens: ``eos_token_ids`` together with ``eos_token_id``; if neither is given,
        the model configuration's.  A stop token ends its sequence and is part of the output.
        ``prefill_batch``: prompts run in portions of that many tokens a sequence (0: whole, in one step).
        ``on_token(request, token)`` is called for every new token; if it returns ``False`` that sequence ends there
        (``finish_reason`` "cancelled").
        """
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        out = self._generate(prompts, self.engine, None, None, max_new_tokens=max_new_tokens, temperature=temperature,
                             top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=repetition_penalty,
                             repeat_last_n=repeat_last_n, presence_penalty=presence_penalty,
                             frequency_penalty=frequency_penalty, seed=seed, eos_token_id=eos_token_id,
                             eos_token_ids=eos_token_ids, max_batch_size=max_batch_size, prefill_batch=prefill_batch,
                             on_token=on_token, return_details=return_details)
        return out[0] if single else out

    def conversation(self) -> "Conversation":
        """A sequence whose cache is kept between calls (see ``Conversation``); close it to give its slot back."""
        return Conversation(self)

    def _generate(self, prompts, engine, cached, lookahead, max_new_tokens: int = 64, temperature: float = 0.0,
                  top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                  repeat_last_n: int = 0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                  seed: int = 0, eos_token_id: Optional[int] = None, eos_token_ids: Optional[Sequence[int]] = None,
                  max_batch_size: Optional[int] = None, prefill_batch: int = 0, on_token=None,
                  return_details: bool = False):
        if eos_token_id is None and eos_token_ids is None:
            stop: Tuple[int, ...] = tuple(self.model.stop_token_ids)
        else:
            stop = tuple(eos_token_ids or ()) + ((eos_token_id,) if eos_token_id is not None else ())
        params = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                                repetition_penalty=repetition_penalty, repeat_last_n=repeat_last_n,
                                presence_penalty=presence_penalty, frequency_penalty=frequency_penalty,
                                seed=seed)
        sampler = Sampler(params, self.engine.device)
        opts = GenerationOptions(max_new_tokens=max_new_tokens, stop_token_ids=stop, sampling=params,
                                 max_batch_size=max_batch_size, prefill_batch=prefill_batch,
                                 **({} if lookahead is None else {"lookahead": lookahead}))
        results, stats = run_generation(engine, sampler.sample_to_host, prompts, opts, on_token=on_token, cached=cached)
        self.last_stats = stats
        return results if return_details else [r.tokens for r in results]


class _HeldSlot:
    """The engine as the generation loop knows it, with ONE slot that is open already and stays open: ``open`` hands
    that slot out, ``close`` leaves it alone.  Everything else is the engine's."""

    def __init__(self, engine, slot: int):
        self._engine, self._slot = engine, slot
        self.max_seqs = 1

    def open(self) -> int:
        return self._slot

    def close(self, slot: int) -> None:
        pass

    def __getattr__(self, name):
        return getattr(self._engine, name)


class Conversation:
    """One sequence whose cache is kept between calls, so that a prompt which goes on from the last call's tokens
    runs only what is new (the reference keeps a ``KvCache`` between the turns of a chat the same way:
    ``generate_streaming_resume``, crates/synaptix-models/llm/qwen3/src/pipeline.rs:134-147, generate.rs:248-250).

    ``generate(prompt, ...)`` takes the WHOLE sequence so far (earlier prompts, earlier answers and what is new) and
    the options of ``LLM.generate``.  If the cached tokens are the prompt's beginning only the rest runs; otherwise
    the cache is dropped and the whole prompt runs (``reusable`` / ``invalidate``, as the reference's
    ``LlmKvSession``, crates/synaptix/src/facade/llm.rs:515-590)."""

    def __init__(self, llm: "LLM"):
        self.llm = llm
        self.slot: Optional[int] = llm.engine.open()
        self.tokens: List[int] = []          # the tokens whose keys and values the cache holds, in order

    @property
    def cached_tokens(self) -> int:
        return len(self.tokens)

    def reusable(self, prompt: Sequence[int]) -> int:
        """How many tokens of ``prompt`` the cache holds already: all cached tokens, if they are the prompt's beginning
        and the prompt brings at least one more (its last token always runs: the first logits come from it); else 0."""
        n = len(self.tokens)
        return n if 0 < n < len(prompt) and list(prompt[:n]) == self.tokens else 0

    def invalidate(self) -> None:
        """Forget the cached tokens (the slot's pages go back; the sequence starts anew)."""
        if self.slot is None:
            raise ValueError("this conversation is closed")
        self.llm.engine.close(self.slot)
        self.slot = self.llm.engine.open()
        self.tokens = []

    def generate(self, prompt: Sequence[int], **kw) -> List[int]:
        if self.slot is None:
            raise ValueError("this conversation is closed")
        prompt = list(prompt)
        n = self.reusable(prompt)
        if n == 0 and self.tokens:
            self.invalidate()
        # one step at a time (no step launched ahead), so that the cache ends with exactly the tokens that were drawn
        out = self.llm._generate([prompt], _HeldSlot(self.llm.engine, self.slot), [n], 1, **kw)[0]
        held = self.llm.engine.cache.slots.length(self.slot)
        self.tokens = (prompt + out)[:held]     # every token that went through the model: all but the last one drawn
        return out

    def close(self) -> None:
        if self.slot is not None:
            self.llm.engine.close(self.slot)
            self.slot = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def load_llm(model_dir: str, **kw) -> LLM:
    return LLM(model_dir, **kw)


def generate(model_dir: str, prompts: Sequence[Sequence[int]], compute_dtype="bf16", device="cuda:0",
             max_tokens: Optional[int] = None, **gen_kw) -> List[List[int]]:
    """One-shot: load ``model_dir`` and generate for ``prompts`` (lists of token ids)."""
    if max_tokens is None:
        new = gen_kw.get("max_new_tokens", 64)
        max_tokens = sum(((len(p) + new + 63) // 64) * 64 for p in prompts)
    return LLM(model_dir, compute_dtype=compute_dtype, device=device, max_tokens=max_tokens).generate(
        prompts, **gen_kw)
