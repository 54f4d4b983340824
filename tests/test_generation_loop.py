"""The generation loop's decisions, with a fake engine and a fake sampler (CPU).

The fake model is a counter: the next token is always the last token + 1 (the idea of the
reference's CounterLm, crates/synaptix-infer/tests/engine_ops.rs:19-37).
"""
import pytest

from synaptix_b200.cache import CacheFull, PagePool, SequenceSlots, pages_for
from synaptix_b200.engine import GenerationOptions, plan_batches, run_generation
from synaptix_b200.sampling import SamplingParams


class CounterEngine:
    def __init__(self, max_tokens=4096, max_seqs=8):
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.slots = SequenceSlots(max_seqs, [PagePool(pages_for(max_tokens))])
        self.steps = []          # per step: list of (slot, n_tokens)
        self.opened, self.closed = [], []

    def open(self):
        s = self.slots.open()
        self.opened.append(s)
        return s

    def close(self, slot):
        self.slots.close(slot)
        self.closed.append(slot)

    def step(self, entries, keep=True):
        self.slots.reserve_many([e.slot for e in entries], [len(e.tokens) for e in entries])
        for e in entries:
            self.slots.advance(e.slot, len(e.tokens))
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        # "logits": the next token for each wanted place
        return [e.tokens[w] + 1 for e in entries for w in e.want]


def counter_sample(logits, request_index, step, contexts):
    return list(logits)


def test_greedy_to_max_length_counts_the_first_token():
    eng = CounterEngine()
    res, st = run_generation(eng, counter_sample, [[5, 6, 7]], GenerationOptions(max_new_tokens=4))
    assert res[0].tokens == [8, 9, 10, 11] and res[0].finish_reason == "length"
    assert eng.steps[0] == [(0, 3)] and len(eng.steps) == 4          # 1 prompt step + 3 single-token steps
    assert st.new_tokens == 4 and st.prompt_tokens == 3 and st.decode_steps == 3
    assert eng.slots.n_live == 0


def test_stop_token_is_part_of_the_output():
    eng = CounterEngine()
    res, _ = run_generation(eng, counter_sample, [[1]], GenerationOptions(max_new_tokens=50, stop_token_ids=(4,)))
    assert res[0].tokens == [2, 3, 4] and res[0].finish_reason == "stop"
    # a stop token sampled from the prompt ends the sequence with no decode step
    eng = CounterEngine()
    res, _ = run_generation(eng, counter_sample, [[3]], GenerationOptions(max_new_tokens=50, stop_token_ids=(4,)))
    assert res[0].tokens == [4] and len(eng.steps) == 1


def test_unequal_batch_shrinks_as_sequences_end():
    eng = CounterEngine()
    prompts = [[10], [20, 21], [30, 31, 32]]
    opts = GenerationOptions(max_new_tokens=10, stop_token_ids=(12, 25))
    res, st = run_generation(eng, counter_sample, prompts, opts)
    assert res[0].tokens == [11, 12] and res[1].tokens == [22, 23, 24, 25]
    assert res[2].tokens == list(range(33, 43)) and res[2].finish_reason == "length"
    assert eng.steps[0] == [(0, 1), (1, 2), (2, 3)]
    assert [len(s) for s in eng.steps[1:]] == [3, 2, 2, 1, 1, 1, 1, 1, 1]
    assert eng.slots.n_live == 0 and sorted(eng.closed) == [0, 1, 2]
    # slots are given back as soon as a sequence ends, not at the batch's end
    assert eng.closed[0] == 0


def test_batches_run_one_after_another_in_reused_slots():
    eng = CounterEngine(max_tokens=4096, max_seqs=8)
    prompts = [[i * 100] for i in range(7)]
    res, st = run_generation(eng, counter_sample, prompts, GenerationOptions(max_new_tokens=3, max_batch_size=3))
    assert st.batches == 3
    assert [r.tokens for r in res] == [[i * 100 + 1, i * 100 + 2, i * 100 + 3] for i in range(7)]
    assert max(eng.opened) <= 2          # the second and third batch run in the slots of the first
    assert eng.slots.pools[0].n_free == eng.slots.pools[0].n_pages


def test_batches_are_cut_to_the_cache():
    # 4 pages: each request of 60 + 10 tokens needs 2
    assert plan_batches([60, 60, 60], 10, 256, 8, None) == [[0, 1], [2]]
    assert plan_batches([60, 60, 60], 4, 256, 8, None) == [[0, 1, 2]]       # 60 + 3 fed back = 63: one page each
    assert plan_batches([10] * 5, 5, 64 * 100, 2, None) == [[0, 1], [2, 3], [4]]
    with pytest.raises(CacheFull, match="prompt"):
        plan_batches([300], 5, 256, 8, None)


def test_sequence_ends_by_capacity_when_the_cache_is_full():
    eng = CounterEngine(max_tokens=128, max_seqs=4)          # 2 pages
    res, _ = run_generation(eng, counter_sample, [[0] * 60], GenerationOptions(max_new_tokens=500))
    r = res[0]
    assert r.finish_reason == "capacity"
    # 128 tokens fit the cache; the token sampled from the last of them is still produced
    assert len(r.tokens) == 128 - 60 + 1
    assert eng.slots.n_live == 0


def test_zero_new_tokens_and_empty_prompt():
    eng = CounterEngine()
    res, _ = run_generation(eng, counter_sample, [[1, 2]], GenerationOptions(max_new_tokens=0))
    assert res[0].tokens == [] and eng.steps == []
    with pytest.raises(ValueError, match="empty"):
        run_generation(eng, counter_sample, [[]], GenerationOptions())


def test_sampler_gets_request_index_step_and_context():
    eng = CounterEngine()
    seen = []

    def spy(logits, request_index, step, contexts):
        seen.append((list(request_index), list(step), None if contexts is None else [list(c) for c in contexts]))
        return list(logits)

    opts = GenerationOptions(max_new_tokens=3, sampling=SamplingParams(repetition_penalty=1.5), stop_token_ids=(7,))
    run_generation(eng, spy, [[5], [8, 9]], opts)
    assert seen[0] == ([0, 1], [0, 0], [[5], [8, 9]])
    assert seen[1] == ([0, 1], [1, 1], [[5, 6], [8, 9, 10]])
    assert seen[2] == ([1], [2], [[8, 9, 10, 11]])           # request 0 stopped at token 7


def test_on_token_streams_in_order():
    eng = CounterEngine()
    got = []
    run_generation(eng, counter_sample, [[1], [50]], GenerationOptions(max_new_tokens=2),
                   on_token=lambda i, t: got.append((i, t)))
    assert got == [(0, 2), (1, 51), (0, 3), (1, 52)]
