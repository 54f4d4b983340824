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
        self.sessions = []

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

    def check_kernels(self):
        self.checks = getattr(self, "checks", 0) + 1

    def start_decode(self, rows, sampling=None):
        self.sessions.append(CounterSession(self, rows, sampling))
        return self.sessions[-1]


class CounterSession:
    """The engine's decode session, faked: the token after ``t`` is ``t + 1``; a step's tokens are
    known when it is launched but handed out only by ``collect``, in order."""

    def __init__(self, engine, rows, sampling):
        self.engine, self.sampling = engine, sampling
        self.rows = list(rows)
        self.next = [r.token for r in rows]
        self.queue = []
        self.most_in_flight = 0

    @property
    def in_flight(self):
        return len(self.queue)

    def launch(self):
        eng = self.engine
        eng.slots.reserve_many([r.slot for r in self.rows], [1] * len(self.rows))
        for r in self.rows:
            eng.slots.advance(r.slot, 1)
        eng.steps.append([(r.slot, 1) for r in self.rows])
        self.next = [t + 1 for t in self.next]
        self.queue.append(list(self.next))
        self.most_in_flight = max(self.most_in_flight, len(self.queue))

    def collect(self):
        return self.queue.pop(0)

    def drop(self, rows):
        assert not self.queue, "rows dropped while steps are in flight"
        gone = set(rows)
        self.rows = [r for i, r in enumerate(self.rows) if i not in gone]
        self.next = [t for i, t in enumerate(self.next) if i not in gone]


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
    # a stop token is seen when the next step is already launched: that step still has the stopped row
    assert [len(s) for s in eng.steps[1:]] == [3, 3, 2, 2, 1, 1, 1, 1, 1]
    assert eng.sessions[0].most_in_flight == 2
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


def test_sampler_and_session_get_request_index_step_and_context():
    eng = CounterEngine()
    seen = []

    def spy(logits, request_index, step, contexts):
        seen.append((list(request_index), list(step), None if contexts is None else [list(c) for c in contexts]))
        return list(logits)

    params = SamplingParams(repetition_penalty=1.5)
    opts = GenerationOptions(max_new_tokens=3, sampling=params, stop_token_ids=(7,))
    res, _ = run_generation(eng, spy, [[5], [6], [8, 9]], opts)
    # the prompt step is sampled by the function; request 1 stops at once (token 7)
    assert seen == [([0, 1, 2], [0, 0, 0], [[5], [6], [8, 9]])]
    assert [r.tokens for r in res] == [[6, 7], [7], [10, 11, 12]]
    # the session samples the rest: it is told each row's request, how many tokens it has, and its context
    sess = eng.sessions[0]
    assert sess.sampling == params
    assert len(eng.sessions) == 1


def test_session_rows_carry_what_the_sampler_needs():
    eng = CounterEngine()
    opts = GenerationOptions(max_new_tokens=2, sampling=SamplingParams(presence_penalty=0.5))
    rows = []
    real = eng.start_decode

    def spy(r, sampling=None):
        rows.extend(r)
        return real(r, sampling)

    eng.start_decode = spy
    run_generation(eng, counter_sample, [[5], [8, 9]], opts)
    assert [(r.slot, r.token, r.request, r.sampled_so_far, list(r.context)) for r in rows] == [
        (0, 6, 0, 1, [5, 6]), (1, 10, 1, 1, [8, 9, 10])]
    # without penalties no context is carried
    eng, rows[:] = CounterEngine(), []
    real = eng.start_decode
    eng.start_decode = spy
    run_generation(eng, counter_sample, [[5]], GenerationOptions(max_new_tokens=2))
    assert rows[0].context is None


def test_a_sequence_that_ends_by_length_runs_no_step_too_many():
    eng = CounterEngine()
    run_generation(eng, counter_sample, [[1], [2]], GenerationOptions(max_new_tokens=5))
    assert len(eng.steps) == 1 + 4 and all(len(s) == 2 for s in eng.steps)
    # lookahead 1: every step's tokens are read before the next is launched
    eng = CounterEngine()
    res, _ = run_generation(eng, counter_sample, [[1]], GenerationOptions(max_new_tokens=4, stop_token_ids=(3,), lookahead=1))
    assert res[0].tokens == [2, 3] and len(eng.steps) == 2 and eng.sessions[0].most_in_flight == 1


def test_the_step_after_a_stop_token_is_dropped():
    eng = CounterEngine()
    got = []
    res, st = run_generation(eng, counter_sample, [[1], [10]], GenerationOptions(max_new_tokens=6, stop_token_ids=(4,)),
                             on_token=lambda i, t: got.append((i, t)))
    assert res[0].tokens == [2, 3, 4] and res[0].finish_reason == "stop"
    assert res[1].tokens == [11, 12, 13, 14, 15, 16]
    assert (0, 5) not in got                      # the extra step's token never reaches the caller
    assert st.new_tokens == 9
    assert eng.slots.n_live == 0 and eng.slots.pools[0].n_free == eng.slots.pools[0].n_pages


def test_kernel_status_is_checked_and_stops_generation():
    eng = CounterEngine()
    run_generation(eng, counter_sample, [[1]], GenerationOptions(max_new_tokens=2))
    assert eng.checks >= 1

    class Broken(CounterEngine):
        def check_kernels(self):
            raise RuntimeError("a bounded wait inside the kernel ran out")

    with pytest.raises(RuntimeError, match="bounded wait"):
        run_generation(Broken(), counter_sample, [[1]], GenerationOptions(max_new_tokens=2))


def test_on_token_streams_in_order():
    eng = CounterEngine()
    got = []
    run_generation(eng, counter_sample, [[1], [50]], GenerationOptions(max_new_tokens=2),
                   on_token=lambda i, t: got.append((i, t)))
    assert got == [(0, 2), (1, 51), (0, 3), (1, 52)]


def test_prompts_in_portions_run_the_same_tokens_in_more_steps():
    """``prefill_batch`` (the reference's name, generate.rs:255-271): prompts go through the step function in portions
    of that many tokens a sequence; a sequence's first token comes from the step that holds its last prompt token."""
    prompts = [[10, 11, 12], list(range(20, 29)), list(range(40, 50))]
    def sample(logits, requests, steps, ctx):
        return list(logits)
    whole_eng, part_eng = CounterEngine(), CounterEngine()
    whole, _ = run_generation(whole_eng, sample, prompts, GenerationOptions(max_new_tokens=3))
    parts, stats = run_generation(part_eng, sample, prompts, GenerationOptions(max_new_tokens=3, prefill_batch=4))
    assert [r.tokens for r in parts] == [r.tokens for r in whole] == [[13, 14, 15], [29, 30, 31], [50, 51, 52]]
    assert [sorted(n for _, n in st) for st in whole_eng.steps[:1]] == [[3, 9, 10]]
    assert [sorted(n for _, n in st) for st in part_eng.steps[:3]] == [[3, 4, 4], [4, 4], [1, 2]]
    assert stats.prompt_tokens == 22
    # a portion at least as long as every prompt: one step, as without it
    eng = CounterEngine()
    run_generation(eng, sample, prompts, GenerationOptions(max_new_tokens=2, prefill_batch=10))
    assert sorted(n for _, n in eng.steps[0]) == [3, 9, 10]


def test_a_token_callback_that_returns_false_ends_its_sequence():
    """The reference's sink cancels by returning false from ``on_token`` (generate.rs:67-75); here per sequence."""
    prompts = [[10], [20], [30]]
    seen = []
    def on_token(request, token):
        seen.append((request, token))
        return not (request == 1 and token == 22)          # None or True goes on; False ends request 1 at its second token
    eng = CounterEngine()
    results, _ = run_generation(eng, lambda logits, *a: list(logits), prompts, GenerationOptions(max_new_tokens=4), on_token=on_token)
    assert [r.tokens for r in results] == [[11, 12, 13, 14], [21, 22], [31, 32, 33, 34]]
    assert [r.finish_reason for r in results] == ["length", "cancelled", "length"]
    assert sorted(eng.closed) == sorted(eng.opened) and eng.slots.n_live == 0
    assert (1, 22) in seen and (1, 23) not in seen


def test_a_prompt_whose_beginning_is_cached_runs_only_the_rest():
    """``cached``: a sequence that goes on from an earlier call (the reference's resume, generate.rs:248-250)."""
    sample = lambda logits, *a: list(logits)
    eng = CounterEngine()
    results, stats = run_generation(eng, sample, [[1, 2, 3, 4, 5], [7, 8]], GenerationOptions(max_new_tokens=2), cached=[3, 0])
    assert sorted(n for _, n in eng.steps[0]) == [2, 2] and stats.prompt_tokens == 4
    assert [r.tokens for r in results] == [[6, 7], [9, 10]] and [r.prompt_tokens for r in results] == [5, 2]
    with pytest.raises(ValueError):
        run_generation(CounterEngine(), sample, [[1, 2, 3]], GenerationOptions(max_new_tokens=2), cached=[3])


def test_cached_tokens_and_portions_together():
    """A prompt whose beginning is cached, run in portions: the portions are cut from what is left to run."""
    sample = lambda logits, *a: list(logits)
    eng = CounterEngine()
    prompt = list(range(100, 112))                                   # 12 tokens, 5 of them cached: 7 run, in 3 + 3 + 1
    results, stats = run_generation(eng, sample, [prompt], GenerationOptions(max_new_tokens=2, prefill_batch=3), cached=[5])
    assert [n for st in eng.steps[:3] for _, n in st] == [3, 3, 1] and stats.prompt_tokens == 7
    assert results[0].tokens == [112, 113]
