"""Decode sessions (sampling and the move to the next token kept on the device) against the plain
implementation: the loop that generation and the benchmark both run.

Reference for the semantics: the graph replay loop of crates/synaptix-models/llm/qwen3/src/pipeline.rs:279-302
and its test that graph and eager decoding give the same greedy tokens
(crates/synaptix/tests/cuda_graph_decode.rs:95-139).
"""
import functools

import pytest
import torch

import plain_qwen3 as P
from helpers import assert_close, folder, oracle, oracle_logits, poison_cache
from tiny import random_tokens

pytestmark = pytest.mark.gpu


@functools.lru_cache(maxsize=None)
def greedy_ref(name, prompt, n):
    cfg, W = oracle(name)
    return P.greedy_generate(cfg, W, list(prompt), n)


def run_session(eng, prompts, n_steps, lookahead=2, sampling=None):
    """Prompts in one step, then ``n_steps`` steps of a session; returns (slots, tokens per sequence)."""
    from synaptix_b200.engine import DecodeRow, Entry
    slots = [eng.open() for _ in prompts]
    lg = eng.step([Entry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = lg.argmax(-1).tolist()
    outs = [[t] for t in first]
    sess = eng.start_decode([DecodeRow(s, t, i, 1) for i, (s, t) in enumerate(zip(slots, first))], sampling)
    launched = 0
    while launched < n_steps or sess.in_flight:
        if launched < n_steps and sess.in_flight < lookahead:
            sess.launch()
            launched += 1
            continue
        for o, t in zip(outs, sess.collect()):
            o.append(t)
    return slots, outs, sess


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("name", ["A", "B", "W", "S", "G"])
def test_float32_session_equals_the_oracle_over_page_and_window_edges(name, graphs):
    import synaptix_b200
    from synaptix_b200.engine import Entry
    cfg, W = oracle(name)
    V = cfg["vocab_size"]
    n_steps = 140                                  # every sequence crosses two page boundaries (64 tokens a page)
    prompts = [random_tokens(V, n, 2000 + n) for n in (5, 60, 33)]
    llm = synaptix_b200.LLM(folder(name), compute_dtype="f32", max_tokens=1024, graph=graphs)
    eng = llm.engine
    poison_cache(eng)
    slots, outs, sess = run_session(eng, prompts, n_steps)
    for p, o in zip(prompts, outs):
        assert o == greedy_ref(name, tuple(p), n_steps + 1)
    # the slots go on through the step function: the cache holds what the session wrote
    sess.drop([0, 1, 2])
    lg = eng.step([Entry(s, [o[-1]], [0]) for s, o in zip(slots, outs)])
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert_close(lg[i:i + 1], oracle_logits(name, tuple(p + o))[-1:], "float32", f"{name} after the session, row {i}")
    for s in slots:
        eng.close(s)
    # a second session in the slots and pages the first gave back (other prompts, two rows: another bucket)
    prompts2 = [random_tokens(V, n, 2100 + n) for n in (70, 2)]
    slots2, outs2, sess2 = run_session(eng, prompts2, 20, lookahead=1)
    assert set(slots2) <= set(slots)
    for p, o in zip(prompts2, outs2):
        assert o == greedy_ref(name, tuple(p), 21)
    sess2.drop([0, 1])
    for s in slots2:
        eng.close(s)
    assert eng.cache.slots.n_live == 0
    assert all(pool.n_free == pool.n_pages for pool in eng.cache.slots.pools)


@pytest.mark.parametrize("name", ["F", "S", "B"])
def test_bfloat16_session_follows_the_oracle_when_fed_its_tokens(name):
    """bfloat16 rounding may flip a close choice, after which two greedy runs part for good.  So the session is
    fed the oracle's token at every step (the control word of a step) and its own choice is compared wherever
    the oracle's choice wins by a clear margin."""
    import synaptix_b200
    from synaptix_b200.engine import DecodeRow, Entry
    cfg, W = oracle(name)
    V = cfg["vocab_size"]
    n_steps = 80
    prompts = [random_tokens(V, n, 2200 + n) for n in (50, 7, 120)]
    refs = [greedy_ref(name, tuple(p), n_steps + 1) for p in prompts]
    eng = synaptix_b200.LLM(folder(name), compute_dtype="bf16", max_tokens=1024).engine
    poison_cache(eng)
    slots = [eng.open() for _ in prompts]
    eng.step([Entry(s, p, []) for s, p in zip(slots, prompts)])
    sess = eng.start_decode([DecodeRow(s, r[0], i, 1) for i, (s, r) in enumerate(zip(slots, refs))])
    checked = 0
    for k in range(n_steps):
        sess.launch(tokens=[r[k] for r in refs])
        got = sess.collect()
        for i, (p, r) in enumerate(zip(prompts, refs)):
            lg = oracle_logits(name, tuple(p + r[:k + 1]))[-1]
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) >= 0.06 * float(lg.abs().max()):       # twice the bfloat16 logit tolerance
                assert got[i] == r[k + 1], f"{name} row {i} step {k}"
                checked += 1
    assert checked >= n_steps          # of 3 x n_steps choices, at least a third are clear


def test_session_rows_that_leave_and_a_cache_that_fills():
    import synaptix_b200
    from synaptix_b200.cache import CacheFull
    from synaptix_b200.engine import StepError
    cfg, W = oracle("B")
    prompts = [random_tokens(389, n, 2300 + n) for n in (60, 62, 10)]
    eng = synaptix_b200.LLM(folder("B"), compute_dtype="f32", max_tokens=5 * 64).engine     # 5 pages
    slots, outs, sess = run_session(eng, prompts, 3)                 # the rows now hold 63, 65 and 13 tokens: 4 pages
    with pytest.raises(StepError, match="collect"):
        sess.launch()
        sess.drop([0])
    sess.collect()
    # row 0 takes the fifth page with its 65th token; the cache is full when row 1 wants a third page
    for _ in range(200):
        try:
            sess.launch()
        except CacheFull:
            break
        sess.collect()
    else:
        raise AssertionError("the cache never filled")
    assert sess.in_flight == 0
    lens = [eng.length(s) for s in slots]
    sess.drop([1])                                       # the longest leaves, its pages come back
    eng.close(slots[1])
    sess.launch()
    toks = sess.collect()
    assert len(toks) == 2 and [eng.length(slots[0]), eng.length(slots[2])] == [lens[0] + 1, lens[2] + 1]


def test_kernel_launch_count_of_a_replayed_step_equals_the_eager_one():
    import synaptix_b200
    eng = synaptix_b200.LLM(folder("F"), compute_dtype="bf16", max_tokens=512).engine
    prompts = [random_tokens(1000, n, 2400 + n) for n in (9, 3)]
    l0 = eng.kernel_launches
    slots, outs, sess = run_session(eng, prompts, 1)
    first = eng.kernel_launches
    sess.launch(), sess.collect()
    per_step = eng.kernel_launches - first
    assert per_step > 0
    sess.launch(), sess.collect()
    assert eng.kernel_launches - first == 2 * per_step
