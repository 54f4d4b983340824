"""Generation through the Python entry point and the command line, against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
from helpers import folder, oracle, oracle_logits
from tiny import random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def margin_ok(name, prompt, out, min_margin):
    """True if every greedy choice of the oracle along ``out`` wins by at least ``min_margin``
    (a smaller margin may legitimately flip under bfloat16 rounding)."""
    seq = list(prompt)
    for t in out:
        lg = oracle_logits(name, tuple(seq))[-1]
        top = torch.topk(lg, 2).values
        if float(top[0] - top[1]) < min_margin:
            return False
        seq.append(t)
    return True


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_greedy_generation_float32_equals_the_oracle(name):
    import synaptix_b200
    cfg, W = oracle(name)
    prompts = [random_tokens(cfg["vocab_size"], n, 800 + n) for n in (3, 11, 1, 40, 7)]
    llm = synaptix_b200.LLM(folder(name), compute_dtype="f32", max_tokens=640)
    outs = llm.generate(prompts, max_new_tokens=12, eos_token_ids=[])
    for p, o in zip(prompts, outs):
        assert o == P.greedy_generate(cfg, W, p, 12)
    # more requests than one batch holds: batches one after another, same tokens
    outs2 = llm.generate(prompts, max_new_tokens=12, eos_token_ids=[], max_batch_size=2)
    assert outs2 == outs and llm.last_stats.batches == 3
    assert llm.engine.cache.slots.n_live == 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_bfloat16_follows_the_oracle(name):
    import synaptix_b200
    cfg, W = oracle(name)
    prompts = [random_tokens(cfg["vocab_size"], n, 900 + n) for n in (5, 9, 13, 70)]
    llm = synaptix_b200.LLM(folder(name), compute_dtype="bf16", max_tokens=640)
    outs = llm.generate(prompts, max_new_tokens=8, eos_token_ids=[])
    scale = max(oracle_logits(name, tuple(p)).abs().max().item() for p in prompts)
    checked = 0
    for p, o in zip(prompts, outs):
        ref = P.greedy_generate(cfg, W, p, 8)
        if margin_ok(name, p, ref, 0.06 * scale):       # twice the bfloat16 logit tolerance
            assert o == ref
            checked += 1
    assert len(outs) == 4 and checked >= 1, "no prompt whose greedy choices are all clear: pick other seeds"


def test_stop_tokens_end_sequences_early():
    import synaptix_b200
    cfg, W = oracle("B")
    prompts = [random_tokens(389, n, 1000 + n) for n in (4, 6, 8)]
    free = [P.greedy_generate(cfg, W, p, 10) for p in prompts]
    stop = free[1][3]
    llm = synaptix_b200.LLM(folder("B"), compute_dtype="f32", max_tokens=512)
    res = llm.generate(prompts, max_new_tokens=10, eos_token_ids=[stop], return_details=True)
    for r, f, p in zip(res, free, prompts):
        want = P.greedy_generate(cfg, W, p, 10, stop_ids=[stop])
        assert r.tokens == want
        assert r.finish_reason == ("stop" if want[-1] == stop else "length")
    assert res[1].tokens[-1] == stop and len(res[1].tokens) <= 4
    # the configuration's own stop tokens are the default (11 and 12 for this model)
    assert tuple(llm.model.stop_token_ids) == (11, 12)


def test_temperature_sampling_is_seeded_and_batch_independent():
    import synaptix_b200
    prompts = [random_tokens(389, n, 1100 + n) for n in (1, 7, 31, 64)]
    llm = synaptix_b200.LLM(folder("B"), compute_dtype="f32", max_tokens=1024)
    kw = dict(max_new_tokens=16, temperature=0.8, seed=7, eos_token_ids=[])
    a = llm.generate(prompts, **kw)
    b = llm.generate(prompts, **kw)
    assert a == b
    assert llm.generate(prompts, **dict(kw, seed=8)) != a
    # every drawn token is consistent with the oracle's distribution and the stream's word
    cfg, W = oracle("B")
    for i, (p, o) in enumerate(zip(prompts, a)):
        seq = list(p)
        for step, t in enumerate(o):
            v = P.processed_logits(oracle_logits("B", tuple(seq))[-1].numpy(), temperature=0.8)
            cum = P.multinomial_intervals(v)
            u = float(P.uniform_from_u32(P.philox_u32(7, step, i)))
            lo = cum[t - 1] if t > 0 else 0.0
            assert lo - 1e-3 <= u <= cum[t] + 1e-3, f"request {i} step {step}"
            seq.append(t)
    # request 0 alone draws the same tokens as in the batch
    assert llm.generate([prompts[0]], **kw)[0] == a[0]


def test_penalties_change_greedy_output_as_the_oracle_says():
    import synaptix_b200
    cfg, W = oracle("A")
    prompt = random_tokens(256, 6, 1200)
    llm = synaptix_b200.LLM(folder("A"), compute_dtype="f32", max_tokens=256)
    out = llm.generate([prompt], max_new_tokens=8, repetition_penalty=1.8, presence_penalty=0.3,
                       frequency_penalty=0.2, eos_token_ids=[])[0]
    seq, ref = list(prompt), []
    for _ in range(8):
        v = P.processed_logits(oracle_logits("A", tuple(seq))[-1].numpy(), context=seq, repetition_penalty=1.8,
                               presence_penalty=0.3, frequency_penalty=0.2)
        t = P.greedy(torch.from_numpy(v))
        ref.append(t)
        seq.append(t)
    assert out == ref


def test_command_line_run(tmp_path):
    cfg, W = oracle("A")
    prompt = random_tokens(256, 9, 1300)
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "synaptix_b200", "run", folder("A"), ",".join(map(str, prompt)),
                        "--max-tokens", "6", "--temperature", "0", "--compute-dtype", "f32", "--stop-ids", "",
                        "--json"], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["outputs"][0]["tokens"] == P.greedy_generate(cfg, W, prompt, 6)
    assert out["prompt_tokens"] == 9 and out["new_tokens"] == 6


def test_penalties_in_a_batch_whose_sequences_end_at_different_times():
    """Penalties look at each sequence's own context, which a decode session keeps on the device and writes
    anew when a sequence leaves the batch.  Three prompts, one of which stops early."""
    import synaptix_b200
    cfg, W = oracle("B")
    prompts = [random_tokens(389, n, 1400 + n) for n in (6, 20, 3)]
    kw = dict(repetition_penalty=1.6, presence_penalty=0.4, frequency_penalty=0.3, repeat_last_n=12)

    def plain(prompt, n, stop=()):
        seq, out = list(prompt), []
        while len(out) < n and not (out and out[-1] in stop):
            v = P.processed_logits(oracle_logits("B", tuple(seq))[-1].numpy(), context=seq, repetition_penalty=1.6,
                                   presence_penalty=0.4, frequency_penalty=0.3, repeat_last_n=12)
            t = P.greedy(torch.from_numpy(v))
            out.append(t)
            seq.append(t)
        return out

    free = [plain(p, 14) for p in prompts]
    stop = free[1][4]                         # request 1 ends with its fifth token (or earlier)
    llm = synaptix_b200.LLM(folder("B"), compute_dtype="f32", max_tokens=512)
    res = llm.generate(prompts, max_new_tokens=14, eos_token_ids=[stop], return_details=True, **kw)
    for r, p in zip(res, prompts):
        assert r.tokens == plain(p, 14, stop=(stop,))
    assert res[1].finish_reason == "stop" and len(res[1].tokens) <= 5
    assert any(len(r.tokens) == 14 for r in res)


def test_prompts_in_portions_generate_the_same_tokens():
    """``prefill_batch``: the prompts in portions of 50 tokens a sequence instead of one step; float32, so the
    greedy tokens are the plain implementation's either way."""
    import synaptix_b200
    cfg, W = oracle("B")
    prompts = [random_tokens(389, n, 1400 + n) for n in (3, 120, 51, 100)]
    llm = synaptix_b200.LLM(folder("B"), compute_dtype="f32", max_tokens=1024)
    want = [P.greedy_generate(cfg, W, p, 5) for p in prompts]
    assert llm.generate(prompts, max_new_tokens=5, eos_token_ids=[], prefill_batch=50) == want
    assert llm.generate(prompts, max_new_tokens=5, eos_token_ids=[]) == want


@pytest.mark.parametrize("name", ["B", "W"])
def test_a_conversation_keeps_its_cache_between_calls(name):
    """``LLM.conversation()``: the second and third call run only the new tokens of their prompts and draw what a
    fresh generation from the whole prompt draws (float32, greedy: the plain implementation's tokens).  W has layers
    with a window of 24 keys, whose pages are given back while the conversation goes on."""
    import synaptix_b200
    cfg, W = oracle(name)
    llm = synaptix_b200.LLM(folder(name), compute_dtype="f32", max_tokens=1024)
    turns = [random_tokens(cfg["vocab_size"], n, 1500 + n) for n in (70, 9, 31)]
    with llm.conversation() as conv:
        seq = []
        for k, new in enumerate(turns):
            seq = seq + new
            out = conv.generate(seq, max_new_tokens=6, eos_token_ids=[])
            assert out == P.greedy_generate(cfg, W, seq, 6), f"turn {k}"
            assert llm.last_stats.prompt_tokens == len(new) + (1 if k else 0)     # + the last token drawn in the turn before
            seq = seq + out
            assert conv.tokens == seq[:-1]
        assert conv.cached_tokens == len(seq) - 1 and conv.reusable(seq + [1]) == len(seq) - 1
        assert conv.reusable(seq[:-3]) == 0 and conv.reusable([1] + seq[1:] + [5]) == 0
        # a prompt that does not go on from the cached tokens: the cache is dropped and the whole prompt runs
        other = [1] + seq[1:40]
        assert conv.generate(other, max_new_tokens=3, eos_token_ids=[]) == P.greedy_generate(cfg, W, other, 3)
        assert llm.last_stats.prompt_tokens == len(other)
        seq = other + conv.generate(other, max_new_tokens=3, eos_token_ids=[])     # nothing new either: whole again
        assert llm.last_stats.prompt_tokens == len(other)
        # a stop token ends a turn; the conversation goes on after it
        stop = P.greedy_generate(cfg, W, seq + [3], 4)[1]
        out = conv.generate(seq + [3], max_new_tokens=4, eos_token_ids=[stop])
        assert out[-1] == stop and len(out) <= 2
        seq = seq + [3] + out
        assert conv.generate(seq + [8], max_new_tokens=3, eos_token_ids=[]) == P.greedy_generate(cfg, W, seq + [8], 3)
    assert llm.engine.cache.slots.n_live == 0
    # other requests run beside an open conversation
    conv = llm.conversation()
    a = conv.generate(turns[0], max_new_tokens=3, eos_token_ids=[])
    assert llm.generate([turns[1], turns[2]], max_new_tokens=3, eos_token_ids=[]) == [P.greedy_generate(cfg, W, t, 3) for t in turns[1:]]
    assert conv.generate(turns[0] + a + [4], max_new_tokens=3, eos_token_ids=[]) == P.greedy_generate(cfg, W, turns[0] + a + [4], 3)
    # requests that would fill the whole cache are cut into batches around what the conversation holds
    many = [random_tokens(cfg["vocab_size"], 100, 1600 + i) for i in range(8)]           # 8 x 2 pages = the 16 pages of the cache
    assert llm.generate(many, max_new_tokens=3, eos_token_ids=[]) == [P.greedy_generate(cfg, W, p, 3) for p in many]
    assert llm.last_stats.batches == 2
    conv.close()
    assert llm.engine.cache.slots.n_live == 0
