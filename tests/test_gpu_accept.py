"""Acceptance at the benchmark model's layer sizes and the benchmark's lengths.

The model has the Qwen3-4B layer sizes (width 2,560, 32 heads over 8 kv heads of 128, feed-forward 9,728)
with 2 of its 36 layers and a vocabulary of 32,003, so that the plain implementation finishes on the CPU.
Compared with it, in 32-bit (1e-4 of the largest logit, the same greedy choice) and in bfloat16:

* the correctness batch of the measurement targets: 8 prompts with seeded lengths uniform in [16, 2,048] in
  one step of unequal lengths, then 8 single-token steps;
* one prompt of 2,048 tokens (the benchmark's prompt step), every position wanted;
* the same prompt without its last 32 tokens, then those one by one;
* 8 sequences that hold about 4,060 tokens and are stepped to 4,096: the decode step the benchmark times
  (64 pages a sequence, the page splits chosen for 8 rows), and the same at 1 row.

The plain implementation runs each sequence once, whole; where several engine sequences are prefixes of one
token sequence they share that run (logits at a position depend only on the tokens up to it).
"""
import functools

import pytest
import torch

import plain_qwen3 as P
from helpers import assert_close, folder, oracle, poison_cache
from tiny import random_tokens

pytestmark = pytest.mark.gpu
V = 32003


@functools.lru_cache(maxsize=None)
def hidden(tokens: tuple) -> torch.Tensor:
    cfg, W = oracle("WIDE")
    return P.hidden_states(cfg, W, list(tokens))


def ref_rows(tokens, rows) -> torch.Tensor:
    cfg, W = oracle("WIDE")
    return P.logits_of(cfg, W, hidden(tuple(tokens))[list(rows)])


def check(got, ref, dtype, what):
    assert_close(got, ref, dtype, what)
    if dtype == "float32":
        # the same greedy choice wherever the plain implementation's choice is not a near-tie
        top = torch.topk(ref, 2, dim=-1).values
        clear = (top[:, 0] - top[:, 1]) > 4e-4 * ref.abs().max()
        assert torch.equal(got.cpu().argmax(-1)[clear], ref.argmax(-1)[clear]), what


@pytest.fixture(scope="module")
def engines():
    from synaptix_b200.engine import Engine
    from synaptix_b200.models import load_model
    made = {}

    def get(dtype):
        if dtype not in made:
            made.clear()                              # one engine at a time
            torch.cuda.empty_cache()
            made[dtype] = Engine(load_model(folder("WIDE"), dtype=dtype), max_tokens=8 * 4160 + 4096)
            poison_cache(made[dtype])
        return made[dtype]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_correctness_batch_of_eight_unequal_prompts(engines, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(dtype)
    g = torch.Generator().manual_seed(2048)
    lens = torch.randint(16, 2049, (8,), generator=g).tolist()
    n_dec = 8
    seqs = [random_tokens(V, n + n_dec, 500 + i) for i, n in enumerate(lens)]
    slots = [eng.open() for _ in seqs]
    got = eng.step([Entry(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, lens)])
    check(got, torch.cat([ref_rows(s, [n - 1]) for s, n in zip(seqs, lens)]), dtype, f"prompts of {lens}")
    for j in range(n_dec):
        got = eng.step([Entry(sl, [s[n + j]], [0]) for sl, s, n in zip(slots, seqs, lens)])
        check(got, torch.cat([ref_rows(s, [n + j]) for s, n in zip(seqs, lens)]), dtype, f"decode step {j}")
    for sl in slots:
        eng.close(sl)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompt_of_2048_tokens_whole_and_with_its_last_32_one_by_one(engines, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(dtype)
    T = 2048
    seq = random_tokens(V, T, 600)
    ref = ref_rows(seq, range(T))
    s = eng.open()
    got = eng.step([Entry(s, seq, list(range(T)))])
    eng.close(s)
    check(got, ref, dtype, "2,048 tokens whole, every position")
    s = eng.open()
    a = eng.step([Entry(s, seq[:T - 32], [T - 33])])
    rest = [eng.step([Entry(s, [seq[t]], [0])]) for t in range(T - 32, T)]
    eng.close(s)
    check(torch.cat([a] + rest), ref[T - 33:], dtype, "2,016 tokens, then 32 one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_at_context_4096(engines, dtype):
    from synaptix_b200.engine import DecodeRow, Entry
    eng = engines(dtype)
    L = 4096
    seq = random_tokens(V, L, 700)
    starts = [4060 - 9 * i for i in range(8)]            # 8 sequences, all prefixes of ``seq``, 3,997 to 4,060 tokens
    slots = [eng.open() for _ in starts]
    for i in range(0, 8, 2):                             # prompts two at a time
        got = eng.step([Entry(slots[k], seq[:starts[k]], [starts[k] - 1]) for k in (i, i + 1)])
        check(got, ref_rows(seq, [starts[i] - 1, starts[i + 1] - 1]), dtype, f"prompts {i}, {i + 1}")
    # the benchmark's decode step: 8 rows, 63 to 64 pages each, through the step function ...
    n_steps = L - starts[0]                              # the longest sequence ends at 4,096 tokens
    for j in range(n_steps // 2):
        got = eng.step([Entry(sl, [seq[st + j]], [0]) for sl, st in zip(slots, starts)])
        check(got, ref_rows(seq, [st + j for st in starts]), dtype, f"8 rows, step {j}")
    # ... and through a decode session fed the sequence's tokens: its choices are the plain implementation's
    half = n_steps // 2
    sess = eng.start_decode([DecodeRow(sl, seq[st + half], i, 0) for i, (sl, st) in enumerate(zip(slots, starts))])
    for j in range(half, n_steps):
        sess.launch(tokens=[seq[st + j] for st in starts])
        got = sess.collect()
        ref = ref_rows(seq, [st + j for st in starts])
        top = torch.topk(ref, 2, dim=-1).values
        margin = (4e-4 if dtype == "float32" else 6e-2) * ref.abs().max()
        for r in range(8):
            if float(top[r, 0] - top[r, 1]) > margin:
                assert got[r] == int(ref[r].argmax()), f"session step {j} row {r}"
    assert eng.length(slots[0]) == L
    sess.drop(list(range(8)))
    # one row alone at the same context (other page splits)
    for sl in slots[1:]:
        eng.close(sl)
    s = eng.open()
    eng.step([Entry(s, seq[:4070], [])])
    got = torch.cat([eng.step([Entry(s, [seq[t]], [0])]) for t in range(4070, 4080)])
    check(got, ref_rows(seq, range(4070, 4080)), dtype, "1 row at context 4,070 to 4,080")
    eng.close(s)
    eng.close(slots[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_seqs", [20, 40])
def test_a_few_dozen_rows_at_the_benchmark_sizes(engines, dtype, n_seqs):
    """Steps of 17 to 128 rows at the real layer sizes: in bfloat16 these are the rows the weight-streaming tcgen05
    product takes, with the split norm between the products.  Three short prompts in one step (a few dozen tokens),
    then ``n_seqs`` sequences of unequal lengths decoding together for 5 steps, through ``Engine.step`` (eager) and,
    in slots used again, through a decode session (one graph a step)."""
    from synaptix_b200.engine import DecodeRow, Entry
    eng = engines(dtype)
    # a prompt step of 11 + 25 + 40 = 76 rows
    short = [random_tokens(V, n, 900 + n) for n in (11, 25, 40)]
    slots = [eng.open() for _ in short]
    got = eng.step([Entry(sl, s, [len(s) - 1]) for sl, s in zip(slots, short)])
    check(got, torch.cat([ref_rows(s, [len(s) - 1]) for s in short]), dtype, "three short prompts in one step")
    for sl in slots:
        eng.close(sl)
    # n_seqs sequences: prompts of 3 to 70 tokens, then 5 single-token steps of n_seqs rows
    n_dec = 5
    lens = [3 + (7 * i) % 68 for i in range(n_seqs)]
    seqs = [random_tokens(V, n + n_dec, 1300 + i) for i, n in enumerate(lens)]
    slots = [eng.open() for _ in seqs]
    eng.step([Entry(sl, s[:n], []) for sl, s, n in zip(slots, seqs, lens)])
    for j in range(n_dec):
        got = eng.step([Entry(sl, [s[n + j]], [0]) for sl, s, n in zip(slots, seqs, lens)])
        check(got, torch.cat([ref_rows(s, [n + j]) for s, n in zip(seqs, lens)]), dtype, f"{n_seqs} rows, decode step {j}")
    for sl in slots:
        eng.close(sl)
    # the same through a decode session with forced tokens: its greedy choices are those of the plain implementation
    slots = [eng.open() for _ in seqs]
    eng.step([Entry(sl, s[:n], []) for sl, s, n in zip(slots, seqs, lens)])
    session = eng.start_decode([DecodeRow(sl, s[n], i, 0) for i, (sl, s, n) in enumerate(zip(slots, seqs, lens))])
    for j in range(n_dec):
        session.launch(tokens=None if j == 0 else [s[n + j] for s, n in zip(seqs, lens)])
        picked = session.collect()
        ref = torch.cat([ref_rows(s, [n + j]) for s, n in zip(seqs, lens)])
        top = torch.topk(ref, 2, dim=-1).values
        clear = (top[:, 0] - top[:, 1]) > (4e-4 if dtype == "float32" else 6e-2) * ref.abs().max()
        assert clear.any()
        assert [p for p, c in zip(picked, clear.tolist()) if c] == [int(t) for t, c in zip(ref.argmax(-1).tolist(), clear.tolist()) if c]
    session.close()
    for sl in slots:
        eng.close(sl)
