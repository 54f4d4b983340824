"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way
of cutting the work into steps and batches."""
import pytest
import torch

from helpers import assert_close, folder, oracle, oracle_logits, poison_cache
from tiny import random_tokens

pytestmark = pytest.mark.gpu

NAMES = ["A", "B", "W", "F", "S", "G", "O"]
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def engines():
    from synaptix_b200.engine import Engine
    from synaptix_b200.models import load_model
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=max_tokens)
            poison_cache(eng)
            made[key] = eng
        assert made[key].cache.slots.n_live == 0
        return made[key]
    return get


def vocab(name):
    return oracle(name)[0]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(engines, name, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    for i, n in enumerate([1, 2, 17, 64, 65, 150]):
        toks = random_tokens(vocab(name), n, 100 + i)
        s = eng.open()
        got = eng.step([Entry(s, toks, list(range(n)))])
        eng.close(s)
        assert_close(got, oracle_logits(name, tuple(toks)), dtype, f"{name} {dtype} whole n={n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(engines, name, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    for i, n in enumerate([33, 96, 140]):
        toks = random_tokens(vocab(name), n, 200 + i)
        ref = oracle_logits(name, tuple(toks))
        s = eng.open()
        head = n - 32
        got = [eng.step([Entry(s, toks[:head], [head - 1])])]
        for j in range(head, n):
            got.append(eng.step([Entry(s, [toks[j]], [0])]))
        eng.close(s)
        assert_close(torch.cat(got), ref[head - 1:], dtype, f"{name} {dtype} n={n} last 32 one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(engines, name, dtype):
    """Batches of unequal prompts; shorter requests end earlier; the next batch runs in the
    slots and pages the first gave back (the cache holds little more than one batch)."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype, max_tokens=448)          # 7 pages
    V = vocab(name)
    for b, (lens, decodes) in enumerate([([5, 70, 1, 33], [3, 40, 12, 20]),
                                         ([64, 9, 128], [10, 30, 2]),
                                         ([2, 3, 100, 31], [25, 1, 27, 33])]):
        seqs = [random_tokens(V, n + d, 300 + 10 * b + i) for i, (n, d) in enumerate(zip(lens, decodes))]
        refs = [oracle_logits(name, tuple(s)) for s in seqs]
        slots = [eng.open() for _ in seqs]
        got = eng.step([Entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)])
        assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), dtype, f"{name} {dtype} batch {b} prompts")
        live = list(range(len(seqs)))
        for j in range(max(decodes)):
            for i in [i for i in live if decodes[i] <= j]:
                eng.close(slots[i])                      # this request ended earlier
                live.remove(i)
            got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
            assert_close(got, torch.stack([refs[i][lens[i] + j] for i in live]), dtype,
                         f"{name} {dtype} batch {b} decode step {j} live {live}")
        for i in live:
            eng.close(slots[i])
        assert eng.cache.slots.n_live == 0
    assert all(p.n_free == p.n_pages for p in eng.cache.slots.pools)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "W"])
def test_long_decoding(engines, name, dtype):
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 3 + 260, 400)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, toks[:3], [2])])]
    for j in range(3, len(toks)):
        got.append(eng.step([Entry(s, [toks[j]], [0])]))
    eng.close(s)
    assert_close(torch.cat(got), ref[2:], dtype, f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens_of_a_sequence(engines, name, dtype):
    """Position 0 alone, then position 1 alone, then a chunk: the start of a sequence has no past."""
    from synaptix_b200.engine import Entry
    eng = engines(name, dtype)
    toks = random_tokens(vocab(name), 12, 500)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    got = [eng.step([Entry(s, [toks[0]], [0])]), eng.step([Entry(s, [toks[1]], [0])]),
           eng.step([Entry(s, toks[2:12], list(range(10)))])]
    eng.close(s)
    assert_close(torch.cat(got), ref, dtype, f"{name} {dtype} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_step_and_empty_want(engines, dtype):
    """A step may mix a new prompt, a continued chunk and a single token, and may want nothing."""
    from synaptix_b200.engine import Entry
    name = "B"
    eng = engines(name, dtype)
    V = vocab(name)
    a, b, c = random_tokens(V, 40, 601), random_tokens(V, 90, 602), random_tokens(V, 20, 603)
    sa, sb, sc = eng.open(), eng.open(), eng.open()
    out = eng.step([Entry(sa, a[:30], []), Entry(sb, b[:10], [])])
    assert out.shape[0] == 0
    got = eng.step([Entry(sa, [a[30]], [0]), Entry(sb, b[10:80], [0, 69]), Entry(sc, c, [19])])
    ra, rb, rc = (oracle_logits(name, tuple(x)) for x in (a, b, c))
    assert_close(got, torch.stack([ra[30], rb[10], rb[79], rc[19]]), dtype, f"mixed step {dtype}")
    for s in (sa, sb, sc):
        eng.close(s)


def test_step_errors_change_nothing(engines):
    from synaptix_b200.cache import CacheFull, SlotError
    from synaptix_b200.engine import Entry, StepError
    eng = engines("A", "float32", max_tokens=128)
    s = eng.open()
    with pytest.raises(StepError, match="token ids"):
        eng.step([Entry(s, [1, 999], [0])])
    with pytest.raises(StepError, match="wanted place"):
        eng.step([Entry(s, [1, 2], [2])])
    with pytest.raises(StepError, match="twice"):
        eng.step([Entry(s, [1], [0]), Entry(s, [2], [0])])
    with pytest.raises(CacheFull):
        eng.step([Entry(s, [1] * 200, [0])])
    with pytest.raises(SlotError):
        eng.step([Entry(s + 1, [1], [0])])
    assert eng.length(s) == 0
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["W", "S", "G"])
def test_prompt_in_portions_across_a_window_whose_pages_were_given_back(name, dtype):
    """Layers with a window give pages back while the sequence runs; their table entries then read as page 0,
    which no sequence owns.  A later portion of several tokens loads such an entry as part of a key block whose
    other keys are visible: the keys of page 0 must count for nothing, whatever finite values lie there.  Every
    other page starts as NaN, page 0 as large numbers."""
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    eng = Engine(load_model(folder(name), dtype=dtype), max_tokens=1024)
    poison_cache(eng)
    g = torch.Generator().manual_seed(5)
    for t in eng.cache._k + eng.cache._v:
        t[:, 0] = (torch.randn(t[:, 0].shape, generator=g) * 1e4).to(t.dtype).to(t.device)
    portions = [100, 2, 1, 90, 70, 3]
    toks = random_tokens(vocab(name), sum(portions), 3100)
    ref = oracle_logits(name, tuple(toks))
    s = eng.open()
    at = 0
    for n in portions:
        got = eng.step([Entry(s, toks[at:at + n], list(range(n)))])
        assert_close(got, ref[at:at + n], dtype, f"{name} {dtype} portion of {n} at {at}")
        at += n
    assert any(-1 in eng.cache.slots.table(s, g_) for g_ in range(eng.cache.n_block_tables)), "no page was given back"
    eng.close(s)
