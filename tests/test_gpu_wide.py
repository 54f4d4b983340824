"""The benchmark model's layer sizes (two layers of them) against the plain implementation, in
32-bit and in bfloat16, whole and cut: this is where the tensor-core kernels, the split products
and the fused prologues run at the shapes they were written for."""
import numpy as np
import pytest
import torch

from helpers import assert_close, folder, oracle_logits, poison_cache
from tiny import random_tokens

pytestmark = pytest.mark.gpu
V = 32003


@pytest.fixture(scope="module")
def wide_engine():
    from synaptix_b200.engine import Engine
    from synaptix_b200.models import load_model
    made = {}

    def get(dtype):
        if dtype not in made:
            made[dtype] = Engine(load_model(folder("WIDE"), dtype=dtype), max_tokens=4096)
            poison_cache(made[dtype])
        return made[dtype]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_model_whole_cut_and_batched(wide_engine, dtype):
    from synaptix_b200.engine import Entry
    eng = wide_engine(dtype)
    lens = [300, 70, 129, 1, 33, 200, 17, 64, 90]                 # 9 sequences: more than 8 rows in decode steps
    seqs = [random_tokens(V, n + 6, 40 + i) for i, n in enumerate(lens)]
    refs = [oracle_logits("WIDE", tuple(s)) for s in seqs]
    # one request alone and whole, every position wanted (many-row products, prompt attention)
    s = eng.open()
    got = eng.step([Entry(s, seqs[0], list(range(len(seqs[0]))))])
    eng.close(s)
    assert_close(got, refs[0], dtype, f"wide {dtype} whole")
    # all prompts in one step, then six single-token steps; the batch shrinks from 9 to 2 rows
    slots = [eng.open() for _ in seqs]
    got = eng.step([Entry(sl, q[:n], [n - 1]) for sl, q, n in zip(slots, seqs, lens)])
    assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), dtype, f"wide {dtype} prompts")
    live = list(range(len(seqs)))
    for j in range(6):
        if j == 2:
            for i in (1, 3, 5, 7):                                 # four requests end early
                eng.close(slots[i]); live.remove(i)
        if j == 4:
            for i in (0, 2, 8):
                eng.close(slots[i]); live.remove(i)
        got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
        assert_close(got, torch.stack([refs[i][lens[i] + j] for i in live]), dtype, f"wide {dtype} decode {j} rows {len(live)}")
    for i in live:
        eng.close(slots[i])
    # a continued chunk: 100 tokens, then 40 more at once (prompt attention over an existing past)
    s = eng.open()
    a = eng.step([Entry(s, seqs[0][:100], [99])])
    b = eng.step([Entry(s, seqs[0][100:140], list(range(40)))])
    eng.close(s)
    assert_close(torch.cat([a, b]), refs[0][99:140], dtype, f"wide {dtype} continued chunk")


def test_wide_model_greedy_tokens_float32():
    import plain_qwen3 as P
    import synaptix_b200
    from helpers import oracle
    cfg, W = oracle("WIDE")
    prompts = [random_tokens(V, n, 70 + n) for n in (5, 40)]
    llm = synaptix_b200.LLM(folder("WIDE"), compute_dtype="f32", max_tokens=512)
    outs = llm.generate(prompts, max_new_tokens=4, eos_token_ids=[])
    assert outs == [P.greedy_generate(cfg, W, p, 4) for p in prompts]


def test_wide_vocabulary_sampling_in_a_replayed_step_equals_the_eager_one():
    """At this vocabulary the draw runs in the kernel that spreads a row over a cluster of blocks; a decode session
    records it into its graph.  Replayed and eager steps draw the same tokens, a request alone the same as in its
    batch, and every drawn token passes the filters applied to the engine's own logits."""
    import plain_qwen3 as P
    import synaptix_b200
    from synaptix_b200.engine import Entry
    prompts = [random_tokens(V, n, 90 + n) for n in (3, 17, 66)]
    kw = dict(max_new_tokens=6, temperature=0.9, top_k=30, top_p=0.85, seed=5, eos_token_ids=[])
    outs = {}
    for graphs in (True, False):
        llm = synaptix_b200.LLM(folder("WIDE"), compute_dtype="f32", max_tokens=1024, graph=graphs)
        outs[graphs] = llm.generate(prompts, **kw)
        if graphs:
            assert llm.generate([prompts[0]], **kw)[0] == outs[True][0]
    assert outs[True] == outs[False]
    eng = llm.engine
    for p, o in zip(prompts, outs[True]):
        s = eng.open()
        lg = eng.step([Entry(s, p + o[:-1], list(range(len(p) - 1, len(p) + len(o) - 1)))]).float().cpu().numpy()
        eng.close(s)
        for row, t in zip(lg, o):
            assert np.isfinite(P.processed_logits(row, temperature=0.9, top_k=30, top_p=0.85)[t])
