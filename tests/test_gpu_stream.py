"""The fused layer kernel (a run of layers of a single-token step as one persistent kernel) against
the plain implementation: long decoding over page and window edges, batches that shrink, a slot
used again, a schedule with layers the kernel cannot take in between and a run that reads another
run's cache.  Every test checks that the kernel really ran and that none of its waits ran out."""
import pytest
import torch

import plain_qwen3 as P
from helpers import assert_close, folder, oracle_logits, poison_cache
from tiny import CONFIGS, random_tokens

pytestmark = pytest.mark.gpu


def fused_plans(engine):
    return [p for _, _, p in engine.model._stream_segments(engine.cache) if p is not None]


@pytest.mark.parametrize("name", ["S", "F"])
def test_long_decode_through_the_fused_kernel(name, monkeypatch):
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    monkeypatch.setenv("SYNAPTIX_STREAM", "1")
    V = CONFIGS[name][0]["vocab_size"]
    eng = Engine(load_model(folder(name), dtype="bfloat16"), max_tokens=2048)
    poison_cache(eng)
    steps = 75                                               # over a page edge (64) and the window of S (40)
    lens = [70, 5, 130, 1, 33]
    seqs = [random_tokens(V, n + steps, 300 + i) for i, n in enumerate(lens)]
    refs = [oracle_logits(name, tuple(s)) for s in seqs]
    for batch in ([0, 1, 2, 3, 4], [3, 0]):                  # the second batch runs in slots used before
        slots = {i: eng.open() for i in batch}
        got = eng.step([Entry(slots[i], seqs[i][:lens[i]], [lens[i] - 1]) for i in batch])
        assert_close(got, torch.stack([refs[i][lens[i] - 1] for i in batch]), "bfloat16", f"{name} prompts")
        live = list(batch)
        for j in range(steps):
            if j == 20 and len(live) > 2:                    # two requests end early
                for i in live[1:3]:
                    eng.close(slots[i])
                live = [live[0]] + live[3:]
            got = eng.step([Entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live])
            assert_close(got, torch.stack([refs[i][lens[i] + j] for i in live]), "bfloat16",
                         f"{name} decode step {j} rows {len(live)}")
        for i in live:
            eng.close(slots[i])
    plans = fused_plans(eng)
    assert plans and sum(p.n_layers for p in plans) == CONFIGS[name][0]["num_hidden_layers"]
    assert eng.model.stream_status() == 0


def test_fused_and_unfused_steps_agree(monkeypatch):
    """The same requests with the fused kernel on and off: both within tolerance of the plain
    implementation, and the same greedy tokens where the plain implementation's margin is clear."""
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    V = CONFIGS["S"][0]["vocab_size"]
    seq = random_tokens(V, 90, 77)
    ref = oracle_logits("S", tuple(seq))
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("SYNAPTIX_STREAM", flag)
        eng = Engine(load_model(folder("S"), dtype="bfloat16"), max_tokens=512)
        s = eng.open()
        rows = [eng.step([Entry(s, seq[:50], [49])])]
        for j in range(50, 90):
            rows.append(eng.step([Entry(s, [seq[j]], [0])]))
        outs[flag] = torch.cat(rows)
        assert_close(outs[flag], ref[49:90], "bfloat16", f"stream={flag}")
        assert bool(fused_plans(eng)) == (flag == "1") or flag == "0"
    top2 = ref[49:90].topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * ref.abs().max()
    assert torch.equal(outs["1"].argmax(-1).cpu()[clear], outs["0"].argmax(-1).cpu()[clear])


def make_mixed():
    """Layers the fused kernel takes (head size 64) around one it does not (head size 16); layer 1
    runs twice, and the last run is layer 0 again, reading the cache its first run wrote."""
    import dataclasses
    from typing import ClassVar, Tuple
    from synaptix_b200.config import ModelConfig, register_architecture, take
    from synaptix_b200.models import DecoderModel, LayerRun
    from synaptix_b200.parts import (Attention, Embedding, NoPosition, OutputHead, PreNormBlock, RMSNorm, RotaryHalf,
                                     SwiGLU)

    @dataclasses.dataclass(frozen=True)
    class MixedConfig(ModelConfig):
        architectures: ClassVar[Tuple[str, ...]] = ("ToyMixedStreamLM",)
        model_types: ClassVar[Tuple[str, ...]] = ("toy_mixed_stream",)
        vocab: int = 0
        width: int = 0
        eps: float = 0.0

        @classmethod
        def from_dict(cls, d):
            return cls(vocab=take(d, "vocab", int), width=take(d, "width", int), eps=take(d, "eps", float))

        def to_dict(self):
            return {"architectures": ["ToyMixedStreamLM"], "vocab": self.vocab, "width": self.width, "eps": self.eps}

        def validate(self):
            pass

    def build(cfg):
        w = cfg.width
        emb = Embedding("emb.weight", cfg.vocab, w)

        def blk(p, att, inter):
            return PreNormBlock(RMSNorm(p + "n1.weight", w, cfg.eps), att, RMSNorm(p + "n2.weight", w, cfg.eps),
                                SwiGLU(p + "ff.", w, inter))
        l0 = blk("l0.", Attention("l0.att.", w, 2, 1, 64, position=NoPosition()), 96)
        l1 = blk("l1.", Attention("l1.att.", w, 4, 2, 64, position=RotaryHalf(64, 10000.0), qk_norm_eps=cfg.eps,
                                  window=48), 160)
        l2 = blk("l2.", Attention("l2.att.", w, 4, 4, 16, position=RotaryHalf(16, 500.0)), 64)
        schedule = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(2, 2), LayerRun(1, 3), LayerRun(0, 0, write_cache=False)]
        return DecoderModel(cfg, emb, [l0, l1, l2], RMSNorm("norm.weight", w, cfg.eps),
                            OutputHead("head.weight", cfg.vocab, w, False, emb), schedule=schedule)

    register_architecture(MixedConfig, build)
    return MixedConfig


def mixed_plain(W, tokens, eps):
    T = len(tokens)
    pos = torch.arange(T)
    h = W["emb.weight"][torch.tensor(tokens)]

    def att(h, p, nh, nkv, hd, theta, qk, window, reuse=None):
        x = P.rms_norm(h, W[p + "n1.weight"], eps)
        q = (x @ W[p + "att.q_proj.weight"].T).view(T, nh, hd)
        if reuse is None:
            k = (x @ W[p + "att.k_proj.weight"].T).view(T, nkv, hd)
            v = (x @ W[p + "att.v_proj.weight"].T).view(T, nkv, hd)
        else:
            k, v = reuse
        if qk:
            q = P.rms_norm(q, W[p + "att.q_norm.weight"], eps)
            if reuse is None:
                k = P.rms_norm(k, W[p + "att.k_norm.weight"], eps)
        if theta is not None:
            f = P.rotary_freqs(theta, hd)
            q = P.rope_rotate_half(q, pos, f)
            if reuse is None:
                k = P.rope_rotate_half(k, pos, f)
        o = P.causal_gqa_attention(q, k, v, hd ** -0.5, window).reshape(T, nh * hd)
        h = h + o @ W[p + "att.o_proj.weight"].T
        y = P.rms_norm(h, W[p + "n2.weight"], eps)
        h = h + P.swiglu(y, W[p + "ff.gate_proj.weight"], W[p + "ff.up_proj.weight"], W[p + "ff.down_proj.weight"])
        return h, (k, v)

    h, kv0 = att(h, "l0.", 2, 1, 64, None, False, None)
    h, _ = att(h, "l1.", 4, 2, 64, 10000.0, True, 48)
    h, _ = att(h, "l2.", 4, 4, 16, 500.0, False, None)
    h, _ = att(h, "l1.", 4, 2, 64, 10000.0, True, 48)
    h, _ = att(h, "l0.", 2, 1, 64, None, False, None, reuse=kv0)
    return P.rms_norm(h, W["norm.weight"], eps) @ W["head.weight"].T


def test_schedule_with_fused_and_unfused_runs(tmp_path, monkeypatch):
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    from synaptix_b200.weights import write_model_folder
    monkeypatch.setenv("SYNAPTIX_STREAM", "1")
    Cfg = make_mixed()
    cfg = Cfg(vocab=211, width=128, eps=1e-5)
    d = write_model_folder(cfg, str(tmp_path / "mixed"), 5, std_matrix=0.08, std_embedding=0.3, std_gain=0.1)
    eng = Engine(load_model(d, dtype="bfloat16"), max_tokens=1024, max_seqs=4)
    poison_cache(eng)
    _, W = P.load_folder(d)
    g = torch.Generator().manual_seed(4)
    lens = [60, 7, 100]
    steps = 12
    seqs = [torch.randint(0, 211, (n + steps,), generator=g).tolist() for n in lens]
    refs = [mixed_plain(W, s, 1e-5) for s in seqs]
    slots = [eng.open() for _ in seqs]
    got = eng.step([Entry(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, lens)])
    assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), "bfloat16", "mixed prompts")
    for j in range(steps):
        got = eng.step([Entry(sl, [s[n + j]], [0]) for sl, s, n in zip(slots, seqs, lens)])
        assert_close(got, torch.stack([r[n + j] for r, n in zip(refs, lens)]), "bfloat16", f"mixed decode {j}")
    segs = eng.model._stream_segments(eng.cache)
    assert [(a, b, p is not None) for a, b, p in segs] == [(0, 1, True), (1, 2, True), (2, 3, False), (3, 4, True),
                                                          (4, 5, True)]
    assert eng.model.stream_status() == 0


@pytest.mark.parametrize("rows", [8, 6, 1])
def test_benchmark_layer_sizes_through_the_fused_kernel(rows, monkeypatch):
    """Two layers of the benchmark model's sizes: with 6 and 8 rows the down product's activations
    do not fit in shared memory whole and are brought chunk by chunk."""
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    monkeypatch.setenv("SYNAPTIX_STREAM", "1")
    V = CONFIGS["WIDE"][0]["vocab_size"]
    eng = Engine(load_model(folder("WIDE"), dtype="bfloat16"), max_tokens=2048)
    poison_cache(eng)
    lens = [61, 3, 20, 64, 9, 40, 1, 30][:rows]
    steps = 6
    seqs = [random_tokens(V, n + steps, 500 + i) for i, n in enumerate(lens)]
    refs = [oracle_logits("WIDE", tuple(s)) for s in seqs]
    slots = [eng.open() for _ in seqs]
    got = eng.step([Entry(sl, s[:n], [n - 1]) for sl, s, n in zip(slots, seqs, lens)])
    assert_close(got, torch.stack([r[n - 1] for r, n in zip(refs, lens)]), "bfloat16", "wide prompts")
    for j in range(steps):
        got = eng.step([Entry(sl, [s[n + j]], [0]) for sl, s, n in zip(slots, seqs, lens)])
        assert_close(got, torch.stack([r[n + j] for r, n in zip(refs, lens)]), "bfloat16", f"wide rows {rows} decode {j}")
    assert fused_plans(eng) and eng.model.stream_status() == 0
