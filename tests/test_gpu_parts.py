"""Each part of a layer alone, bound from tensors made here, against the plain functions;
and a toy mixer with state of its own, defined here, registered, built and stepped without a
change to the package's files."""
import dataclasses
import json
import math
import os
from typing import ClassVar, Tuple

import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


def rt(dtype):
    from synaptix_b200.parts import Runtime
    return Runtime(torch.device("cuda:0"), dtype)


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def simple_ctx(lens_past, lens_new, runtime, block_tables):
    from synaptix_b200.parts import StepContext
    pos = torch.cat([torch.arange(p, p + n) for p, n in zip(lens_past, lens_new)]).to(torch.int32).cuda()
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(lens_new)]).to(torch.int32).cuda()
    return StepContext(positions=pos, seq_of_token=sot, block_tables=block_tables, n_tokens=sum(lens_new),
                       n_seqs=len(lens_new), runtime=runtime)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from synaptix_b200.parts import RMSNorm
    n = RMSNorm("x.weight", 50, 3e-5)
    assert n.tensor_specs()["x.weight"].shape == (50,)
    w = (1 + 0.2 * torch.randn(50)).to(torch.bfloat16)
    n.bind({"x.weight": w}, rt(dtype))
    assert n.weight.dtype == torch.float32                     # gains are kept in 32-bit
    h = torch.randn(4, 50).cuda()
    d = torch.randn(4, 50).to(dtype).cuda()
    ref_h = h.cpu() + d.float().cpu()
    y = n.add_forward(h, d)
    assert torch.allclose(h.cpu(), ref_h, atol=1e-6)
    assert torch.allclose(y.float().cpu(), P.rms_norm(ref_h, w.float(), 3e-5), **tol(dtype))
    assert torch.allclose(n.forward(h).float().cpu(), P.rms_norm(ref_h, w.float(), 3e-5), **tol(dtype))


@pytest.mark.parametrize("rows", [1, 2, 5, 16, 20, 128, 150, 170])
def test_a_deferred_product_through_the_norm_and_the_next_product(rows):
    """A branch's last product handed on unrun (PendingLinear): the norm lets it add itself into h and hands scaled
    rows to the next product (2 to 160 rows), or runs it and norms as ever; either way the numbers are the plain ones.
    A norm that does not say it takes such a thing never sees one (the block runs the product first)."""
    from synaptix_b200.parts import Linear, RMSNorm
    from synaptix_b200.parts.base import PendingLinear, ScaledRows
    width, inner, out = 96, 160, 72
    bf = torch.bfloat16
    n = RMSNorm("n.weight", width, 2e-5)
    gain = 1 + 0.2 * torch.randn(width)
    n.bind({"n.weight": gain}, rt(bf))
    down = Linear("d.weight", inner, width)
    nxt = Linear("q.weight", width, out)
    wd = (torch.randn(width, inner) / math.sqrt(inner)).to(bf)
    wq = (torch.randn(out, width) / math.sqrt(width)).to(bf)
    down.bind({"d.weight": wd}, rt(bf))
    nxt.bind({"q.weight": wq}, rt(bf))
    z = torch.randn(rows, inner).to(bf)
    h0 = torch.randn(rows, width) * 3
    ref_h = h0.double() + z.double() @ wd.double().T
    ref_y = P.rms_norm(ref_h.float(), gain, 2e-5).double() @ wq.double().T
    for lazy in (True, False):
        h = h0.clone().cuda()
        x = n.add_forward(h, down.deferred(z.cuda()), lazy=lazy)
        assert isinstance(x, ScaledRows) == (lazy and 1 < rows <= 160)
        y = nxt.forward(x, out_dtype=torch.float32)
        h_after = x.h_after() if hasattr(x, "h_after") else h        # a lazy norm says where the sum went
        assert torch.allclose(h_after.cpu().double(), ref_h, atol=3e-2, rtol=1e-2)          # the branch is rounded to bf16 when run alone
        assert torch.allclose(y.cpu().double(), ref_y, atol=3e-2, rtol=2e-2)
        if isinstance(x, ScaledRows):
            assert torch.allclose(x.materialize().float().cpu(), P.rms_norm(ref_h.float(), gain, 2e-5), atol=3e-2, rtol=2e-2)
    pl = PendingLinear(z.cuda(), down.weight)
    assert pl.shape == (rows, width) and pl.materialize() is pl.materialize()


def test_rotary_part_has_the_plain_frequencies():
    from synaptix_b200.parts import RotaryHalf
    r = RotaryHalf(48, 77777.0, rotary_dim=32)
    r.bind({}, rt(torch.float32))
    inv, dim = r.rotation()
    assert dim == 32 and torch.equal(inv.cpu(), P.rotary_freqs(77777.0, 32))
    with pytest.raises(ValueError):
        RotaryHalf(48, 1e4, rotary_dim=50)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_part_stacks_named_matrices(dtype):
    from synaptix_b200.parts import Linear
    lin = Linear(["a.weight", "b.weight"], 40, [24, 8])
    assert {k: v.shape for k, v in lin.tensor_specs().items()} == {"a.weight": (24, 40), "b.weight": (8, 40)}
    a, b = torch.randn(24, 40).to(torch.bfloat16), torch.randn(8, 40).to(torch.bfloat16)
    lin.bind({"a.weight": a, "b.weight": b}, rt(dtype))
    x = torch.randn(19, 40).to(dtype)
    y = lin.forward(x.cuda())
    ref = x.float() @ torch.cat([a, b]).float().T
    assert y.dtype == dtype and torch.allclose(y.float().cpu(), ref, atol=(1e-4 if dtype == torch.float32 else 0.1), rtol=tol(dtype)["rtol"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from synaptix_b200.parts import SwiGLU
    f = SwiGLU("m.", 24, 56)
    w = {"m.gate_proj.weight": torch.randn(56, 24) * 0.3, "m.up_proj.weight": torch.randn(56, 24) * 0.3,
         "m.down_proj.weight": torch.randn(24, 56) * 0.3}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    assert set(f.all_tensor_specs()) == set(w)
    f.bind_all(w, rt(dtype))
    x = torch.randn(7, 24).to(dtype)
    y = f.forward(x.cuda(), None)
    ref = P.swiglu(x.float(), *(w[k].float() for k in ("m.gate_proj.weight", "m.up_proj.weight", "m.down_proj.weight")))
    assert torch.allclose(y.float().cpu(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,qk_norm", [(None, True), (20, True), (None, False)])
def test_attention_part_over_its_own_cache(dtype, window, qk_norm):
    """Two sequences, a prompt step and single-token steps, against whole-sequence attention."""
    from synaptix_b200.cache import Cache
    from synaptix_b200.parts import Attention, RotaryHalf
    width, nh, nkv, hd, eps, theta = 40, 6, 2, 16, 1e-5, 3000.0
    att = Attention("a.", width, nh, nkv, hd, position=RotaryHalf(hd, theta), qk_norm_eps=eps if qk_norm else None,
                    window=window)
    specs = att.all_tensor_specs()
    assert ("a.q_norm.weight" in specs) == qk_norm
    g = torch.Generator().manual_seed(0)
    w = {n: (torch.randn(s.shape, generator=g) * 0.3 + (1.0 if s.kind == "gain" else 0.0)).to(torch.bfloat16)
         for n, s in specs.items()}
    att.bind_all(w, rt(dtype))
    cache = Cache([att.cache_request()], max_tokens=512, max_seqs=4, dtype=dtype, device="cuda")
    for t in cache._k + cache._v:
        t.fill_(float("nan"))
    lens = [70, 45]
    xs = [torch.randn(n, width).to(dtype) for n in lens]

    def whole(x):
        cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=eps, rope_theta=theta)
        W = {("a." + k): v.float() for k, v in ((n[2:], t) for n, t in w.items())}
        T = x.shape[0]
        q = (x @ W["a.q_proj.weight"].T).view(T, nh, hd)
        k = (x @ W["a.k_proj.weight"].T).view(T, nkv, hd)
        v = (x @ W["a.v_proj.weight"].T).view(T, nkv, hd)
        if qk_norm:
            q, k = P.rms_norm(q, W["a.q_norm.weight"], eps), P.rms_norm(k, W["a.k_norm.weight"], eps)
        f = P.rotary_freqs(theta, hd)
        pos = torch.arange(T)
        q, k = P.rope_rotate_half(q, pos, f), P.rope_rotate_half(k, pos, f)
        return P.causal_gqa_attention(q, k, v, 1 / math.sqrt(hd), window).reshape(T, nh * hd) @ W["a.o_proj.weight"].T

    refs = [whole(x.float()) for x in xs]
    slots = [cache.open(), cache.open()]
    past = [0, 0]
    plan = [[60, 40], [1, 1], [1, 1], [8, 3]]
    for new in plan:
        cache.slots.reserve_many(slots, new)
        maxp = max((p + n + 63) // 64 for p, n in zip(past, new))
        bt = torch.zeros(2, maxp, dtype=torch.int32)
        for i, s in enumerate(slots):
            tb = cache.slots.table(s, 0)[:maxp]
            bt[i, :len(tb)] = torch.tensor(tb).clamp(min=0)
        ctx = simple_ctx(past, new, att, [bt.cuda()])
        x = torch.cat([xs[i][past[i]:past[i] + new[i]] for i in range(2)]).cuda()
        y = att.forward(x, ctx, cache.view(0)).float().cpu()
        ref = torch.cat([refs[i][past[i]:past[i] + new[i]] for i in range(2)])
        # outputs are of size ~10 here: measure against the largest value, as for logits
        rel = ((y - ref).abs().max() / ref.abs().max()).item()
        assert rel <= (1e-5 if dtype == torch.float32 else 2e-2), f"step {new}: {rel}"
        for i, s in enumerate(slots):
            cache.slots.advance(s, new[i])
            past[i] += new[i]


@pytest.mark.parametrize("tied", [True, False, None])
def test_embedding_and_output_head(tied):
    from synaptix_b200.parts import Embedding, OutputHead
    emb = Embedding("e.weight", 33, 12)
    head = OutputHead("h.weight", 33, 12, tied, emb)
    E, H = torch.randn(33, 12).to(torch.bfloat16), torch.randn(33, 12).to(torch.bfloat16)
    tensors = {"e.weight": E} if tied in (True, None) else {"e.weight": E, "h.weight": H}
    assert head.tensor_specs()["h.weight"].optional == (tied is not False)
    r = rt(torch.float32)
    emb.bind(tensors, r)
    head.bind(tensors, r)
    assert head.is_tied == (tied is not False)
    ids = torch.tensor([3, 32, 0], dtype=torch.int32).cuda()
    h = emb.forward(ids)
    assert torch.equal(h.cpu(), E.float()[[3, 32, 0]])
    x = torch.randn(2, 12).cuda()
    lg = head.forward(x)
    assert lg.dtype == torch.float32
    assert torch.allclose(lg.cpu(), x.cpu() @ (E if head.is_tied else H).float().T, atol=1e-5)


# ---------------------------------------------------------------------------------------------
# a toy architecture defined here: a mixer with a running state of its own in layer 0, attention
# in layer 1, and a schedule that runs layer 1 twice
# ---------------------------------------------------------------------------------------------
def make_toy(device_state: bool = False):
    """``device_state``: the mixer updates its state on the device from ``ctx.seq_slots`` in single-token steps,
    so those steps can be captured as CUDA graphs (registered under a name of its own)."""
    from synaptix_b200.cache import StateRequest
    from synaptix_b200.config import ModelConfig, register_architecture, take
    from synaptix_b200.models import DecoderModel, LayerRun
    from synaptix_b200.parts import (Attention, Embedding, Linear, Mixer, NoPosition, OutputHead, PreNormBlock,
                                     RMSNorm, SwiGLU)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architectures: ClassVar[Tuple[str, ...]] = ("ToyRunningMeanGraphLM" if device_state else "ToyRunningMeanLM",)
        model_types: ClassVar[Tuple[str, ...]] = ("toy_running_mean_graph" if device_state else "toy_running_mean",)
        vocab: int = 0
        width: int = 0
        eps: float = 0.0
        decay: float = 0.0

        @classmethod
        def from_dict(cls, d):
            return cls(vocab=take(d, "vocab", int), width=take(d, "width", int), eps=take(d, "eps", float),
                       decay=take(d, "decay", float))

        def to_dict(self):
            return {"architectures": list(self.architectures), "vocab": self.vocab, "width": self.width,
                    "eps": self.eps, "decay": self.decay}

        def validate(self):
            pass

    class DecayedSum(Mixer):
        """state <- decay * state + x_t ; out_t = W state.  The state [width] lives in the
        cache's per-sequence state region and goes on across steps."""
        graph_safe = device_state

        def __init__(self, prefix, width, decay):
            self.width, self.decay = width, decay
            self.proj = Linear(prefix + "proj.weight", width, width)

        def children(self):
            return [self.proj]

        def cache_request(self):
            return StateRequest((self.width,), torch.float32)

        def forward(self, x, ctx, state, write_cache=True):
            if device_state and ctx.all_single:
                # one token per sequence: the state rows of the step's slots, read and written on the device
                # (rows that pad a captured step carry the cache's spare slot, which no sequence owns)
                idx = ctx.seq_slots.long()
                s = self.decay * state.index_select(0, idx) + x.float()
                state.index_copy_(0, idx, s)
                return self.proj.forward(s.to(x.dtype))
            out = torch.empty_like(x)
            cu, slots = ctx.host["cu_seqlens"], ctx.host["seq_slots"]
            for i, slot in enumerate(slots):
                s = state[slot]
                for t in range(cu[i], cu[i + 1]):
                    s = self.decay * s + x[t].float()
                    out[t] = s.to(x.dtype)
                state[slot] = s
            return self.proj.forward(out)

    def build(cfg):
        emb = Embedding("emb.weight", cfg.vocab, cfg.width)
        l0 = PreNormBlock(RMSNorm("l0.n1.weight", cfg.width, cfg.eps), DecayedSum("l0.mix.", cfg.width, cfg.decay),
                          RMSNorm("l0.n2.weight", cfg.width, cfg.eps), SwiGLU("l0.ff.", cfg.width, 2 * cfg.width))
        l1 = PreNormBlock(RMSNorm("l1.n1.weight", cfg.width, cfg.eps),
                          Attention("l1.att.", cfg.width, 2, 1, 16, position=NoPosition()),
                          RMSNorm("l1.n2.weight", cfg.width, cfg.eps), SwiGLU("l1.ff.", cfg.width, 3 * cfg.width))
        # layer 1 runs twice, each run with a cache entry of its own
        schedule = [LayerRun(0, 0), LayerRun(1, 1), LayerRun(1, 2)]
        return DecoderModel(cfg, emb, [l0, l1], RMSNorm("norm.weight", cfg.width, cfg.eps),
                            OutputHead("head.weight", cfg.vocab, cfg.width, False, emb), schedule=schedule)

    register_architecture(ToyConfig, build)
    return ToyConfig


def toy_plain(cfg, W, tokens):
    """The toy model on one whole sequence, plain float32."""
    h = W["emb.weight"][torch.tensor(tokens)]
    T = len(tokens)

    def ff(x, p):
        return P.swiglu(x, W[p + "gate_proj.weight"], W[p + "up_proj.weight"], W[p + "down_proj.weight"])

    x = P.rms_norm(h, W["l0.n1.weight"], cfg["eps"])
    s = torch.zeros(cfg["width"])
    run = []
    for t in range(T):
        s = cfg["decay"] * s + x[t]
        run.append(s)
    h = h + torch.stack(run) @ W["l0.mix.proj.weight"].T
    h = h + ff(P.rms_norm(h, W["l0.n2.weight"], cfg["eps"]), "l0.ff.")
    for _ in range(2):
        x = P.rms_norm(h, W["l1.n1.weight"], cfg["eps"])
        q = (x @ W["l1.att.q_proj.weight"].T).view(T, 2, 16)
        k = (x @ W["l1.att.k_proj.weight"].T).view(T, 1, 16)
        v = (x @ W["l1.att.v_proj.weight"].T).view(T, 1, 16)
        h = h + P.causal_gqa_attention(q, k, v, 0.25, None).reshape(T, 32) @ W["l1.att.o_proj.weight"].T
        h = h + ff(P.rms_norm(h, W["l1.n2.weight"], cfg["eps"]), "l1.ff.")
    return P.rms_norm(h, W["norm.weight"], cfg["eps"]) @ W["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stateful_mixer_with_state_on_the_device_under_captured_steps(tmp_path, dtype):
    """Three live sequences run in a captured step of four rows: the padding row must not touch any live
    sequence's state (it carries the cache's spare slot).  Through the step function and through a decode session."""
    from helpers import assert_close
    from synaptix_b200.engine import DecodeRow, Engine, Entry
    from synaptix_b200.models import load_model
    from synaptix_b200.weights import write_model_folder
    ToyConfig = make_toy(device_state=True)
    cfg = ToyConfig(vocab=71, width=24, eps=1e-5, decay=0.9)
    d = write_model_folder(cfg, str(tmp_path / "toyg"), 4, std_matrix=0.2, std_embedding=0.5, std_gain=0.1)
    model = load_model(d, dtype=dtype)
    assert model.all_graph_safe()
    eng = Engine(model, max_tokens=1024, max_seqs=3)          # slots 0, 1, 2 are all in use
    assert eng.use_graphs and eng.cache.spare_slot == 3
    cfgd, W = P.load_folder(d)
    g = torch.Generator().manual_seed(2)
    n_dec = 40
    seqs = [torch.randint(0, 71, (n + n_dec,), generator=g).tolist() for n in (30, 75, 9)]
    refs = [toy_plain(cfgd, W, s) for s in seqs]
    slots = [eng.open() for _ in seqs]
    cut = [len(s) - n_dec for s in seqs]
    got = eng.step([Entry(sl, s[:c], [c - 1]) for sl, s, c in zip(slots, seqs, cut)])
    assert_close(got, torch.stack([r[c - 1] for r, c in zip(refs, cut)]), dtype, "prompts")
    half = n_dec // 2
    for j in range(half):                                     # captured steps of the step function (3 rows in 4)
        got = eng.step([Entry(sl, [s[c + j]], [0]) for sl, s, c in zip(slots, seqs, cut)])
        assert_close(got, torch.stack([r[c + j] for r, c in zip(refs, cut)]), dtype, f"step {j}")
    assert any(c.graph is not None for c in eng._captured.values())
    # the rest through a decode session, fed the sequences' own tokens; its choices are the plain model's
    sess = eng.start_decode([DecodeRow(sl, s[c + half], i, 0) for i, (sl, s, c) in enumerate(zip(slots, seqs, cut))])
    for j in range(half, n_dec):
        sess.launch(tokens=[s[c + j] for s, c in zip(seqs, cut)])
        got = sess.collect()
        if dtype == "float32":
            assert got == [int(r[c + j].argmax()) for r, c in zip(refs, cut)], f"session step {j}"
    assert sess.cap.graph is not None and sess.cap.layout.S == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer(tmp_path, dtype):
    from helpers import assert_close
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    from synaptix_b200.weights import write_model_folder
    ToyConfig = make_toy()
    cfg = ToyConfig(vocab=71, width=24, eps=1e-5, decay=0.9)
    d = write_model_folder(cfg, str(tmp_path / "toy"), 3, std_matrix=0.2, std_embedding=0.5, std_gain=0.1)
    model = load_model(d, dtype=dtype)                      # the class is chosen by config.json
    assert type(model.config).__name__ == "ToyConfig" and not model.all_graph_safe()
    eng = Engine(model, max_tokens=512, max_seqs=3)
    assert len(eng.cache.kv_groups) == 1 and len(eng.cache.state_groups) == 1
    cfgd, W = P.load_folder(d)
    g = torch.Generator().manual_seed(1)
    seqs = [torch.randint(0, 71, (n,), generator=g).tolist() for n in (30, 75, 9, 20)]
    refs = [toy_plain(cfgd, W, s) for s in seqs]
    # two batches, so that the second runs in slots whose state the first left behind
    for batch in ([0, 1, 2], [3, 0]):
        slots = {i: eng.open() for i in batch}
        cut = {i: len(seqs[i]) - 5 for i in batch}
        got = eng.step([Entry(slots[i], seqs[i][:cut[i]], [cut[i] - 1]) for i in batch])
        assert_close(got, torch.stack([refs[i][cut[i] - 1] for i in batch]), dtype, "toy prompts")
        for j in range(5):
            got = eng.step([Entry(slots[i], [seqs[i][cut[i] + j]], [0]) for i in batch])
            assert_close(got, torch.stack([refs[i][cut[i] + j] for i in batch]), dtype, f"toy decode {j}")
        for i in batch:
            eng.close(slots[i])


# ---------------------------------------------------------------------------------------------
# a second toy architecture defined here: a feed-forward with routing (a router picks one of three
# experts per token) and a position encoding of another law (half of every head rotated, with
# frequencies that fall off as 1 / (1 + i)); layer 1's attention also has a window, so the two
# layers' keys live in storage groups of their own
# ---------------------------------------------------------------------------------------------
def make_routed_toy():
    from synaptix_b200 import ops
    from synaptix_b200.config import ModelConfig, register_architecture, take
    from synaptix_b200.models import DecoderModel
    from synaptix_b200.parts import (Attention, Embedding, FeedForward, Linear, OutputHead, PositionEncoding,
                                     PreNormBlock, RMSNorm, SwiGLU)

    @dataclasses.dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architectures: ClassVar[Tuple[str, ...]] = ("ToyRoutedLM",)
        model_types: ClassVar[Tuple[str, ...]] = ("toy_routed",)
        vocab: int = 0
        width: int = 0
        eps: float = 0.0
        experts: int = 0
        inner: int = 0
        base: float = 0.0

        @classmethod
        def from_dict(cls, d):
            return cls(vocab=take(d, "vocab", int), width=take(d, "width", int), eps=take(d, "eps", float),
                       experts=take(d, "experts", int), inner=take(d, "inner", int), base=take(d, "base", float))

        def to_dict(self):
            return {"architectures": ["ToyRoutedLM"], "vocab": self.vocab, "width": self.width, "eps": self.eps,
                    "experts": self.experts, "inner": self.inner, "base": self.base}

        def validate(self):
            pass

    class HarmonicHalfRotary(PositionEncoding):
        """The first ``rotary_dim`` elements of a head are rotated by ``position * base / (1 + i)``."""

        def __init__(self, rotary_dim, base):
            self.rotary_dim, self.base = rotary_dim, base
            self.inv_freq = None

        def bind(self, tensors, rt):
            self.inv_freq = (self.base / (1.0 + torch.arange(self.rotary_dim // 2, dtype=torch.float32))).to(rt.device)

        def rotation(self):
            return self.inv_freq, self.rotary_dim

    class OneOfExperts(FeedForward):
        """``out_t = p_t[e_t] * expert_{e_t}(x_t)`` with ``p_t = softmax(router x_t)`` in float32 and ``e_t`` its
        largest entry.  The router and the experts are the framework's ``Linear`` and ``SwiGLU``; picking the
        tokens of an expert is this part's own business."""
        graph_safe = False            # the number of tokens per expert is read on the host

        def __init__(self, prefix, width, experts, inner):
            self.router = Linear(prefix + "router.weight", width, experts)
            self.experts = [SwiGLU(prefix + f"e{e}.", width, inner) for e in range(experts)]

        def children(self):
            return [self.router] + self.experts

        def forward(self, x, ctx):
            logits = self.router.forward(x, out_dtype=torch.float32)
            p = torch.softmax(logits, dim=-1)
            top = logits.argmax(dim=-1)
            out = torch.zeros_like(x)
            for e, expert in enumerate(self.experts):
                idx = (top == e).nonzero().squeeze(1)
                if idx.numel():
                    y = expert.forward(x.index_select(0, idx).contiguous(), ctx)
                    out.index_copy_(0, idx, (y.float() * p[idx, e][:, None]).to(x.dtype))
            return out

    def build(cfg):
        emb = Embedding("emb.weight", cfg.vocab, cfg.width)
        layers = []
        for i, window in enumerate((None, 9)):
            layers.append(PreNormBlock(
                RMSNorm(f"l{i}.n1.weight", cfg.width, cfg.eps),
                Attention(f"l{i}.att.", cfg.width, 3, 1, 32, position=HarmonicHalfRotary(16, cfg.base), window=window),
                RMSNorm(f"l{i}.n2.weight", cfg.width, cfg.eps),
                OneOfExperts(f"l{i}.ff.", cfg.width, cfg.experts, cfg.inner)))
        return DecoderModel(cfg, emb, layers, RMSNorm("norm.weight", cfg.width, cfg.eps),
                            OutputHead("head.weight", cfg.vocab, cfg.width, False, emb))

    register_architecture(RoutedConfig, build)
    return RoutedConfig


def routed_toy_plain(cfg, W, tokens):
    """The routed toy model on one whole sequence, plain float32."""
    T = len(tokens)
    h = W["emb.weight"][torch.tensor(tokens)]
    pos = torch.arange(T)
    freqs = cfg["base"] / (1.0 + torch.arange(8, dtype=torch.float32))

    def rotate(x):                                                  # the first 16 of 32 elements
        return torch.cat([P.rope_rotate_half(x[..., :16], pos, freqs), x[..., 16:]], dim=-1)

    for i, window in enumerate((None, 9)):
        x = P.rms_norm(h, W[f"l{i}.n1.weight"], cfg["eps"])
        q = rotate((x @ W[f"l{i}.att.q_proj.weight"].T).view(T, 3, 32))
        k = rotate((x @ W[f"l{i}.att.k_proj.weight"].T).view(T, 1, 32))
        v = (x @ W[f"l{i}.att.v_proj.weight"].T).view(T, 1, 32)
        a = P.causal_gqa_attention(q, k, v, 1.0 / math.sqrt(32), window).reshape(T, 96)
        h = h + a @ W[f"l{i}.att.o_proj.weight"].T
        x = P.rms_norm(h, W[f"l{i}.n2.weight"], cfg["eps"])
        logits = x @ W[f"l{i}.ff.router.weight"].T
        p = torch.softmax(logits, dim=-1)
        out = torch.zeros_like(x)
        for t in range(T):
            e = int(logits[t].argmax())
            pre = f"l{i}.ff.e{e}."
            out[t] = p[t, e] * P.swiglu(x[t:t + 1], W[pre + "gate_proj.weight"], W[pre + "up_proj.weight"],
                                        W[pre + "down_proj.weight"])[0]
        h = h + out
    return P.rms_norm(h, W["norm.weight"], cfg["eps"]) @ W["head.weight"].T


def test_toy_architecture_with_routed_experts_and_another_rotation(tmp_path):
    """Registered, built, loaded and stepped without a change to the framework's files.  In float32 only: the
    choice of an expert is a step function of the router's logits, and a near-tie flipped by bfloat16 rounding
    changes a token's output wholesale, which says nothing about the parts under test."""
    from helpers import assert_close
    from synaptix_b200.engine import Engine, Entry
    from synaptix_b200.models import load_model
    from synaptix_b200.weights import write_model_folder
    RoutedConfig = make_routed_toy()
    cfg = RoutedConfig(vocab=83, width=40, eps=2e-5, experts=3, inner=56, base=0.7)
    d = write_model_folder(cfg, str(tmp_path / "routed"), 5, std_matrix=0.2, std_embedding=0.5, std_gain=0.1)
    model = load_model(d, dtype="float32")
    assert type(model.config).__name__ == "RoutedConfig" and not model.all_graph_safe()
    eng = Engine(model, max_tokens=1024, max_seqs=3)
    assert len(eng.cache.kv_groups) == 2                           # all keys, and a window of them
    cfgd, W = P.load_folder(d)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 83, (n,), generator=g).tolist() for n in (41, 90, 7, 26)]
    refs = [routed_toy_plain(cfgd, W, s) for s in seqs]
    used = set()
    for s in seqs:                                                   # every expert is used by some token
        x = P.rms_norm(W["emb.weight"][torch.tensor(s)], W["l0.n1.weight"], cfgd["eps"])
        used |= set((x @ W["l0.ff.router.weight"].T).argmax(-1).tolist())
    assert len(used) >= 2
    for batch in ([0, 1, 2], [3, 1]):
        slots = {i: eng.open() for i in batch}
        cut = {i: len(seqs[i]) - 5 for i in batch}
        got = eng.step([Entry(slots[i], seqs[i][:cut[i]], [0, cut[i] - 1]) for i in batch])
        want = torch.stack([refs[i][j] for i in batch for j in (0, cut[i] - 1)])
        assert_close(got, want, "float32", "routed prompts")
        for j in range(5):
            got = eng.step([Entry(slots[i], [seqs[i][cut[i] + j]], [0]) for i in batch])
            assert_close(got, torch.stack([refs[i][cut[i] + j] for i in batch]), "float32", f"routed decode {j}")
        for i in batch:
            eng.close(slots[i])
