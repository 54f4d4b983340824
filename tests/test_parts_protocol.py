"""What a block hands between its parts, decided on the host: checked here with fake parts on the CPU.

A branch's last product may travel unrun (``PendingLinear``) only between parts that both say they can handle it;
everybody else gets plain tensors, so a part written without knowledge of the deferred forms keeps working.
"""
import torch

from synaptix_b200.parts import FeedForward, Mixer, Norm, PendingLinear, PreNormBlock


class FakeProduct(PendingLinear):
    """A deferred product that needs no kernel: materialises to a tensor of ones."""

    def __init__(self, rows, width):
        super().__init__(torch.zeros(rows, 3), torch.zeros(width, 3))
        self.runs = 0

    def materialize(self):
        self.runs += 1
        return torch.ones(self.shape)


class PlainNorm(Norm):
    def __init__(self):
        self.seen = []

    def add_forward(self, h, delta, rows=None, lazy=False):
        self.seen.append(delta)
        if delta is not None:
            h += delta
        return h.clone()


class TakingNorm(PlainNorm):
    takes_pending_product = True

    def add_forward(self, h, delta, rows=None, lazy=False):
        self.seen.append(delta)
        if isinstance(delta, PendingLinear):
            delta = delta.materialize()
        if delta is not None:
            h += delta
        return h.clone()


class PlainMixer(Mixer):
    def __init__(self):
        self.kwargs = []

    def forward(self, x, ctx, cache_view, write_cache=True, **kw):
        self.kwargs.append(kw)
        return torch.full_like(x, 2.0)


class DeferringMixer(PlainMixer):
    can_defer_output = True

    def forward(self, x, ctx, cache_view, write_cache=True, defer_output=False):
        self.kwargs.append({"defer_output": defer_output})
        return FakeProduct(*x.shape) if defer_output else torch.ones_like(x)


class PlainFF(FeedForward):
    def __init__(self):
        self.kwargs = []

    def forward(self, x, ctx, **kw):
        self.kwargs.append(kw)
        return torch.full_like(x, 3.0)


class DeferringFF(PlainFF):
    can_defer_output = True

    def forward(self, x, ctx, defer_output=False):
        self.kwargs.append({"defer_output": defer_output})
        return FakeProduct(*x.shape) if defer_output else torch.ones_like(x)


def test_parts_that_know_nothing_of_deferred_products_never_see_one():
    n1, n2, mx, ff = PlainNorm(), PlainNorm(), PlainMixer(), PlainFF()
    blk = PreNormBlock(n1, mx, n2, ff)
    h = torch.zeros(4, 5)
    pending = FakeProduct(4, 5)
    h2, m = blk.forward(h, pending, None, None)
    assert pending.runs == 1 and isinstance(n1.seen[0], torch.Tensor)       # run before the norm saw it
    assert mx.kwargs == [{}] and ff.kwargs == [{}]                            # nobody was asked to defer
    assert isinstance(n2.seen[0], torch.Tensor) and isinstance(m, torch.Tensor)
    assert torch.equal(h2, torch.full((4, 5), 3.0))                           # 1 (pending) + 2 (mixer); m is not added yet


def test_a_product_is_deferred_only_towards_a_norm_that_takes_it():
    # the mixer could defer, but the norm after it does not take such a thing: it is not asked to
    n1, n2, mx, ff = TakingNorm(), PlainNorm(), DeferringMixer(), PlainFF()
    PreNormBlock(n1, mx, n2, ff).forward(torch.zeros(2, 3), None, None, None)
    assert mx.kwargs == [{"defer_output": False}] and isinstance(n2.seen[0], torch.Tensor)
    # both agree: the norm gets the product unrun
    n1, n2, mx, ff = TakingNorm(), TakingNorm(), DeferringMixer(), DeferringFF()
    blk = PreNormBlock(n1, mx, n2, ff)
    pending = FakeProduct(2, 3)
    h, m = blk.forward(torch.zeros(2, 3), pending, None, None)
    assert n1.seen[0] is pending and pending.runs == 1                        # handed on unrun; the norm ran it
    assert mx.kwargs == [{"defer_output": True}] and isinstance(n2.seen[0], FakeProduct)
    assert ff.kwargs == [{"defer_output": True}] and isinstance(m, FakeProduct) and m.runs == 0
    assert torch.equal(h, torch.full((2, 3), 2.0))                            # 1 (pending) + 1 (the mixer's product)


def test_a_block_says_whether_its_pending_input_may_be_deferred():
    assert PreNormBlock.takes_pending_product is True
    assert Norm.takes_pending_product is False and Mixer.can_defer_output is False and FeedForward.can_defer_output is False
