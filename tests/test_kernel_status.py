"""The host side of the kernels' bounded waits, with fake status words (CPU).

A tensor-memory kernel whose wait on a barrier runs out stores a code in its library's status
word and returns without (all of) its output.  ``ops.check_status`` is what the engine calls
where the host has waited for the device anyway (after the prompt step, at every collected
decode step): it must name the kernel and the code, put the word back to 0, and leave the next
check clean.  No GPU is made to wait here: the words are Python objects.
"""
import pytest

from synaptix_b200 import ops
from synaptix_b200.ops import KernelError


class Word:
    def __init__(self, code=0):
        self.code, self.resets, self.reads = code, 0, 0

    def __call__(self, reset=False):
        self.reads += 1
        v = self.code
        if reset:
            self.code = 0
            self.resets += 1
        return v


def test_clean_words_raise_nothing():
    a, b = Word(), Word()
    ops.check_status({"gemm_tc": ("the product", a), "attn_tc": ("the attention", b)})
    assert a.reads == 1 and b.reads == 1 and a.resets == 0


def test_a_wait_that_ran_out_is_named_and_cleared():
    a, b = Word(), Word(7)
    with pytest.raises(KernelError, match=r"the attention.*status 7"):
        ops.check_status({"gemm_tc": ("the product", a), "attn_tc": ("the attention", b)})
    assert b.code == 0 and b.resets == 1
    ops.check_status({"gemm_tc": ("the product", a), "attn_tc": ("the attention", b)})       # clean again


def test_libraries_never_loaded_are_not_looked_at():
    # on a machine without a GPU nothing was loaded: the check is a no-op, not a build
    ops.check_status()
