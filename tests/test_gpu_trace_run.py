"""bin/trace_run driven as a user drives it: a subprocess, JSON lines on standard input,
``done <step>`` lines on standard output, logits files compared with the plain implementation.
The same requests are replayed whole, with the last 32 tokens one by one, and in batches of
unequal lengths whose shorter requests end earlier, one batch after another in a cache that
holds little more than one batch."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import assert_close, folder, oracle, oracle_logits
from tiny import random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Replay:
    def __init__(self, model_dir, dtype, out_dir, max_tokens):
        self.out_dir = out_dir
        self.proc = subprocess.Popen(
            [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step_no = 0

    def step(self, entries, end=()):
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        assert line.strip() == f"done {self.step_no}", f"got {line!r}"
        n = self.step_no
        self.step_no += 1
        path = os.path.join(self.out_dir, f"{n}.f32")
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(data.reshape(wanted, -1).copy())

    def finish(self):
        self.proc.stdin.close()
        assert self.proc.wait(timeout=120) == 0


def requests_for(name):
    V = oracle(name)[0]["vocab_size"]
    lens = [40, 97, 33, 150, 64]
    return {f"r{i}": random_tokens(V, n, 700 + i) for i, n in enumerate(lens)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_three_ways(tmp_path, name, dtype):
    reqs = requests_for(name)
    V = oracle(name)[0]["vocab_size"]

    # 1. each request alone and whole, every position wanted
    rp = Replay(folder(name), dtype, str(tmp_path / "whole"), max_tokens=192)
    for rid, toks in reqs.items():
        got = rp.step([{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], end=[rid])
        assert got.shape == (len(toks), V)
        assert_close(got, oracle_logits(name, tuple(toks)), dtype, f"{name} {dtype} whole {rid}")
    rp.finish()

    # 2. whole but for the last 32 tokens, which are decoded one by one
    rp = Replay(folder(name), dtype, str(tmp_path / "tail"), max_tokens=192)
    for rid, toks in reqs.items():
        ref = oracle_logits(name, tuple(toks))
        head = len(toks) - 32
        got = [rp.step([{"id": rid, "tokens": toks[:head], "want": [head - 1]}])]
        for j in range(head, len(toks)):
            got.append(rp.step([{"id": rid, "tokens": [toks[j]], "want": [0]}],
                               end=[rid] if j == len(toks) - 1 else []))
        assert_close(torch.cat(got), ref[head - 1:], dtype, f"{name} {dtype} tail {rid}")
    rp.finish()

    # 3. batches of unequal lengths; shorter requests end earlier; a second batch follows in
    #    the pages the first gave back (6 pages hold one batch and no more)
    rp = Replay(folder(name), dtype, str(tmp_path / "batch"), max_tokens=384)
    for batch in (["r0", "r1", "r2"], ["r3", "r4", "r2"]):
        prompt = {rid: len(reqs[rid]) - 32 if rid != "r2" else len(reqs[rid]) - 8 for rid in batch}
        got = rp.step([{"id": rid, "tokens": reqs[rid][:prompt[rid]], "want": [prompt[rid] - 1]} for rid in batch])
        ref = torch.stack([oracle_logits(name, tuple(reqs[rid]))[prompt[rid] - 1] for rid in batch])
        assert_close(got, ref, dtype, f"{name} {dtype} batch prompts {batch}")
        live = list(batch)
        j = 0
        while live:
            ending = [rid for rid in live if prompt[rid] + j == len(reqs[rid]) - 1]
            got = rp.step([{"id": rid, "tokens": [reqs[rid][prompt[rid] + j]], "want": [0]} for rid in live], end=ending)
            ref = torch.stack([oracle_logits(name, tuple(reqs[rid]))[prompt[rid] + j] for rid in live])
            assert_close(got, ref, dtype, f"{name} {dtype} batch {batch} step {j} live {live}")
            live = [rid for rid in live if rid not in ending]
            j += 1
    rp.finish()


def test_replay_wants_nothing_and_exits_zero(tmp_path):
    rp = Replay(folder("A"), "float32", str(tmp_path / "o"), max_tokens=128)
    assert rp.step([{"id": "x", "tokens": [1, 2, 3], "want": []}]) is None
    got = rp.step([{"id": "x", "tokens": [4], "want": [0]}], end=["x"])
    assert_close(got, oracle_logits("A", (1, 2, 3, 4))[3:], "float32", "after a step that wanted nothing")
    rp.finish()
