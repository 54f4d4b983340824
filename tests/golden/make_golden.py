#!/usr/bin/env python3
"""Makes tests/golden/reference_ops.safetensors: small slices of the tensors that the reference's
OWN op-level oracles produce (scripts/reference/gen_norm.py, gen_pos.py, gen_ffn.py,
gen_attention.py, gen_infer.py: PyTorch generators whose outputs the reference's Rust tests
compare against at 1e-5, crates/synaptix-test-utils/src/lib.rs:43-90).

The reference's model code is Rust and cannot be built where this library is developed (no Rust
toolchain), so a whole-model comparison is not possible; these generators are the part of the
reference that does run here.  tests/test_golden.py checks the plain implementation
(tests/plain_qwen3.py) against the slices, which anchors its norm, rotation, feed-forward,
attention, head mapping, argmax and temperature formulas to the reference's.

    python tests/golden/make_golden.py /path/to/reference

Only slices of the OUTPUTS are kept (a few rows, heads and columns), so the committed file stays
small; the test regenerates the inputs from the generators' seeds.
"""
import importlib.util
import os
import sys
import tempfile

import torch
from safetensors import safe_open
from safetensors.torch import save_file

CASES = [("gen_norm.py", "case_rms_norm", "rms_norm"),
         ("gen_pos.py", "case_rope_split", "rope_split"),
         ("gen_ffn.py", "case_swiglu", "swiglu"),
         ("gen_attention.py", "case_scaled_dot_causal", "scaled_dot_causal"),
         ("gen_attention.py", "case_gqa", "gqa"),
         ("gen_infer.py", "case_greedy_argmax", "greedy_argmax"),
         ("gen_infer.py", "case_temperature_scaling", "temperature_scaling")]


def load(path):
    with safe_open(path, "pt") as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>")
    ref = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        os.chdir(tmp)
        for script, fn, name in CASES:
            spec = importlib.util.spec_from_file_location("gen_" + fn, os.path.join(ref, "scripts", "reference", script))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            getattr(mod, fn)()
            found = [os.path.join(dp, f) for dp, _, fs in os.walk(tmp) for f in fs if f == name + ".safetensors"]
            t = load(found[0])
            # Only OUTPUTS are kept (sliced); tests/test_golden.py regenerates the inputs from the same
            # torch seeds and shapes as the reference's generator functions.
            if name == "rms_norm":                       # output [4,32,256]
                out["rms_norm.output"] = t["output"][0, :4]
            elif name == "rope_split":                   # q_out [2,8,32,64]: batch 0, heads 0..1
                out["rope_split.q_out"] = t["q_out"][0, :2]
                out["rope_split.k_out"] = t["k_out"][0, :2]
            elif name == "swiglu":                       # output [2,16,256]: batch 0, 4 rows
                out["swiglu.output"] = t["output"][0, :4]
            elif name == "scaled_dot_causal":            # [2,8,32,64]: batch 0, heads 0..1
                out["sdpa_causal.output"] = t["output"][0, :2]
            elif name == "gqa":                          # [2,8,32,64]: batch 1, heads 0,3,4,7 (both kv heads, both ends of a group)
                out["gqa.output"] = t["output"][1][[0, 3, 4, 7]]
            elif name == "greedy_argmax":
                out["greedy.tokens"] = t["tokens"]
            elif name == "temperature_scaling":
                out["temperature.scaled_logits"] = t["scaled_logits"][:2, :64]
                out["temperature.probs"] = t["probs"][:2, :64]
                out["temperature.vocab"] = torch.tensor([t["logits"].shape[1], t["logits"].shape[0]])
    save_file({k: v.contiguous().clone() for k, v in out.items()}, os.path.join(here, "reference_ops.safetensors"))
    print("wrote", os.path.join(here, "reference_ops.safetensors"), sum(v.numel() * v.element_size() for v in out.values()), "bytes")


if __name__ == "__main__":
    main()
