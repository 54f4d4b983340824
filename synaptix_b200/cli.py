"""Command line, in the manner of the reference's ``synaptix run`` and ``synaptix bench``
(crates/synaptix-cli/src/bin/synaptix.rs:49-129): the same option names and meanings where
the reference has them.  Prompts are token ids (comma or blank separated), since
tokenizers are outside this library; ``--prompt-file`` holds one prompt per line and makes
a batch.  ``random`` writes a model folder with seeded random weights.

    python -m synaptix_b200 run MODEL "5 17 3" --max-tokens 16 --temperature 0
    python -m synaptix_b200 bench MODEL --n-tokens 128 --prompt-tokens 2048 --batch-size 8
    python -m synaptix_b200 random CONFIG.json OUT_DIR --seed 0
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from typing import List


def parse_ids(text: str) -> List[int]:
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"a prompt is a list of token ids (integers), got {text!r}") from None


def _dtype_arg(s: str) -> str:
    table = {"f32": "float32", "fp32": "float32", "float32": "float32",
             "bf16": "bfloat16", "bfloat16": "bfloat16"}
    if s.lower() == "f16":
        raise SystemExit("compute dtype f16 is not built: use bf16 or f32")
    if s.lower() not in table:
        raise SystemExit(f"unknown dtype {s!r}: use bf16 or f32")
    return table[s.lower()]


_ATTN = {"auto": None, "flash-decode": None, "flash_decode": None, "decode": None,
         "fa2": False, "flash2": False, "flash-attn-2": False, "fa4": True, "flash4": True, "flash-attn-4": True}
_ATTN_HELP = ("attention backend, the reference's names (synaptix-core/src/backend/attn.rs:47-56): auto (default); "
              "fa4: prompt attention on the tcgen05 tensor cores; fa2: on mma.sync tiles; flash-decode: accepted, equals "
              "auto here (single-token steps always run the split-KV decode kernel)")


def _set_attn(name) -> None:
    """``--attn``: which prompt-attention kernel runs (an option of this process, ``ops.set_options(attn_tc=...)``)."""
    if name is None:
        return
    key = name.strip().lower()
    if key not in _ATTN:
        raise SystemExit(f"unknown --attn {name!r}: use auto, flash-decode, fa2 or fa4")
    if _ATTN[key] is not None:
        from . import ops
        ops.set_options(attn_tc=_ATTN[key])


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="synaptix_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="generate from a prompt of token ids")
    run.add_argument("model", help="folder with config.json and model.safetensors")
    run.add_argument("prompt", nargs="?", default="", help="token ids, comma or blank separated")
    run.add_argument("--prompt-file", help="one prompt per line (a batch)")
    run.add_argument("--max-tokens", type=int, default=128, help="new tokens per prompt")
    run.add_argument("--temperature", type=float, default=1.0, help="<= 0 is greedy")
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--top-k", type=int, default=0)
    run.add_argument("--top-p", type=float, default=1.0)
    run.add_argument("--min-p", type=float, default=0.0)
    run.add_argument("--repetition-penalty", type=float, default=1.0)
    run.add_argument("--repeat-last-n", type=int, default=0)
    run.add_argument("--presence-penalty", type=float, default=0.0)
    run.add_argument("--frequency-penalty", type=float, default=0.0)
    run.add_argument("--device", default="cuda", help="cuda or cuda:N (there is no CPU path)")
    run.add_argument("--prefill-batch", type=int, default=0,
                     help="run the prompt in portions of N tokens (0: the whole prompt in one step)")
    run.add_argument("--max-seq", type=int, default=None,
                     help="cache capacity per sequence; default prompt + max-tokens")
    run.add_argument("--attn", default=None, help=_ATTN_HELP)
    run.add_argument("--compute-dtype", default="bf16", help="bf16 or f32 (f32: everything in true 32-bit)")
    run.add_argument("--no-graph", action="store_true", help="do not replay decode steps as CUDA graphs")
    run.add_argument("--nvtx", action="store_true", help="name every step for a profiler's timeline (NVTX ranges)")
    run.add_argument("--warmup", action="store_true", help="run one prompt step and one token before timing")
    run.add_argument("--stop-ids", default=None, help="stop token ids; default: the model's eos_token_id")
    run.add_argument("--json", action="store_true", help="print one JSON object instead of text")

    bench = sub.add_parser("bench", help="time prompt processing and decoding with synthetic ids")
    bench.add_argument("model")
    bench.add_argument("--n-tokens", type=int, default=128, help="decoded tokens per sequence")
    bench.add_argument("--prompt-tokens", type=int, default=0, help="prompt length (0: 32)")
    bench.add_argument("--batch-size", type=int, default=1)
    bench.add_argument("--warmup", type=int, default=3)
    bench.add_argument("--device", default="cuda")
    bench.add_argument("--attn", default=None, help=_ATTN_HELP)
    bench.add_argument("--dtype", default="bf16")

    ins = sub.add_parser("inspect", help="list the tensors of a safetensors file, or of a model folder with what its configuration says")
    ins.add_argument("file", help="a .safetensors file, or a folder with config.json and model.safetensors")
    ins.add_argument("-v", "--verbose", action="store_true", help="bytes of every tensor too")
    ins.add_argument("-f", "--filter", default=None, help="only tensors whose name contains this")

    rnd = sub.add_parser("random", help="write a model folder with seeded random weights")
    rnd.add_argument("config", help="a config.json (or a folder holding one)")
    rnd.add_argument("out_dir")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--std", type=float, default=0.02, help="standard deviation of matrices and embeddings")
    rnd.add_argument("--std-gain", type=float, default=0.05, help="norm gains are 1 + N(0, std-gain)")
    return ap


def _device(s: str) -> str:
    if s == "cuda":
        return "cuda:0"
    if not s.startswith("cuda"):
        raise SystemExit(f"device {s!r}: only CUDA devices are supported (there is no CPU path)")
    return s


def cmd_run(a) -> int:
    from .api import LLM
    _set_attn(a.attn)
    prompts: List[List[int]] = []
    if a.prompt_file:
        with open(a.prompt_file) as f:
            prompts = [parse_ids(line) for line in f if line.strip()]
    elif a.prompt.strip():
        prompts = [parse_ids(a.prompt)]
    if not prompts:
        raise SystemExit("give a prompt (token ids) or --prompt-file")
    per_seq = a.max_seq or max(len(p) for p in prompts) + a.max_tokens
    max_tokens = sum(((min(per_seq, len(p) + a.max_tokens) + 63) // 64) * 64 for p in prompts)
    t0 = time.perf_counter()
    llm = LLM(a.model, compute_dtype=_dtype_arg(a.compute_dtype), device=_device(a.device),
              max_tokens=max_tokens, graph=not a.no_graph, nvtx=a.nvtx)
    load_s = time.perf_counter() - t0
    kw = dict(max_new_tokens=a.max_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
              min_p=a.min_p, repetition_penalty=a.repetition_penalty, repeat_last_n=a.repeat_last_n,
              presence_penalty=a.presence_penalty, frequency_penalty=a.frequency_penalty, seed=a.seed,
              prefill_batch=a.prefill_batch)
    if a.stop_ids is not None:
        kw["eos_token_ids"] = parse_ids(a.stop_ids)
    if a.warmup:
        llm.generate([prompts[0]], **dict(kw, max_new_tokens=2))
    results = llm.generate(prompts, return_details=True, **kw)
    st = llm.last_stats
    if a.json:
        print(json.dumps({"outputs": [{"tokens": r.tokens, "finish_reason": r.finish_reason} for r in results],
                          "prompt_tokens": st.prompt_tokens, "new_tokens": st.new_tokens,
                          "prefill_ms": st.prefill_ms, "decode_ms": st.decode_ms}))
    else:
        for r in results:
            print(" ".join(str(t) for t in r.tokens))
        dec = max(st.new_tokens - len(results), 0)
        print(f"[load {load_s:.2f} s | prompt {st.prompt_tokens} tok in {st.prefill_ms:.1f} ms | "
              f"decode {dec} tok in {st.decode_ms:.1f} ms"
              + (f" = {dec / st.decode_ms * 1e3:.1f} tok/s" if st.decode_ms > 0 and dec else "") + "]",
              file=sys.stderr)
    return 0


def cmd_inspect(a) -> int:
    """As the reference's ``inspect`` for safetensors (crates/synaptix-cli/src/commands/inspect.rs:66-93): every
    tensor with its dtype and shape, how many were shown, and the total of bytes.  For a model folder first what the
    configuration gives: the architecture, its sizes, the cache's bytes a token.  Needs no GPU."""
    import os
    from .weights.safetensors_io import SafetensorsFile
    path = a.file
    if os.path.isdir(path):
        from .config import load_config
        cfg = load_config(path)
        d = cfg.to_dict()
        print(f"=== model folder: {path} ===")
        print(f"  architecture: {(d.get('architectures') or ['?'])[0]} ({d.get('model_type', '?')})")
        for k in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                  "intermediate_size", "vocab_size", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
                  "max_position_embeddings"):
            if k in d:
                print(f"  {k}: {d[k]}")
        if all(k in d for k in ("num_hidden_layers", "num_key_value_heads", "head_dim")):
            print(f"  cache, bfloat16: {2 * d['num_hidden_layers'] * d['num_key_value_heads'] * d['head_dim'] * 2} bytes a token")
        print()
        path = os.path.join(path, "model.safetensors")
    f = SafetensorsFile(path)
    print(f"=== SafeTensors: {path} ===")
    print(f"  total tensors: {len(f.tensors)}")
    print()
    shown = total_bytes = params = 0
    for name, info in f.tensors.items():
        total_bytes += info.end - info.begin
        n = 1
        for x in info.shape:
            n *= x
        params += n
        if a.filter is not None and a.filter not in name:
            continue
        shape = ",".join(str(x) for x in info.shape)
        if a.verbose:
            print(f"  {name} dtype={info.dtype} shape=[{shape}] bytes={info.end - info.begin}")
        else:
            print(f"  {name:<60} {info.dtype} [{shape}]")
        shown += 1
    print()
    print(f"  shown {shown} of {len(f.tensors)} tensors, {params} elements, total {total_bytes} bytes "
          f"({total_bytes / 1024.0 / 1024.0:.2f} MB)")
    return 0


def cmd_bench(a) -> int:
    from .api import LLM
    _set_attn(a.attn)
    n_prompt = a.prompt_tokens or 32
    B = a.batch_size
    llm = LLM(a.model, compute_dtype=_dtype_arg(a.dtype), device=_device(a.device),
              max_tokens=B * (((n_prompt + a.n_tokens + 63) // 64) * 64))
    vocab = llm.model.vocab_size
    # synthetic ids as the reference's perf tools make them (qwen3/examples/format_perf.rs:70,94)
    prompts = [[((i * 7 + 13 + b) % min(200, vocab - 5)) + 5 for i in range(n_prompt)] for b in range(B)]
    for _ in range(a.warmup):
        llm.generate(prompts, max_new_tokens=2, eos_token_ids=[])
    best = None
    for _ in range(2):
        llm.generate(prompts, max_new_tokens=a.n_tokens, eos_token_ids=[])
        st = llm.last_stats
        if best is None or st.decode_ms < best.decode_ms:
            best = st
    dec = best.new_tokens - B
    print(f"prefill: {best.prompt_tokens} tok in {best.prefill_ms:.2f} ms = "
          f"{best.prompt_tokens / best.prefill_ms * 1e3:.1f} tok/s")
    print(f"decode : {dec} tok in {best.decode_ms:.2f} ms = {dec / best.decode_ms * 1e3:.1f} tok/s (batch {B})")
    return 0


def cmd_random(a) -> int:
    from .config import load_config
    from .weights import write_model_folder
    cfg = load_config(a.config)
    write_model_folder(cfg, a.out_dir, a.seed, std_matrix=a.std, std_gain=a.std_gain)
    print(a.out_dir)
    return 0


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    return {"run": cmd_run, "bench": cmd_bench, "random": cmd_random, "inspect": cmd_inspect}[a.command](a)
