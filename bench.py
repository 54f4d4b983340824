#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-4B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 4b|8b|32b] [--batch B] [--context C]

A step is one decode step of the whole batch (default batch 8, context 4,096: every
sequence holds a prompt and decodes up to 4,096 tokens, the timed steps being the last 5 x K).
One JSON line is printed: ``value`` = decoded tokens per second timed on the device over K
steps of a decode session (the loop ``LLM.generate`` runs: one CUDA graph a step, sampling and
the next token kept on the device), median of 5 such regions back to back; ``e2e`` = the same
steps from the same prompts through the Python entry point (``LLM.generate``), host tokens in
and out, and its greedy tokens must equal the timed run's;
``prefill`` = one 2,048-token prompt step (median of 5, timed before the decode runs and again after them: the
faster of the two, with both times beside it); ``points`` = decoding at batch 1 and 64; ``roofline`` =
bytes a decode step has to read (every weight once, the cache of the live sequences) over
its time, against the measured copy bandwidth; ``further`` = short runs at contexts 8,192 and 16,384 and at
the 8B and 32B shapes (all their layers), made after everything else.  Inputs are larger than L2 (a step streams
all weights, ~8 GB), so L2 is not flushed between steps.
"""
import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-4B shape (the benchmark configuration): every size named here goes into "config"
QWEN3_4B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=2560,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960,
    hidden_act="silu", attention_bias=False, use_sliding_window=False)
# the other shapes the measurement targets name (--shape); the default run is the 4B shape
SHAPES = {
    "4b": QWEN3_4B,
    "0.6b": dict(QWEN3_4B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, intermediate_size=3072),
    "1.7b": dict(QWEN3_4B, num_hidden_layers=28, hidden_size=2048, num_attention_heads=16, intermediate_size=6144),
    "8b": dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False),
    "14b": dict(QWEN3_4B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408,
                tie_word_embeddings=False),
    "32b": dict(QWEN3_4B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600,
                tie_word_embeddings=False),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)):
                    out[k] = float(d[k])
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None
        self.first = 0

    def mark(self):
        """The timed region begins: only what is sampled from here on counts.  (The sampler is started before the
        untimed steps, because nvidia-smi's own start-up can hold the GPU up for tens of milliseconds.)"""
        self.first = len(self.rows)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in (self.rows[self.first:] or self.rows):
            try:
                mhz.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def decode_bytes(cfg, layers, batch, mean_context):
    """Bytes one decode step has to read: every matrix once, the embedding rows of the batch,
    and the keys and values of the live sequences (bfloat16)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((nh + 2 * nkv) * hd * H + nh * hd * H + 3 * I * H + 2 * H + 2 * hd) * 2
    head = V * H * 2
    kv = 2 * nkv * hd * 2 * layers * mean_context * batch
    return layers * per_layer + head + batch * H * 2 + kv


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    mat = ((nh + 2 * nkv) * hd * H + nh * hd * H + 3 * I * H) * 2 * T
    att = 2 * 2 * nh * hd * T * (T + 1) / 2
    return layers * (mat + att) + 2 * V * H


def further_points(torch, pk, graph):
    """Decoding and the prompt step at further sizes, one short run each: the 4B shape at contexts 8,192 and 16,384
    (batch 1 and 8), and the 8B and 32B shapes at context 4,096 (batch 8, all their layers).  Flat: name -> number;
    ``*_hbm_frac`` is the decode step's bytes over its time over the copy bandwidth, ``*_prefill_frac`` the
    2,048-token prompt step's flops over its time over the burst peak."""
    from synaptix_b200.api import LLM
    from synaptix_b200.config import Qwen3Config
    from synaptix_b200.engine import DecodeRow, Entry
    from synaptix_b200.models import model_skeleton
    from synaptix_b200.parts import Runtime
    from synaptix_b200.weights import RandomSource
    out = {}
    K, REGIONS, TOTAL = 20, 5, 255
    g = torch.Generator().manual_seed(2)

    def decode(llm, cfg, cfgd, B, context, key):
        engine = llm.engine
        prompts = [torch.randint(0, cfg.vocab_size, (context - TOTAL - 1,), generator=g).tolist() for _ in range(B)]
        slots = [engine.open() for _ in prompts]
        first = []
        for i in range(0, B, 4):
            lg = engine.step([Entry(s, p, [len(p) - 1]) for s, p in zip(slots[i:i + 4], prompts[i:i + 4])], keep=False)
            first += lg.argmax(-1).tolist()
        session = engine.start_decode([DecodeRow(s, t, i, 1) for i, (s, t) in enumerate(zip(slots, first))])
        events = [torch.cuda.Event(enable_timing=True) for _ in range(REGIONS + 1)]
        for _ in range(TOTAL - REGIONS * K):
            session.launch()
        events[0].record()
        for r in range(REGIONS):
            for _ in range(K):
                session.launch()
            events[r + 1].record()
        torch.cuda.synchronize()
        ms = sorted(events[r].elapsed_time(events[r + 1]) for r in range(REGIONS))[REGIONS // 2] / K
        for _ in range(TOTAL):
            session.collect()
        session.drop(list(range(B)))
        for s in slots:
            engine.close(s)
        nbytes = decode_bytes(cfgd, cfgd["num_hidden_layers"], B, context - REGIONS * K / 2.0)
        out[key] = round(B / (ms / 1e3), 1)
        out[key + "_hbm_frac"] = round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def prefill(llm, cfg, cfgd, key):
        engine, T = llm.engine, 2048
        toks = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        times = []
        for it in range(3 + 5):
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            engine.step([Entry(s, toks, [T - 1])], keep=False)
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        ms = sorted(times)[len(times) // 2]
        out[key + "_ms"] = round(ms, 2)
        out[key + "_frac"] = round(prefill_flops(cfgd, cfgd["num_hidden_layers"], T) / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 4)

    for shape_name, runs in (("4b", [(8192, 1), (8192, 8), (16384, 1), (16384, 8)]), ("8b", [(4096, 8)]), ("32b", [(4096, 8)])):
        cfgd = dict(SHAPES[shape_name])
        cfg = Qwen3Config.from_dict(cfgd)
        model = model_skeleton(cfg)
        src = RandomSource(model.all_tensor_specs(), seed=0, std_matrix=0.02, std_gain=0.05, device="cuda:0")
        model.load(src, Runtime(torch.device("cuda:0"), torch.bfloat16), where="random weights")
        llm = LLM.from_model(model, max_tokens=max(B * (c + 64) for c, B in runs), graph=graph)
        if shape_name != "4b":
            prefill(llm, cfg, cfgd, f"qwen3_{shape_name}_prefill_2048")
        for context, B in runs:
            decode(llm, cfg, cfgd, B, context, f"qwen3_{shape_name}_ctx{context}_decode_b{B}")
        del llm, model, src
        gc.collect()                             # engines and models hold reference cycles
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--shape", default="4b", choices=sorted(SHAPES), help="layer sizes: Qwen3-4B (the default) or another size of the family")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch-1/64 points, the prefill and the e2e run")
    ap.add_argument("--phase", default="all", choices=["all", "prefill"],
                    help="prefill: time only the 2,048-token prompt step (small cases for profilers)")
    ap.add_argument("--no-graph", action="store_true", help="run decode steps eagerly instead of replaying CUDA graphs")
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="length of the timed prompt step (the line's figure is for 2,048)")
    ap.add_argument("--further-only", action="store_true", help="only the short runs at further sizes, as a JSON object")
    ap.add_argument("--no-further", action="store_true",
                    help="skip the short runs at further contexts and at the 8B and 32B shapes (the default run of the 4B shape makes them)")
    ap.add_argument("--short", action="store_true",
                    help="decode only 5 x --steps + --warmup tokens instead of at least 255 (small cases for profilers: "
                         "every launch under a profiler costs a good part of a second)")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "VitaminDB/synaptix is a Rust workspace (no Python package, no Rust toolchain offline) whose "
                          "kernels are NVRTC sources for sm_80/sm_120a with no sm_100 path; it cannot be installed or run here"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures one GPU: this library runs on a single B200 (asked for --gpus {a.gpus})")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    if a.further_only:
        try:
            print(json.dumps(further_points(torch, peaks(), not a.no_graph)))
        except Exception as e:                   # noqa: BLE001 - reported in the caller's line
            print(json.dumps({"error": f"{type(e).__name__}: {e}"[:300]}))
        return 0
    from synaptix_b200.api import LLM
    from synaptix_b200.config import Qwen3Config
    from synaptix_b200.engine import DecodeRow, Entry
    from synaptix_b200.models import model_skeleton
    from synaptix_b200.parts import Runtime
    from synaptix_b200.weights import RandomSource

    shape = SHAPES[a.shape]
    full_layers = shape["num_hidden_layers"]
    name = f"Qwen3-{a.shape.upper()} shape"
    if a.layers is None:
        a.layers = full_layers
    cfgd = dict(shape, num_hidden_layers=a.layers)
    cfg = Qwen3Config.from_dict(cfgd)
    dev = torch.device("cuda:0")
    model = model_skeleton(cfg)
    src = RandomSource(model.all_tensor_specs(), seed=0, std_matrix=0.02, std_gain=0.05, device="cuda:0")
    model.load(src, Runtime(dev, torch.bfloat16), where="random weights")
    pk = peaks()

    batches = [a.batch] if a.no_points else sorted({a.batch, 1, 64})
    K, W = a.steps, a.warmup
    # Every sequence decodes at least 255 tokens, the timed steps (5 regions of K) being the last ones, which end at
    # the context length.  A generation that short would be mostly the GPU coming back from the prompt step: the
    # first 15 to 20 single-token steps after a long prompt step run about a quarter slower (measured; the SM clock
    # is still low from the power cap of the prompt step's products), and the end-to-end figure below has them all.
    total_steps = 5 * K + W if a.short else max(5 * K + W, 255)
    start_len = a.context - total_steps - 1
    if start_len < 1:
        raise SystemExit("--context is too short for 5 x --steps + --warmup")
    llm = LLM.from_model(model, max_tokens=max(max(batches) * (a.context + 64), a.prefill_tokens + 64) if a.phase == "all" else a.prefill_tokens + 2048,
                         graph=not a.no_graph)
    engine = llm.engine
    g = torch.Generator().manual_seed(1)

    def time_prefill():
        """Median time of a 2,048-token prompt step of one sequence, a fresh slot each time."""
        T = a.prefill_tokens
        toks = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
        times = []
        for it in range(3 + 5):
            s = engine.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            engine.step([Entry(s, toks, [T - 1])], keep=False)
            e1.record()
            torch.cuda.synchronize()
            engine.close(s)
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        pms = sorted(times)[len(times) // 2]
        fl = prefill_flops(cfgd, a.layers, T)
        return {"value": round(T / (pms / 1e3), 1), "tokens": T, "ms": round(pms, 3),
                "frac": round(fl / (pms / 1e3) / 1e12 / pk["bf16_tflops"], 4), "of": pk["source"],
                "tflops": round(fl / (pms / 1e3) / 1e12, 1)}

    if a.phase == "prefill":
        print(json.dumps({"metric": f"prefill tok/s at {a.prefill_tokens:,} tokens ({name}, bf16, random weights)", "impl": "ours",
                          "layers": a.layers, "layers_of_config": full_layers, "prefill": time_prefill()}))
        return 0

    REGIONS = 5                                   # the K-step region is timed this many times, back to back
    settle = total_steps - REGIONS * K            # untimed steps before them (at least the W warm-up steps)

    def prompts_for(B):
        return [torch.randint(0, cfg.vocab_size, (start_len,), generator=g).tolist() for _ in range(B)]

    def fill(prompts, whole):
        """Open a slot per prompt and run the prompts: all in one step as ``LLM.generate`` does (``whole``), or a
        few sequences a step."""
        slots = [engine.open() for _ in prompts]
        first = []
        per = len(prompts) if whole else 4
        for i in range(0, len(prompts), per):
            lg = engine.step([Entry(s, p, [len(p) - 1]) for s, p in zip(slots[i:i + per], prompts[i:i + per])], keep=False)
            first += lg.argmax(-1).tolist()
        return slots, first

    # The prompt step is timed twice, before the decode runs and after them (medians of 5): which of the two states of
    # the GPU is the faster differs from run to run (clocks under the power cap, what ran before this process), so the
    # line carries both and ``prefill.value`` is the faster one.
    prefill_first = None if a.no_points else time_prefill()
    results = {}
    clocks = None
    launches = 0
    device_tokens = main_prompts = None
    for B in batches:
        prompts = prompts_for(B)
        slots, first = fill(prompts, whole=(B == a.batch))
        session = engine.start_decode([DecodeRow(s, t, i, 1) for i, (s, t) in enumerate(zip(slots, first))])
        events = [torch.cuda.Event(enable_timing=True) for _ in range(REGIONS + 1)]
        with ClockSampler() as cs:
            for _ in range(settle):
                session.launch()
            torch.cuda.synchronize()
            l0 = engine.kernel_launches
            cs.mark()
            events[0].record()
            for r in range(REGIONS):
                for _ in range(K):
                    session.launch()
                events[r + 1].record()
            torch.cuda.synchronize()
        region_ms = sorted(events[r].elapsed_time(events[r + 1]) for r in range(REGIONS))
        ms = region_ms[REGIONS // 2]
        results[B] = {"ms_per_step": ms / K, "tok_s": B * K / (ms / 1e3), "best_tok_s": B * K / (region_ms[0] / 1e3),
                      "region_ms": [round(events[r].elapsed_time(events[r + 1]), 3) for r in range(REGIONS)]}
        toks = [session.collect() for _ in range(total_steps)]
        if B == a.batch:
            clocks = cs.summary()
            launches = (engine.kernel_launches - l0) // REGIONS
            device_tokens = [[first[i]] + [t[i] for t in toks] for i in range(B)]
            main_prompts = prompts
        session.drop(list(range(B)))
        for s in slots:
            engine.close(s)

    main_r = results[a.batch]
    mean_ctx = a.context - REGIONS * K / 2.0
    nbytes = decode_bytes(cfgd, a.layers, a.batch, mean_ctx)
    achieved = nbytes / (main_r["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s ({name}, bf16, random weights)", "value": round(main_r["tok_s"], 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(main_r["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": f"{name}, random weights", "global_batch": a.batch, "seq_len": a.context,
                   "parallelism": "1 GPU", "layers": a.layers, "layers_of_config": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "tied_head": bool(shape["tie_word_embeddings"]),
                   "prefill_tokens": a.prefill_tokens, "l2": "inputs larger than L2 (a step streams all weights, 8 GB or more)"},
        "gpu_launches": launches,
        "clocks": clocks,
        "timing": {"regions": REGIONS, "steps_per_region": K, "value_is": "median region",
                   "best": round(main_r["best_tok_s"], 2), "region_ms": main_r["region_ms"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"], "bytes_per_step": int(nbytes)},
    }

    if not a.no_points:
        line["points"] = {f"decode_b{B}": round(r["tok_s"], 2) for B, r in results.items() if B != a.batch}
        line["points"][f"decode_b{a.batch}"] = round(main_r["tok_s"], 2)
        line["points_hbm_frac"] = {
            f"decode_b{B}": round(decode_bytes(cfgd, a.layers, B, mean_ctx) / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            for B, r in results.items()}
        prefill_after = time_prefill()
        line["prefill"] = dict(min(prefill_first, prefill_after, key=lambda r: r["ms"]))
        line["prefill"]["ms_before_decoding"] = prefill_first["ms"]
        line["prefill"]["ms_after_decoding"] = prefill_after["ms"]
        # end to end through the Python entry point, from the same prompts: host tokens in, every step's control
        # words up from pinned memory and its tokens back down; greedy, so the tokens must be the timed run's
        llm.generate(main_prompts[:1], max_new_tokens=W + 1, eos_token_ids=[])
        llm.generate(main_prompts, max_new_tokens=W + 1, eos_token_ids=[], max_batch_size=a.batch)
        runs = []
        same = True
        for _ in range(3):                       # the whole generation three times; the median run is reported
            outs = llm.generate(main_prompts, max_new_tokens=total_steps + 1, eos_token_ids=[], max_batch_size=a.batch)
            runs.append(llm.last_stats)
            same = same and outs == device_tokens
        runs.sort(key=lambda st: st.decode_ms / max(st.decode_steps, 1))
        st = runs[1]
        line["e2e"] = {"value": round(a.batch * st.decode_steps / (st.decode_ms / 1e3), 2), "unit": "tokens/s",
                       "h2d_bytes_per_step": st.decode_h2d_bytes // max(st.decode_steps, 1),
                       "d2h_bytes_per_step": st.decode_d2h_bytes // max(st.decode_steps, 1),
                       "steps": st.decode_steps, "runs": 3, "value_is": "median run",
                       "best": round(a.batch * runs[0].decode_steps / (runs[0].decode_ms / 1e3), 2),
                       "tokens_equal_device_timed_run": same}
        if not same:
            bad = next(i for i in range(a.batch) if outs[i] != device_tokens[i])
            k = next(k for k, (x, y) in enumerate(zip(outs[bad], device_tokens[bad])) if x != y)
            print(json.dumps(line))
            raise SystemExit(f"LLM.generate and the device-timed decode run disagree: request {bad}, token {k}: "
                             f"{outs[bad][k]} against {device_tokens[bad][k]}")
    if not a.no_points and not a.no_further and a.shape == "4b" and a.layers == full_layers:
        # After everything the line's other figures need, and in a process of its own with a time limit: a failure
        # there costs these figures alone.
        del session, llm, engine, model, src
        gc.collect()
        torch.cuda.empty_cache()
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--further-only"] + (["--no-graph"] if a.no_graph else []),
                               capture_output=True, text=True, timeout=240)
            line["further"] = json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 and r.stdout.strip() else \
                {"error": f"exit code {r.returncode}: {r.stderr.strip()[-200:]}"}
        except Exception as e:                   # noqa: BLE001 - the line above is measured and is printed whatever happens here
            line["further"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
