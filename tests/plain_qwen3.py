"""A plain, slow implementation of the Qwen3 dense decoder and of the samplers: the oracle.

Whole sequences, no cache, float32 on the CPU, one function for each part, written from the
reference's formulas (each function cites the file and lines; paths are relative to the
reference project's root).  It shares no code with ``synaptix_b200``: it reads the model
folder with ``json`` and the ``safetensors`` package and computes with plain torch tensor
arithmetic.

The reference's own model code is Rust and cannot be compiled or imported where these
tests run (no Rust toolchain), so this file rests on the formulas; the reference's
op-level PyTorch generators (scripts/reference/gen_*.py) state the same formulas and are
compared once in tests/golden/.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch
from safetensors import safe_open


# ----------------------------------------------------------------------------------------
# model folder
# ----------------------------------------------------------------------------------------
def load_folder(model_dir: str):
    """config.json as a dict and every tensor of model.safetensors widened to float32."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), "pt") as f:
        for k in f.keys():
            W[k] = f.get_tensor(k).to(torch.float32)
    return cfg, W


def head_dim_of(cfg) -> int:
    hd = cfg.get("head_dim")
    return hd if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer: int) -> Optional[int]:
    """None = every earlier key.  The reference forces full attention for Qwen3
    (crates/synaptix-models/llm/qwen3/src/config.rs:117-118); a window applies only when
    config.json switches it on with use_sliding_window, per layer by layer_types or
    max_window_layers."""
    if not cfg.get("use_sliding_window", False):
        return None
    lt = cfg.get("layer_types")
    if lt is not None:
        return cfg["sliding_window"] if lt[layer] == "sliding_attention" else None
    mwl = cfg.get("max_window_layers")
    first = cfg["num_hidden_layers"] if mwl is None else mwl
    return cfg["sliding_window"] if layer >= first else None


# ----------------------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------------------
def embedding(E: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h0[t] = E[id_t], no scale (crates/synaptix-ops/src/embed/token_embed.rs:4-15)."""
    return E[torch.tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """v = mean(x^2) over the last dim; out = x / sqrt(v + eps) * w, plain gain w
    (crates/synaptix-ops/src/norm/rms_norm.rs:17-26; qwen3/src/config.rs:100)."""
    v = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(v + eps)) * w


def rotary_freqs(theta: float, head_dim: int) -> torch.Tensor:
    """f_i = theta^(-(2 i)/head_dim), i < head_dim/2, in float32
    (crates/synaptix-ops/src/pos/rope_cache.rs:21-26)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    exponent = -(np.float32(2.0) * i) / np.float32(head_dim)
    return torch.from_numpy(np.power(np.float32(theta), exponent).astype(np.float32))


def rope_rotate_half(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x [T, n, d]; angle = position * f_i (float32); for i < d/2:
    o[i] = x[i] cos - x[i+d/2] sin, o[i+d/2] = x[i] sin + x[i+d/2] cos
    (crates/synaptix-ops/src/pos/rope_cache.rs:27-35; crates/synaptix-ops/src/pos/rope.rs:84-100)."""
    half = x.shape[-1] // 2
    ang = positions.to(torch.float32)[:, None] * freqs[None, :]        # [T, d/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                         window: Optional[int] = None) -> torch.Tensor:
    """q [T, nh, d], k and v [T, nkv, d] of ONE whole sequence.  s[i,j] = q_i . k_j * scale;
    key j visible to query i iff j <= i (and j > i - window); softmax with the maximum
    subtracted; o_i = sum_j P_ij v_j; query head h reads kv head h // (nh / nkv)
    (crates/synaptix-ops/src/attention/softmax/scaled_dot.rs:7-37;
    crates/synaptix-models/llm/common/src/model.rs:2569-2602;
    crates/synaptix-kernels-cuda/src/cu/fused/attention/flash_decode.cu:108-110)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    for h in range(nh):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        s = s - s.max(dim=-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """g = x Wg^T, u = x Wu^T, z = silu(g) * u with silu(a) = a / (1 + exp(-a)), out = z Wd^T
    (crates/synaptix-models/llm/common/src/model.rs:1670-1691;
    crates/synaptix-kernels-cuda/src/cu/fused/mlp/silu_and_mul.cu:11-25)."""
    g = x @ wg.T
    u = x @ wu.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ wd.T


def attention_layer(x: torch.Tensor, W, p: str, cfg, positions: torch.Tensor,
                    window: Optional[int]) -> torch.Tensor:
    """Projections without bias -> per-head RMSNorm of q and k -> rotation -> attention -> Wo
    (crates/synaptix-models/llm/common/src/model.rs:1715-1734,1872-1878)."""
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    T = x.shape[0]
    q = (x @ W[p + "q_proj.weight"].T).view(T, nh, d)
    k = (x @ W[p + "k_proj.weight"].T).view(T, nkv, d)
    v = (x @ W[p + "v_proj.weight"].T).view(T, nkv, d)
    q = rms_norm(q, W[p + "q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, W[p + "k_norm.weight"], cfg["rms_norm_eps"])
    f = rotary_freqs(rope_theta_of(cfg), d)
    q = rope_rotate_half(q, positions, f)
    k = rope_rotate_half(k, positions, f)
    o = causal_gqa_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return o.reshape(T, nh * d) @ W[p + "o_proj.weight"].T


def rope_theta_of(cfg) -> float:
    if cfg.get("rope_theta") is not None:
        return cfg["rope_theta"]
    return cfg["rope_parameters"]["rope_theta"]


def block(h: torch.Tensor, W, layer: int, cfg, positions: torch.Tensor) -> torch.Tensor:
    """r = h; h = r + Attn(RMS(h, w_in)); r2 = h; h = r2 + MLP(RMS(h, w_post))
    (crates/synaptix-models/llm/common/src/model.rs:1179-1199)."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    a = attention_layer(rms_norm(h, W[p + "input_layernorm.weight"], eps), W, p + "self_attn.", cfg,
                        positions, layer_window(cfg, layer))
    h = h + a
    m = swiglu(rms_norm(h, W[p + "post_attention_layernorm.weight"], eps),
               W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    return h + m


def hidden_states(cfg, W, tokens: Sequence[int]) -> torch.Tensor:
    """The residual stream [T, width] after the last block of one whole sequence: embedding -> blocks
    (crates/synaptix-models/llm/common/src/model.rs:1057-1066)."""
    with torch.no_grad():
        h = embedding(W["model.embed_tokens.weight"], tokens)
        positions = torch.arange(len(tokens))
        for layer in range(cfg["num_hidden_layers"]):
            h = block(h, W, layer, cfg, positions)
        return h


def logits_of(cfg, W, h: torch.Tensor) -> torch.Tensor:
    """Final norm -> output head on the rows of ``h`` (the head is tied to the embedding unless
    lm_head.weight is there and tie_word_embeddings is not true)
    (crates/synaptix-models/llm/common/src/model.rs:757-772, 1068-1117)."""
    with torch.no_grad():
        n = rms_norm(h, W["model.norm.weight"], cfg["rms_norm_eps"])
        tied = cfg.get("tie_word_embeddings")
        if tied is None:
            tied = "lm_head.weight" not in W
        head = W["model.embed_tokens.weight"] if tied else W["lm_head.weight"]
        return n @ head.T


def forward(cfg, W, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence."""
    return logits_of(cfg, W, hidden_states(cfg, W, tokens))


# ----------------------------------------------------------------------------------------
# sampling (host-side, as the reference does it)
# ----------------------------------------------------------------------------------------
def greedy(logits: torch.Tensor) -> int:
    """argmax; among equal maxima the last index, as Rust's max_by returns
    (crates/synaptix-infer/src/sampling/greedy.rs:8-12)."""
    v = logits.to(torch.float32).numpy()
    m = v.max()
    return int(np.nonzero(v == m)[0][-1])


def greedy_generate(cfg, W, prompt: Sequence[int], max_new_tokens: int,
                    stop_ids: Sequence[int] = ()) -> List[int]:
    """Whole-sequence recomputation at every step; stops after emitting a stop token, which is
    part of the output (crates/synaptix-models/llm/common/src/generate.rs:275-292)."""
    seq = list(prompt)
    out: List[int] = []
    while len(out) < max_new_tokens:
        if out and out[-1] in stop_ids:
            break
        t = greedy(forward(cfg, W, seq)[-1])
        out.append(t)
        seq.append(t)
    return out


_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox4x32(counter, key):
    """Philox4x32-10 block (crates/synaptix-ops/src/rng.rs:82-97)."""
    c = list(counter)
    k = list(key)
    for _ in range(10):
        p0 = _M0 * c[0]
        p1 = _M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + _W0) & 0xFFFFFFFF, (k[1] + _W1) & 0xFFFFFFFF]
    return c


def philox_u32(seed: int, step: int, seq_index: int = 0) -> int:
    """Word number `step` of the stream with key (seed lo, seed hi): block step // 4 with counter
    (block, seq_index, 0, 0), word step % 4.  seq_index 0 is the reference's single stream
    (crates/synaptix-ops/src/rng.rs:16-25,58-66)."""
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return philox4x32((step // 4, seq_index, 0, 0), key)[step % 4]


def uniform_from_u32(word: int) -> np.float32:
    """u = (word as f64 as f32) / (u32::MAX as f32) (crates/synaptix-infer/src/sampling/multinomial.rs:30-32)."""
    return np.float32(np.float32(np.float64(word)) / np.float32(4294967295))


def apply_repetition(logits: np.ndarray, ids: Sequence[int], penalty: float, last_n: int) -> None:
    """Once per occurrence in the window: logit > 0 ? /= p : *= p
    (crates/synaptix-infer/src/sampling/repetition.rs:7-41)."""
    ids = list(ids)
    win = ids if last_n == 0 or last_n >= len(ids) else ids[len(ids) - last_n:]
    for t in win:
        if t < len(logits):
            logits[t] = logits[t] / np.float32(penalty) if logits[t] > 0 else logits[t] * np.float32(penalty)


def apply_presence_frequency(logits: np.ndarray, ids: Sequence[int], presence: float, frequency: float,
                             last_n: int) -> None:
    """logit -= presence + frequency * count, once per distinct token of the window
    (crates/synaptix-infer/src/sampling/repetition.rs:43-77)."""
    ids = list(ids)
    win = ids if last_n == 0 or last_n >= len(ids) else ids[len(ids) - last_n:]
    counts: Dict[int, int] = {}
    for t in win:
        counts[t] = counts.get(t, 0) + 1
    for t, c in counts.items():
        if t < len(logits):
            logits[t] -= np.float32(presence) + np.float32(frequency) * np.float32(c)


def filter_top_k(logits: np.ndarray, k: int) -> None:
    """Keep the k largest, the rest -> -inf (crates/synaptix-infer/src/sampling/top_k.rs:8-24)."""
    if k == 0 or k >= len(logits):
        return
    order = np.argsort(-logits, kind="stable")
    logits[order[k:]] = -np.inf


def filter_top_p(logits: np.ndarray, p: float) -> None:
    """exp(x - max), sorted descending; cut at the first place where the sum BEFORE it exceeds
    p * total (crates/synaptix-infer/src/sampling/top_p.rs:8-44)."""
    if p >= 1.0:
        return
    mx = logits.max()
    probs = np.exp(logits - mx).astype(np.float32)
    total = probs.sum(dtype=np.float32)
    idx = [i for i in range(len(logits)) if np.isfinite(logits[i])]
    idx.sort(key=lambda i: -probs[i])
    thresh = np.float32(p) * total
    cum = np.float32(0)
    cutoff = len(idx)
    for pos, i in enumerate(idx):
        if cum > thresh:
            cutoff = pos
            break
        cum += probs[i]
    for i in idx[cutoff:]:
        logits[i] = -np.inf


def filter_min_p(logits: np.ndarray, min_p: float) -> None:
    """Drop prob < min_p * max prob (crates/synaptix-infer/src/sampling/min_p.rs:8-24)."""
    mx = logits.max()
    e = np.exp(logits - mx).astype(np.float32)
    probs = e / e.sum(dtype=np.float32)
    logits[probs < np.float32(min_p) * probs.max()] = -np.inf


def processed_logits(logits, context: Sequence[int] = (), temperature: float = 0.0, top_k: int = 0,
                     top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0,
                     repeat_last_n: int = 0, presence_penalty: float = 0.0,
                     frequency_penalty: float = 0.0) -> np.ndarray:
    """The processor chain in the reference's order
    (crates/synaptix-models/llm/common/src/generate.rs:304-332)."""
    v = np.array(logits, dtype=np.float32)
    if repetition_penalty != 1.0:
        apply_repetition(v, context, repetition_penalty, repeat_last_n)
    if presence_penalty != 0.0 or frequency_penalty != 0.0:
        apply_presence_frequency(v, context, presence_penalty, frequency_penalty, repeat_last_n)
    if temperature > 0.0 and temperature != 1.0:
        v = v / np.float32(temperature)
    if top_k > 0:
        filter_top_k(v, top_k)
    if top_p < 1.0:
        filter_top_p(v, top_p)
    if min_p > 0.0:
        filter_min_p(v, min_p)
    return v


def multinomial_intervals(v: np.ndarray):
    """Cumulative probabilities (float64) of softmax(v): token i is drawn when
    cum[i-1] <= u < cum[i] (crates/synaptix-infer/src/sampling/multinomial.rs:8-28)."""
    e = np.exp(v.astype(np.float64) - np.max(v))
    p = e / e.sum()
    return np.cumsum(p)


def multinomial(v: np.ndarray, u: float) -> int:
    probs = np.exp(v - v.max()).astype(np.float32)
    probs = probs / probs.sum(dtype=np.float32)
    cum = np.float32(0)
    for i, p in enumerate(probs):
        cum += p
        if u < cum:
            return i
    return len(probs) - 1
