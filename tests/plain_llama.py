"""A plain, slow implementation of the Llama-style decoder, written from the reference's formulas.

It rests on the formulas of artalis-io/bitnet.c's CPU path (each function cites file:line) and is
compared once with that code itself: ``tests/golden/`` holds logits that the reference's own
compiled CPU engine produced on two tiny random models, and ``tests/test_plain_vs_golden.py``
checks this file against them.

Whole sequences, no cache, no batching, one function per part, NumPy only.  It shares no code
with the library under test.  Arithmetic is float64 except where the reference fixes float32
(the rotation angles); that makes it the more exact of the two, and the tolerances of the tests
are those of float32 rounding in the engine.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# ---- reading a model folder (own reader: the library's loader is not used here) ----------------
def read_safetensors(path: str, keep=np.float64) -> Dict[str, np.ndarray]:
    """Every tensor of the file as ``keep`` (float64; float32 for models of real layer sizes,
    whose products are then taken row block by row block in float64, see ``linear``)."""
    out: Dict[str, np.ndarray] = {}
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = np.frombuffer(data, dtype=np.uint8, count=e - b, offset=b)
        dt = info["dtype"]
        if dt == "F32":
            a = raw.view(np.float32).astype(keep)
        elif dt == "BF16":
            a = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).astype(keep)
        elif dt == "F16":
            a = raw.view(np.float16).astype(keep)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(info["shape"])
    return out


def read_model(folder: str, keep=np.float64):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"), keep)


def linear(h: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = h W^T with W [out, in] row-major, float64 products and sums (src/quant/f32_scalar.c:4-32).
    A matrix kept in float32 is widened 8,192 rows at a time, so that no float64 copy of it exists."""
    if w.dtype == np.float64:
        return h @ w.T
    out = np.empty((h.shape[0], w.shape[0]), dtype=np.float64)
    for r in range(0, w.shape[0], 8192):
        out[:, r:r + 8192] = h @ w[r:r + 8192].astype(np.float64).T
    return out


def to_bf16(a: np.ndarray) -> np.ndarray:
    """Round to bfloat16 (nearest even) and return as float64."""
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).astype(np.float64)


# ---- parts --------------------------------------------------------------------------------------
def embed(tokens: Sequence[int], table: np.ndarray) -> np.ndarray:
    """x = float(E[token, :]), no scale for this architecture (src/model_embed.c:6-28)."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(np.float64)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """scale = 1/sqrt(mean(x^2) + eps); out = x * scale * w (src/transformer/rmsnorm_scalar.c:4-13)."""
    ss = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ss + eps)) * w


def rope_angles(pos: int, dims: int, theta: float) -> np.ndarray:
    """angle_0 = pos, angle_{i+1} = angle_i * powf(theta, -2/dims), all float32
    (src/model_arch.c:322-338)."""
    half = dims // 2
    scale = np.power(np.float32(theta), np.float32(-2.0) / np.float32(dims)).astype(np.float32)
    out = np.empty(half, dtype=np.float32)
    a = np.float32(pos)
    for i in range(half):
        out[i] = a
        a = np.float32(a * scale)
    return out


def apply_rope(x: np.ndarray, positions: Sequence[int], theta: float, dims: Optional[int] = None) -> np.ndarray:
    """x: [T, heads, head_dim].  Pairs (i, i + half): x_i = a cos - b sin, x_{i+half} = a sin + b cos
    with cosf/sinf of the float32 angle (src/transformer/cpu_backend.c:283-296, src/transformer.c:143-162)."""
    T, _, hd = x.shape
    dims = dims or hd
    half = dims // 2
    out = x.copy()
    for t in range(T):
        ang = rope_angles(int(positions[t]), dims, theta)
        c = np.cos(ang).astype(np.float64)
        s = np.sin(ang).astype(np.float64)
        a, b = x[t, :, :half], x[t, :, half:dims]
        out[t, :, :half] = a * c - b * s
        out[t, :, half:dims] = a * s + b * c
    return out


def softmax(s: np.ndarray) -> np.ndarray:
    """max-subtracted softmax (src/transformer/math_scalar.c:33-68)."""
    e = np.exp(s - np.max(s))
    return e / np.sum(e)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int = 0) -> np.ndarray:
    """q: [T, H, hd], k, v: [T, KV, hd] of one whole sequence, already rotated.  Query head h uses
    key/value head h // (H // KV); token t sees keys 0..t (the last ``window`` of them if window > 0);
    scores = q.k * scale, softmax, weighted sum of values (src/transformer/gqa_scalar.c:61-121,
    src/transformer/batched_attn_scalar.c:97-169)."""
    T, H, hd = q.shape
    KV = k.shape[1]
    mul = H // KV
    out = np.zeros_like(q)
    for t in range(T):
        lo = max(0, t - window + 1) if window > 0 else 0
        for h in range(H):
            kvh = h // mul
            s = (k[lo:t + 1, kvh] @ q[t, h]) * scale
            p = softmax(s)
            out[t, h] = p @ v[lo:t + 1, kvh]
    return out


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def swiglu(h: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray) -> np.ndarray:
    """y = W_down (silu(W_gate h) * (W_up h)) (src/transformer/cpu.c:1247-1303)."""
    return linear(silu(linear(h, w_gate)) * linear(h, w_up), w_down)


def attention_block(h, w, prefix, cfg, positions, round_fn=None):
    """q, k, v projections, rotary on q and k, causal attention, output projection
    (src/transformer/cpu.c:859-939)."""
    H = cfg["num_attention_heads"]
    KV = cfg.get("num_key_value_heads") or H
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    r = round_fn or (lambda a: a)
    T = h.shape[0]
    q = r(linear(h, w[prefix + "self_attn.q_proj.weight"])).reshape(T, H, hd)
    k = r(linear(h, w[prefix + "self_attn.k_proj.weight"])).reshape(T, KV, hd)
    v = r(linear(h, w[prefix + "self_attn.v_proj.weight"])).reshape(T, KV, hd)
    theta = float(cfg.get("rope_theta") or 10000.0)
    q, k = r(apply_rope(q, positions, theta)), r(apply_rope(k, positions, theta))
    a = r(attention(q, k, v, hd ** -0.5, int(cfg.get("sliding_window") or 0))).reshape(T, H * hd)
    return r(linear(a, w[prefix + "self_attn.o_proj.weight"]))


def forward(cfg: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], round_fn=None) -> np.ndarray:
    """Logits [T, vocab] at every position of one whole sequence (order of operations:
    src/transformer/cpu.c:491-987, final norm and head: src/transformer/logits.c:236-323).

    ``round_fn`` rounds the tensors that the bfloat16 engine stores in bfloat16 (products'
    outputs and normed activations); the residual stream stays unrounded as it does there.
    """
    r = round_fn or (lambda a: a)
    eps = float(cfg.get("rms_norm_eps") or 1e-5)
    T = len(tokens)
    positions = list(range(T))
    x = embed(tokens, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = r(rmsnorm(x, w[p + "input_layernorm.weight"], eps))
        x = x + attention_block(h, w, p, cfg, positions, round_fn)
        h = r(rmsnorm(x, w[p + "post_attention_layernorm.weight"], eps))
        gu_g, gu_u = r(linear(h, w[p + "mlp.gate_proj.weight"])), r(linear(h, w[p + "mlp.up_proj.weight"]))
        x = x + r(linear(r(silu(gu_g) * gu_u), w[p + "mlp.down_proj.weight"]))
    h = r(rmsnorm(x, w["model.norm.weight"], eps))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(h, head)


# ---- sampling (src/sampler.c) ---------------------------------------------------------------------
MASK64 = (1 << 64) - 1


class Xorshift64Star:
    """src/sampler.c:6-15; seed 0 becomes 42 (src/sampler.c:22)."""

    def __init__(self, seed: int):
        self.state = (seed or 42) & MASK64

    def next_u32(self) -> int:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & MASK64
        s ^= s >> 27
        self.state = s
        return ((s * 0x2545F4914F6CDD1D) & MASK64) >> 32

    def next_float(self) -> np.float32:
        return np.float32(self.next_u32() >> 8) / np.float32(16777216.0)


def apply_repeat_penalty(logits: np.ndarray, recent: Sequence[int], penalty: float) -> np.ndarray:
    """Each distinct recent id once: logit > 0 ? logit / p : logit * p (src/sampler.c:139-157)."""
    out = logits.copy()
    for tok in dict.fromkeys(recent):
        if 0 <= tok < len(out):
            out[tok] = out[tok] / penalty if out[tok] > 0 else out[tok] * penalty
    return out


def argmax_first(logits: np.ndarray) -> int:
    """First maximum wins (src/sampler_backend.c:129-135)."""
    return int(np.argmax(logits))


def sample(logits: np.ndarray, temperature: float, topp: float, rng: Xorshift64Star) -> int:
    """src/sampler.c:159-173: temperature 0 is argmax; else softmax(logits / T) in float32 and either
    the plain multinomial walk (src/sampler.c:77-85) or the nucleus (src/sampler.c:95-135)."""
    if temperature == 0.0:
        return argmax_first(logits)
    x = logits.astype(np.float32) / np.float32(temperature)
    e = np.exp(x - x.max()).astype(np.float32)
    p = e / e.sum(dtype=np.float32)
    n = len(p)
    if topp <= 0.0 or topp >= 1.0:
        r = rng.next_float()
        cdf = np.cumsum(p, dtype=np.float32)
        hit = np.nonzero(r < cdf)[0]
        return int(hit[0]) if len(hit) else n - 1
    cutoff = np.float32((1.0 - topp) / (n - 1))
    cand = np.nonzero(p >= cutoff)[0]
    order = cand[np.argsort(-p[cand], kind="stable")]
    cum = np.cumsum(p[order], dtype=np.float32)
    over = np.nonzero(cum > np.float32(topp))[0]
    last = int(over[0]) if len(over) else len(order) - 1
    r = rng.next_float() * cum[last]
    hit = np.nonzero(r < cum[:last + 1])[0]
    return int(order[hit[0]]) if len(hit) else int(order[last])


def generate(cfg: dict, w: Dict[str, np.ndarray], prompt: Sequence[int], max_new: int, temperature: float = 0.0,
             topp: float = 1.0, seed: int = 42, stop_ids: Sequence[int] = (), repeat_penalty: float = 1.0,
             repeat_window: int = 64) -> List[int]:
    """The reference's loop (src/generate.c:143-231): sample; a stop id ends the sequence without
    being emitted; after ``max_new`` tokens no further forward pass runs.  With a repeat penalty
    the prompt's ids and every emitted id enter the recent window (src/main.c:1648,
    src/generate.c:178-179)."""
    rng = Xorshift64Star(seed)
    toks = list(prompt)
    recent = list(prompt)[-repeat_window:] if repeat_penalty != 1.0 else []
    out: List[int] = []
    for _ in range(max_new):
        logits = forward(cfg, w, toks)[-1]
        if repeat_penalty != 1.0:
            logits = apply_repeat_penalty(logits, recent, repeat_penalty)
        nxt = sample(logits, temperature, topp, rng)
        if nxt in stop_ids:
            break
        out.append(nxt)
        toks.append(nxt)
        if repeat_penalty != 1.0:
            recent = (recent + [nxt])[-repeat_window:]
    return out
