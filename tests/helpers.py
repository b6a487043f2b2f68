"""Shared by the GPU tests: tiny model folders, traces of steps, and comparison with the plain implementation."""
import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np

import plain_llama

# Largest allowed |engine - plain| on logits.  float32: the target of this build (1e-4, logits
# of size ~1).  bfloat16: see ``bf16_bound``.
TOL_F32 = 1e-4


def bf16_bound(plain_logits: np.ndarray) -> float:
    """Bound for the bfloat16 engine against the float64 plain implementation.

    Activations are rounded to bfloat16 (relative 2^-9) at about six places per layer; the
    errors add up like a random walk through the layers and are carried into logits of
    magnitude max|logit|.  3 * 2^-8 * max|logit| (at least 3 * 2^-8) is a few such roundings
    and is far below the spacing that would change which kernel or cache slot was wrong.
    """
    return 3.0 * 2.0 ** -8 * max(1.0, float(np.abs(plain_logits).max()))


BF16_GAP_FACTOR = 3.0


def sharp_std(cfg: dict) -> float:
    """The matrix scale of the "sharp" variant of a tiny configuration: 1 / sqrt(width).

    With the stock N(0, 0.02) matrices a tiny model's attention scores are all near zero and
    attention is a running mean: rotation, softmax scale and the weighting of the keys then move
    the logits by less than bfloat16 rounding does.  With this scale queries and keys have
    components of size ~1, the scores of a row spread over 2 to 4 and logits reach 3 to 5, so
    that a missing rotation, a wrong softmax scale, a dropped key or a wrong key/value head moves
    them by 0.7 to 6 (tests/test_sharp_models.py asserts it)."""
    return float(cfg["hidden_size"]) ** -0.5


def measured_bf16_bound(cfg: dict, w, tokens, ref: np.ndarray = None) -> float:
    """Bound for a bfloat16 engine on one request of a sharp model: BF16_GAP_FACTOR times the gap
    between the plain implementation and the plain implementation with every stored activation
    rounded to bfloat16 (``round_fn``).  The engine rounds at a few more places than that and adds
    in other orders; a factor of three of one such set of roundings covers it, and the faults a
    test is there to catch are another factor of three to thirty beyond."""
    ref = plain_llama.forward(cfg, w, tokens) if ref is None else ref
    rounded = plain_llama.forward(cfg, w, tokens, round_fn=plain_llama.to_bf16)
    return BF16_GAP_FACTOR * float(np.abs(ref - rounded).max())


def make_model_dir(tmp_path, cfg: dict, seed: int, storage: str, matrix_std: float = 0.02) -> str:
    from bitnet_c_b200.weights import write_random_model
    d = os.path.join(str(tmp_path), f"model_{seed}_{storage}")
    write_random_model(d, cfg, seed, dtype=storage, matrix_std=matrix_std)
    return d


def random_tokens(seed: int, n: int, vocab: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


Step = dict  # {"step": int, "entries": [{"id", "tokens", "want"}], "end": [ids]}


def trace_whole(reqs: Dict[str, List[int]]) -> List[Step]:
    """Each request alone and whole, logits wanted everywhere."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(reqs.items())]


def trace_tail(reqs: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    """Each request alone: all but the last ``tail`` tokens in one step, then one token per step."""
    steps, n = [], 0
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_batches(batches: Sequence[Dict[str, Tuple[List[int], int]]]) -> List[Step]:
    """Batches one after another.  In a batch every request brings its first ``len - d`` tokens in
    one step (d = its number of decoded tokens), then one token per step; a request with fewer
    decode steps ends earlier and its slot is free for the next batch."""
    steps, n = [], 0
    for batch in batches:
        first = {"step": n, "entries": [], "end": []}
        for rid, (toks, d) in batch.items():
            head = len(toks) - d
            first["entries"].append({"id": rid, "tokens": toks[:head], "want": list(range(head))})
            if d == 0:
                first["end"].append(rid)
        steps.append(first)
        n += 1
        for j in range(max(d for _t, d in batch.values())):
            st = {"step": n, "entries": [], "end": []}
            for rid, (toks, d) in batch.items():
                if j < d:
                    st["entries"].append({"id": rid, "tokens": [toks[len(toks) - d + j]], "want": [0]})
                    if j == d - 1:
                        st["end"].append(rid)
            steps.append(st)
            n += 1
    return steps


def trace_chunks(reqs: Dict[str, List[int]], pieces: Sequence[int] = (1, 7, 64, 130), stagger: int = 1) -> List[Step]:
    """Every request in pieces of ``pieces`` tokens (taken in turn, each request starting at
    another place of the list), request i joining at step ``i * stagger``: steps then mix a fresh
    prompt, a continuation of many tokens behind cached ones and a continuation of one token."""
    ids = list(reqs)
    at = {r: 0 for r in ids}
    steps, n = [], 0
    while any(at[r] < len(reqs[r]) for r in ids):
        st = {"step": len(steps), "entries": [], "end": []}
        for i, r in enumerate(ids):
            if n < i * stagger or at[r] >= len(reqs[r]):
                continue
            toks = reqs[r][at[r]:at[r] + pieces[(n + i) % len(pieces)]]
            st["entries"].append({"id": r, "tokens": toks, "want": list(range(len(toks)))})
            at[r] += len(toks)
            if at[r] >= len(reqs[r]):
                st["end"].append(r)
        if st["entries"]:  # nobody may be live between one request's end and the next one's start
            steps.append(st)
        n += 1
    return steps


def replay(model, cache, steps: List[Step]) -> Dict[str, Dict[int, np.ndarray]]:
    """Run steps through Model.step in process; returns id -> position -> logits."""
    from bitnet_c_b200.engine import SeqStep
    slots, pos, out = {}, {}, {}
    for st in steps:
        seqs = []
        for e in st["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = cache.open()
                pos[e["id"]] = 0
                out.setdefault(e["id"], {})
            seqs.append(SeqStep(slots[e["id"]], e["tokens"], e["want"]))
        logits = model.step(cache, seqs)
        if logits is not None:
            arr = logits.float().cpu().numpy()
            r = 0
            for e in st["entries"]:
                for w in e["want"]:
                    out[e["id"]][pos[e["id"]] + w] = arr[r]
                    r += 1
        for e in st["entries"]:
            pos[e["id"]] += len(e["tokens"])
        for rid in st["end"]:
            cache.close(slots.pop(rid))
        cache.check()
    assert not slots
    return out


def collect_trace_output(steps: List[Step], out_dir: str, vocab: int) -> Dict[str, Dict[int, np.ndarray]]:
    """The same mapping from the files bin/trace_run wrote."""
    pos, out = {}, {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        arr = None
        if n_want:
            arr = np.fromfile(os.path.join(out_dir, f"{st['step']}.f32"), dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in st["entries"]:
            pos.setdefault(e["id"], 0)
            out.setdefault(e["id"], {})
            for w in e["want"]:
                out[e["id"]][pos[e["id"]] + w] = arr[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
    return out


def plain_logits(model_dir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_llama.read_model(model_dir)
    return {rid: plain_llama.forward(cfg, w, toks) for rid, toks in reqs.items()}


def compare(got: Dict[str, Dict[int, np.ndarray]], want: Dict[str, np.ndarray], tol_fn, what: str) -> float:
    """``tol_fn``: a function of a request's plain logits, or a dict from request id to its bound."""
    worst = 0.0
    for rid, per_pos in got.items():
        ref = want[rid]
        tol = tol_fn[rid] if isinstance(tol_fn, dict) else tol_fn(ref)
        for p, l in sorted(per_pos.items()):
            err = float(np.abs(l.astype(np.float64) - ref[p]).max())
            worst = max(worst, err)
            assert err <= tol, (f"{what}: request {rid} position {p} (of {len(ref)}): "
                                f"max |diff| {err:.3e} > {tol:.3e}; first wrong place is where to look")
    return worst


def steps_to_jsonl(steps: List[Step]) -> str:
    return "".join(json.dumps(s) + "\n" for s in steps)
