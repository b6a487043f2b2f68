"""The Python side of the C interface (capi/bn_api.c): plain functions over ints, bytes and
objects, so that the C side needs only a handful of CPython calls.  Everything here goes through
the library's public engine; nothing is computed in this file."""
from __future__ import annotations

import numpy as np


def _bn():
    import bitnet_c_b200 as bn
    return bn


class ModelHandle:
    def __init__(self, model_dir: str, dtype: str, max_seq: int, max_tokens: int, max_seqs: int):
        bn = _bn()
        self.model = bn.load_model(model_dir, dtype=dtype, max_seq=max_seq)
        max_seqs = max(1, max_seqs)
        if max_tokens <= 0:
            max_tokens = max_seqs * self.model.spec.max_positions
        self.cache = self.model.new_cache(max_tokens=max_tokens, max_seqs=max_seqs)
        self.vocab = self.model.spec.vocab_size
        self.seq_len = self.model.spec.max_positions
        self.engine = None  # the generation engine of bn_generate_batch, kept from call to call


class SessionHandle:
    def __init__(self, m: ModelHandle):
        self.m = m
        self.slot = m.cache.open()
        self.logits = None

    def pos(self) -> int:
        return self.m.cache.length(self.slot)

    def close(self) -> None:
        if self.slot is not None:
            self.m.cache.close(self.slot)
            self.slot = None

    def reset(self) -> None:
        self.m.cache.close(self.slot)
        self.slot = self.m.cache.open()


def model_load(model_dir, dtype, max_seq, max_tokens, max_seqs):
    return ModelHandle(model_dir, dtype, max_seq, max_tokens, max_seqs)


def session_create(m):
    return SessionHandle(m)


def _ints(buf: bytes):
    return np.frombuffer(buf, dtype=np.int32).tolist()


def prefill(m: ModelHandle, s: SessionHandle, tokens: bytes, pos0: int, no_prefill: int, want: int):
    """want: 0 no logits, 1 the last token's, 2 every token's.  Returns float32 bytes or b''."""
    bn = _bn()
    toks = _ints(tokens)
    if pos0 != s.pos():
        raise ValueError(f"pos0={pos0}, but the session holds {s.pos()} tokens")
    n = len(toks)
    if no_prefill and n > 1:
        rows = []
        for i, t in enumerate(toks):
            w = [0] if (want == 2 or (want == 1 and i == n - 1)) else []
            out = m.model.step(m.cache, [bn.SeqStep(s.slot, [t], w)])
            if out is not None:
                rows.append(out.cpu().numpy())
        m.model.check_kernels()
        return np.concatenate(rows).astype("<f4").tobytes() if rows else b""
    w = list(range(n)) if want == 2 else ([n - 1] if want == 1 else [])
    out = m.model.step(m.cache, [bn.SeqStep(s.slot, toks, w)])
    m.model.check_kernels()
    return out.cpu().numpy().astype("<f4").tobytes() if out is not None else b""


def step(m: ModelHandle, sessions, n_new: bytes, tokens: bytes, want: int):
    bn = _bn()
    counts, toks = _ints(n_new), _ints(tokens)
    if sum(counts) != len(toks) or len(counts) != len(sessions):
        raise ValueError("n_new does not add up to the tokens given")
    seqs, at = [], 0
    for s, c in zip(sessions, counts):
        seqs.append(bn.SeqStep(s.slot, toks[at:at + c], [c - 1] if want else []))
        at += c
    out = m.model.step(m.cache, seqs)
    m.model.check_kernels()
    return out.cpu().numpy().astype("<f4").tobytes() if out is not None else b""


class SamplerHandle:
    """One request's sampler on the device: the library's own sampling kernels."""

    def __init__(self, vocab, temperature, topp, penalty, window, seed):
        import torch
        from bitnet_c_b200.sampling import Sampler, SamplingParams
        self.torch = torch
        self.vocab = vocab
        params = SamplingParams(temperature=temperature, top_p=topp if 0.0 < topp < 1.0 else 1.0, seed=int(seed),
                                repeat_penalty=penalty, repeat_window=max(1, window))
        self.sampler = Sampler(params, 1, vocab, torch.device("cuda:0"), first_index=0, prompts=[[]])

    def accept(self, token):
        if self.sampler.penalised:
            self.sampler.accept(self.torch.tensor([token], dtype=self.torch.int32, device="cuda:0"), None)

    def sample(self, logits: bytes) -> int:
        row = self.torch.frombuffer(bytearray(logits), dtype=self.torch.float32).reshape(1, self.vocab).to("cuda:0")
        return int(self.sampler.sample(row, None).cpu().item())


def sampler_create(vocab, temperature, topp, penalty, window, seed):
    return SamplerHandle(vocab, temperature, topp, penalty, window, seed)


def generate_batch(m: ModelHandle, prompts, max_new, temperature, topp, penalty, window, seed, stop_ids: bytes):
    """prompts: list of int32 byte strings.  Returns a list of int32 byte strings."""
    from bitnet_c_b200.engine import ModelEngine, generate
    from bitnet_c_b200.sampling import SamplingParams
    params = SamplingParams(temperature=temperature, top_p=topp if 0.0 < topp < 1.0 else 1.0, seed=int(seed),
                            repeat_penalty=penalty, repeat_window=max(1, window))
    eng = m.engine
    if eng is None or eng.params != params:
        eng = m.engine = ModelEngine(m.model, m.cache, params)
    out = generate(eng, [_ints(p) for p in prompts], [int(max_new)] * len(prompts), stop_ids=tuple(_ints(stop_ids)))
    return [np.asarray(c.tokens, dtype="<i4").tobytes() for c in out]
