"""The model: embedding, blocks in schedule order, final norm, output head — and its step function.

The reference's model is an immutable ``BnModel`` shared by all sessions, with per-request
state in ``BnSession`` (include/model.h:14-20, include/session.h:13-20).  Here ``Model`` is the
shared, immutable half; ``Cache`` (cache/cache.py) is the per-sequence half.  The reference has
two forward entry points, many tokens of one sequence (bn_transformer_prefill,
src/transformer/prefill.c:2494) and one token (bn_transformer_forward, src/transformer.c:183);
``Model.step`` is both at once, for a batch of sequences.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from ..cache import Cache, CacheFull
from ..config import ConfigError, ModelSpec, architecture_of, read_config_json
from ..csrc import build as kernel_build
from ..csrc import ops
from ..parts import BuildContext, ParamSpec, Part, build_part
from ..parts.base import Normed
from .batch import SeqStep, StepContext, pack_step

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """A step that cannot run: a token outside the vocabulary, a slot that is not open, a wanted
    place outside the step's tokens.  Raised before anything is launched or reserved."""


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


def _walk(prefix: str, part: Part, out: Dict[str, tuple]) -> None:
    for name, p in part.params().items():
        out[f"{prefix}.{name}"] = (part, name, p)
    for cname, child in part.children().items():
        _walk(f"{prefix}.{cname}", child, out)


class Model:
    def __init__(self, spec: ModelSpec, dtype="bfloat16", device="cuda:0", arch=None, config=None):
        spec.validate()
        self.spec, self.arch, self.config = spec, arch, config
        self.dtype = resolve_dtype(dtype)
        self.device = torch.device(device) if device is not None else None
        b = BuildContext(dtype=self.dtype, device=self.device)
        self.blocks = [build_part("block", bs, b) for bs in spec.blocks]
        self.final_norm = build_part("norm", spec.final_norm, b)
        self.head_part = build_part("head", spec.head, b)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self._bad_token: Optional[torch.Tensor] = None
        self.diagnostics = None  # engine/diagnostics.py: tensor dumps, top logits, kernel timers
        self._owners: Dict[str, tuple] = {}
        for i, blk in enumerate(self.blocks):
            _walk(f"blocks.{i}", blk, self._owners)
        _walk("final_norm", self.final_norm, self._owners)
        _walk("head", self.head_part, self._owners)  # a head's own parameters; the matrix is "head.weight"
        if "head.weight" in self._owners:
            raise ConfigError("a head part must not name a parameter 'weight': 'head.weight' is the head matrix")

    # ---- parameters -----------------------------------------------------------------------
    def parameter_table(self) -> Dict[str, ParamSpec]:
        """Every parameter of the model by path, e.g. ``blocks.0.mixer.q``."""
        t: Dict[str, ParamSpec] = {"embedding.table": ParamSpec((self.spec.vocab_size, self.spec.width))}
        for path, (_part, _name, p) in self._owners.items():
            t[path] = p
        if not self.spec.tie_embeddings:
            t["head.weight"] = ParamSpec((self.spec.vocab_size, self.spec.width))
        return t

    def graph_safe(self) -> bool:
        """True when every part reads its step from device buffers only, so that a decode step can
        be recorded once and replayed (parts say so with ``graph_safe = True``)."""
        def ok(part) -> bool:
            return bool(getattr(part, "graph_safe", False)) and all(ok(c) for c in part.children().values())
        return all(ok(b) for b in self.blocks) and ok(self.final_norm) and ok(self.head_part)

    def decode_blocks_per_sequence(self) -> int:
        """The most thread blocks any part launches per sequence in a decode step (0: no part takes
        a work list); what ``DecodeRunner`` sizes a batch's work list by."""
        return max((b.decode_blocks_per_sequence() for b in self.blocks), default=0)

    def kernel_families(self) -> List[str]:
        fams = ["embed", "linear"]
        for blk in self.blocks:
            fams.extend(blk.all_kernels())
        fams.extend(self.final_norm.all_kernels())
        fams.extend(self.head_part.all_kernels())
        return list(dict.fromkeys(fams))

    def bind(self, tensors: Dict[str, torch.Tensor]) -> "Model":
        """Hand every parameter to the part that owns it.  ``tensors`` maps paths to device tensors
        (None, or no entry, for an optional parameter that the model does not have)."""
        table = self.parameter_table()
        tensors = dict(tensors)
        for path, p in table.items():
            if p.optional:
                tensors.setdefault(path, None)
        missing = sorted(set(table) - set(tensors))
        extra = sorted(set(tensors) - set(table))
        if missing or extra:
            raise ValueError(f"bind: missing {missing}, unexpected {extra}")
        per_part: Dict[int, tuple] = {}
        for path, (part, name, _p) in self._owners.items():
            per_part.setdefault(id(part), (part, {}))[1][name] = tensors[path]
        for part, group in per_part.values():
            part.bind(group)
        self.embedding = tensors["embedding.table"]
        self.head = tensors["head.weight"] if not self.spec.tie_embeddings else self.embedding
        self._bad_token = torch.zeros(1, dtype=torch.int32, device=self.device)
        return self

    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0", max_seq: int = 0) -> "Model":
        """Load ``config.json`` and the safetensors weights of ``model_dir``; the model class is
        chosen by ``architectures[0]``."""
        from ..weights import load_weights
        cfg_dict = read_config_json(model_dir)
        arch = architecture_of(cfg_dict)
        cfg = arch.read_config(cfg_dict)
        if max_seq:
            cfg = arch.cap_positions(cfg, max_seq)
        model = cls(arch.to_spec(cfg), dtype=dtype, device=device, arch=arch, config=cfg)
        require_cuda(model.device)
        kernel_build.ensure_built(model.kernel_families())
        tensors = load_weights(model_dir, model.parameter_table(), arch.tensor_name, model.dtype, model.device)
        return model.bind(tensors)

    @classmethod
    def from_random(cls, config: Dict[str, Any], seed: int = 0, dtype="bfloat16", device="cuda:0",
                    matrix_std: float = 0.02, norm_std: float = 0.1) -> "Model":
        """A model of ``config`` (config.json keys) with the weights of ``write_random_model(folder,
        config, seed, dtype)`` drawn on the device instead of written to a folder and loaded: the
        same seeded generator (``weights.random_init``), for sizes whose file would be large."""
        from ..weights import random_parameters
        arch = architecture_of(config)
        cfg = arch.read_config(config)
        model = cls(arch.to_spec(cfg), dtype=dtype, device=device, arch=arch, config=cfg)
        require_cuda(model.device)
        kernel_build.ensure_built(model.kernel_families())
        tensors = {path: t for path, _name, t in random_parameters(model.spec, arch.tensor_name, seed, model.dtype,
                                                                   matrix_std, norm_std, model.device)}
        return model.bind(tensors)

    # ---- cache ----------------------------------------------------------------------------
    def new_cache(self, max_tokens: int, max_seqs: Optional[int] = None, allocate: bool = True) -> Cache:
        sched = self.spec.schedule
        kv = [self.blocks[e.block].cache_request() for e in sched]
        st = [self.blocks[e.block].state_request() for e in sched]
        return Cache(kv, [e.cache_of for e in sched], st, max_tokens, self.spec.max_positions, self.dtype,
                     self.device, max_seqs=max_seqs, allocate=allocate)

    # ---- the step -------------------------------------------------------------------------
    def check_kernels(self) -> None:
        """Raise if a kernel with bounded waits reported that a wait gave up since the last call
        (the results of that launch are not valid).  Synchronises with the device."""
        if self.device is not None and self.device.type == "cuda":
            ops.check_tc_status(self.device)
            if self._bad_token is not None and int(self._bad_token.item()):
                self._bad_token.zero_()
                raise StepError("a token id outside the embedding table reached the device (its row was taken as "
                                "zero); ids fed back on the device are not checked on the host")

    def check_step(self, cache: Cache, seqs: Sequence[SeqStep]) -> List[int]:
        if not seqs:
            raise StepError("a step needs at least one sequence")
        seen = set()
        lengths = []
        V = self.spec.vocab_size
        length_of = cache.length
        for s in seqs:
            slot, toks = s.slot, s.tokens
            if slot in seen:
                raise StepError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            lengths.append(length_of(slot))
            n = len(toks)
            if n == 0:
                raise StepError(f"slot {slot} brings no token")
            if not (0 <= min(toks) and max(toks) < V):
                bad = next(t for t in toks if not 0 <= int(t) < V)
                raise StepError(f"token {bad} is outside the vocabulary of {V}")
            for w in s.want:
                if not 0 <= w < n:
                    raise StepError(f"wanted place {w} is outside the {n} tokens of slot {slot}")
        return lengths

    def step(self, cache: Cache, seqs: Sequence[SeqStep]) -> Optional[torch.Tensor]:
        """Run the given tokens of the given sequences as one batch from the cache.

        Returns float32 logits ``[wanted, vocab]`` in the order of ``seqs`` and of each
        ``want``, or None when nothing is wanted.  On return the sequences are longer by the
        tokens they brought.  If the cache cannot hold them, nothing has changed.
        """
        lengths = self.check_step(cache, seqs)
        reserved = []
        try:
            for s in seqs:
                cache.reserve(s.slot, len(s.tokens))
                reserved.append(s)
        except CacheFull:
            for s in reserved:  # give back what this step took
                cache.unreserve(s.slot)
            raise
        try:
            cache.sync()
            ctx = pack_step(seqs, lengths, self.device)
            logits = self.forward(cache, ctx)
        except BaseException:
            for s in seqs:  # the step did not happen: its pages go back, the lengths stay
                cache.unreserve(s.slot)
            raise
        for s in seqs:
            cache.advance(s.slot, len(s.tokens))
        return logits

    def forward(self, cache: Cache, ctx: StepContext) -> Optional[torch.Tensor]:
        """Embedding, every scheduled run, final norm and head at the wanted rows."""
        x = torch.empty((ctx.n_tokens, self.spec.width), dtype=torch.float32, device=self.device)
        ops.embed_gather(self.embedding, ctx.tokens, x, self._bad_token, self.spec.embedding_scale)
        diag = ctx.diag = self.diagnostics
        ctx.layer = -1
        ctx.tap("inp", x)
        pending = None
        sched = self.spec.schedule
        for i, e in enumerate(sched):
            blk = self.blocks[e.block]
            if diag is not None:
                if i > 0:
                    ctx.tap("lout", lambda: _residual_after(x, pending))
                ctx.layer = i
            if not getattr(blk, "accepts_normed", False):
                pending = blk.forward(x, pending, ctx, cache.view(i), cache.state(i))
                continue
            # the norm after this block, if whoever applies it can take its output ready-made:
            # the next block's first norm, or the final norm when every row's logits are wanted
            if i + 1 < len(sched):
                nxt = self.blocks[sched[i + 1].block]
                next_norm = nxt.entry_norm() if getattr(nxt, "accepts_normed", False) else None
            else:
                next_norm = self.final_norm if ctx.rows is not None and ctx.rows_all else None
            pending = blk.forward(x, pending, ctx, cache.view(i), cache.state(i), next_norm=next_norm)
        if diag is not None:
            ctx.tap("lout", lambda: _residual_after(x, pending))
            ctx.layer = -1
        if ctx.rows is None:
            return None
        if isinstance(pending, Normed):
            h = pending.value
        else:
            h = self.final_norm.add_norm(x, pending, ctx, rows=ctx.rows)
        logits = self.head_part.forward(h, self.head, ctx)
        if diag is not None:
            ctx.tap("result_norm", h, rows=ctx.host_rows)
            ctx.tap("result_output", logits, rows=ctx.host_rows)
        return logits


def _residual_after(x: torch.Tensor, pending) -> torch.Tensor:
    """The residual stream with a block's last delta added (the delta is otherwise added by the next
    norm; a product that prepared that norm in its epilogue has added it already)."""
    if pending is None or isinstance(pending, Normed):
        return x
    return x + (pending.sum(0) if pending.dim() == 3 else pending).float()


def require_cuda(device) -> None:
    if device is None or torch.device(device).type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this library runs on a CUDA device only (no CPU path); "
                           f"asked for device {device!r}, torch.cuda.is_available()={torch.cuda.is_available()}")


def parameter_table(spec: ModelSpec) -> Dict[str, ParamSpec]:
    """The parameters a model of ``spec`` has, without building anything on a device."""
    return Model(spec, dtype="float32", device=None).parameter_table()
