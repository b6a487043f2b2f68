"""Each part alone against the plain implementation, and the proof that a new part needs no change
to the library: a toy mixer with state of its own, defined here, is registered, built and stepped."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import bitnet_c_b200 as bn
from bitnet_c_b200.config import (AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NoPositionSpec, RmsNormSpec,
                                  RotarySpec, ScheduleEntry)
from bitnet_c_b200.engine import Model, SeqStep, pack_step
from bitnet_c_b200.parts import (BuildContext, FeedForward, Mixer, ParamSpec, Position, StateRequest, build_part,
                                 register_ffn, register_mixer, register_position, unregister)
import plain_llama
from helpers import bf16_bound

pytestmark = pytest.mark.gpu


def ctx_for(dev, lengths_new):
    """A step of fresh sequences of the given lengths in slots 0..n-1."""
    seqs = [SeqStep(i, [0] * n) for i, n in enumerate(lengths_new)]
    return pack_step(seqs, [0] * len(seqs), dev)


def randn(gen, *shape, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(cuda_device, dtype):
    g = torch.Generator().manual_seed(0)
    part = build_part("norm", RmsNormSpec(width=72, eps=3e-6), BuildContext(dtype, cuda_device))
    assert part.params()["weight"].shape == (72,)
    w = (1 + randn(g, 72, scale=0.1)).to(dtype)
    part.bind({"weight": w.to(cuda_device)})
    x, d = randn(g, 5, 72), randn(g, 5, 72).to(dtype)
    xd = x.to(cuda_device)
    h = part.add_norm(xd, d.to(cuda_device), None)
    ref = plain_llama.rmsnorm(x.double().numpy() + d.double().numpy(), w.double().numpy(), 3e-6)
    assert h.dtype == dtype
    assert np.abs(h.double().cpu().numpy() - ref).max() < (1e-5 if dtype == torch.float32 else 3e-2)
    assert np.abs(xd.double().cpu().numpy() - (x.double() + d.double()).numpy()).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_part(cuda_device, dtype):
    g = torch.Generator().manual_seed(1)
    part = build_part("position", RotarySpec(head_dim=48, theta=50000.0), BuildContext(dtype, cuda_device))
    ctx = ctx_for(cuda_device, [5, 130])
    x = randn(g, 135, 3 * 48).to(dtype)
    xd = x.to(cuda_device).contiguous()
    part.rotate(xd, 2, 48, ctx)  # only the first two heads
    pos = list(range(5)) + list(range(130))
    heads = x.double().numpy().reshape(135, 3, 48)
    ref = plain_llama.apply_rope(heads[:, :2], pos, 50000.0)
    got = xd.double().cpu().numpy().reshape(135, 3, 48)
    assert np.abs(got[:, :2] - ref).max() < (2e-6 if dtype == torch.float32 else 2e-2)
    assert np.array_equal(got[:, 2], heads[:, 2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(cuda_device, dtype):
    g = torch.Generator().manual_seed(2)
    part = build_part("ffn", GatedMlpSpec(width=40, intermediate=104), BuildContext(dtype, cuda_device))
    w = {"gate": randn(g, 104, 40, scale=0.2).to(dtype), "up": randn(g, 104, 40, scale=0.2).to(dtype),
         "down": randn(g, 40, 104, scale=0.2).to(dtype)}
    part.bind({k: v.to(cuda_device) for k, v in w.items()})
    for rows in (3, 50):  # few rows: own kernel; many rows: library product
        h = randn(g, rows, 40).to(dtype)
        out = part.forward(h.to(cuda_device), None)
        ref = plain_llama.swiglu(h.double().numpy(), *(w[k].double().numpy() for k in ("gate", "up", "down")))
        assert np.abs(out.double().cpu().numpy() - ref).max() < (2e-5 if dtype == torch.float32 else 5e-2)


def tiny_spec(mixers, schedule=None, width=32, vocab=50, max_positions=256):
    norm = RmsNormSpec(width=width, eps=1e-5)
    blocks = tuple(BlockSpec(mixer=m, ffn=GatedMlpSpec(width=width, intermediate=48), mixer_norm=norm, ffn_norm=norm)
                   for m in mixers)
    schedule = schedule or [ScheduleEntry(i) for i in range(len(blocks))]
    return ModelSpec(vocab_size=vocab, width=width, blocks=blocks, schedule=tuple(schedule), final_norm=norm,
                     max_positions=max_positions)


def random_bind(model, seed, scale=0.3):
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for path, p in model.parameter_table().items():
        t = (1 + randn(g, *p.shape, scale=0.1)) if p.init == "ones" else randn(g, *p.shape, scale=scale)
        tensors[path] = t.to(model.dtype).to(model.device)
    model.bind(tensors)
    return {k: v.double().cpu().numpy() for k, v in tensors.items()}


def plain_forward_spec(spec, w, tokens):
    """The plain parts put together for a spec of attention blocks (window and shared caches included)."""
    T = len(tokens)
    x = w["embedding.table"][np.asarray(tokens)]
    kv_of = {}
    for run, e in enumerate(spec.schedule):
        b, p = spec.blocks[e.block], f"blocks.{e.block}."
        a = b.mixer
        h = plain_llama.rmsnorm(x, w[p + "mixer_norm.weight"], b.mixer_norm.eps)
        q = (h @ w[p + "mixer.q"].T).reshape(T, a.n_heads, a.head_dim)
        rot = (lambda z: plain_llama.apply_rope(z, range(T), a.position.theta)) if a.position.kind == "rotary" else (lambda z: z)
        if e.cache_of is None:
            k = rot((h @ w[p + "mixer.k"].T).reshape(T, a.n_kv_heads, a.head_dim))
            v = (h @ w[p + "mixer.v"].T).reshape(T, a.n_kv_heads, a.head_dim)
            kv_of[run] = (k, v)
        else:
            k, v = kv_of[e.cache_of]
        o = plain_llama.attention(rot(q), k, v, a.softmax_scale, a.window).reshape(T, -1)
        x = x + o @ w[p + "mixer.o"].T
        h = plain_llama.rmsnorm(x, w[p + "ffn_norm.weight"], b.ffn_norm.eps)
        x = x + plain_llama.swiglu(h, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
    h = plain_llama.rmsnorm(x, w["final_norm.weight"], spec.final_norm.eps)
    return h @ w["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_blocks_differ_layer_by_layer_and_schedule_is_data(cuda_device, dtype):
    """One model with a full-attention block, a windowed block without position encoding and other head
    counts, a block that runs twice, and a run that reads another run's cache."""
    full = AttentionSpec(width=32, n_heads=4, n_kv_heads=2, head_dim=16, position=RotarySpec(16, 10000.0))
    win = AttentionSpec(width=32, n_heads=2, n_kv_heads=1, head_dim=32, position=NoPositionSpec(), window=70)
    spec = tiny_spec([full, win], [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(0, cache_of=0),
                                   ScheduleEntry(1)])
    model = Model(spec, dtype=dtype, device=cuda_device)
    w = random_bind(model, 5, scale=0.12)
    cache = model.new_cache(max_tokens=1024, max_seqs=3)
    assert len(cache.groups) == 2 and cache.groups[0].entries == [0, 2] and cache.groups[1].entries == [1, 4]
    toks = {"x": np.random.default_rng(0).integers(0, 50, 200).tolist(), "y": [3, 4, 5]}
    plain = {k: plain_forward_spec(spec, w, v) for k, v in toks.items()}
    from helpers import compare, replay, trace_batches, trace_tail
    for steps in (trace_tail(toks, 40), trace_batches([{"x": (toks["x"], 90), "y": (toks["y"], 2)}])):
        got = replay(model, cache, steps)
        compare(got, plain, (lambda r: 1e-4) if dtype == "float32" else bf16_bound, "mixed blocks")
    # the windowed group gave back the pages that fell out of its window
    assert cache.groups[1].pool.n_free == cache.groups[1].pool.n_pages


@dataclass(frozen=True)
class DecayMixSpec:
    """A toy mixer with a state of its own: s_t = decay * s_{t-1} + h_t, out = W s_t."""
    width: int
    decay: float
    kind: str = "toy_decay_mix"


def test_a_new_mixer_with_state_needs_no_change_to_the_library(cuda_device):
    @register_mixer("toy_decay_mix")
    class DecayMix(Mixer):
        def params(self):
            return {"w": ParamSpec((self.spec.width, self.spec.width))}

        def bind(self, tensors):
            self.w = tensors["w"]

        def state_request(self):
            return StateRequest((self.spec.width,), torch.float32)

        def forward(self, h, ctx, kv, state):
            out = torch.empty_like(h, dtype=torch.float32)
            at = 0
            for slot, n in zip(ctx.host_slots, ctx.host_new):
                s = state[slot]
                for t in range(at, at + n):
                    s = self.spec.decay * s + h[t].float()
                    out[t] = s
                state[slot] = s
                at += n
            return (out @ self.w.float().t()).to(h.dtype)

    try:
        attn = AttentionSpec(width=32, n_heads=2, n_kv_heads=2, head_dim=16, position=RotarySpec(16, 10000.0))
        spec = tiny_spec([DecayMixSpec(32, 0.9), attn, DecayMixSpec(32, 0.5)])
        model = Model(spec, dtype="float32", device=cuda_device)
        assert "blocks.0.mixer.w" in model.parameter_table() and "blocks.1.mixer.q" in model.parameter_table()
        w = random_bind(model, 6)
        cache = model.new_cache(max_tokens=512, max_seqs=2)
        assert set(cache.states) == {0, 2} and cache.states[0].shape == (2, 32) and len(cache.groups) == 1

        def plain(tokens):
            T = len(tokens)
            x = w["embedding.table"][np.asarray(tokens)]
            for i, b in enumerate(spec.blocks):
                p = f"blocks.{i}."
                h = plain_llama.rmsnorm(x, w[p + "mixer_norm.weight"], 1e-5)
                if b.mixer.kind == "toy_decay_mix":
                    s, rows = np.zeros(32), []
                    for t in range(T):
                        s = b.mixer.decay * s + h[t]
                        rows.append(s)
                    x = x + np.stack(rows) @ w[p + "mixer.w"].T
                else:
                    q = plain_llama.apply_rope((h @ w[p + "mixer.q"].T).reshape(T, 2, 16), range(T), 10000.0)
                    k = plain_llama.apply_rope((h @ w[p + "mixer.k"].T).reshape(T, 2, 16), range(T), 10000.0)
                    v = (h @ w[p + "mixer.v"].T).reshape(T, 2, 16)
                    x = x + plain_llama.attention(q, k, v, 0.25).reshape(T, 32) @ w[p + "mixer.o"].T
                h = plain_llama.rmsnorm(x, w[p + "ffn_norm.weight"], 1e-5)
                x = x + plain_llama.swiglu(h, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
            return plain_llama.rmsnorm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T

        from helpers import compare, replay, trace_batches, trace_tail, trace_whole
        toks = {"p": np.random.default_rng(1).integers(0, 50, 70).tolist(), "q": [9, 8, 7, 6]}
        ref = {k: plain(v) for k, v in toks.items()}
        for steps in (trace_whole(toks), trace_tail(toks, 32), trace_batches([{"p": (toks["p"], 10), "q": (toks["q"], 3)}]),
                      trace_batches([{"q": (toks["q"], 1)}, {"p": (toks["p"], 5)}])):  # the last reuses q's slot: state must be zeroed
            compare(replay(model, cache, steps), ref, lambda r: 2e-4, "toy mixer")
    finally:
        unregister("mixer", "toy_decay_mix")


@dataclass(frozen=True)
class RoutedToySpec:
    """A toy feed-forward with routing: every token goes to the expert with the largest router
    logit, weighted by that expert's softmax probability; an expert is W_out relu(W_in h)."""
    width: int
    intermediate: int
    n_experts: int
    kind: str = "toy_routed"


@dataclass(frozen=True)
class PositionScaleSpec:
    """A toy position encoding: the heads of a token at position p are divided by 1 + rate * p."""
    head_dim: int
    rate: float
    kind: str = "toy_position_scale"


def test_a_routed_feed_forward_and_another_position_encoding_need_no_change_to_the_library(cuda_device):
    """Both are defined here, registered, built by the model from its spec like any other part,
    and stepped whole, token by token and in unequal batches.  The attention mixer finds no fast
    paths on this position encoding and takes its general ones."""
    @register_ffn("toy_routed")
    class RoutedToy(FeedForward):
        def params(self):
            s = self.spec
            return {"router": ParamSpec((s.n_experts, s.width)), "w_in": ParamSpec((s.n_experts * s.intermediate, s.width)),
                    "w_out": ParamSpec((s.n_experts * s.width, s.intermediate))}

        def bind(self, tensors):
            s = self.spec
            self.router = tensors["router"].float()
            self.w_in = tensors["w_in"].float().reshape(s.n_experts, s.intermediate, s.width)
            self.w_out = tensors["w_out"].float().reshape(s.n_experts, s.width, s.intermediate)

        def forward(self, h, ctx):
            hf = h.float()
            prob = torch.softmax(hf @ self.router.t(), dim=-1)
            top = prob.argmax(dim=-1)
            out = torch.zeros_like(hf)
            for e in range(self.spec.n_experts):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    x = hf[rows]
                    out[rows] = (torch.relu(x @ self.w_in[e].t()) @ self.w_out[e].t()) * prob[rows, e][:, None]
            return out.to(h.dtype)

    @register_position("toy_position_scale")
    class PositionScale(Position):
        graph_safe = True

        def rotate(self, x, n_heads, head_dim, ctx):
            scale = 1.0 / (1.0 + self.spec.rate * ctx.tok_pos.to(torch.float32))
            part = x[:, : n_heads * head_dim]
            part.copy_((part.float() * scale[:, None]).to(x.dtype))

    try:
        width, E, inter = 32, 3, 40
        norm = RmsNormSpec(width=width, eps=1e-5)
        attn = AttentionSpec(width=width, n_heads=2, n_kv_heads=1, head_dim=16, position=PositionScaleSpec(16, 0.05))
        blocks = (BlockSpec(mixer=attn, ffn=RoutedToySpec(width, inter, E), mixer_norm=norm, ffn_norm=norm),
                  BlockSpec(mixer=attn, ffn=GatedMlpSpec(width=width, intermediate=48), mixer_norm=norm, ffn_norm=norm))
        spec = ModelSpec(vocab_size=50, width=width, blocks=blocks, schedule=(ScheduleEntry(0), ScheduleEntry(1)),
                         final_norm=norm, max_positions=256)
        model = Model(spec, dtype="float32", device=cuda_device)
        assert "blocks.0.ffn.router" in model.parameter_table()
        w = random_bind(model, 9, scale=0.12)
        # a decisive router: top-1 routing is a discontinuous function, and the comparison with the
        # plain implementation only means something where rounding cannot flip a choice
        model.blocks[0].ffn.router *= 16
        w["blocks.0.ffn.router"] = w["blocks.0.ffn.router"] * 16

        def plain(tokens):
            T = len(tokens)
            x = w["embedding.table"][np.asarray(tokens)]
            pos_scale = 1.0 / (1.0 + 0.05 * np.arange(T))
            for i, b in enumerate(spec.blocks):
                p = f"blocks.{i}."
                h = plain_llama.rmsnorm(x, w[p + "mixer_norm.weight"], 1e-5)
                q = (h @ w[p + "mixer.q"].T).reshape(T, 2, 16) * pos_scale[:, None, None]
                k = (h @ w[p + "mixer.k"].T).reshape(T, 1, 16) * pos_scale[:, None, None]
                v = (h @ w[p + "mixer.v"].T).reshape(T, 1, 16)
                x = x + plain_llama.attention(q, k, v, 0.25).reshape(T, 32) @ w[p + "mixer.o"].T
                h = plain_llama.rmsnorm(x, w[p + "ffn_norm.weight"], 1e-5)
                if b.ffn.kind == "toy_routed":
                    logits = h @ w[p + "ffn.router"].T
                    prob = np.exp(logits - logits.max(-1, keepdims=True))
                    prob /= prob.sum(-1, keepdims=True)
                    w_in = w[p + "ffn.w_in"].reshape(E, inter, width)
                    w_out = w[p + "ffn.w_out"].reshape(E, width, inter)
                    y = np.zeros_like(h)
                    for t in range(T):
                        e = int(np.argmax(prob[t]))
                        y[t] = (np.maximum(h[t] @ w_in[e].T, 0) @ w_out[e].T) * prob[t, e]
                    x = x + y
                else:
                    x = x + plain_llama.swiglu(h, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
            return plain_llama.rmsnorm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T

        from helpers import compare, replay, trace_batches, trace_tail, trace_whole
        toks = {"p": np.random.default_rng(3).integers(0, 50, 90).tolist(), "q": [9, 8, 7, 6, 5]}
        ref = {k: plain(v) for k, v in toks.items()}
        cache = model.new_cache(max_tokens=512, max_seqs=2)
        for steps in (trace_whole(toks), trace_tail(toks, 32), trace_batches([{"p": (toks["p"], 12), "q": (toks["q"], 4)}])):
            compare(replay(model, cache, steps), ref, lambda r: 2e-4, "toy routed feed-forward and position encoding")
    finally:
        unregister("ffn", "toy_routed")
        unregister("position", "toy_position_scale")


def test_norms_fused_into_products_agree_with_norm_kernels(cuda_device, monkeypatch):
    """With few rows in bfloat16 the products before a norm add to the residual and prepare the
    norm's output themselves (``ops.RowScaled``).  The logits must agree with the path through
    the norm kernels to a few bfloat16 roundings, for prompts in one step and for decode steps,
    and a request for only some rows' logits must still take the final norm kernel."""
    from bitnet_c_b200.csrc import ops
    from tiny_configs import TINY_D
    model = Model.from_random(dict(TINY_D), seed=5, dtype="bfloat16", device=cuda_device)
    toks = [torch.randint(0, TINY_D["vocab_size"], (n,), generator=torch.Generator().manual_seed(n)).tolist()
            for n in (40, 9, 23)]

    def run(fused):
        monkeypatch.setattr(ops, "USE_FUSED_NORM", fused)
        cache = model.new_cache(max_tokens=1024, max_seqs=3)
        slots = [cache.open() for _ in toks]
        outs = [model.step(cache, [SeqStep(s, t, list(range(len(t)))) for s, t in zip(slots, toks)])]  # 72 rows: kernels
        outs.append(model.step(cache, [SeqStep(s, [7, 8, 9], [0, 1, 2]) for s in slots]))  # 9 rows, all wanted
        outs.append(model.step(cache, [SeqStep(s, [3], [0]) for s in slots]))              # decode
        outs.append(model.step(cache, [SeqStep(s, [4, 5], [1]) for s in slots]))           # only some rows wanted
        model.check_kernels()
        return [o.double().cpu().numpy() for o in outs]

    launches = []
    real = ops.add_rmsnorm
    monkeypatch.setattr(ops, "add_rmsnorm", lambda *a, **k: (launches.append(1), real(*a, **k))[1])
    a = run(False)
    n_unfused = len(launches)
    del launches[:]
    b = run(True)
    n_fused = len(launches)
    # 2 layers: 5 norm launches per step unfused; fused: all five in the prompt step (72 rows), one
    # (the first norm) in the steps of few rows, two (first and final) when only some rows are wanted
    assert n_unfused == 20 and n_fused == 5 + 1 + 1 + 2
    for x, y in zip(a, b):
        assert np.abs(x - y).max() <= bf16_bound(x)


@dataclass(frozen=True)
class BiasedHeadSpec:
    """A toy output head: logits = W h + bias, the bias being a parameter of the head's own that a
    file may lack."""
    vocab: int
    kind: str = "toy_biased_head"


def test_the_output_head_is_a_part_chosen_by_the_spec(cuda_device):
    """The stock head with a logit scale and the reference's final soft-cap
    (src/transformer/logits.c:325-333), and a toy head with an optional bias of its own that is
    defined here: both come out of the model's spec; nothing in the library names them."""
    from bitnet_c_b200.config import LinearHeadSpec
    from bitnet_c_b200.parts import Head, register_head
    from bitnet_c_b200.csrc import ops
    from helpers import compare, replay, trace_tail, trace_whole

    @register_head("toy_biased_head")
    class BiasedHead(Head):
        def params(self):
            return {"bias": ParamSpec((self.spec.vocab,), init="zeros", optional=True)}

        def bind(self, tensors):
            self.bias = tensors["bias"]

        def forward(self, h, table, ctx):
            logits = ops.linear(h, table, out_dtype=torch.float32)
            return logits if self.bias is None else logits + self.bias.float()

    try:
        attn = AttentionSpec(width=32, n_heads=2, n_kv_heads=1, head_dim=16, position=RotarySpec(16, 10000.0))
        toks = {"p": np.random.default_rng(5).integers(0, 50, 40).tolist(), "q": [1, 2, 3]}
        base = tiny_spec([attn])
        for head, fn in ((LinearHeadSpec(scale=0.5, softcap=2.0), lambda l, w: np.tanh(0.5 * l / 2.0) * 2.0),
                         (BiasedHeadSpec(50), lambda l, w: l + w["head.bias"]),
                         (BiasedHeadSpec(50), lambda l, w: l)):
            import dataclasses
            spec = dataclasses.replace(base, head=head)
            model = Model(spec, dtype="float32", device=cuda_device)
            table = model.parameter_table()
            assert ("head.bias" in table) == (head.kind == "toy_biased_head") and "head.weight" in table
            w = random_bind(model, 12, scale=0.4)
            if head.kind == "toy_biased_head" and fn(np.zeros(1), {"head.bias": np.ones(1)})[0] == 0:
                # the same model without the optional tensor: bound with None
                tensors = {k: torch.from_numpy(v).float().to(cuda_device) for k, v in w.items() if k != "head.bias"}
                model.bind(tensors)
                assert model.head_part.bias is None
            elif head.kind == "toy_biased_head":
                bias = torch.randn(50, generator=torch.Generator().manual_seed(1))
                model.head_part.bias = bias.to(cuda_device)
                w["head.bias"] = bias.double().numpy()
            plain = {k: fn(plain_forward_spec(base, w, v), w) for k, v in toks.items()}
            cache = model.new_cache(max_tokens=256, max_seqs=2)
            for steps in (trace_whole(toks), trace_tail(toks, 8)):
                compare(replay(model, cache, steps), plain, lambda r: 1e-4, f"head {head}")
    finally:
        unregister("head", "toy_biased_head")


@dataclass(frozen=True)
class NarrowValueSpec:
    """A toy mixer whose cached values are narrower than its keys: one head, keys of ``k_dim``,
    values of ``v_dim``, plain causal softmax attention, output W_o (v_dim -> width)."""
    width: int
    k_dim: int
    v_dim: int
    kind: str = "toy_narrow_values"


def test_keys_and_values_of_different_widths_get_storage_of_their_own_shape(cuda_device):
    from bitnet_c_b200.parts import KvRequest
    from helpers import compare, replay, trace_batches, trace_tail, trace_whole

    @register_mixer("toy_narrow_values")
    class NarrowValues(Mixer):
        def params(self):
            s = self.spec
            return {"qk": ParamSpec((2 * s.k_dim, s.width)), "v": ParamSpec((s.v_dim, s.width)), "o": ParamSpec((s.width, s.v_dim))}

        def bind(self, tensors):
            self.w = torch.cat([tensors["qk"], tensors["v"]]).float()
            self.o = tensors["o"].float()

        def cache_request(self):
            return KvRequest(n_kv_heads=1, head_dim=self.spec.k_dim, v_head_dim=self.spec.v_dim)

        def forward(self, h, ctx, kv, state):
            s = self.spec
            qkv = h.float() @ self.w.t()  # [T, k_dim (q) | k_dim (k) | v_dim]
            kv.append(qkv, s.k_dim, 2 * s.k_dim, ctx)
            out = torch.zeros(h.shape[0], s.v_dim, device=h.device)
            at = 0
            for slot, n, p0 in zip(ctx.host_slots, ctx.host_new, ctx.host_pos0):
                for j in range(n):
                    L = p0 + j + 1
                    pages = kv.page_table[slot, : (L + 63) // 64].long()
                    keys = kv.k[pages, 0].reshape(-1, s.k_dim)[:L].float()
                    vals = kv.v[pages, 0].reshape(-1, s.v_dim)[:L].float()
                    p = torch.softmax(keys @ qkv[at + j, : s.k_dim] * s.k_dim ** -0.5, dim=0)
                    out[at + j] = p @ vals
                at += n
            return (out @ self.o.t()).to(h.dtype)

    try:
        spec = tiny_spec([NarrowValueSpec(32, 16, 8), AttentionSpec(width=32, n_heads=2, n_kv_heads=2, head_dim=16,
                                                                    position=RotarySpec(16, 10000.0))])
        model = Model(spec, dtype="float32", device=cuda_device)
        w = random_bind(model, 21, scale=0.3)
        cache = model.new_cache(max_tokens=512, max_seqs=2)
        narrow = [g for g in cache.groups if g.request.v_head_dim][0]
        assert narrow.k.shape[-1] == 16 and narrow.v.shape[-1] == 8 and len(cache.groups) == 2
        assert narrow.bytes_per_token(4) == (16 + 8) * 4

        def plain(tokens):
            T = len(tokens)
            x = w["embedding.table"][np.asarray(tokens)]
            h = plain_llama.rmsnorm(x, w["blocks.0.mixer_norm.weight"], 1e-5)
            qk = h @ w["blocks.0.mixer.qk"].T
            q, k = qk[:, None, :16], qk[:, None, 16:]
            v = (h @ w["blocks.0.mixer.v"].T)[:, None, :]
            o = np.zeros((T, 8))
            for t in range(T):
                o[t] = plain_llama.softmax(k[: t + 1, 0] @ q[t, 0] * 0.25) @ v[: t + 1, 0]
            x = x + o @ w["blocks.0.mixer.o"].T
            h = plain_llama.rmsnorm(x, w["blocks.0.ffn_norm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, w["blocks.0.ffn.gate"], w["blocks.0.ffn.up"], w["blocks.0.ffn.down"])
            p = "blocks.1."
            h = plain_llama.rmsnorm(x, w[p + "mixer_norm.weight"], 1e-5)
            q2 = plain_llama.apply_rope((h @ w[p + "mixer.q"].T).reshape(T, 2, 16), range(T), 10000.0)
            k2 = plain_llama.apply_rope((h @ w[p + "mixer.k"].T).reshape(T, 2, 16), range(T), 10000.0)
            v2 = (h @ w[p + "mixer.v"].T).reshape(T, 2, 16)
            x = x + plain_llama.attention(q2, k2, v2, 0.25).reshape(T, 32) @ w[p + "mixer.o"].T
            h = plain_llama.rmsnorm(x, w[p + "ffn_norm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
            return plain_llama.rmsnorm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T

        toks = {"p": np.random.default_rng(2).integers(0, 50, 150).tolist(), "q": [4, 5, 6, 7]}
        ref = {k: plain(v) for k, v in toks.items()}
        for steps in (trace_whole(toks), trace_tail(toks, 20), trace_batches([{"p": (toks["p"], 9), "q": (toks["q"], 2)}])):
            compare(replay(model, cache, steps), ref, lambda r: 2e-4, "narrow values")
    finally:
        unregister("mixer", "toy_narrow_values")


def test_a_mixer_with_state_inside_recorded_decode_steps(cuda_device):
    """The toy decaying-sum mixer written against the step's device arrays (``ctx.slots``), so that
    it may be recorded: generation through the engine replays decode steps as CUDA graphs with the
    state of fixed size updated inside them; requests one after another reuse a slot, whose state
    must start at zero again."""
    from bitnet_c_b200.engine import ModelEngine, generate
    from bitnet_c_b200.sampling import SamplingParams

    @register_mixer("toy_decay_mix")
    class DecayMix(Mixer):
        graph_safe = True

        def params(self):
            return {"w": ParamSpec((self.spec.width, self.spec.width))}

        def bind(self, tensors):
            self.w = tensors["w"]

        def state_request(self):
            return StateRequest((self.spec.width,), torch.float32)

        def forward(self, h, ctx, kv, state):
            hf = h.float()
            if ctx.decode:  # one token per sequence: row b is sequence b; device arrays only
                idx = ctx.slots.long()
                s = state[idx] * self.spec.decay + hf
                state.index_copy_(0, idx, s)
                out = s
            else:
                out = torch.empty_like(hf)
                at = 0
                for slot, n in zip(ctx.host_slots, ctx.host_new):
                    s = state[slot]
                    for t in range(at, at + n):
                        s = self.spec.decay * s + hf[t]
                        out[t] = s
                    state[slot] = s
                    at += n
            return (out @ self.w.float().t()).to(h.dtype)

    try:
        attn = AttentionSpec(width=32, n_heads=2, n_kv_heads=2, head_dim=16, position=RotarySpec(16, 10000.0))
        spec = tiny_spec([DecayMixSpec(32, 0.8), attn])
        model = Model(spec, dtype="float32", device=cuda_device)
        assert model.graph_safe()
        w = random_bind(model, 31, scale=0.5)

        def plain_logits(tokens):
            T = len(tokens)
            x = w["embedding.table"][np.asarray(tokens)]
            h = plain_llama.rmsnorm(x, w["blocks.0.mixer_norm.weight"], 1e-5)
            s, rows = np.zeros(32), []
            for t in range(T):
                s = 0.8 * s + h[t]
                rows.append(s)
            x = x + np.stack(rows) @ w["blocks.0.mixer.w"].T
            h = plain_llama.rmsnorm(x, w["blocks.0.ffn_norm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, w["blocks.0.ffn.gate"], w["blocks.0.ffn.up"], w["blocks.0.ffn.down"])
            p = "blocks.1."
            h = plain_llama.rmsnorm(x, w[p + "mixer_norm.weight"], 1e-5)
            q = plain_llama.apply_rope((h @ w[p + "mixer.q"].T).reshape(T, 2, 16), range(T), 10000.0)
            k = plain_llama.apply_rope((h @ w[p + "mixer.k"].T).reshape(T, 2, 16), range(T), 10000.0)
            v = (h @ w[p + "mixer.v"].T).reshape(T, 2, 16)
            x = x + plain_llama.attention(q, k, v, 0.25).reshape(T, 32) @ w[p + "mixer.o"].T
            h = plain_llama.rmsnorm(x, w[p + "ffn_norm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, w[p + "ffn.gate"], w[p + "ffn.up"], w[p + "ffn.down"])
            return plain_llama.rmsnorm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T

        def plain_generate(prompt, n):
            toks = list(prompt)
            for _ in range(n):
                toks.append(int(np.argmax(plain_logits(toks)[-1])))
            return toks[len(prompt):]

        prompts = [np.random.default_rng(i).integers(0, 50, n).tolist() for i, n in enumerate([9, 1, 30, 4, 17])]
        new = [12, 5, 8, 12, 3]
        want = [plain_generate(p, n) for p, n in zip(prompts, new)]
        for max_batch in (5, 2, 1):  # together; two at a time; one after another in the same slot
            cache = model.new_cache(max_tokens=64 * max_batch * 2, max_seqs=max_batch)
            eng = ModelEngine(model, cache, SamplingParams(temperature=0.0))
            got = generate(eng, prompts, new, stop_ids=(), max_batch=max_batch)
            assert [c.tokens for c in got] == want, f"max_batch={max_batch}"
            assert eng.use_graphs and eng.runners and all(r.graphs for r in eng.runners.values())  # decode steps were recorded
    finally:
        unregister("mixer", "toy_decay_mix")
