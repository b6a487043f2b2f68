"""Two layers of the real layer sizes end to end against the plain implementation.

Fewer layers is not a smaller configuration: width, heads, head size, feed-forward width and
vocabulary are those of the 8B sizes (32 heads on 8 key/value heads of 128, vocabulary 128,256)
and of the 13B sizes (40 heads, none shared, vocabulary 32,000) that the benchmark and the kernel
tests use.  Every other model-level test runs at widths up to 256; here the tcgen05 products,
the TMA-fed attention kernels and the float32 path meet their real shapes inside a whole model.

The folder is written once in bfloat16 with the seeded generator evaluated on the device; the
bfloat16 engine loads it as it is and the float32 engine widens the same values, so one run of
the plain implementation (float32-kept weights, float64 products) serves both.
"""
import numpy as np
import pytest

import bitnet_c_b200 as bn
import plain_llama
from helpers import TOL_F32, compare, measured_bf16_bound, random_tokens, replay, trace_batches, trace_tail, trace_whole

pytestmark = [pytest.mark.gpu, pytest.mark.slow]

SIZES = {
    "8b": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336,
           "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
           "vocab_size": 128256, "max_position_embeddings": 4096, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
           "tie_word_embeddings": False, "hidden_act": "silu"},
    "13b": {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 5120, "intermediate_size": 13824,
            "num_hidden_layers": 2, "num_attention_heads": 40, "num_key_value_heads": 40, "head_dim": 128,
            "vocab_size": 32000, "max_position_embeddings": 4096, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "tie_word_embeddings": False, "hidden_act": "silu"},
}
LENGTHS = {"long": 300, "b0": 70, "b1": 200, "b2": 33}


@pytest.fixture(scope="module", params=list(SIZES))
def real(request, tmp_path_factory, cuda_device):
    cfg = SIZES[request.param]
    d = str(tmp_path_factory.mktemp("real") / request.param)
    bn.write_random_model(d, cfg, seed=17, dtype="bfloat16", device=cuda_device)
    pcfg, w = plain_llama.read_model(d, keep=np.float32)
    reqs = {r: random_tokens(500 + i, n, cfg["vocab_size"]) for i, (r, n) in enumerate(LENGTHS.items())}
    plain = {r: plain_llama.forward(pcfg, w, t) for r, t in reqs.items()}
    bounds = {r: measured_bf16_bound(pcfg, w, t, plain[r]) for r, t in reqs.items()}
    del w
    return dict(dir=d, reqs=reqs, plain=plain, bounds=bounds, models={})


def _model(real, dtype):
    if dtype not in real["models"]:
        real["models"].clear()  # one at a time on the device
        real["models"][dtype] = bn.load_model(real["dir"], dtype=dtype)
    return real["models"][dtype]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_whole_tail_and_unequal_batches_at_real_layer_sizes(real, dtype):
    m = _model(real, dtype)
    reqs, plain = real["reqs"], real["plain"]
    tol = real["bounds"] if dtype == "bfloat16" else (lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())))
    cache = m.new_cache(max_tokens=2048, max_seqs=4)
    got = replay(m, cache, trace_whole(reqs))
    compare(got, plain, tol, f"whole, {dtype}")
    got = replay(m, cache, trace_tail({"long": reqs["long"]}, 32))
    compare(got, plain, tol, f"last 32 one by one, {dtype}")
    batch = {"b0": (reqs["b0"], 6), "b1": (reqs["b1"], 12), "b2": (reqs["b2"], 3)}
    got = replay(m, cache, trace_batches([batch, {"long": (reqs["long"], 8)}]))
    compare(got, plain, tol, f"unequal batch, {dtype}")
    assert cache.slots.n_free == cache.slots.n_slots
    m.check_kernels()


def test_the_bfloat16_bounds_at_real_sizes_are_a_few_roundings(real):
    for r, ref in real["plain"].items():
        assert real["bounds"][r] < 0.05 * float(np.abs(ref).max()), (r, real["bounds"][r], float(np.abs(ref).max()))


def test_a_step_of_more_than_2048_rows_takes_the_own_products_and_agrees_with_the_library_ones(real, monkeypatch):
    """At 2,048 rows and more the default policy sends the gate|up product (SwiGLU epilogue) and the O
    product (residual + norm epilogue) to the library's own tcgen05 kernel.  One ragged step of 2,100 + 40
    tokens: the last positions' logits are those of the same step with every many-row product on the
    library product and separate kernels, within the bound of a few roundings."""
    from bitnet_c_b200.csrc import ops
    from bitnet_c_b200.engine import SeqStep
    m = _model(real, "bfloat16")
    cfg_vocab = real["plain"]["long"].shape[-1]
    reqs = [random_tokens(900, 2100, cfg_vocab), random_tokens(901, 40, cfg_vocab)]

    def run():
        cache = m.new_cache(max_tokens=2304, max_seqs=2)
        slots = [cache.open() for _ in reqs]
        out = m.step(cache, [SeqStep(slot=s, tokens=t, want=[len(t) - 1]) for s, t in zip(slots, reqs)])
        for s in slots:
            cache.close(s)
        return out.float().cpu().numpy()

    assert ops.USE_OWN_GEMM == "fused"
    kinds = []
    real_gemm = ops.gemm_tc
    monkeypatch.setattr(ops, "gemm_tc", lambda *a, **k: (kinds.append("sink" if k.get("sink") is not None else
                                                                      "swiglu" if k.get("swiglu") else "plain"),
                                                         real_gemm(*a, **k))[1])
    own = run()
    assert "sink" in kinds and "swiglu" in kinds
    monkeypatch.setattr(ops, "USE_OWN_GEMM", False)
    kinds.clear()
    lib = run()
    assert not kinds
    bound = max(real["bounds"].values())
    assert np.abs(own - lib).max() < bound, (float(np.abs(own - lib).max()), bound)
    m.check_kernels()
