"""Each CUDA kernel alone against a plain PyTorch/NumPy float32-or-better reference of the same
operation, at sizes other than the engine's test models."""
import numpy as np
import pytest
import torch

import bitnet_c_b200  # noqa: F401
from bitnet_c_b200.csrc import ops
import plain_llama

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == "float32" else bf16


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab", [(72, 101), (4096, 777)])
def test_embed_gather(cuda_device, dtype, width, vocab):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(vocab, width, generator=g).to(DT[dtype]).to(cuda_device)
    toks = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32, device=cuda_device)
    out = torch.full((5, width), 7.0, device=cuda_device)
    bad = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    ops.embed_gather(table, toks, out, bad)
    assert torch.equal(out, table.float()[toks.long()])
    assert bad.item() == 0
    toks[2] = vocab  # outside: zero row and flag, nothing read out of bounds
    ops.embed_gather(table, toks, out, bad)
    assert bad.item() == 1 and out[2].abs().max().item() == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,width,eps", [(5, 72, 1e-5), (3, 4096, 1e-6), (2, 13000, 1e-3)])
def test_add_rmsnorm(cuda_device, dtype, rows, width, eps):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(rows, width, generator=g).to(cuda_device) * 3
    delta = torch.randn(rows, width, generator=g).to(DT[dtype]).to(cuda_device)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DT[dtype]).to(cuda_device)
    ref_x = x.double() + delta.double()
    ref = ref_x / torch.sqrt((ref_x * ref_x).mean(-1, keepdim=True) + eps) * w.double()
    out = torch.empty(rows, width, dtype=DT[dtype], device=cuda_device)
    x1 = x.clone()
    ops.add_rmsnorm(x1, delta, w, eps, out)
    assert (x1.double() - ref_x).abs().max().item() < 1e-6
    assert (out.double() - ref).abs().max().item() < tol(dtype, 1e-5, 3e-2)
    # with a row index: only those rows, x untouched, no delta
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=cuda_device)
    out2 = torch.empty(2, width, dtype=DT[dtype], device=cuda_device)
    x2 = x.clone()
    ops.add_rmsnorm(x2, None, w, eps, out2, rows=idx)
    r2 = x.double()[idx.long()]
    r2 = r2 / torch.sqrt((r2 * r2).mean(-1, keepdim=True) + eps) * w.double()
    assert torch.equal(x2, x)
    assert (out2.double() - r2).abs().max().item() < tol(dtype, 1e-5, 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_silu_mul(cuda_device, dtype):
    g = torch.Generator().manual_seed(3)
    h = (torch.randn(7, 2 * 200, generator=g) * 3).to(DT[dtype]).to(cuda_device)
    out = torch.empty(7, 200, dtype=DT[dtype], device=cuda_device)
    ops.silu_mul(h, out)
    hh = h.double().reshape(7, 25, 2, 8)  # alternating blocks of 8 gate and 8 up values
    gte, up = hh[:, :, 0].reshape(7, 200), hh[:, :, 1].reshape(7, 200)
    ref = gte / (1 + torch.exp(-gte)) * up
    err = (out.double() - ref).abs()
    # one rounding of the result: relative 2^-9 in bfloat16, 2^-24 in float32 (plus expf's ulps)
    rel = 2.0 ** -8 if dtype == "bfloat16" else 1e-6
    assert (err <= rel * ref.abs() + 1e-6).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 50, 72), (8, 333, 4096), (11, 17, 200), (16, 1000, 64)])
def test_linear_skinny(cuda_device, dtype, M, N, K):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, K, generator=g).to(DT[dtype]).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(DT[dtype]).to(cuda_device)
    y = ops.linear(x, w, out_dtype=torch.float32)
    ref = x.double() @ w.double().t()
    assert y.dtype == torch.float32 and y.shape == (M, N)
    assert (y.double() - ref).abs().max().item() < 1e-4 * max(1.0, K / 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_linear_many_rows_is_float32_exact(cuda_device, dtype):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(100, 512, generator=g).to(DT[dtype]).to(cuda_device)
    w = (torch.randn(300, 512, generator=g) * 0.05).to(DT[dtype]).to(cuda_device)
    y = ops.linear(x, w, out_dtype=torch.float32)
    ref = x.double() @ w.double().t()
    # float32 accumulation of exact products: no tf32, no bf16 output rounding
    assert (y.double() - ref).abs().max().item() < 2e-5


def _paged_cache(cuda_device, dtype, n_pages, kv, hd, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n_pages, kv, 64, hd, generator=g).to(DT[dtype]).to(cuda_device)
    v = torch.randn(n_pages, kv, 64, hd, generator=g).to(DT[dtype]).to(cuda_device)
    return k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,rd,theta,pos", [(4, 2, 16, 16, 1e4, [0, 5, 63, 64]), (3, 1, 48, 48, 5e5, [700, 1, 129, 130]),
                                                  (5, 5, 128, 128, 1e6, [4000, 4001, 3, 64]),
                                                  (3, 3, 64, 32, 1e4, [7, 8, 200, 64]), (2, 1, 64, 40, 1e4, [7, 8, 200, 64])])
def test_rope_append(cuda_device, dtype, H, KV, hd, rd, theta, pos):
    """Rotation in place and the cache write; ``rd`` rotary dimensions of ``hd`` (the last case is
    no multiple of 16 and takes the element-wise kernel in bfloat16 too)."""
    T = len(pos)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(T, (H + 2 * KV) * hd, generator=g).to(DT[dtype]).to(cuda_device)
    x0 = x.clone()
    # two sequences: tokens 0,1 in slot 2; tokens 2,3 in slot 0; scattered pages
    tok_seq = torch.tensor([0, 0, 1, 1], dtype=torch.int32, device=cuda_device)
    tok_pos = torch.tensor(pos, dtype=torch.int32, device=cuda_device)
    slots = torch.tensor([2, 0], dtype=torch.int32, device=cuda_device)
    n_pages, per_seq = 200, 64
    perm = torch.randperm(n_pages, generator=g)[: 3 * per_seq].reshape(3, per_seq).to(torch.int32).to(cuda_device)
    k, v = _paged_cache(cuda_device, dtype, n_pages, KV, hd, 7)
    k0, v0 = k.clone(), v.clone()
    scale = float(np.power(np.float32(theta), np.float32(-2.0) / np.float32(rd)))
    ops.rope_append(x, H + KV, hd, rd, scale, tok_pos, k_off=H * hd, v_off=(H + KV) * hd, n_kv_heads=KV,
                    tok_seq=tok_seq, slots=slots, page_table=perm, k_cache=k, v_cache=v)
    heads = x0.double().cpu().numpy().reshape(T, H + 2 * KV, hd)
    rot = plain_llama.apply_rope(heads[:, : H + KV], pos, theta, dims=rd)
    got = x.double().cpu().numpy().reshape(T, H + 2 * KV, hd)
    t_ = tol(dtype, 2e-6, 2e-2)
    assert np.abs(got[:, : H + KV] - rot).max() < t_
    assert np.array_equal(got[:, H + KV:], heads[:, H + KV:])  # values untouched
    touched = torch.zeros_like(k, dtype=torch.bool)
    for t in range(T):
        slot = [2, 2, 0, 0][t]
        page = perm[slot, pos[t] // 64].item()
        row = pos[t] % 64
        assert np.abs(k[page, :, row].double().cpu().numpy() - got[t, H:H + KV]).max() == 0
        assert torch.equal(v[page, :, row], x0.reshape(T, H + 2 * KV, hd)[t, H + KV:])
        touched[page, :, row] = True
    assert torch.equal(k[~touched], k0[~touched]) and torch.equal(v[~touched], v0[~touched])


def _attention_reference(q, k_seq, v_seq, scale, window):
    return plain_llama.attention(q, k_seq, v_seq, scale, window)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,lens,news,window", [
    (4, 2, 16, [5, 64, 130], [5, 1, 3], 0),
    (3, 1, 48, [200, 1, 65], [200, 1, 1], 0),
    (8, 2, 128, [300, 129], [2, 129], 0),
    (2, 2, 256, [70], [70], 0),
    (4, 4, 32, [150, 40], [150, 1], 17),
])
def test_attention_general(cuda_device, dtype, H, KV, hd, lens, news, window):
    """Sequences of total length ``lens`` whose last ``news`` tokens are new; keys live in
    scattered pages; one query and key are scaled so that a far key dominates its row."""
    g = torch.Generator().manual_seed(8)
    n_seq, n_pages, per_seq = len(lens), 64, 8
    perm = torch.randperm(n_pages, generator=g)[: n_seq * per_seq].reshape(n_seq, per_seq).to(torch.int32)
    k, v = _paged_cache(cuda_device, dtype, n_pages, KV, hd, 9)
    ks = [torch.randn(L, KV, hd, generator=g).to(DT[dtype]) for L in lens]
    vs = [torch.randn(L, KV, hd, generator=g).to(DT[dtype]) for L in lens]
    qs = [torch.randn(n, H, hd, generator=g).to(DT[dtype]) * 0.5 for n in news]
    # a far key that must win: key 1 of sequence 0 (if it has one) lines up with the last query
    if lens[0] > 2 and window == 0:
        ks[0][1, 0] = (qs[0][-1, 0].float() * 4).to(DT[dtype])
    slots = list(range(n_seq))[::-1]
    for s, L in enumerate(lens):
        for p in range(L):
            page = perm[slots[s], p // 64].item()
            k[page, :, p % 64] = ks[s][p].to(cuda_device)
            v[page, :, p % 64] = vs[s][p].to(cuda_device)
    q = torch.cat([x.reshape(x.shape[0], H * hd) for x in qs]).contiguous().to(cuda_device)
    T = q.shape[0]
    tok_seq = torch.tensor(sum(([s] * n for s, n in enumerate(news)), []), dtype=torch.int32, device=cuda_device)
    tok_pos = torch.tensor(sum((list(range(L - n, L)) for L, n in zip(lens, news)), []), dtype=torch.int32,
                           device=cuda_device)
    out = torch.empty(T, H * hd, dtype=DT[dtype], device=cuda_device)
    ops.attention_general(q, H * hd, out, T, H, KV, hd, hd ** -0.5, window, tok_seq, tok_pos,
                          torch.tensor(slots, dtype=torch.int32, device=cuda_device), perm.to(cuda_device), k, v)
    got = out.double().cpu().numpy().reshape(T, H, hd)
    at = 0
    for s, (L, n) in enumerate(zip(lens, news)):
        qfull = np.zeros((L, H, hd))
        qfull[L - n:] = qs[s].double().numpy()
        ref = _attention_reference(qfull, ks[s].double().numpy(), vs[s].double().numpy(), hd ** -0.5, window)[L - n:]
        err = np.abs(got[at:at + n] - ref).max()
        assert err < tol(dtype, 2e-5, 2e-2), f"sequence {s}: {err}"
        at += n


def test_argmax_ties_and_sizes(cuda_device):
    g = torch.Generator().manual_seed(10)
    logits = torch.randn(5, 3001, generator=g).to(cuda_device)
    logits[0, 100] = logits[0, 2000] = 50.0  # tie: lower index wins
    logits[1, 3000] = 60.0
    logits[2, 0] = 60.0
    got = ops.argmax(logits).cpu().tolist()
    ref = [int(np.argmax(r)) for r in logits.cpu().numpy()]
    assert got == ref and got[0] == 100


def test_sample_temperature_follows_the_reference_walk(cuda_device):
    V, rows, temp = 1013, 6, 0.8
    g = torch.Generator().manual_seed(11)
    logits = (torch.randn(rows, V, generator=g) * 2).to(cuda_device)
    seeds = [42, 1, 7, 123456789, 99, 2**40 + 5]
    state = torch.tensor(seeds, dtype=torch.int64, device=cuda_device)
    rngs = [plain_llama.Xorshift64Star(s) for s in seeds]
    for _ in range(5):
        got = ops.sample_temperature(logits, temp, state).cpu().tolist()
        for r in range(rows):
            want = plain_llama.sample(logits[r].cpu().numpy(), temp, 1.0, rngs[r])
            if got[r] != want:
                # only a draw within rounding of a boundary of the cumulative sum may differ, by one place
                assert abs(got[r] - want) == 1, (r, got[r], want)
        assert state.cpu().tolist() == [np.int64(np.uint64(x.state)) for x in rngs]


@pytest.mark.parametrize("V,topp,temp", [(1013, 0.9, 0.8), (50, 0.51, 1.3), (128256, 0.9, 0.7), (4099, 0.999, 1.0),
                                         (331, 0.05, 0.6)])
def test_sample_topp_follows_the_reference_nucleus(cuda_device, V, topp, temp):
    """Nucleus sampling against the plain sort-based one: peaked and flat rows, rows with many equal
    logits (ties go by index), a row where one token holds nearly all the mass, large vocabularies.
    (The plain running sums are float32 in sorted order, as the reference's; the kernel's masses are
    exact.  They can part only where a sum lands within rounding of topp or of the draw, so no
    case here puts a sum of equal probabilities exactly on topp.)"""
    rows = 6
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(rows, V, generator=g) * 2
    logits[1] = torch.round(logits[1])            # many ties
    logits[2] *= 4                                # peaked
    logits[3] *= 0.05                             # flat: almost everything is a candidate
    logits[4, 7] = 60.0                           # one token takes the whole nucleus
    logits[5] = 0.0                               # all equal
    logits = logits.to(cuda_device)
    seeds = [42, 1, 7, 123456789, 99, 2**40 + 5]
    state = torch.tensor(seeds, dtype=torch.int64, device=cuda_device)
    rngs = [plain_llama.Xorshift64Star(s) for s in seeds]
    differ = 0
    for _ in range(4):
        got = ops.sample_topp(logits, temp, topp, state).cpu().tolist()
        for r in range(rows):
            want = plain_llama.sample(logits[r].cpu().numpy(), temp, topp, rngs[r])
            if got[r] != want:
                # only a draw within float32 rounding of a boundary of a running sum may differ
                # (the plain sums run in float32 in sorted order, the kernel's are exact)
                differ += 1
                pl = torch.softmax(logits[r].double().cpu() / temp, 0)
                assert abs(pl[got[r]].item() - pl[want].item()) <= 1e-3 * max(pl[got[r]].item(), pl[want].item()) + 1e-9 or \
                    abs(torch.argsort(-pl, stable=True).tolist().index(got[r]) - torch.argsort(-pl, stable=True).tolist().index(want)) <= 1, (r, got[r], want)
        assert state.cpu().tolist() == [np.int64(np.uint64(x.state)) for x in rngs]
    # a float32 running sum over V terms is off by up to about V * 2^-24 of the total; that is below
    # one token's mass only while V is small, so only there must (nearly) every draw agree exactly
    if V < 5000:
        assert differ <= 2


def test_repeat_penalty(cuda_device):
    logits = torch.tensor([[1.0, -2.0, 3.0, 4.0, -5.0], [1.0, 1.0, 1.0, 1.0, 1.0]], device=cuda_device)
    recent = torch.tensor([[2, 4, 2, 9, 0], [1, 1, 1, 1, 1]], dtype=torch.int32, device=cuda_device)
    n = torch.tensor([4, 2], dtype=torch.int32, device=cuda_device)
    ops.repeat_penalty(logits, recent, n, 2.0)
    assert logits.cpu().tolist() == [[1.0, -2.0, 1.5, 4.0, -10.0], [1.0, 0.5, 1.0, 1.0, 1.0]]


@pytest.mark.parametrize("M,N,K", [(1, 64, 128), (3, 50, 72), (8, 333, 4096), (9, 1000, 200), (16, 64, 1000),
                                   (33, 130, 264), (64, 272, 2048)])
@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
def test_linear_small_batch_store_and_partials(cuda_device, monkeypatch, impl, M, N, K):
    """The tensor-core small-batch products (tcgen05 in linear_tc.cu; mma.sync in linear_mma.cu, the
    second implementation, reached with ``ops.USE_TCGEN05`` off): every row count up to 64, sizes
    that are no multiple of their tiles."""
    monkeypatch.setattr(ops, "USE_TCGEN05", impl == "tcgen05")
    g = torch.Generator().manual_seed(12)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    ref = x.double() @ w.double().t()
    bound = 2e-5 * max(1.0, K / 64)
    y = ops.linear(x, w, out_dtype=torch.float32)
    assert y.shape == (M, N) and (y.double() - ref).abs().max().item() < bound
    yb = ops.linear(x, w)
    assert yb.dtype == torch.bfloat16 and ((yb.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + bound).all()
    parts = ops.linear(x, w, partial_sums=True)
    if K >= 1024:
        assert parts.dim() == 3 and parts.dtype == torch.float32 and parts.shape[0] > 1
    total = parts.double().sum(0) if parts.dim() == 3 else parts.double()
    assert (total - ref).abs().max().item() < (bound if parts.dim() == 3 else 2.0 ** -7 * ref.abs().max().item() + bound)
    # partial sums feed the residual add of the norm
    if parts.dim() == 3:
        xres = torch.randn(M, N, generator=g).to(cuda_device)
        wn = torch.ones(N, device=cuda_device)
        out = torch.empty(M, N, device=cuda_device)
        x2 = xres.clone()
        ops.add_rmsnorm(x2, parts, wn, 1e-5, out)
        assert (x2.double() - (xres.double() + ref)).abs().max().item() < bound + 1e-6


@pytest.mark.parametrize("M,I,K", [(1, 16, 64), (8, 176, 64), (20, 200, 120), (64, 256, 96)])
@pytest.mark.parametrize("impl", ["tcgen05", "mma"])
def test_linear_small_batch_swiglu_epilogue(cuda_device, monkeypatch, impl, M, I, K):
    monkeypatch.setattr(ops, "USE_TCGEN05", impl == "tcgen05")
    g = torch.Generator().manual_seed(13)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    gate = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16).to(cuda_device)
    up = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16).to(cuda_device)
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[:8], gate[:8]) and torch.equal(w[8:16], up[:8]) and torch.equal(w[16:24], gate[8:16])
    a, b = x.double() @ gate.double().t(), x.double() @ up.double().t()
    ref = a / (1 + torch.exp(-a)) * b
    y = ops.linear(x, w, out_dtype=torch.float32, swiglu=True)
    assert y.shape == (M, I) and (y.double() - ref).abs().max().item() < 1e-4
    # many rows: library product, then the activation kernel on the same layout
    xl = torch.randn(80, K, generator=g).to(torch.bfloat16).to(cuda_device)
    a, b = xl.double() @ gate.double().t(), xl.double() @ up.double().t()
    yl = ops.linear(xl, w, swiglu=True)
    refl = a / (1 + torch.exp(-a)) * b
    assert yl.shape == (80, I) and ((yl.double() - refl).abs() <= 2.0 ** -6 * refl.abs() + 2e-2).all()


@pytest.mark.parametrize("H,KV,hd,lens,window", [
    (4, 2, 16, [1, 5, 64, 130], 0), (3, 1, 48, [200, 129, 128], 0), (32, 8, 128, [700, 3], 0),
    (2, 2, 256, [257], 0), (40, 40, 64, [100, 300], 0), (12, 1, 32, [150, 40, 260], 17), (4, 4, 80, [513], 130),
    (32, 1, 64, [300, 70], 0), (40, 1, 128, [200, 513], 0), (80, 2, 64, [140, 66], 0),  # 32 and 40 query heads on one key/value head
])
def test_attention_decode(cuda_device, H, KV, hd, lens, window):
    """One new token per sequence over scattered pages; a far key is made to dominate one row."""
    g = torch.Generator().manual_seed(14)
    n_seq, n_pages, per_seq = len(lens), 80, 16
    perm = torch.randperm(n_pages, generator=g)[: n_seq * per_seq].reshape(n_seq, per_seq).to(torch.int32)
    k, v = _paged_cache(cuda_device, "bfloat16", n_pages, KV, hd, 15)
    ks = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]
    vs = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]
    q = (torch.randn(n_seq, H, hd, generator=g) * 0.5).to(torch.bfloat16)
    if lens[0] > 140 and window == 0:
        ks[0][2, 0] = (q[0, 0].float() * 4).to(torch.bfloat16)  # key 2, three chunks back, must win for head 0
    slots = list(range(n_seq))[::-1]
    for s, L in enumerate(lens):
        for p in range(L):
            page = perm[slots[s], p // 64].item()
            k[page, :, p % 64] = ks[s][p].to(cuda_device)
            v[page, :, p % 64] = vs[s][p].to(cuda_device)
    # q sits in a wider row, as in the packed q|k|v buffer
    wide = torch.zeros(n_seq, H * hd + 32, dtype=torch.bfloat16, device=cuda_device)
    wide[:, : H * hd] = q.reshape(n_seq, H * hd).to(cuda_device)
    out = torch.empty(n_seq, H * hd, dtype=torch.bfloat16, device=cuda_device)
    ops.attention_decode(wide, wide.shape[1], out, n_seq, H, KV, hd, hd ** -0.5, window,
                         torch.tensor([L - 1 for L in lens], dtype=torch.int32, device=cuda_device),
                         torch.tensor(slots, dtype=torch.int32, device=cuda_device), perm.to(cuda_device), k, v,
                         max(lens))
    got = out.double().cpu().numpy().reshape(n_seq, H, hd)
    for s, L in enumerate(lens):
        qfull = np.zeros((L, H, hd))
        qfull[L - 1] = q[s].double().numpy()
        ref = plain_llama.attention(qfull, ks[s].double().numpy(), vs[s].double().numpy(), hd ** -0.5, window)[L - 1]
        assert np.abs(got[s] - ref).max() < 2e-2, f"sequence {s}"


@pytest.mark.parametrize("H,KV,hd,lens,news,window", [
    (4, 2, 16, [5, 64, 130], [5, 1, 3], 0),
    (3, 1, 48, [200, 1, 65], [200, 1, 1], 0),
    (8, 2, 128, [300, 129], [2, 129], 0),
    (2, 2, 256, [70, 200], [70, 136], 0),
    (4, 4, 32, [150, 40], [150, 1], 17),
    (6, 3, 80, [513], [260], 100),
    (32, 8, 128, [700], [700], 0),
    (5, 5, 64, [130, 300, 64], [128, 129, 64], 0),
    (4, 1, 112, [400, 90], [399, 3], 130),
])
@pytest.mark.parametrize("impl", ["mma", "tcgen05"])
def test_attention_prefill(cuda_device, impl, H, KV, hd, lens, news, window):
    """The tensor-core prefill kernels (mma.sync with 64-row blocks, tcgen05 with 128-row blocks):
    ragged runs of new tokens after cached ones, scattered pages, head sizes that are padded inside
    the kernel, windows, a far key that must dominate, a late key that raises a row's maximum by
    far more than the rescaling threshold, and non-finite leftovers behind a sequence's end."""
    if impl == "tcgen05" and hd > 128:
        pytest.skip("the tcgen05 kernel takes head sizes up to 128")
    from bitnet_c_b200.engine import SeqStep, pack_step
    g = torch.Generator().manual_seed(16)
    n_seq, n_pages, per_seq = len(lens), 64, 16
    perm = torch.randperm(n_pages, generator=g)[: n_seq * per_seq].reshape(n_seq, per_seq).to(torch.int32)
    k, v = _paged_cache(cuda_device, "bfloat16", n_pages, KV, hd, 17)
    ks = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]
    vs = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]
    qs = [(torch.randn(n, H, hd, generator=g) * 0.5).to(torch.bfloat16) for n in news]
    if lens[0] > 2 and window == 0:
        ks[0][1, 0] = (qs[0][-1, 0].float() * 4).to(torch.bfloat16)
    if lens[0] > 200:
        ks[0][lens[0] - 3, 0] = (qs[0][-1, 0].float() * 9).to(torch.bfloat16)
    slots = list(range(n_seq))[::-1]
    for s, L in enumerate(lens):
        for p in range(L):
            page = perm[slots[s], p // 64].item()
            k[page, :, p % 64] = ks[s][p].to(cuda_device)
            v[page, :, p % 64] = vs[s][p].to(cuda_device)
        if L % 64:  # whatever lies behind the sequence's end in its last page must not reach the result
            page = perm[slots[s], (L - 1) // 64].item()
            k[page, :, L % 64:] = float("nan")
            v[page, :, L % 64:] = float("inf")
    T = sum(news)
    wide = torch.zeros(T, H * hd + 2 * KV * hd, dtype=torch.bfloat16, device=cuda_device)
    wide[:, : H * hd] = torch.cat([x.reshape(x.shape[0], H * hd) for x in qs]).to(cuda_device)
    ctx = pack_step([SeqStep(slots[i], [0] * news[i]) for i in range(n_seq)], [L - n for L, n in zip(lens, news)],
                    cuda_device)
    out = torch.full((T, H * hd), 7.0, dtype=torch.bfloat16, device=cuda_device)
    if impl == "mma":
        ops.attention_prefill(wide, wide.shape[1], out, H, KV, hd, hd ** -0.5, window, ctx.tile_seq, ctx.tile_row0,
                              ctx.seq_start, ctx.seq_pos0, ctx.slots, perm.to(cuda_device), k, v)
    else:
        ops.attention_prefill_tc(wide, wide.shape[1], out, H, KV, hd, hd ** -0.5, window, ctx.wide_tile_seq,
                                 ctx.wide_tile_row0, ctx.seq_start, ctx.seq_pos0, ctx.slots, perm.to(cuda_device), k, v)
        ops.check_tc_status(cuda_device)
    got = out.double().cpu().numpy().reshape(T, H, hd)
    at = 0
    for s, (L, n) in enumerate(zip(lens, news)):
        qfull = np.zeros((L, H, hd))
        qfull[L - n:] = qs[s].double().numpy()
        ref = plain_llama.attention(qfull, ks[s].double().numpy(), vs[s].double().numpy(), hd ** -0.5, window)[L - n:]
        err = np.abs(got[at:at + n] - ref).max()
        assert err < 2e-2, f"sequence {s}: {err}"
        at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_add_rmsnorm_with_partial_sums_and_few_rows(cuda_device, dtype):
    """Wide rows and few of them take the path that spreads a row over a cluster of blocks."""
    g = torch.Generator().manual_seed(18)
    rows, width, parts = 6, 2048, 5
    x = torch.randn(rows, width, generator=g).to(cuda_device)
    delta = torch.randn(parts, rows, width, generator=g).to(cuda_device)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DT[dtype]).to(cuda_device)
    ref_x = x.double() + delta.double().sum(0)
    ref = ref_x / torch.sqrt((ref_x * ref_x).mean(-1, keepdim=True) + 1e-5) * w.double()
    out = torch.empty(rows, width, dtype=DT[dtype], device=cuda_device)
    x1 = x.clone()
    ops.add_rmsnorm(x1, delta, w, 1e-5, out)
    assert (x1.double() - ref_x).abs().max().item() < 1e-5
    assert (out.double() - ref).abs().max().item() < tol(dtype, 1e-5, 3e-2)
    idx = torch.tensor([4, 1], dtype=torch.int32, device=cuda_device)
    out2 = torch.empty(2, width, dtype=DT[dtype], device=cuda_device)
    x2 = x.clone()
    ops.add_rmsnorm(x2, delta, w, 1e-5, out2, rows=idx)
    assert torch.equal(x2, x)
    assert (out2.double() - ref[idx.long()]).abs().max().item() < tol(dtype, 1e-5, 3e-2)


def test_rope_partial_rotation_and_plain_append(cuda_device):
    """rotary_dims below head_dim leaves the upper dimensions as they are (they still reach the cache);
    with no rotation at all the kernel is a plain append."""
    H, KV, hd, rd, theta = 2, 2, 32, 16, 10000.0
    g = torch.Generator().manual_seed(19)
    x = torch.randn(3, (H + 2 * KV) * hd, generator=g).to(cuda_device)
    x0 = x.clone()
    tok_seq = torch.zeros(3, dtype=torch.int32, device=cuda_device)
    tok_pos = torch.tensor([62, 63, 64], dtype=torch.int32, device=cuda_device)
    slots = torch.tensor([1], dtype=torch.int32, device=cuda_device)
    pt = torch.tensor([[0, 0], [5, 2]], dtype=torch.int32, device=cuda_device)
    k = torch.zeros(8, KV, 64, hd, device=cuda_device)
    v = torch.zeros(8, KV, 64, hd, device=cuda_device)
    scale = float(np.power(np.float32(theta), np.float32(-2.0) / np.float32(rd)))
    ops.rope_append(x, H + KV, hd, rd, scale, tok_pos, k_off=H * hd, v_off=(H + KV) * hd, n_kv_heads=KV,
                    tok_seq=tok_seq, slots=slots, page_table=pt, k_cache=k, v_cache=v)
    heads = x0.double().cpu().numpy().reshape(3, H + 2 * KV, hd)
    rot = plain_llama.apply_rope(heads[:, : H + KV], [62, 63, 64], theta, dims=rd)
    got = x.double().cpu().numpy().reshape(3, H + 2 * KV, hd)
    assert np.abs(got[:, : H + KV] - rot).max() < 2e-6
    assert np.array_equal(got[:, : H + KV, rd:], heads[:, : H + KV, rd:])
    for t, (page, row) in enumerate([(5, 62), (5, 63), (2, 0)]):
        assert np.array_equal(k[page, :, row].double().cpu().numpy(), got[t, H:H + KV])
        assert np.array_equal(v[page, :, row].double().cpu().numpy(), heads[t, H + KV:])
    k2, v2 = torch.zeros_like(k), torch.zeros_like(v)
    ops.rope_append(x0.clone(), 0, hd, 0, 1.0, tok_pos, k_off=H * hd, v_off=(H + KV) * hd, n_kv_heads=KV,
                    tok_seq=tok_seq, slots=slots, page_table=pt, k_cache=k2, v_cache=v2)
    assert np.array_equal(k2[5, :, 62].double().cpu().numpy(), heads[0, H:H + KV]) and torch.equal(v2, v)


def test_argmax_large_vocabulary(cuda_device):
    g = torch.Generator().manual_seed(20)
    logits = torch.randn(9, 128256, generator=g).to(cuda_device)
    logits[0, 77] = logits[0, 100000] = 40.0
    logits[1, 128255] = 41.0
    logits[2, :] = -float("inf")
    got = ops.argmax(logits).cpu().tolist()
    ref = [int(np.argmax(r)) for r in logits.cpu().numpy()]
    assert got == ref and got[0] == 77 and got[2] == 0
    assert ops.argmax(logits).cpu().tolist() == ref  # the tickets were left at zero


def _last_row_attention(q, k, v, scale, window):
    """Attention of the last position only (q [H, hd], k and v [L, KV, hd]) in float64, the formulas
    of plain_llama.attention restricted to one row so that long sequences stay cheap."""
    L, KV, _ = k.shape
    H = q.shape[0]
    lo = max(0, L - window) if window else 0
    out = np.zeros_like(q)
    for h in range(H):
        kh = h // (H // KV)
        sc = k[lo:, kh] @ q[h] * scale
        w = np.exp(sc - sc.max())
        out[h] = (w / w.sum()) @ v[lo:, kh]
    return out


@pytest.mark.parametrize("H,KV,hd,rd,lens,window", [
    (4, 2, 16, 16, [1, 5, 64, 130], 0), (3, 1, 48, 48, [200, 129, 128], 0), (32, 8, 128, 128, [700, 3, 513], 0),
    (2, 2, 256, 64, [257], 0), (40, 40, 64, 0, [100, 300], 0), (12, 1, 32, 32, [150, 40, 260], 17),
    (40, 40, 128, 128, [3000, 17, 2049], 0), (32, 8, 64, 64, [2303, 1], 0), (8, 2, 128, 128, [5000, 4097], 1024),
    (4, 2, 64, 40, [70, 200], 0),  # rotary dimensions that are no multiple of 16
    (8, 1, 128, 128, [20000], 0),  # one long sequence: more blocks than a cluster holds, chosen by the policy
    # more than 16 query heads on one key/value head: two and three blocks of 16 rows per head
    (32, 1, 64, 64, [300, 70, 1100], 0), (40, 1, 128, 128, [200, 513], 0), (80, 2, 64, 64, [140, 1030], 0),
    # 60 sequences x 8 key/value heads = 480 blocks without splits: more than the GPU holds at once
    (32, 8, 128, 128, [130 + (37 * i) % 300 for i in range(56)] + [192, 193, 256, 257], 0),
])
@pytest.mark.parametrize("splits", [0, 3, 12, "list1", "list2", "list4"])
def test_attention_decode_fused(cuda_device, monkeypatch, splits, H, KV, hd, rd, lens, window):
    """The one-launch decode attention against plain rotary + attention: the new key and value must land
    in the cache (rotated / as they are) and the result must see them.  ``splits``: blocks per
    sequence, 0 = chosen from the batch; up to eight merge inside a thread-block cluster, more
    through global memory and a ticket.  "listN": a work list in groups of N (``ops.decode_items``):
    the sequences with more than 1/N of the longest one's pages get N blocks, the others one."""
    work_list = int(splits[4:]) if isinstance(splits, str) else 0
    if len(lens) > 8 and splits not in (0, "list2"):
        pytest.skip("the many-sequence case is there for launches without splits")
    monkeypatch.setattr(ops, "_FORCE_SPLITS", 0 if work_list else splits)
    g = torch.Generator().manual_seed(23)
    theta = 10000.0
    n_seq = len(lens)
    per_seq = max(16, (max(lens) + 63) // 64 + 1)
    n_pages = max(80, n_seq * per_seq + 7)
    perm = torch.randperm(n_pages, generator=g)[: n_seq * per_seq].reshape(n_seq, per_seq).to(torch.int32)
    k, v = _paged_cache(cuda_device, "bfloat16", n_pages, KV, hd, 24)
    ks = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]  # already rotated, cached
    vs = [torch.randn(L, KV, hd, generator=g).to(torch.bfloat16) for L in lens]
    raw = (torch.randn(n_seq, H + 2 * KV, hd, generator=g) * 0.7).to(torch.bfloat16)  # the new token's q|k|v
    slots = list(range(n_seq))[::-1]
    scale = float(np.power(np.float32(theta), np.float32(-2.0) / np.float32(rd))) if rd else 1.0
    pos = [L - 1 for L in lens]
    for s, L in enumerate(lens):
        if L < 1000:
            continue
        # among thousands of random keys a far one would hardly count: make the key at a third of
        # the sequence point along the first query of each group, so that its value is the result
        r = raw[s].double().numpy()
        rot = plain_llama.apply_rope(r[None, :H], [pos[s]], theta, dims=rd)[0] if rd else r[:H]
        for kh in range(KV):
            qv = rot[kh * (H // KV)]
            ks[s][L // 3, kh] = torch.from_numpy(qv / np.linalg.norm(qv) * 16.0 * hd ** 0.5 / np.linalg.norm(qv)).to(torch.bfloat16)
    for s, L in enumerate(lens):
        for p in range(L - 1):  # the last position is written by the kernel
            page = perm[slots[s], p // 64].item()
            k[page, :, p % 64] = ks[s][p].to(cuda_device)
            v[page, :, p % 64] = vs[s][p].to(cuda_device)
        # whatever lies behind the new position in its page must not reach the result
        page, row = perm[slots[s], (L - 1) // 64].item(), (L - 1) % 64
        k[page, :, row + 1:] = float("nan")
        v[page, :, row + 1:] = float("inf")
    k_before, v_before = k.clone(), v.clone()
    out = torch.empty(n_seq, H * hd, dtype=torch.bfloat16, device=cuda_device)
    extra = {}
    if work_list:
        group, items = ops.decode_items([p // 64 + 1 for p in pos], KV * ((H // KV + 15) // 16), group=work_list)
        assert group == work_list and len(items) % group == 0 and sorted(i & 0xFFFF for i in items if i >= 0 and not (i >> 16) & 0xFF) == list(range(n_seq))
        extra = {"items": torch.tensor(items, dtype=torch.int32, device=cuda_device), "item_group": group}
    ops.attention_decode_fused(raw.reshape(n_seq, -1).contiguous().to(cuda_device), H * hd, (H + KV) * hd, out, n_seq,
                               H, KV, hd, hd ** -0.5, window, rd, scale,
                               torch.tensor(pos, dtype=torch.int32, device=cuda_device),
                               torch.tensor(slots, dtype=torch.int32, device=cuda_device), perm.to(cuda_device), k, v,
                               max(lens), **extra)
    got = out.double().cpu().numpy().reshape(n_seq, H, hd)
    touched = torch.zeros_like(k, dtype=torch.bool)
    for s, L in enumerate(lens):
        r = raw[s].double().numpy()
        rot = plain_llama.apply_rope(r[None, : H + KV], [pos[s]], theta, dims=rd)[0] if rd else r[: H + KV]
        rot = plain_llama.to_bf16(rot)
        page, row = perm[slots[s], pos[s] // 64].item(), pos[s] % 64
        assert np.abs(k[page, :, row].double().cpu().numpy() - rot[H:]).max() < 2e-2
        assert np.array_equal(v[page, :, row].double().cpu().numpy(), r[H + KV:])
        touched[page, :, row] = True
        kfull = np.concatenate([ks[s][: L - 1].double().numpy(), rot[None, H:]])
        vfull = np.concatenate([vs[s][: L - 1].double().numpy(), r[None, H + KV:]])
        ref = _last_row_attention(rot[:H], kfull, vfull, hd ** -0.5, window)
        assert np.abs(got[s] - ref).max() < 2e-2, f"sequence {s}"
        if L >= 1000 and not window:
            for kh in range(KV):  # the marked key decides the first head of each group
                assert np.abs(ref[kh * (H // KV)] - vfull[L // 3, kh]).max() < 0.1
    bits = lambda t: t.view(torch.int16)
    assert torch.equal(bits(k)[~touched], bits(k_before)[~touched]) and torch.equal(bits(v)[~touched], bits(v_before)[~touched])
    ops.check_tc_status(cuda_device)


@pytest.mark.parametrize("M,N,K", [(65, 264, 72), (128, 256, 64), (200, 1000, 200), (333, 512, 4096), (1000, 6144, 512),
                                   (2048, 272, 1032), (2048, 4096, 576)])
@pytest.mark.parametrize("pairs", [True, False])
def test_gemm_tc_store_swiglu_and_norm_epilogues(cuda_device, pairs, M, N, K):
    """The many-row tcgen05 product with its epilogues: plain store (bfloat16 and float32), SwiGLU on
    the interleaved gate/up layout, residual add + next norm's gain + sums of squares, and rows that
    still lack their scale (the output of that epilogue) as input.  Sizes that are no multiples of
    the 128 x 256 x 64 tiles; more tiles than blocks.  ``pairs``: two blocks work as one
    (cta_group::2, tiles of 256 x 256) or every block alone."""
    ops.gemm_pairs(pairs)
    g = torch.Generator().manual_seed(40)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    ref = x.double() @ w.double().t()
    bound = 2e-5 * max(1.0, K / 64)
    y = ops.gemm_tc(x, w, out_dtype=torch.float32)
    assert y.shape == (M, N) and (y.double() - ref).abs().max().item() < bound
    yb = ops.gemm_tc(x, w)
    assert yb.dtype == torch.bfloat16 and ((yb.double() - ref).abs() <= 2.0 ** -8 * ref.abs() + bound).all()
    # SwiGLU: N/2 gate and N/2 up rows interleaved in blocks of 8
    I = N // 16 * 8
    gate, up = w[:I], (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    a, b = x.double() @ gate.double().t(), x.double() @ up.double().t()
    refs = a / (1 + torch.exp(-a)) * b
    ys = ops.gemm_tc(x, ops.interleave_gate_up(gate, up), out_dtype=torch.float32, swiglu=True)
    assert ys.shape == (M, I) and (ys.double() - refs).abs().max().item() < 10 * bound
    # residual + norm epilogue, then a product that consumes the rows that still lack their scale
    res = torch.randn(M, N, generator=g).to(cuda_device)
    gain = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(cuda_device)
    eps = 1e-5
    res2 = res.clone()
    rs = ops.gemm_tc(x, w, sink=ops.NormSink(res2, gain, eps))
    new = res.double() + ref
    assert (res2.double() - new).abs().max().item() < bound + 1e-6
    assert isinstance(rs, ops.RowScaled) and rs.ss.shape == ((N + 255) // 256, M)
    assert torch.equal(rs.dense(), ops.gemm_tc(x, w, sink=ops.NormSink(res.clone(), gain, eps)).dense())  # and the same again
    assert ((rs.ss.double().sum(0) - (new * new).sum(1)).abs() <= 1e-4 * (new * new).sum(1)).all()
    normed = new / torch.sqrt((new * new).mean(1, keepdim=True) + eps) * gain.double()
    assert (rs.dense().double() - normed).abs().max().item() < 3e-2
    w2 = (torch.randn(80, N, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    y2 = ops.gemm_tc(rs, w2, out_dtype=torch.float32)
    # the reference uses the rounded rows the kernel multiplied, then the scale
    xg = rs.x.double()
    scale = 1.0 / torch.sqrt(rs.ss.double().sum(0) / N + eps)
    assert (y2.double() - (xg @ w2.double().t()) * scale[:, None]).abs().max().item() < 2e-4 * max(1.0, N / 256)
    ops.check_tc_status(cuda_device)
    ops.gemm_pairs(True)


def test_linear_takes_the_own_gemm_when_asked(cuda_device, monkeypatch):
    g = torch.Generator().manual_seed(41)
    x = torch.randn(100, 512, generator=g).to(torch.bfloat16).to(cuda_device)
    w = (torch.randn(304, 512, generator=g) * 0.05).to(torch.bfloat16).to(cuda_device)
    a = ops.linear(x, w, out_dtype=torch.float32)
    monkeypatch.setattr(ops, "USE_OWN_GEMM", True)
    calls = []
    real = ops.gemm_tc
    monkeypatch.setattr(ops, "gemm_tc", lambda *p, **k: (calls.append(1), real(*p, **k))[1])
    b = ops.linear(x, w, out_dtype=torch.float32)
    assert calls and (a - b).abs().max().item() < 1e-4
