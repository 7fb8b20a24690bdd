"""Every mechanism of the Palilix family alone: the framework's op (sm_100a kernel on the `gpu` tier, its PyTorch path on the
plumbing tier) against the float64 oracle's function of the same mechanism.  Inputs are made so that a fault shows: a far
key that one query singles out among hundreds, keys on both sides of page borders, values beyond the clamp, a decay of
exactly one, rows wider than a kernel's register tile, odd widths that take the scalar paths."""
import math

import pytest
import torch

from colossalai_b200 import ops
from colossalai_b200.ops import mixers as M
from colossalai_b200.ops.moe import gather_combine

from . import oracle as O

TIERS = ["plumbing", pytest.param("gpu", marks=pytest.mark.gpu)]
F64 = torch.float64


def _dev(tier):
    if tier == "gpu" and not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return "cuda" if tier == "gpu" else "cpu"


def _rand(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def _close(got, want, tol):
    err = (got.double().cpu() - want).abs().max().item() / max(want.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e}"


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("dims,width", [(8, 8), (4, 12), (0, 6), (32, 32)])
def test_rotary_half_turns_the_first_channels_of_every_head(tier, dims, width):
    dev = _dev(tier)
    T, H, pad = 9, 3, 5                                  # heads sit `pad` columns into a wider row, strided out as well
    src = _rand(T, H * (width + pad) + 3, seed=1)
    pos = torch.tensor([0, 1, 2, 700, 701, 5, 31, 32, 4095], dtype=torch.int32)
    table = M.rotary_table(5000, max(dims, 2), 1e4, dev) if dims else torch.zeros(5000, 0, device=dev)
    dst = torch.zeros(T, H * (width + 1), device=dev)
    M.rotary_half(src.to(dev), dst, H, width + pad, pad, width + 1, 1, width, dims, table, pos.to(dev))
    x = torch.stack([src[:, h * (width + pad) + pad: h * (width + pad) + pad + width] for h in range(H)], 1).to(F64)
    want = O.rotate(x, pos.tolist(), dims, 1e4) if dims else x
    got = torch.stack([dst[:, h * (width + 1) + 1: (h + 1) * (width + 1)] for h in range(H)], 1)
    _close(got, want, 2e-6)
    assert float(dst[:, 0].abs().max()) == 0.0            # the column in front of every head is left alone


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("W", [48, 50, 1024, 8196])
@pytest.mark.parametrize("kind", ["layer", "rms", None])
def test_stream_sum_and_norm(tier, W, kind):
    dev = _dev(tier)
    T = 5
    x = _rand(T, W, seed=2, scale=3.0) + 1.5                       # a mean that a layer norm must take off
    a16 = _rand(T, W, seed=3).to(torch.bfloat16)
    a32 = _rand(T, W, seed=4)
    b16 = _rand(T, W + 8, seed=5).to(torch.bfloat16)[:, 8:]          # a column slice: row stride wider than the row
    row = _rand(W, seed=6)
    w = (1.0 + _rand(W, seed=7, scale=0.3)).to(torch.bfloat16)
    xs = x.clone().to(dev)
    h = M.stream_add_norm(xs, [a16.to(dev), a32.to(dev), b16.to(dev)], row=row.to(dev), weight=w.to(dev), eps=1e-5,
                          kind=kind, out_dtype=torch.float32)
    want_x = x.to(F64) + ((a16.to(F64) + a32.to(F64)) + b16.to(F64) + row.to(F64))
    _close(xs, want_x, 1e-6)
    if kind is None:
        assert h is None
        return
    want = O.layer_norm(want_x, w.to(F64), 1e-5) if kind == "layer" else O.rms(want_x, 1e-5) * w.to(F64)
    _close(h, want, 3e-6)
    # nothing to add: the stream is left as it is and only normalised
    xs2 = x.clone().to(dev)
    h2 = M.stream_add_norm(xs2, (), weight=w.to(dev), eps=1e-5, kind=kind, out_dtype=torch.bfloat16)
    assert torch.equal(xs2.cpu(), x) and h2.dtype == torch.bfloat16
    want2 = O.layer_norm(x.to(F64), w.to(F64), 1e-5) if kind == "layer" else O.rms(x.to(F64), 1e-5) * w.to(F64)
    _close(h2, want2, 1e-2)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("I,dtype", [(24, torch.float32), (17, torch.float32), (64, torch.bfloat16)])
def test_clamped_gated_unit(tier, I, dtype):
    dev = _dev(tier)
    gu = (_rand(11, 2 * I, seed=8, scale=2.5)).to(dtype)            # many values beyond the limit on both sides
    limit, alpha = 1.25, 1.702
    got = ops.clamped_glu(gu.to(dev), limit, alpha)
    g, u = gu.to(F64)[:, :I], gu.to(F64)[:, I:]
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    want = g * torch.sigmoid(alpha * g) * (u + 1.0)
    assert float((gu.float()[:, :I] > limit).sum()) > 0 and float((gu.float()[:, I:] < -limit).sum()) > 0
    _close(got, want, 2e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("tier", TIERS)
def test_gather_combine_sums_a_tokens_rows_in_fp32(tier):
    dev = _dev(tier)
    T, k, H = 7, 3, 40
    rows = _rand(T * k, H, seed=9).to(torch.bfloat16)
    perm = torch.randperm(T * k, generator=torch.Generator().manual_seed(1)).view(T, k)
    w = torch.rand(T, k, generator=torch.Generator().manual_seed(2))
    got = gather_combine(rows.to(dev), perm.to(dev), w.to(dev))
    want = (rows.to(F64)[perm] * w.to(F64)[..., None]).sum(1)
    assert got.dtype == torch.float32
    _close(got, want, 1e-6)


def _retention_oracle(q, k, v, decay, pos, dims, base):
    """read-outs of one sequence, [L, H, dv]"""
    L, H, d = q.shape
    q = O.rotate(q, pos, dims, base)
    k = O.rotate(k, pos, dims, base) * d ** -0.5
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = torch.zeros(L, H, v.shape[-1], dtype=F64)
    for t in range(L):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("d,dv,dims", [(16, 24, 8), (32, 40, 32), (24, 8, 0), (160, 8, 64)])
def test_retention_scan_carries_its_state_through_portions_and_slots(tier, d, dv, dims):
    """Two sequences in three steps: a whole prompt beside a portion, two-token portions, single tokens; the second
    sequence takes a slot that held another sequence before.  One head never forgets (decay 1)."""
    dev = _dev(tier)
    H, base = 3, 1000.0
    decay = [1.0, 0.9, 0.5]
    La, Lb = 37, 21
    qa, ka, va = (_rand(La, H * w, seed=s) for s, w in ((10, d), (11, d), (12, dv)))
    qb, kb, vb = (_rand(Lb, H * w, seed=s) for s, w in ((13, d), (14, d), (15, dv)))
    want_a = _retention_oracle(qa.view(La, H, d).to(F64), ka.view(La, H, d).to(F64), va.view(La, H, dv).to(F64), decay,
                               list(range(La)), dims, base)
    want_b = _retention_oracle(qb.view(Lb, H, d).to(F64), kb.view(Lb, H, d).to(F64), vb.view(Lb, H, dv).to(F64), decay,
                               list(range(Lb)), dims, base)
    state = torch.full((2, H, d, dv), 7.0, device=dev)                 # stale contents of reused slots
    table = M.rotary_table(64, dims, base, dev) if dims else None
    dec = torch.tensor(decay, device=dev)
    got_a, got_b = [], []
    # (tokens of a, tokens of b) per step; a sits in slot 1, b in slot 0
    at_a = at_b = 0
    for na, nb in [(20, 2), (2, 2), (1, 1), (14, 16)]:
        q = torch.cat([qa[at_a:at_a + na], qb[at_b:at_b + nb]]).to(dev)
        k = torch.cat([ka[at_a:at_a + na], kb[at_b:at_b + nb]]).to(dev)
        v = torch.cat([va[at_a:at_a + na], vb[at_b:at_b + nb]]).to(dev)
        meta = M.RaggedMeta.build([na, nb], [at_a, at_b], [1, 0], dev)
        o = M.state_scan_decay(q, k, v, dec, state, meta, H, d, dv, act_silu=False, rot_table=table, rot_dims=dims,
                               k_scale=d ** -0.5)
        got_a.append(o[:na])
        got_b.append(o[na:])
        at_a, at_b = at_a + na, at_b + nb
    _close(torch.cat(got_a).view(La, H, dv), want_a, 3e-6)
    _close(torch.cat(got_b).view(Lb, H, dv), want_b, 3e-6)


@pytest.mark.parametrize("tier", TIERS)
def test_unit_rms_read_out_with_silu_gate(tier):
    dev = _dev(tier)
    T, H, dv = 6, 3, 20
    o = _rand(T, H * dv, seed=16, scale=30.0)
    gate = _rand(T, H * dv, seed=17)
    got = M.gated_group_rms_norm(o.to(dev), None, gate.to(dev), dv, 1e-5, torch.float32, gate_act="silu")
    want = O.rms(o.to(F64).view(T, H, dv), 1e-5).reshape(T, H * dv) * O.silu(gate.to(F64))
    _close(got, want, 2e-6)


def _latent_setup(dev, dtype, L, R, r, bs, seed):
    """A sequence of L tokens whose cache rows sit on scattered pages; returns (z, cache, tables, normalised latent c,
    rotated key part) with c / key part from the oracle's pieces."""
    z = _rand(L, R + r, seed=seed).to(dtype)
    w = (1.0 + _rand(R, seed=seed + 1, scale=0.2)).to(dtype)
    pages = (L + bs - 1) // bs
    order = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(seed)).tolist()[:pages]
    tables = torch.tensor([order], dtype=torch.int32, device=dev)
    cache = torch.zeros(pages + 3, bs, 1, R + r, dtype=dtype, device=dev)
    c = O.rms(z.to(F64)[:, :R], 1e-5) * w.to(F64)
    kr = O.rotate(z.to(F64)[:, None, R:], list(range(L)), r, 5e5)[:, 0]
    return z, w, cache, tables, c, kr


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,r", [(40, 8), (168, 24), (36, 6)])
def test_latent_cache_rows_and_attention_in_the_latent_space(tier, dtype, R, r):
    """Rows [normalised latent | rotated key part] written in two portions; queries of the second portion and of a
    decoded token attend over them; values are the rows' latent columns.  Row widths of 48 and 192 (two tile widths of
    the tensor-core kernel in 16 bits) and 42 (no multiple of 8: the CUDA-core kernel)."""
    dev = _dev(tier)
    L, bs, H = 300, 16, 4
    z, w, cache, tables, c, kr = _latent_setup(dev, dtype, L, R, r, bs, seed=20)
    table = M.rotary_table(L, r, 5e5, dev)
    first = 203                                                    # a cut inside a page
    for lo, hi in ((0, first), (first, L)):
        meta = M.RaggedMeta.build([hi - lo], [lo], [0], dev)
        M.latent_kv_write(z[lo:hi].to(dev), w.to(dev), 1e-5, R, table, cache, tables, meta)
    rows = torch.cat([c, kr], -1)
    flat = cache.view(-1, R + r)[(tables[0].long()[:, None] * bs + torch.arange(bs, device=dev)[None]).reshape(-1)][:L]
    _close(flat, rows, 2e-6 if dtype == torch.float32 else 8e-3)
    q = _rand(L - first, H * (R + r), seed=23, scale=0.5).to(dtype)
    meta = M.RaggedMeta.build([L - first], [first], [0], dev)
    got = M.paged_bias_attention(q.to(dev), cache, cache, tables, meta, 0.3, vdim=R)
    stored = flat.double().cpu()                                    # what the kernel reads (rounded once)
    want = torch.zeros(L - first, H, R, dtype=F64)
    for i in range(L - first):
        for h in range(H):
            s = stored[: first + i + 1] @ q.to(F64).view(-1, H, R + r)[i, h] * 0.3
            want[i, h] = torch.softmax(s, 0) @ stored[: first + i + 1, :R]
    _close(got.view(-1, H, R), want, 3e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("tier", TIERS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("portion", [1, 23])
@pytest.mark.parametrize("target", [0, 1, 15, 16, 17, 255, 256, 511])
def test_one_far_key_singled_out_among_hundreds(tier, dtype, target, portion):
    """The query of the last token points at ONE key (the first tokens, both sides of a page border and of a key chunk's
    edge, far back): the result must be that key's latent, whatever page it lies on - for a token decoded alone and for
    the last token of a prompt's portion (the other rows of the portion carry small random queries)."""
    dev = _dev(tier)
    L, R, r, bs, H = 520, 32, 8, 16, 2
    z, w, cache, tables, c, kr = _latent_setup(dev, dtype, L, R, r, bs, seed=30 + target)
    table = M.rotary_table(L, r, 5e5, dev)
    M.latent_kv_write(z.to(dev), w.to(dev), 1e-5, R, table, cache, tables, M.RaggedMeta.build([L], [0], [0], dev))
    row = torch.cat([c, kr], -1)[target]
    q = _rand(portion, H * (R + r), seed=50 + target, scale=0.3).to(F64)
    q[-1] = torch.stack([row * 6.0, -row * 6.0]).reshape(H * (R + r))              # head 1 looks away from it
    q = q.to(dtype)
    meta = M.RaggedMeta.build([portion], [L - portion], [0], dev)
    got = M.paged_bias_attention(q.to(dev), cache, cache, tables, meta, 1.0, vdim=R).view(portion, H, R).double().cpu()
    keys = torch.cat([c, kr], -1)
    qd = q.to(F64).view(portion, H, R + r)
    want = torch.zeros(portion, H, R, dtype=F64)
    for i in range(portion):
        n = L - portion + i + 1
        for h in range(H):
            want[i, h] = torch.softmax(keys[:n] @ qd[i, h], 0) @ c[:n]
    p = torch.softmax(keys @ qd[-1, 0], 0)
    assert p[target] > 0.99                                         # the crafted key does stand out
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert (got - want).abs().max() < tol * c.abs().max()
    assert (got[-1, 0] - c[target]).abs().max() < 0.05 * c.abs().max()


@pytest.mark.parametrize("tier", TIERS)
def test_router_takes_the_largest_scores_and_renormalises(tier):
    dev = _dev(tier)
    from colossalai_b200.models.config import ExpertFFSpec, ModelConfig
    from colossalai_b200.models.moe import ClampedExpertFF

    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=32, vocab_size=16, num_hidden_layers=1, num_attention_heads=1)
    for dtype in (torch.float32, torch.bfloat16):
        ff = ClampedExpertFF(cfg, ExpertFFSpec(experts=6, top=3, ff=8, limit=1.0, shared_ff=0)).to(dev).to(dtype)
        with torch.no_grad():
            ff.router.weight.copy_(_rand(6, 32, seed=40, scale=0.7))
        x = _rand(9, 32, seed=41).to(dtype)
        w, idx = ff.route(x.to(dev))
        s = torch.softmax(x.to(F64) @ ff.router.weight.detach().to(F64).cpu().T, -1)
        for t in range(9):
            chosen = sorted(range(6), key=lambda e: -float(s[t, e]))[:3]
            assert sorted(idx[t].tolist()) == sorted(chosen)
            tot = sum(float(s[t, e]) for e in chosen)
            for j in range(3):
                assert abs(float(w[t, j]) - float(s[t, int(idx[t, j])]) / tot) < 1e-5
        assert abs(float(w.sum(-1).min()) - 1.0) < 1e-5
