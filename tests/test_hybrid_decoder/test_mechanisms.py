"""Each mechanism of the hybrid decoder alone: the op (CPU path here, sm_100a kernel under the gpu marker) against the
plain float64 functions of `oracle.py`, on ragged steps with carried state, permuted pages and crafted inputs."""
import math

import pytest
import torch

from colossalai_b200.ops import mixers as M

from . import oracle as O

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _dev(device):
    if device == "cuda" and not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return device


def _close(got, want, tol):
    got, want = got.detach().double().cpu(), want.double()
    err = (got - want).abs().max().item()
    assert err <= tol * max(want.abs().max().item(), 1e-3), f"max error {err:.3e} (scale {want.abs().max().item():.3e})"


def _steps(total, cuts):
    """[(start, n)] portions that cover `total` tokens: the given sizes, then single tokens."""
    out, at = [], 0
    for n in cuts:
        n = min(n, total - at)
        if n > 0:
            out.append((at, n))
            at += n
    while at < total:
        out.append((at, 1))
        at += 1
    return out


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("B,D", [(8, 20), (10, 40), (16, 300), (6, 7), (32, 1000)])
def test_bucket_starts_match_the_formula(device, B, D):
    starts = M.log_bucket_starts(B, D)
    for n in range(0, 3 * D + 5):
        want = O.bucket(n, B, D)
        got = max(b for b in range(B) if starts[b] <= n)
        assert got == want, (n, got, want)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,cuts", [(4, [1, 1, 2, 9, 3]), (3, [40]), (2, [2, 2, 1]), (1, [5, 1]), (5, [1, 1, 1, 1, 1, 1])])
@pytest.mark.parametrize("C", [70, 72])              # 72: the 16-byte vector kernel; 70: the scalar one
def test_short_conv_carries_its_window(device, dtype, taps, cuts, C):
    dev = _dev(device)
    g = torch.Generator().manual_seed(taps)
    L, slots = 44, 3
    x = torch.randn(L, C, generator=g).to(dtype)
    w = (torch.randn(C, taps, generator=g) * 0.5).to(dtype)
    want = O.silu(O.short_conv(x.double(), w.double()))
    state = torch.full((slots, max(taps - 1, 0), C), 7.0, dtype=dtype, device=dev)      # stale content of a used slot
    outs = []
    for at, n in _steps(L, cuts):
        meta = M.RaggedMeta.build([n], [at], [2], dev)
        outs.append(M.short_conv_silu(x[at:at + n].to(dev), w.to(dev), state, meta))
    _close(torch.cat(outs), want, 1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,d,dv", [(3, 16, 24), (2, 48, 8), (1, 128, 130), (5, 8, 33)])
def test_decay_scan_matches_token_by_token(device, H, d, dv):
    dev = _dev(device)
    g = torch.Generator().manual_seed(H * d)
    L = 37
    q, k = torch.randn(L, H * d, generator=g) * 0.5, torch.randn(L, H * d, generator=g) * 0.5
    v = torch.randn(L, H * dv, generator=g)
    decay = torch.tensor([0.5, 0.9, 0.999, 0.97, 1.0][:H], dtype=torch.float64)
    want = O.lightning(O.silu(q.double()).view(L, H, d), O.silu(k.double()).view(L, H, d),
                       O.silu(v.double()).view(L, H, dv), decay.tolist()).reshape(L, H * dv)
    state = torch.full((2, H, d, dv), 3.0, device=dev)
    outs = []
    for at, n in _steps(L, [5, 1, 1, 17, 2]):
        meta = M.RaggedMeta.build([n], [at], [1], dev)
        outs.append(M.state_scan_decay(q[at:at + n].to(dev), k[at:at + n].to(dev), v[at:at + n].to(dev),
                                       decay.float().to(dev), state, meta, H, d, dv))
    _close(torch.cat(outs), want, 2e-5)


def _delta_inputs(L, H, G, d, dv, seed):
    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(L, G * d, generator=g), torch.randn(L, G * d, generator=g)
    v = torch.randn(L, H * dv, generator=g)
    a, b = torch.randn(L, H * d, generator=g) * 2, torch.randn(L, H, generator=g) * 2
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5, torch.randn(H * d, generator=g)
    return q, k, v, a, b, a_log, dt_bias


def _delta_oracle(q, k, v, a, b, a_log, dt_bias, H, G, d, dv):
    L = q.shape[0]
    q, k = q.double().view(L, G, d), k.double().view(L, G, d)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    gdec = torch.exp(-torch.exp(a_log.double())[None, :, None]
                     * torch.log1p(torch.exp(a.double() + dt_bias.double())).view(L, H, d))
    return O.delta_rule(q, k, v.double().view(L, H, dv), gdec, torch.sigmoid(b.double())).reshape(L, H * dv)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 24), (3, 3, 32, 8), (2, 1, 128, 40), (6, 2, 24, 136)])
def test_delta_scan_matches_token_by_token(device, H, G, d, dv):
    dev = _dev(device)
    L = 41
    q, k, v, a, b, a_log, dt_bias = _delta_inputs(L, H, G, d, dv, H + d)
    want = _delta_oracle(q, k, v, a, b, a_log, dt_bias, H, G, d, dv)
    state = torch.full((3, H, d, dv), -2.0, device=dev)
    outs = []
    for at, n in _steps(L, [2, 16, 1, 1, 3]):
        meta = M.RaggedMeta.build([n], [at], [0], dev)
        t = lambda z: z[at:at + n].to(dev)
        outs.append(M.state_scan_delta(t(q), t(k), t(v), t(a), t(b), a_log.to(dev), dt_bias.to(dev), state, meta,
                                       H, G, d, dv))
    _close(torch.cat(outs), want, 3e-5)


@pytest.mark.parametrize("device", DEVICES)
def test_scans_keep_sequences_of_a_batch_apart(device):
    """Three sequences of unequal portions in one step, in shuffled slots, equal each sequence run alone."""
    dev = _dev(device)
    H, G, d, dv = 4, 2, 16, 24
    lens, ctx, slots = [9, 1, 4], [0, 6, 2], [2, 0, 1]
    full = [_delta_inputs(c + n, H, G, d, dv, 10 + i) for i, (n, c) in enumerate(zip(lens, ctx))]
    cat = lambda j: torch.cat([full[i][j][ctx[i]:] for i in range(3)]).to(dev)
    al, db = full[0][5], full[0][6]                   # one a_log / dt_bias per layer
    state = torch.full((3, H, d, dv), 5.0, device=dev)
    for i, c in enumerate(ctx):                       # bring every sequence to its context alone
        if c:
            q, k, v, a, b, _, _ = full[i]
            M.state_scan_delta(q[:c].to(dev), k[:c].to(dev), v[:c].to(dev), a[:c].to(dev), b[:c].to(dev), al.to(dev),
                               db.to(dev), state, M.RaggedMeta.build([c], [0], [slots[i]], dev), H, G, d, dv)
    got = M.state_scan_delta(cat(0), cat(1), cat(2), cat(3), cat(4), al.to(dev), db.to(dev), state,
                             M.RaggedMeta.build(lens, ctx, slots, dev), H, G, d, dv)
    at = 0
    for i, (n, c) in enumerate(zip(lens, ctx)):
        q, k, v, a, b, _, _ = full[i]
        want = _delta_oracle(q, k, v, a, b, al, db, H, G, d, dv)[c:]
        _close(got[at:at + n], want, 3e-5)
        at += n


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W", [72, 75])
def test_norm_kernels(device, dtype, W):
    dev = _dev(device)
    g = torch.Generator().manual_seed(3)
    T, H, dv = 7, 3, 40
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    o, gate = torch.randn(T, H * dv, generator=g) * 3, torch.randn(T, H * dv, generator=g).to(dtype)
    for group, w in ((dv, torch.randn(dv, generator=g).to(dtype)), (H * dv, torch.randn(H * dv, generator=g).to(dtype))):
        y = o.double().view(T, -1, group)
        want = (O.rms(y, 1e-4).reshape(T, -1) * w.double().repeat(H * dv // w.numel())) * torch.sigmoid(gate.double())
        _close(M.gated_group_rms_norm(o.to(dev), w.to(dev), gate.to(dev), group, 1e-4, dtype), want, tol)
    x, y, w = torch.randn(T, W, generator=g), (torch.randn(T, W, generator=g) * 5).to(dtype), (torch.randn(W, generator=g) * 0.2).to(dtype)
    want = x.double() + 0.6 * O.rms(y.double(), 1e-4) * (1 + w.double())
    xd = x.clone().to(dev)
    h = M.rms_norm_residual(xd, y.to(dev), w.to(dev), 1e-4, 0.6, 1.0)
    _close(xd, want, 1e-6)            # the stream itself stays fp32 whatever the compute dtype
    _close(h, want, tol)
    _close(M.rms_norm_f32in(xd, w.to(dev), 1e-4, 1.0), O.rms(want, 1e-4) * (1 + w.double()), tol)


def _paged(L, G, d, dv, bs, dtype, dev, gen):
    """Random K / V of one sequence scattered over shuffled pages of a pool with stale content."""
    nblk = (L + bs - 1) // bs
    pool = nblk + 5
    kc = torch.full((pool, bs, G, d), 9.0, dtype=dtype, device=dev)
    vc = torch.full((pool, bs, G, dv), -9.0, dtype=dtype, device=dev)
    table = torch.randperm(pool, generator=gen)[:nblk].int().view(1, nblk)
    return kc, vc, table


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,bs", [(4, 2, 24, 16, 8), (6, 1, 48, 40, 16), (2, 2, 8, 130, 16), (3, 3, 20, 12, 32),
                                         (8, 2, 128, 128, 16), (4, 4, 64, 32, 64), (5, 1, 16, 72, 8)])
def test_paged_bias_sink_attention(device, dtype, H, G, d, dv, bs):
    dev = _dev(device)
    g = torch.Generator().manual_seed(H + bs)
    L, B, D = 53, 10, 30
    q = torch.randn(L, H * d, generator=g).to(dtype)
    k = torch.randn(L, G * d, generator=g).to(dtype)
    v = torch.randn(L, G * dv, generator=g).to(dtype)
    vo = torch.randn(L, G * dv, generator=g).to(dtype)
    rel = torch.randn(B, H, generator=g)
    lam = 0.3
    vmix = ((1 - lam) * v.float() + lam * vo.float()).to(dtype)
    want = O.sink_attention(q.double().view(L, H, d), k.double().view(L, G, d), vmix.double().view(L, G, dv), 0.3,
                            rel.double(), D).reshape(L, H * dv)
    kc, vc, table = _paged(L, G, d, dv, bs, dtype, dev, g)
    starts = torch.tensor(M.log_bucket_starts(B, D), dtype=torch.int32, device=dev)
    outs = []
    for at, n in _steps(L, [bs - 1, 2, bs + 3, 1, 1, 2]):          # portions end before, on and after page borders
        meta = M.RaggedMeta.build([n], [at], [0], dev)
        t = lambda z: z[at:at + n].to(dev)
        M.paged_kv_write_mix(t(k), t(v), kc, vc, table.to(dev), meta, v_other=t(vo), lam=lam)
        outs.append(M.paged_bias_attention(t(q), kc, vc, table.to(dev), meta, 0.3, rel.to(dev), starts, sink=True))
    _close(torch.cat(outs), want, 2e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("sink,buckets", [(True, 10), (False, 10), (True, 0)])
@pytest.mark.parametrize("q_lens,ctx", [([70, 1, 5, 1, 130], [0, 200, 61, 0, 3]),      # portions beside single tokens
                                        ([1, 1, 3], [700, 0, 300]),                    # few rows, long contexts: split keys
                                        ([300], [129])])                               # 128-row tiles, context + portion
def test_tensor_core_and_exact_attention_kernels_agree(sink, buckets, q_lens, ctx):
    """Mixed steps through both CUDA kernels: the tensor-core one (also with its keys split over CTAs) and the exact one."""
    dev = _dev("cuda")
    g = torch.Generator().manual_seed(5)
    H, G, d, dv, bs = 8, 2, 48, 32, 16
    n, T = len(q_lens), sum(q_lens)
    per = max((c + l + bs - 1) // bs for c, l in zip(ctx, q_lens))
    kc = torch.randn(n * per + 3, bs, G, d, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(n * per + 3, bs, G, dv, generator=g).to(torch.bfloat16).to(dev)
    tables = torch.randperm(n * per + 3, generator=g)[: n * per].int().view(n, per).to(dev)
    q = torch.randn(T, H * d, generator=g).to(torch.bfloat16).to(dev)
    meta = M.RaggedMeta.build(q_lens, ctx, list(range(n)), dev)
    rel = torch.randn(buckets, H, generator=g).to(dev) if buckets else None
    starts = torch.tensor(M.log_bucket_starts(buckets, 90), dtype=torch.int32, device=dev) if buckets else None
    a = M.paged_bias_attention(q, kc, vc, tables, meta, 0.2, rel, starts, sink, tensor_cores=True)
    b = M.paged_bias_attention(q, kc, vc, tables, meta, 0.2, rel, starts, sink, tensor_cores=False)
    _close(a, b.cpu(), 2e-2)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("decode", [False, True])
def test_attention_finds_a_far_key_and_its_bucket_edges(device, decode):
    """One key hundreds of tokens back carries the only large score; the bias table marks single buckets, so a table row
    that is one distance off, a page that is mapped wrongly or a lost sink all change the result by O(1)."""
    dev = _dev(device)
    g = torch.Generator().manual_seed(11)
    H, G, d, dv, bs, L, B, D = 2, 1, 16, 8, 16, 330, 12, 200
    starts_host = M.log_bucket_starts(B, D)
    q = torch.randn(L, H * d, generator=g) * 0.05
    k = torch.randn(L, G * d, generator=g) * 0.05
    v = torch.randn(L, G * dv, generator=g)
    far, last = 7, L - 1
    k[far] = 0
    k[far, 0] = 30.0
    q[last] = 0
    q[last, 0], q[last, d] = 1.0, 1.0                    # both heads look at the far key
    kc, vc, table = _paged(L, G, d, dv, bs, torch.float32, dev, g)
    starts = torch.tensor(starts_host, dtype=torch.int32, device=dev)

    def run(rel):
        cut = L - 1 if decode else L - 5
        outs = []
        for at, n in [(0, cut)] + [(i, 1) for i in range(cut, L)] if decode else [(0, cut), (cut, L - cut)]:
            meta = M.RaggedMeta.build([n], [at], [0], dev)
            M.paged_kv_write_mix(k[at:at + n].to(dev), v[at:at + n].to(dev), kc, vc, table.to(dev), meta)
            outs.append(M.paged_bias_attention(q[at:at + n].to(dev), kc, vc, table.to(dev), meta, 1.0, rel.to(dev),
                                               starts, sink=True))
        return torch.cat(outs).cpu()

    got = run(torch.zeros(B, H))
    want_last = v[far].repeat(H)                          # exp(30) dwarfs the sink and every other key
    assert (got[last] - want_last).abs().max() < 1e-3
    # mark one logarithmic bucket: the keys just inside it win, the key one step outside does not
    for b in (B // 2 + 1, B - 2):
        rel = torch.zeros(B, H)
        rel[b] = 25.0
        got = run(rel)
        i = 300
        lo, hi = starts_host[b], starts_host[b + 1] - 1   # distances of the bucket
        inside = [i - n for n in range(lo, hi + 1)]
        want = O.sink_attention(q[: i + 1].double().view(-1, H, d), k[: i + 1].double().view(-1, G, d),
                                v[: i + 1].double().view(-1, G, dv), 1.0, rel.double(), D)[i].reshape(-1)
        _close(got[i], want, 1e-4)
        mean_inside = v[inside].mean(0)
        assert (got[i, :dv] - mean_inside).abs().max() < 0.2      # dominated by the bucket's keys, edges included
    # the sink: with every score very negative nothing is attended
    rel = torch.full((B, H), -40.0)
    got = run(rel)
    assert got[:200].abs().max() < 1e-6
