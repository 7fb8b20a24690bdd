"""Plain, slow float64 implementation of the hybrid decoder's mechanisms, one function per mechanism, written from the
equations and sharing no code with the package: the yardstick for the kernels, the ragged step function and the engine.

Notation: h is a sublayer's input [L, width]; all products are W h with W stored [out, in].
"""
import json
import math
import os

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def bucket(n, B, D):
    """Distance -> row of the bias table: exact below B/2, logarithmic up to D above, clipped to the last row."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def short_conv(z, w):
    """Causal depthwise convolution over time, zeros before the start; w [C, taps], last column = current token."""
    L, taps = z.shape[0], w.shape[1]
    out = torch.zeros_like(z)
    for t in range(L):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += z[src] * w[:, j]
    return out


def lightning(q, k, v, decay):
    """q, k [L, H, d], v [L, H, dv].  Per head a matrix M [d, dv], zero at the start: each token first shrinks M by
    the head's decay, then adds outer(k, v), then reads M^T q."""
    L, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = []
    for t in range(L):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
        out.append(torch.stack([S[h].T @ q[t, h] for h in range(H)]))
    return torch.stack(out)


def delta_rule(q, k, v, g, beta):
    """q, k [L, H, d] (already unit / scaled), v [L, H, dv], g [L, H, d] row decays, beta [L, H] write strengths.
    Per head a matrix M [d, dv], zero at the start; each token: rows of M times g; error = beta * (v - M^T k);
    M gains outer(k, error); the read-out M^T q comes after the write."""
    L, H, d = q.shape
    S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = []
    for t in range(L):
        row = []
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + torch.outer(k[t, h], u)
            row.append(S[h].T @ q[t, h])
        out.append(torch.stack(row))
    return torch.stack(out)


def sink_attention(q, k, v, scale, rel, D):
    """q [L, H, d], k [L, G, d], v [L, G, dv].  Token i scores every j <= i with scale * <q_i, k_j> plus the table entry
    of (bucket of i - j, head); the softmax has an extra term exp(0) in its denominator that carries no value."""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, v.shape[-1], dtype=F64)
    B = 0 if rel is None else rel.shape[0]
    for i in range(L):
        for h in range(H):
            g = h // (H // G)
            s = torch.stack([scale * (q[i, h] @ k[j, g]) + (rel[bucket(i - j, B, D), h] if B else 0.0)
                             for j in range(i + 1)])
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            p = e / (math.exp(-m) + e.sum())
            out[i, h] = (p[:, None] * v[: i + 1, g]).sum(0)
    return out


def forward(cfg, W, tokens, layers_out=None):
    """Logits [L, vocab] of one sequence.  cfg: the checkpoint's config dict; W: name -> float64 tensor."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    tokens = torch.as_tensor(tokens)
    L = tokens.numel()
    x = W["embed"][tokens] * cfg["embedding"]["scale"]
    v_first = None
    for i, ly in enumerate(cfg["layers"]):
        p, mx, h = f"l{i}.mix.", ly["mixer"], x
        if ly["type"] == "lightning":
            H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
            q = silu(h @ W[p + "q"].T).view(L, H, d)
            k = silu(h @ W[p + "k"].T).view(L, H, d)
            v = silu(h @ W[p + "v"].T).view(L, H, dv)
            o = lightning(q, k, v, mx["decay"]).reshape(L, H * dv)
            o = rms(o, eps) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
        elif ly["type"] == "channel_delta":
            H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            rep = H // G
            q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(L, G, d)
            k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(L, G, d)
            v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(L, H, dv)
            q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
            k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            beta = torch.sigmoid(h @ W[p + "b"].T)
            pre = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
            g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * torch.log1p(torch.exp(pre)).view(L, H, d))
            o = delta_rule(q, k, v, g, beta)
            o = (rms(o, eps) * W[p + "norm"]).reshape(L, H * dv)
            o = o * torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
        else:
            H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            q = rms(h @ W[p + "q"].T + W[p + "q.b"], eps) * W[p + "q.norm"]
            k = rms(h @ W[p + "k"].T + W[p + "k.b"], eps) * W[p + "k.norm"]
            v = (h @ W[p + "v"].T + W[p + "v.b"]).view(L, G, dv)
            if mx.get("v_mix"):
                if v_first is None:
                    v_first = v
                else:
                    lam = W[p + "vmix"]
                    v = (1 - lam) * v + lam * v_first
            o = sink_attention(q.view(L, H, d), k.view(L, G, d), v, mx["scale"], W[p + "rel"], mx["bias_max"])
            o = o.reshape(L, H * dv)
        x = x + m * rms(o @ W[p + "o"].T, eps) * (1 + W[f"l{i}.norm1"])
        if ly["mlp"] is not None:
            u = torch.relu(x @ W[f"l{i}.mlp.up"].T) ** 2
            x = x + m * rms(u @ W[f"l{i}.mlp.down"].T, eps) * (1 + W[f"l{i}.norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * (1 + W["final.norm"])) @ W["head"].T


# ----------------------------------------------------------------------------------------------- checkpoints for the tests
def attention_layer(heads=4, kv_heads=2, dim=24, vdim=16, scale=0.2, bias_max=40, v_mix=False, ff=96):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale, "bias_max": bias_max, "v_mix": v_mix},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def lightning_layer(heads=3, dim=16, vdim=24, decay=(0.7, 0.93, 0.995), ff=96):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def delta_layer(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, ff=96):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def make_config(layers, width=64, vocab=96, eps=1e-5, residual_mult=0.6, embed_scale=1.5):
    return {"architecture": "Gopunex", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
            "residual_mult": residual_mult, "vocab": vocab, "width": width}


def random_weights(cfg, seed=0, buckets=10, decay_rank=6, gate_rank=5):
    """name -> bf16-representable fp32 tensors in the checkpoint's naming."""
    gen = torch.Generator().manual_seed(seed)
    W, Wd = {}, cfg["width"]

    def lin(o, i, s=1.0):
        return torch.randn(o, i, generator=gen) * (s / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + torch.randn(n, generator=gen) * std

    W["embed"] = torch.randn(cfg["vocab"], Wd, generator=gen)
    W["head"] = lin(cfg["vocab"], Wd)
    W["final.norm"] = vec(Wd)
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", ly["mixer"]
        W[p + "norm1"] = vec(Wd)
        if ly["mlp"] is not None:
            W[p + "norm2"] = vec(Wd)
            W[p + "mlp.up"] = lin(ly["mlp"]["ff"], Wd)
            W[p + "mlp.down"] = lin(Wd, ly["mlp"]["ff"])
        p += "mix."
        if ly["type"] == "lightning":
            H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
            for n, o in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                W[p + n] = lin(o, Wd)
            W[p + "norm"] = vec(H * dv, 1.0)
            W[p + "o"] = lin(Wd, H * dv)
        elif ly["type"] == "channel_delta":
            H, G, d, dv, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            for n, o in (("q", G * d), ("k", G * d), ("v", H * dv)):
                W[p + n] = lin(o, Wd, 2.0)
                W[p + n + ".conv"] = torch.randn(o, taps, generator=gen) * 0.5
            W[p + "b"] = lin(H, Wd, 2.0)
            W[p + "A_log"] = vec(H, 0.0, 0.5)
            W[p + "norm"] = vec(dv, 1.0)
            W[p + "a1"], W[p + "a2"] = lin(decay_rank, Wd), lin(H * d, decay_rank, 2.0)
            W[p + "dt_bias"] = vec(H * d, 0.0, 1.0)
            W[p + "g1"], W[p + "g2"] = lin(gate_rank, Wd), lin(H * dv, gate_rank, 2.0)
            W[p + "o"] = lin(Wd, H * dv)
        else:
            H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            for n, o in (("q", H * d), ("k", G * d), ("v", G * dv)):
                W[p + n] = lin(o, Wd)
                W[p + n + ".b"] = vec(o, 0.0, 0.3)
            W[p + "q.norm"], W[p + "k.norm"] = vec(H * d, 1.2, 0.3), vec(G * d, 1.2, 0.3)
            W[p + "rel"] = torch.randn(buckets, H, generator=gen)
            W[p + "vmix"] = torch.tensor(0.35)
            W[p + "o"] = lin(Wd, H * dv)
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}


def write_checkpoint(folder, cfg, W):
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, os.path.join(folder, "model.safetensors"))
    return str(folder)


def to64(W):
    return {k: v.to(F64) for k, v in W.items()}
