"""Plain, slow float64 implementation of the Palilix decoder, one function per mechanism, written from the equations and
sharing no code with the package: the yardstick for the kernels, the ragged step function and the engine.

Notation: h is a layer's normalised input [L, width]; all products are W h with W stored [out, in]; positions count
from 0.  A layer is parallel: x <- x + mixer(h) + ff(h) with ONE layer norm (weight, no bias) in front of both.  A span
of layers may run several times in a row with the same weights ("loop"): every pass gets the embedding output added
again (except the first) plus a learned vector of its own, and every pass keeps caches and states of its own.
"""
import json
import math
import os

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------------------------- small pieces
def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x, pos, dims, base):
    """x [L, H, d]; the first `dims` channels of every head turn by the angle pos * base^(-2i/dims), channel i paired
    with channel i + dims/2; the other channels pass."""
    out = x.clone()
    half = dims // 2
    for t in range(x.shape[0]):
        for i in range(half):
            a = float(pos[t]) * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def latent_attention(h, W, p, mx, eps, pos):
    """Keys and values of all heads are rebuilt from one small latent per token plus one rotated key part that all
    heads share; the softmax is causal and ordinary."""
    L = h.shape[0]
    H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ W[p + "q"].T).view(L, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, mx["rot"]["dims"], mx["rot"]["base"])
    z = h @ W[p + "dkv"].T
    c = rms(z[:, :R], eps) * W[p + "dkv.norm"]
    k_rot = rotate(z[:, None, R:], pos, mx["rot"]["dims"], mx["rot"]["base"])[:, 0]
    k_plain = (c @ W[p + "uk"].T).view(L, H, d)
    v = (c @ W[p + "uv"].T).view(L, H, dv)
    out = torch.zeros(L, H, dv, dtype=F64)
    for i in range(L):
        for hh in range(H):
            s = (k_plain[: i + 1, hh] @ q_plain[i, hh] + k_rot[: i + 1] @ q_rot[i, hh]) * mx["scale"]
            out[i, hh] = torch.softmax(s, 0) @ v[: i + 1, hh]
    return out.reshape(L, H * dv) @ W[p + "o"].T


def retention(h, W, p, mx, eps, pos):
    """Per head a matrix S [d, dv], zero at the start: S <- decay * S + outer(k, v); read-out S^T q after the write; no
    softmax and no denominator.  The read-out of every head is brought to unit root mean square and gated."""
    L = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
    q = rotate((h @ W[p + "q"].T).view(L, H, d), pos, mx["rot"]["dims"], mx["rot"]["base"])
    k = rotate((h @ W[p + "k"].T).view(L, H, d), pos, mx["rot"]["dims"], mx["rot"]["base"]) * d ** -0.5
    v = (h @ W[p + "v"].T).view(L, H, dv)
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(L, H, dv, dtype=F64)
    for t in range(L):
        for hh in range(H):
            S[hh] = mx["decay"][hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            out[t, hh] = S[hh].T @ q[t, hh]
    o = rms(out, eps).reshape(L, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# ----------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p):
    return gelu_tanh(h @ W[p + "up"].T) @ W[p + "down"].T


def clamped_expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def moe_ff(h, W, p, mlp):
    """Every token goes to the `top` experts of largest softmax score, weighted by those scores renormalised to one;
    a shared expert, where the layer has one, takes every token."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.softmax(h @ W[p + "router"].T, -1)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        chosen = sorted(range(E), key=lambda e: -float(s[t, e]))[:top]
        tot = sum(s[t, e] for e in chosen) + 1e-20
        for e in chosen:
            out[t] += s[t, e] / tot * clamped_expert(h[t:t + 1], W, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, W, p + "shared.", mlp["shared"]["limit"])
    return out


# ----------------------------------------------------------------------------------------------- the model
def layer_runs(cfg):
    """[(layer, pass or None)] in the order the layers run."""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = lp["start"], lp["stop"], lp["times"]
    if b <= a:
        return [(i, None) for i in range(n)]
    return [(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + \
        [(i, None) for i in range(b, n)]


def forward(cfg, W, tokens, layers_out=None):
    """Logits [L, vocab] of one sequence.  cfg: the checkpoint's config dict; W: name -> float64 tensor."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens)
    L = tokens.numel()
    pos = list(range(L))
    x0 = W["embed"][tokens] * cfg["embedding"]["scale"]
    x = x0.clone()
    lp = cfg.get("loop")
    for i, t in layer_runs(cfg):
        if t is not None and i == lp["start"]:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        ly = cfg["layers"][i]
        h = layer_norm(x, W[f"l{i}.norm1"], eps)
        fn = {"latent_attention": latent_attention, "retention": retention}[ly["type"]]
        y = fn(h, W, f"l{i}.mix.", ly["mixer"], eps, pos)
        mlp = ly["mlp"]
        if mlp is not None:
            y = y + (dense_ff(h, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(h, W, f"l{i}.mlp.", mlp))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    z = layer_norm(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


# ----------------------------------------------------------------------------------------------- checkpoints for the tests
def dense(ff=80):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=24, limit=0.8, shared_ff=40, shared_limit=1.2):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return m


def latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, scale=0.2, base=10000.0, mlp="dense"):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}},
            "mlp": dense() if mlp == "dense" else mlp}


def retention_layer(heads=3, dim=16, vdim=24, decay=(0.7, 0.93, 0.995), rot_dims=8, base=5000.0, mlp="dense"):
    return {"type": "retention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": rot_dims}},
            "mlp": dense() if mlp == "dense" else mlp}


def make_config(layers, width=48, vocab=96, eps=1e-5, embed_scale=3.0, loop=None, logit_scale=1.5, softcap=10.0):
    cfg = {"architecture": "Palilix", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps},
           "vocab": vocab, "width": width, "logit_scale": logit_scale, "logit_softcap": softcap}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0):
    """name -> bf16-representable fp32 tensors in the checkpoint's naming."""
    gen = torch.Generator().manual_seed(seed)
    W, Wd = {}, cfg["width"]

    def lin(o, i, s=1.0):
        return torch.randn(o, i, generator=gen) * (s / math.sqrt(i))

    def vec(n, mean=0.0, std=0.2):
        return mean + torch.randn(n, generator=gen) * std

    W["embed"] = torch.randn(cfg["vocab"], Wd, generator=gen) * 0.5
    W["head"] = lin(cfg["vocab"], Wd)
    W["final.norm"] = vec(Wd, 1.0)
    if cfg.get("loop"):
        W["loop.step"] = torch.randn(cfg["loop"]["times"], Wd, generator=gen) * 0.5
    for i, ly in enumerate(cfg["layers"]):
        p, mx, mlp = f"l{i}.", ly["mixer"], ly["mlp"]
        W[p + "norm1"] = vec(Wd, 1.0)
        if mlp is not None and mlp["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = lin(mlp["ff"], Wd), lin(Wd, mlp["ff"])
        elif mlp is not None:
            names = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                names.append(("shared.", mlp["shared"]["ff"]))
            for n, ff in names:
                W[p + "mlp." + n + "gate"], W[p + "mlp." + n + "up"] = lin(ff, Wd, 1.5), lin(ff, Wd, 1.5)
                W[p + "mlp." + n + "down"] = lin(Wd, ff)
            W[p + "mlp.router"] = lin(mlp["router"]["experts"], Wd, 2.0)
        p += "mix."
        if ly["type"] == "retention":
            H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
            for n, o in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                W[p + n] = lin(o, Wd)
            W[p + "o"] = lin(Wd, H * dv)
        else:
            H, d, r, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
            W[p + "q"] = lin(H * (d + r), Wd, 2.0)
            W[p + "dkv"] = lin(R + r, Wd, 2.0)
            W[p + "dkv.norm"] = vec(R, 1.0)
            W[p + "uk"], W[p + "uv"] = lin(H * d, R, 2.0), lin(H * dv, R)
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
