"""Venidra restated plainly, in float64, one function per mechanism: what the tests compare the library with.
Nothing here is shared with the package: tensors come in as a dict name -> float64 tensor, the config as the
dict config.json holds.

Notation: x [T, W] the residual stream of one sequence; p the positions 0..T-1; all sums in float64."""
import math

import torch

F = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def angles(T, dims, base, pos0=0):
    """[T, dims/2]: a(p, i) = p * base^(-2i/dims), with the frequency rounded to float32 as a 32-bit product has it."""
    i = torch.arange(dims // 2, dtype=F)
    f = (float(base) ** (-2.0 * i / dims)).to(torch.float32).to(F)
    p = torch.arange(pos0, pos0 + T, dtype=F)
    return (p[:, None] * f[None, :]).to(torch.float32).to(F)


def rotate_halves(x, a):
    """x [T, H, D]: coordinate i pairs with i + dims/2 over the first dims = 2 * a.shape[1] coordinates."""
    n = a.shape[1]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n:]], -1)


def rotate_pairs(x, a):
    """x [T, H, D]: coordinate 2i pairs with 2i + 1 over the first dims = 2 * a.shape[1] coordinates."""
    n = a.shape[1]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


def chunk_mask(T, size):
    i = torch.arange(T)
    return (i[None, :] <= i[:, None]) & ((i[None, :] // size) == (i[:, None] // size))


def window_mask(T, size):
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


def softmax_heads(score, mask, v):
    """score [H, T, T], mask [T, T], v [T, H, Dv] -> [T, H * Dv]."""
    score = score.masked_fill(~mask[None], -math.inf)
    w = torch.softmax(score, -1)
    return torch.einsum("hij,jhd->ihd", w, v).reshape(v.shape[0], -1)


def attention(h, w, pre, m, eps, v_first):
    """Grouped heads, rotation of the first rot.dims coordinates by halves, unit RMS of q and k after it, chunk mask,
    values blended with the first blending layer's. Returns (output, this layer's values before blending)."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads", H), m.get("vdim", D)
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = (h @ w[pre + "v"].T).view(T, G, Dv)
    if m.get("rot") and m["rot"]["dims"]:
        a = angles(T, m["rot"]["dims"], m["rot"]["base"])
        q, k = rotate_halves(q, a), rotate_halves(k, a)
    q, k = rms(q, eps), rms(k, eps)
    v_own = v
    if m.get("v_mix") and v_first is not None:
        lam = w[pre + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rep = H // G
    ke, ve = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    score = torch.einsum("ihd,jhd->hij", q, ke) * m["scale"]
    o = softmax_heads(score, chunk_mask(T, m["mask"]["size"] if m.get("mask") else T), ve)
    return o @ w[pre + "o"].T, v_own


def latent_attention(h, w, pre, m, eps):
    """Queries and keys/values through low-rank latents; one rotated key part for all heads; sliding window."""
    T = h.shape[0]
    H, D, R, Dv, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, D + R)
    kv = h @ w[pre + "dkv"].T
    c = rms(kv[:, :L], eps) * w[pre + "dkv.norm"]
    a = angles(T, m["rot"].get("dims", R), m["rot"]["base"])
    k_rot = rotate_pairs(kv[:, None, L:], a)                       # [T, 1, R]
    q_rot = rotate_pairs(q[..., D:], a)
    k_plain = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, Dv)
    score = (torch.einsum("ihd,jhd->hij", q[..., :D], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    o = softmax_heads(score, window_mask(T, m["mask"]["size"] if m.get("mask") else T), v)
    return o @ w[pre + "o"].T


def feed_forward(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence. ``layers_out``: a list that receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    v_first = None
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}."
        hin = rms(x, eps) * w[pre + "norm1"]
        if lc["type"] == "attention":
            y, v_own = attention(hin, w, pre + "mix.", lc["mixer"], eps, v_first)
            if lc["mixer"].get("v_mix") and v_first is None:
                v_first = v_own
        elif lc["type"] == "latent_attention":
            y = latent_attention(hin, w, pre + "mix.", lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        x = x + rms(y, eps) * w[pre + "norm1b"]
        if lc.get("mlp") is not None:
            y = feed_forward(rms(x, eps) * w[pre + "norm2"], w, pre + "mlp.")
            x = x + rms(y, eps) * w[pre + "norm2b"]
        if layers_out is not None:
            layers_out.append(x.clone())
    xn = rms(x, eps) * w["final.norm"]
    logits = xn @ w["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def read_model(folder):
    """(config dict, name -> float64 tensor) of a model folder."""
    import json
    import os

    from safetensors import safe_open

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k).to(F)
    return cfg, w


def masked_softmax_attention(q, k, v, mask, scale):
    """q [T, H, D], k [T, G, D], v [T, G, Dv], mask [T, T] -> [T, H * Dv], heads grouped onto the G key/value heads."""
    rep = q.shape[1] // k.shape[1]
    score = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, 1)) * scale
    return softmax_heads(score, mask, v.repeat_interleave(rep, 1))
