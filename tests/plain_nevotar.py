"""Nevotar restated plainly: one slow function per mechanism, float64 throughout, straight from the
equations. Shares no code with the package; the tests compare the package with this.

Notation: T tokens of one sequence at positions pos0 .. pos0 + T - 1; W width; H heads, G key/value heads,
D key size, V value size, N state size; weights are [out, in] and act as x @ W.T. ``p`` is a dict of a
part's tensors by their names under the part's prefix, ``m`` the part's entry of the config.
"""
import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, w, eps, groups):
    """The vector in ``groups`` equal consecutive parts, each over its own root mean square, the whole times w."""
    T, n = x.shape
    return rms(x.reshape(T, groups, n // groups), eps).reshape(T, n) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def query_temperature(pos, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    return 1.0 + coef * torch.log(torch.div(pos + 1, every, rounding_mode="floor").to(F) + 1.0)


def rotate_partial(x, pos, dims, base):
    """x [T, heads, D]: coordinate i < dims/2 turns with coordinate i + dims/2 by pos * base^(-2i/dims)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = pos.to(F)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def causal(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window:
        see = see & (i - j < window)
    return see


def softmax_rows(s, see):
    s = torch.where(see, s, torch.full_like(s, -math.inf))
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def diff_lambda(p, diff):
    return float(torch.exp((p["lq1"] * p["lk1"]).sum()) - torch.exp((p["lq2"] * p["lk2"]).sum()) + diff)


def diff_core(q, k, v, scale, lam, diff, eps, q_temp=None, pos0=0):
    """q [T, H, 2, D], k [T, G, 2, D], v [T, G, V] -> [T, H, V]: per head two causal softmax maps over the same values,
    a1 - lam a2, over the head's root mean square, times 1 - diff."""
    T, H = q.shape[:2]
    G, V = k.shape[1], v.shape[2]
    if q_temp:
        q = q * query_temperature(torch.arange(pos0, pos0 + T), q_temp["coef"], q_temp["every"])[:, None, None, None]
    see = causal(T)
    out = torch.zeros(T, H, V, dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        a = [softmax_rows((q[:, hd, j] @ k[:, g, j].T) * scale, see) @ v[:, g] for j in range(2)]
        out[:, hd] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return out


def diff_attention(h, p, m, eps, pos0=0):
    """Two softmax maps per head over the same values, combined as a1 - lambda a2, each head then over its root
    mean square, times 1 - diff."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).reshape(T, H, 2, D)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, G, 2, D)
    v = (h @ p["v"].T + p["v.b"]).reshape(T, G, V)
    out = diff_core(q, k, v, m["scale"], diff_lambda(p, m["diff"]), m["diff"], eps, m.get("q_temp"), pos0)
    return out.reshape(T, H * V) @ p["o"].T


def hgrn2(h, p, m, eps, state=None):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with f = l + (1 - l) sigmoid(W_f h + b)."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].T).reshape(T, H, D)
    v = (h @ p["v"].T).reshape(T, H, V)
    low = p["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).reshape(T, H, D)
    S = torch.zeros(H, D, V, dtype=F) if state is None else state
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms(out, eps) * p["norm"]
    return out.reshape(T, H * V) @ p["o"].T, S


def talking_window_attention(h, p, m, eps, pos0=0):
    """Grouped-query attention with biases, a norm per q and k head, a rotation of the heads' first coordinates,
    the heads' scores mixed by a matrix before the softmax, and a sliding window."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ p["q"].T + p["q.b"]).reshape(T, H, D)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, G, D)
    v = (h @ p["v"].T + p["v.b"]).reshape(T, G, V)
    q, k = rms(q, eps) * p["q.norm"], rms(k, eps) * p["k.norm"]
    rot = m.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_partial(q, pos, rot["dims"], rot["base"]), rotate_partial(k, pos, rot["dims"], rot["base"])
    out = talking_core(q, k, v, p["talk"], m["scale"], m["mask"]["size"] if m.get("mask") else None)
    return out.reshape(T, H * V) @ p["o"].T


def talking_core(q, k, v, talk, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]: score_h <- sum_g talk[h, g] score_g, then the window and the softmax."""
    T, H = q.shape[:2]
    G, V = k.shape[1], v.shape[2]
    s = torch.stack([(q[:, hd] @ k[:, hd // (H // G)].T) * scale for hd in range(H)], 0)       # [H, T, T]
    s = torch.einsum("hg,gij->hij", talk, s)
    see = causal(T, window)
    out = torch.zeros(T, H, V, dtype=F)
    for hd in range(H):
        out[:, hd] = softmax_rows(s[hd], see) @ v[:, hd // (H // G)]
    return out


def conv_taps(u, w, b, before=None):
    """u [T, C], w [C, taps] whose last column is the current token's, b [C]; ``before``: the taps - 1 inputs
    that came before (zeros at a sequence's start)."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F) if before is None else before, u], 0)
    y = torch.zeros_like(u) + b
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y, pad[T:]


def ssd(h, p, m, eps, state=None):
    """The state-space mixer: S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t."""
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    u = h @ p["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    S, before = (torch.zeros(H, N, V, dtype=F), None) if state is None else state
    xbc, before = conv_taps(xbc, p["conv"], p["conv.b"], before)
    xbc = silu(xbc)
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + p["dt_bias"])
    A = torch.exp(p["A_log"])
    grp = torch.arange(H) // (H // G)
    y = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = torch.exp(-A * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][grp][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, C[t][grp]) + p["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = group_norm(y, p["norm"], eps, m["norm_groups"])
    return y @ p["o"].T, (S, before)


def clamped_expert(x, gate, up, down, limit):
    g = torch.clamp(x @ gate.T, max=limit)
    u = torch.clamp(x @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(x, w_router, top):
    """Sigmoid scores; the ``top`` largest (the lower index first among equals); weights = the scores themselves."""
    s = torch.sigmoid(x @ w_router.T)
    idx = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return idx, torch.gather(s, 1, idx)


def moe(x, p, mlp):
    """sum over the chosen experts of expert(weight * x), plus the shared expert."""
    T = x.shape[0]
    idx, wt = route(x, p["router"], mlp["router"]["top"])
    out = torch.zeros(T, p["e0.down"].shape[0], dtype=F)
    for t in range(T):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += clamped_expert(wt[t, j] * x[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"],
                                     mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(x, p["shared.gate"], p["shared.up"], p["shared.down"], mlp["shared"]["limit"])
    return out


def sub(p, prefix):
    return {k[len(prefix):]: v for k, v in p.items() if k.startswith(prefix)}


def mixer(kind, a, p, m, eps, pos0=0, state=None):
    """-> (output, state). ``state``: what a recurrent mixer carries (None at a sequence's start)."""
    if kind == "attention":
        return diff_attention(a, p, m, eps, pos0), None
    if kind == "hgrn2":
        return hgrn2(a, p, m, eps, state)
    if kind == "parallel":
        left = talking_window_attention(a, sub(p, "left."), m["left"], eps, pos0)
        right, state = ssd(a, sub(p, "right."), m["right"], eps, state)
        return m["left_scale"] * left + m["right_scale"] * right, state
    raise ValueError(kind)


def read_model(folder):
    """(config.json as a dict, tensors by name) of a model folder."""
    import json
    import os

    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


def forward(tokens, tensors, cfg, taps=None):
    """Logits [T, vocab] of one whole sequence. ``taps``: a list that receives the stream after every layer run."""
    p = {k: v.to(F) for k, v in tensors.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = p["embed"][torch.tensor(tokens)]
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{lc.get('weights_of', i)}."
        lp = sub(p, pre)
        a = group_norm(x, lp["norm1"], eps, groups)
        d, _ = mixer(lc["type"], a, sub(lp, "mix."), lc["mixer"], eps)
        x = x + d
        if lc.get("mlp"):
            x = x + moe(group_norm(x, lp["norm2"], eps, groups), sub(lp, "mlp."), lc["mlp"])
        if taps is not None:
            taps.append(x.clone())
    return group_norm(x, p["final.norm"], eps, groups) @ p["embed"].T
