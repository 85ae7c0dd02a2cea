"""Plain, slow restatement of the Naguzen decoder for the numerics tests: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batching), float64 by default.  It shares no code with the served model:
weights come in as a ``{checkpoint name: tensor}`` dict and the configuration as the parsed ``config.json`` dict."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(h, w):
    """h [S, C], w [C, taps]: out_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    S, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(S):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_half(x, pos, base, dims):
    """x [..., D]: the first ``dims`` coordinates are rotated, coordinate i paired with i + dims/2."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        a = pos * base ** (-2.0 * i / dims)
        c, s = math.cos(a), math.sin(a)
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def latent_attention(h, P, m, eps):
    S = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, dims, win, scale = m["rot"]["base"], m["rot"]["dims"], m["mask"]["size"], m["scale"]
    cq = rms(h @ P["dq"].T, eps) * P["dq.norm"]
    q = (cq @ P["uq"].T).reshape(S, H, D + R)
    kv = h @ P["dkv"].T
    c, kr = rms(kv[:, :C], eps) * P["dkv.norm"], kv[:, C:]
    ku = (c @ P["uk"].T).reshape(S, H, D)
    vv = (c @ P["uv"].T).reshape(S, H, V)
    out = torch.zeros(S, H, V, dtype=h.dtype)
    for i in range(S):
        qi = q[i].clone()
        qi[:, D:] = rotate_half(q[i, :, D:], i, base, dims)
        lo = max(0, i - win + 1)
        scores = torch.empty(H, i - lo + 1, dtype=h.dtype)
        for j in range(lo, i + 1):
            kj = rotate_half(kr[j], j, base, dims)
            scores[:, j - lo] = ((qi[:, :D] * ku[j]).sum(-1) + qi[:, D:] @ kj) * scale
        p = torch.softmax(scores, -1)
        out[i] = torch.einsum("hj,jhv->hv", p, vv[lo:i + 1])
    return out.reshape(S, H * V) @ P["o"].T


def gla(h, P, m, eps):
    S = h.shape[0]
    H, D, V, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ P["q"].T).reshape(S, H, D) * D ** -0.5
    k = (h @ P["k"].T).reshape(S, H, D)
    v = (h @ P["v"].T).reshape(S, H, V)
    z = (h @ P["a1"].T) @ P["a2"].T + P["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(S, H, D)
    state = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(S, H, V, dtype=h.dtype)
    for t in range(S):
        state = alpha[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", state, q[t])
    o = rms(o, eps) * P["norm"]
    g = h @ P["g"].T
    return (o.reshape(S, H * V) * (g * torch.sigmoid(g))) @ P["o"].T


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rglru(h, P, m):
    S = h.shape[0]
    W, nb = m["width"], m["blocks"]
    y = gelu_tanh(h @ P["y"].T + P["y.b"])
    u = short_conv(h @ P["x"].T + P["x.b"], P["conv"]) + P["conv.b"]
    ub = u.reshape(S, nb, W // nb)
    r = torch.sigmoid(torch.einsum("boi,sbi->sbo", P["ra"], ub) + P["ra.b"]).reshape(S, W)
    i = torch.sigmoid(torch.einsum("boi,sbi->sbo", P["ri"], ub) + P["ri.b"]).reshape(S, W)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(P["lam"]))
    state = torch.zeros(W, dtype=h.dtype)
    out = torch.zeros(S, W, dtype=h.dtype)
    for t in range(S):
        state = a[t] * state + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        out[t] = state
    return (out * y) @ P["o"].T


def xielu(z, act):
    sp = torch.nn.functional.softplus
    pos = sp(act[0]) * z * z + z / 2
    neg = (0.5 + sp(act[1])) * (torch.exp(z) - 1 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def gelu_erf(z):
    return 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))


def dense_ff(h, P):
    return xielu(h @ P["up"].T, P["act"]) @ P["down"].T


def expert(h, up, down):
    return gelu_erf(h @ up.T) @ down.T


def moe_ff(h, P, f):
    E, top, rs = f["router"]["experts"], f["router"]["top"], f["router"]["scale"]
    s = torch.sigmoid(h @ P["router"].T)
    out = torch.zeros(h.shape[0], P["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        chosen = torch.argsort(s[t], descending=True, stable=True)[:top]
        for e in chosen.tolist():
            out[t] += s[t, e] * rs * expert(h[t], P[f"e{e}.up"], P[f"e{e}.down"])
    if f.get("shared"):
        out = out + expert(h, P["shared.up"], P["shared.down"])
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, dtype=torch.float64):
    """tokens: list of ids → (logits [S, vocab], residual stream after every layer [L, S, width])."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens)]
    trail = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = x + short_conv(x, W[p + "canon1"])
        P = sub(W, p + "mix.")
        if L["type"] == "latent_attention":
            y = latent_attention(h, P, L["mixer"], eps)
        elif L["type"] == "gla":
            y = gla(h, P, L["mixer"], eps)
        elif L["type"] == "rglru":
            y = rglru(h, P, L["mixer"])
        else:
            raise ValueError(L["type"])
        x = x + rms(y, eps) * W[p + "norm1"]
        if L.get("mlp"):
            h = x + short_conv(x, W[p + "canon2"])
            P = sub(W, p + "mlp.")
            y = dense_ff(h, P) if L["mlp"]["kind"] == "dense" else moe_ff(h, P, L["mlp"])
            x = x + rms(y, eps) * W[p + "norm2"]
        trail.append(x)
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T, torch.stack(trail)
