"""Plain, slow restatement of the Pinirax decoder for the numerics tests: one function per mechanism, whole sequences only
(no cache, no state carried between calls, no batching), float64 by default.  It shares no code with the served model:
weights come in as a ``{checkpoint name: tensor}`` dict and the configuration as the parsed ``config.json`` dict."""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def embed(tokens, table, scale):
    """Scaled table rows plus interleaved sinusoids: coordinate 2i is sin(p f_i), 2i+1 is cos(p f_i), f_i = 10000^(-2i/width)."""
    W = table.shape[1]
    x = table[tokens] * scale
    for p in range(len(tokens)):
        for i in range(W // 2):
            a = p * 10000.0 ** (-2.0 * i / W)
            x[p, 2 * i] += math.sin(a)
            x[p, 2 * i + 1] += math.cos(a)
        if W % 2:
            x[p, W - 1] += math.sin(p * 10000.0 ** (-(W - 1.0) / W))
    return x


def norm1p(x, w, eps):
    """RMS norm whose stored weight is the gain's offset from one."""
    return rms(x, eps) * (1.0 + w)


def causal_conv(h, w, bias=None):
    """h [S, C], w [C, taps]: out_t = bias + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before the start."""
    S, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for t in range(S):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
        if bias is not None:
            out[t] += bias
    return out


def window_attention(h, P, m, eps):
    """Grouped-query softmax attention over a sliding window: biased projections, per-head RMS norm of queries and keys, no
    positional rotation, tanh-capped scores, one sigmoid gate per head on the output."""
    S = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    win, scale, cap = m["mask"]["size"], m["scale"], m["softcap"]
    q = (h @ P["q"].T + P["q.b"]).reshape(S, H, D)
    k = (h @ P["k"].T + P["k.b"]).reshape(S, G, D)
    v = (h @ P["v"].T + P["v.b"]).reshape(S, G, V)
    q, k = rms(q, eps) * P["q.norm"], rms(k, eps) * P["k.norm"]
    gate = torch.sigmoid(h @ P["g"].T)                                     # [S, H]
    out = torch.zeros(S, H, V, dtype=h.dtype)
    for i in range(S):
        lo = max(0, i - win + 1)
        for hd in range(H):
            g = hd // (H // G)
            sc = (k[lo:i + 1, g] @ q[i, hd]) * scale
            if cap > 0:                                                    # a cap of zero stands for no cap
                sc = cap * torch.tanh(sc / cap)
            p = torch.softmax(sc, 0)
            out[i, hd] = (p[:, None] * v[lo:i + 1, g]).sum(0) * gate[i, hd]
    return out.reshape(S, H * V) @ P["o"].T


def gated_delta_rule(h, P, m, eps):
    """Per head a matrix memory S [dim, vdim]: decay, then an error-correcting write of the value at the key, then the read."""
    S = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ P["q"].T, P["q.conv"])).reshape(S, G, D)
    k = silu(causal_conv(h @ P["k"].T, P["k.conv"])).reshape(S, G, D)
    v = silu(causal_conv(h @ P["v"].T, P["v.conv"])).reshape(S, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P["b"].T)                                     # [S, H]
    decay = torch.exp(-torch.exp(P["A_log"]) * softplus(h @ P["a"].T + P["dt_bias"]))
    o = torch.zeros(S, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        M = torch.zeros(D, V, dtype=h.dtype)
        for t in range(S):
            M = decay[t, hd] * M
            u = beta[t, hd] * (v[t, hd] - M.T @ k[t, g])
            M = M + torch.outer(k[t, g], u)
            o[t, hd] = M.T @ q[t, g]
    o = rms(o, eps) * P["norm"]
    return (o.reshape(S, H * V) * silu(h @ P["g"].T)) @ P["o"].T


def parallel_mixer(h, P, m, eps):
    left = window_attention(h, {k[5:]: v for k, v in P.items() if k.startswith("left.")}, m["left"], eps)
    right = gated_delta_rule(h, {k[6:]: v for k, v in P.items() if k.startswith("right.")}, m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mamba2(h, P, m, eps):
    """Selective state space layer with one scalar decay per head (state [N, vdim] per head)."""
    S = h.shape[0]
    H, V, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * V
    p = h @ P["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P["conv"], P["conv.b"]))
    x = xbc[:, :inner].reshape(S, H, V)
    Bm = xbc[:, inner:inner + G * N].reshape(S, G, N)
    Cm = xbc[:, inner + G * N:].reshape(S, G, N)
    dt = softplus(dt + P["dt_bias"])                                       # [S, H]
    y = torch.zeros(S, H, V, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        M = torch.zeros(N, V, dtype=h.dtype)
        for t in range(S):
            M = torch.exp(-torch.exp(P["A_log"][hd]) * dt[t, hd]) * M + dt[t, hd] * torch.outer(Bm[t, g], x[t, hd])
            y[t, hd] = M.T @ Cm[t, g] + P["D"][hd] * x[t, hd]
    y = y.reshape(S, inner) * silu(z)
    y = rms(y.reshape(S, NG, inner // NG), eps).reshape(S, inner) * P["norm"]
    return y @ P["o"].T


def moe(h, P, f):
    """Softmax router over real and identity experts; an additive correction steers the choice only; weights are not renormalised."""
    r = f["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ P["router"].T, -1)                               # [S, E + I]
    choice = s + P["correction"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(choice[t], top).indices.tolist():
            if e >= E:
                y = h[t]
            else:
                y = (silu(h[t] @ P[f"e{e}.gate"].T) * (h[t] @ P[f"e{e}.up"].T)) @ P[f"e{e}.down"].T
            out[t] += s[t, e] * y
    return out


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg, w, tokens, dtype=torch.float64, taps=None):
    """tokens: list of ids → (logits [S, vocab], residual stream after every layer [L, S, width])."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = embed(torch.tensor(tokens), w["embed"], cfg["embedding"]["scale"])
    stream = []
    for i, spec in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm1p(x, w[p + "norm1"], eps)
        mix = {"parallel": parallel_mixer, "mamba2": mamba2}[spec["type"]](h, sub(w, p + "mix."), spec["mixer"], eps)
        x = x + norm1p(mix, w[p + "norm1b"], eps)
        if spec.get("mlp"):
            h = norm1p(x, w[p + "norm2"], eps)
            x = x + norm1p(moe(h, sub(w, p + "mlp."), spec["mlp"]), w[p + "norm2b"], eps)
        stream.append(x.clone())
    logits = norm1p(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(stream)
