"""Gudarax in plain, slow PyTorch: the statement the engine is held against.

One function per mechanism, whole sequences only, no cache, no batching, nothing shared with the package.  `cfg` is
the raw config.json dictionary, `w` maps tensor names to tensors; everything runs in the type of the weights it is
given (the tests pass float32 or float64 copies).

    embedding        x[p] = embed[token] * embedding.scale + pos[p]
    layer            x += mixer(norm1(x));  x += ff(norm2(x));  then the token's own input (below);
                     norm(y) = y / sqrt(mean(y^2) + eps) * gain
    token input      e = columns [i * d, (i + 1) * d) of side.embed[token] for layer i;  y = proj(gelu_tanh(gate x) * e);
                     x += norm(y) with the gain side.norm
    attention        q, k, v with biases; q and k normed over their whole rows (all heads at once); no turn; the score of
                     key j from position i is scale * q.k - slope_h * (i - j), slope_h = 2^(-8 (h + 1) / heads); key j is
                     visible when 0 <= i - j < mask.size; softmax; from the second layer with `v_mix` on the values are
                     (1 - lambda) v + lambda v_first, v_first being the first such layer's values of the same token
    latent attention queries through a normed latent row (dq, dq.norm, uq); keys and values are maps (uk, uv) of one normed
                     latent row per position (dkv, dkv.norm); every earlier key is visible; softmax of scale * q.k; the
                     heads' outputs times sigmoid(g x); output projection
    delta            q, k, v through a causal convolution over time per channel and silu; q and k heads made unit vectors
                     (q also times dim^-1/2); per head a state S [dim, vdim]:  S *= decay;  u = beta (v - S^T k);
                     S += k u^T;  o = S^T q;  decay = exp(-exp(A_log) softplus(a x + dt_bias)), beta = sigmoid(b x);
                     o divided by its root mean square per head, times a gain and silu(g x); output projection
    feed-forward     dense: down(silu(gate x) * up x);  experts: scores sigmoid(router x), the `top` largest chosen, the
                     output is the sum over the chosen of down(relu(up (s x))^2) with s the expert's score
    head             final norm, logits = head x
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, gain, eps):
    return rms(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(cfg, w, tokens):
    n = len(tokens)
    return w["embed"][tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0)) + w["pos"][:n]


def softmax_rows(scores, visible):
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1)


def slopes(heads, dtype):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def window_visible(n, size):
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    d = i - j
    return (d >= 0) & ((d < size) if size is not None else True)


def attention(m, w, p, h, eps, v_first):
    """Returns (output, the layer's own values before mixing)."""
    n, H, D = h.shape[0], m["heads"], m["dim"]
    G, V, scale = m.get("kv_heads", H), m.get("vdim", D), float(m.get("scale", D ** -0.5))
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = norm(q, w[p + "q.norm"], eps).view(n, H, D)
    k = norm(k, w[p + "k.norm"], eps).view(n, G, D)
    own = v
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1 - lam) * v + lam * v_first
    v = v.view(n, G, V)
    size = (m.get("mask") or {}).get("size")
    visible = window_visible(n, size)
    dist = (torch.arange(n)[:, None] - torch.arange(n)[None, :]).to(h.dtype)
    sl = slopes(H, h.dtype)
    out = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale - sl[a] * dist
        out.append(softmax_rows(s, visible) @ v[:, g])
    return torch.cat(out, dim=-1) @ w[p + "o"].T, own


def latent_attention(m, w, p, h, eps):
    n, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    cq = norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(n, H, D)
    c = norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).view(n, H, D)
    v = (c @ w[p + "uv"].T).view(n, H, V)
    visible = window_visible(n, None)
    out = []
    for a in range(H):
        s = (q[:, a] @ k[:, a].T) * float(m.get("scale", D ** -0.5))
        out.append(softmax_rows(s, visible) @ v[:, a])
    heads = torch.cat(out, dim=-1) * torch.sigmoid(h @ w[p + "g"].T)
    return heads @ w[p + "o"].T


def short_conv(x, taps):
    """x [n, channels], taps [channels, T]: y[t] = sum_i taps[:, T - 1 - i] * x[t - i], zeros before the start."""
    n, T = x.shape[0], taps.shape[1]
    padded = torch.cat([x.new_zeros((T - 1, x.shape[1])), x], dim=0)
    y = torch.zeros_like(x)
    for i in range(T):
        y = y + padded[T - 1 - i:T - 1 - i + n] * taps[:, T - 1 - i]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta(m, w, p, h, eps):
    n, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    G = m.get("kv_heads", H)
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(n, G, D)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(n, G, D)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(n, H, V)
    q = unit(q) * D ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    out = h.new_zeros((n, H, V))
    for a in range(H):
        g = a // (H // G)
        S = h.new_zeros((D, V))
        for t in range(n):
            S = S * decay[t, a]
            u = beta[t, a] * (v[t, a] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, a] = S.T @ q[t, g]
    out = rms(out, eps) * w[p + "norm"]
    out = out.reshape(n, H * V) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def dense_ff(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(mlp, w, p, h):
    """(chosen [n, top], their scores [n, top])."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    val, idx = torch.topk(s, int(mlp["router"]["top"]), dim=-1)
    return idx, val


def experts_ff(mlp, w, p, h):
    idx, val = route(mlp, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            z = torch.relu((s * h[t]) @ w[f"{p}e{e}.up"].T) ** 2
            out[t] = out[t] + z @ w[f"{p}e{e}.down"].T
    return out


def token_input(cfg, w, i, x, tokens, eps):
    d = int(cfg["token_side"]["dim"])
    p = f"l{i}.side."
    e = w["side.embed"][tokens][:, i * d:(i + 1) * d]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return rms(y, eps) * w[p + "norm"]


def forward(cfg, w, tokens, layers_out=None):
    """Logits [n, vocab] of one whole sequence; `layers_out`, a list, receives the residual after every layer."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = embed(cfg, w, tokens)
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            y, own = attention(m, w, p, h, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = own
        elif layer["type"] == "latent_attention":
            y = latent_attention(m, w, p, h, eps)
        else:
            y = delta(m, w, p, h, eps)
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm(x, w[f"l{i}.norm2"], eps)
            x = x + (dense_ff(w, f"l{i}.mlp.", h) if mlp["kind"] == "dense" else experts_ff(mlp, w, f"l{i}.mlp.", h))
        if cfg.get("token_side"):
            x = x + token_input(cfg, w, i, x, tokens, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T
