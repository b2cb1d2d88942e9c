"""Zafilix in plain, slow PyTorch: the statement the engine is held against.

One function per mechanism, whole sequences only, no cache, no batching, nothing shared with the package.  `cfg` is
the raw config.json dictionary, `w` maps tensor names to tensors; everything runs in the type of the weights it is
given (the tests pass float32 or float64 copies).

    embedding        x[p] = embed[token] * embedding.scale
    layer            x += norm1(mixer(x));  x += norm2(ff(x)): the sublayers read x as it is, a norm stands only
                     behind them; norm(y) = y / sqrt(mean(y^2) + eps) * (1 + gain)
    attention        grouped heads; q and k are normed over their whole rows (all heads at once, plain gains) and
                     then turned: pairs (2i, 2i+1) over the first rot.dims elements of a head by the angle
                     p * base^(-2i/dims) / factor; key j is visible from i when j <= i and both lie in the same
                     block of mask.size positions; softmax of scale * q.k; the heads' outputs times sigmoid(g x);
                     output projection
    latent attention one latent row c = norm(first kv_rank rows of dkv x) and one turned key part (the last rot_dim
                     rows, pairs (i, i + dims/2)) per position, shared by all heads; a head's key is [uk c, turned
                     part], its value uv c, its query [dim plain elements, rot_dim turned]; key j is visible from
                     i when 0 <= i - j < mask.size; softmax of scale * q.k; output projection
    feed-forward     down(relu(up x)^2)
    head             final norm, logits = (head x) * logit_scale, then cap * tanh(logits / cap)
    weights_of       a layer that names another layer runs on that layer's tensors
"""
from __future__ import annotations

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, gain, eps):
    return rms(x, eps) * (1 + gain)


def norm_plain(x, gain, eps):
    return rms(x, eps) * gain


def angles(positions, rot, dtype):
    """[n, dims/2]: position * base^(-2i/dims) / factor."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(rot["base"]) ** (-2.0 * i / dims)
    factor = (rot.get("scaling") or {}).get("factor")
    if factor is not None:
        freq = freq / float(factor)
    return (positions.to(torch.float64)[:, None] * freq[None, :]).to(dtype)


def turn_neighbours(x, positions, rot):
    """x [n, heads, d]: the pairs (2i, 2i+1) of the first rot.dims elements turn; the rest stays."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    a = angles(positions, rot, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def turn_halves(x, positions, rot):
    """x [n, heads, d]: the pairs (i, i + dims/2) of the first rot.dims elements turn; the rest stays."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    half = dims // 2
    a = angles(positions, rot, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def seen_in_blocks(n, size):
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return (j <= i) & (i // size == j // size)


def seen_in_window(n, size):
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return (j <= i) & (i - j < size)


def seen_all(n):
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    return j <= i


def softmax_heads(q, k, v, scale, seen):
    """q [n, H, d], k [n, G, d], v [n, G, dv] -> [n, H * dv]."""
    H, G = q.shape[1], k.shape[1]
    heads = []
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(heads, dim=-1)


def attention(m, w, p, h, eps):
    n, H, G, d = h.shape[0], m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    dv = m.get("vdim", d)
    pos = torch.arange(n)
    q = norm_plain(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(n, H, d)
    k = norm_plain(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(n, G, d)
    v = (h @ w[p + "v"].T).view(n, G, dv)
    q, k = turn_neighbours(q, pos, m.get("rot")), turn_neighbours(k, pos, m.get("rot"))
    seen = seen_in_blocks(n, m["mask"]["size"]) if m.get("mask") else seen_all(n)
    mixed = softmax_heads(q, k, v, m.get("scale", d ** -0.5), seen)
    return (mixed * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def latent_attention(m, w, p, h, eps):
    n, H, d, r, dv, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(n)
    q = (h @ w[p + "q"].T).view(n, H, d + r)
    down = h @ w[p + "dkv"].T
    c = norm_plain(down[:, :rank], w[p + "dkv.norm"], eps)
    shared = turn_halves(down[:, rank:].view(n, 1, r), pos, m.get("rot"))
    q_plain, q_turned = q[..., :d], turn_halves(q[..., d:].contiguous(), pos, m.get("rot"))
    k_plain = (c @ w[p + "uk"].T).view(n, H, d)
    v = (c @ w[p + "uv"].T).view(n, H, dv)
    seen = seen_in_window(n, m["mask"]["size"]) if m.get("mask") else seen_all(n)
    heads = []
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_turned[:, a] @ shared[:, 0].T) * m.get("scale", (d + r) ** -0.5)
        s = s.masked_fill(~seen, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, a])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def feed_forward(w, p, h):
    return torch.relu(h @ w[p + "up"].T).square() @ w[p + "down"].T


def owner(cfg, i):
    """The layer whose tensors layer i runs on."""
    src = cfg["layers"][i].get("weights_of")
    return i if src is None else src


def layers(cfg, w, tokens):
    """The residual stream after the embedding's layers, one entry per layer run: [runs, n, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    out = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg, i)}."
        mixer = {"attention": attention, "latent_attention": latent_attention}[layer["type"]]
        x = x + norm_one_plus(mixer(layer["mixer"], w, p + "mix.", x, eps), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + norm_one_plus(feed_forward(w, p + "mlp.", x), w[p + "norm2"], eps)
        out.append(x)
    return torch.stack(out)


def forward(cfg, w, tokens):
    """Logits [n, vocab] of one whole sequence."""
    x = layers(cfg, w, tokens)[-1]
    logits = (norm_one_plus(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return logits if cap is None else cap * torch.tanh(logits / cap)
