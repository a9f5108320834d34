"""Bevadra restated from its equations: whole sequences, no cache, no kernels, one function per mechanism.

Everything runs in the dtype of the tensors it is given (float64 in the tests).  ``config`` is the parsed
``config.json``; ``w`` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def window_mask(tokens, window, like):
    """[T, T] True where query i sees key j: 0 <= i - j < window (no window: j <= i)."""
    i = torch.arange(tokens).unsqueeze(1)
    j = torch.arange(tokens).unsqueeze(0)
    seen = j <= i
    if window is not None:
        seen &= (i - j) < window
    return seen.to(like.device)


def slopes(heads, like):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=like.dtype)


def softmax_with_extra(scores, seen, extra=None):
    """Softmax over the visible keys of [H, T, T] scores; ``extra`` [H] is one more term of the denominator
    per head that has neither key nor value."""
    scores = scores.masked_fill(~seen, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if extra is not None:
        top = torch.maximum(top, extra.view(-1, 1, 1))
    e = torch.exp(scores - top)
    denom = e.sum(-1, keepdim=True)
    if extra is not None:
        denom = denom + torch.exp(extra.view(-1, 1, 1) - top)
    return e / denom


def project_keys_values(h, w, p, m):
    """Keys [T, G, dim] and values [T, G, vdim] of an attention layer that owns them."""
    tokens = h.shape[0]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(tokens, m["kv_heads"], m["dim"])
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(tokens, m["kv_heads"], m["vdim"])
    return k, v


def attention(h, w, p, m, k, v):
    """Grouped-query attention with a linear distance bias, a window, a learned sink and an element-wise gate."""
    tokens = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(tokens, heads, dim)
    rep = heads // groups
    kk = k.repeat_interleave(rep, dim=1)  # head h reads kv head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    pos = torch.arange(tokens, dtype=h.dtype)
    distance = pos.view(-1, 1) - pos.view(1, -1)
    scores = scores - slopes(heads, h).view(-1, 1, 1) * distance
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    weights = softmax_with_extra(scores, window_mask(tokens, window, h), w[p + "sink"])
    out = torch.einsum("hij,jhd->ihd", weights, vv).reshape(tokens, heads * vdim)
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T + w[p + "o.b"]


def rotate_half(x, positions, base, dims):
    """Rotation of the first ``dims`` elements of the last axis; element i pairs with i + dims / 2."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions.to(x.dtype).view(-1, *([1] * (x.dim() - 2)), 1) * freq
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, rest), dim=-1)


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are expanded from a shared low-rank latent, with one rotated key part that
    all heads share."""
    tokens = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(tokens)
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(tokens, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = down[:, rank:]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_half(q_rot, positions, base, dims)
    k_rot = rotate_half(k_rot, positions, base, dims)
    k_plain = (c @ w[p + "uk"].T).view(tokens, heads, dim)
    v = (c @ w[p + "uv"].T).view(tokens, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    window = m.get("mask", {}).get("size") if m.get("mask") else None
    weights = softmax_with_extra(scores, window_mask(tokens, window, h))
    out = torch.einsum("hij,jhd->ihd", weights, v)
    out = out * torch.sigmoid(h @ w[p + "g"].T).unsqueeze(-1)
    return out.reshape(tokens, heads * vdim) @ w[p + "o"].T


def feed_forward(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def forward(config, w, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    streams = []
    for index, layer in enumerate(config["layers"]):
        name = f"l{index}."
        m = layer["mixer"]
        h = layer_norm(x, w[name + "norm1"], w[name + "norm1.b"], eps)
        if layer["type"] == "attention":
            source = m.get("kv_from")
            if source is None:
                kept[index] = project_keys_values(h, w, name + "mix.", m)
                source = index
            mixed = attention(h, w, name + "mix.", m, *kept[source])
        elif layer["type"] == "latent_attention":
            mixed = latent_attention(h, w, name + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            mixed = mixed + feed_forward(h, w, name + "mlp.")
        x = x + mixed
        streams.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = x @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
