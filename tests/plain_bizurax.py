"""Bizurax restated from its equations: whole sequences, no cache, no kernels, one function per mechanism.

Everything runs in the dtype of the tensors it is given (float64 in the tests).  ``config`` is the parsed
``config.json``; ``w`` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def frequencies(rot, like):
    """f_i = base^(-2 i / dims), each divided by the factor of a linear scaling when the layer has one."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=like.dtype)
    scaling = rot.get("scaling")
    return f / scaling["factor"] if scaling else f


def rotate(x, positions, rot, interleaved):
    """Rotation of the first ``dims`` elements of the last axis of ``x [T, ..., d]``.  Pairs are (i, i + dims / 2),
    or (2 i, 2 i + 1) when ``interleaved``; (u, v) becomes (u cos a - v sin a, v cos a + u sin a), a = p f_i."""
    dims = rot["dims"]
    half = dims // 2
    angle = positions.to(x.dtype).view(-1, *([1] * (x.dim() - 2)), 1) * frequencies(rot, x)
    cos, sin = torch.cos(angle), torch.sin(angle)
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def causal(tokens):
    i = torch.arange(tokens)
    return i.view(1, -1) <= i.view(-1, 1)


def softmax_with_extra(scores, seen, extra=None):
    """Softmax over the visible keys of ``[H, T, T]`` scores; ``extra [H]`` is one more term ``exp(extra_h)`` of
    the denominator that has neither key nor value."""
    scores = scores.masked_fill(~seen, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if extra is not None:
        top = torch.maximum(top, extra.view(-1, 1, 1))
    e = torch.exp(scores - top)
    denom = e.sum(-1, keepdim=True)
    if extra is not None:
        denom = denom + torch.exp(extra.view(-1, 1, 1) - top)
    return e / denom


def attention(h, w, p, m, eps):
    """Grouped-query attention: biased projections, rotation, unit q and k, capped scores, a sink in the softmax."""
    tokens = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(tokens)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(tokens, heads, dim)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(tokens, groups, dim)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(tokens, groups, vdim)
    q = rms_norm(rotate(q, positions, m["rot"], False), None, eps)
    k = rms_norm(rotate(k, positions, m["rot"], False), None, eps)
    rep = heads // groups
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)  # head h reads kv head h // rep
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    weights = softmax_with_extra(scores, causal(tokens), w[p + "sink"])
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(tokens, heads * vdim)
    return out @ w[p + "o"].T


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are expanded from one normed latent per token, with one rotated key part
    that all heads share."""
    tokens = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(tokens)
    q = (h @ w[p + "q"].T).view(tokens, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = down[:, rank:]
    q_rot = rotate(q_rot, positions, m["rot"], True)
    k_rot = rotate(k_rot, positions, m["rot"], True)
    k_plain = (c @ w[p + "uk"].T).view(tokens, heads, dim)
    v = (c @ w[p + "uv"].T).view(tokens, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    weights = softmax_with_extra(scores, causal(tokens))
    out = torch.einsum("hij,jhd->ihd", weights, v)
    return out.reshape(tokens, heads * vdim) @ w[p + "o"].T


def retention(h, w, p, m, eps, state=None, start=0):
    """Linear attention with one fixed decay per head, token by token: S_t = a_h S_(t-1) + k_t v_t^T, o_t = S_t^T
    q_t.  Returns the output and the state ``[heads, dim, vdim]`` after the last token."""
    tokens = h.shape[0]
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    positions = torch.arange(start, start + tokens)
    q = rotate((h @ w[p + "q"].T).view(tokens, heads, dim), positions, m["rot"], False)
    k = rotate((h @ w[p + "k"].T).view(tokens, heads, dim), positions, m["rot"], False) * dim**-0.5
    v = (h @ w[p + "v"].T).view(tokens, heads, vdim)
    decay = torch.tensor(m["decay"], dtype=h.dtype).view(heads, 1, 1)
    s = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(tokens):
        s = decay * s + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        outs.append(torch.einsum("hde,hd->he", s, q[t]))
    o = rms_norm(torch.stack(outs), None, eps).reshape(tokens, heads * vdim)
    gate = h @ w[p + "g"].T
    return (o * (gate * torch.sigmoid(gate))) @ w[p + "o"].T, s


def dense_feed_forward(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def gated_unit(h, w, p):
    gate = h @ w[p + "gate"].T
    return (gate * torch.sigmoid(gate) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, top):
    """The chosen units ``[T, top]`` and their weights: a softmax over the chosen logits only."""
    logits = h @ w[p + "router"].T + w[p + "router.b"]
    best = torch.topk(logits, top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def route_following(h, w, p, top, follow, close):
    """The routing of :func:`route`, except that a token whose decision was won by less than ``close`` (in logits)
    takes the units of ``follow [T, top]`` (another implementation's choice, which rounding may have turned)."""
    logits = h @ w[p + "router"].T + w[p + "router.b"]
    ranked = torch.sort(logits, dim=-1, descending=True).values
    units, weights = route(h, w, p, top)
    if logits.shape[-1] == top:
        return units, weights
    for t in range(h.shape[0]):
        theirs = sorted(int(u) for u in follow[t])
        if sorted(units[t].tolist()) != theirs and float(ranked[t, top - 1] - ranked[t, top]) < close:
            units[t] = torch.tensor(theirs)
            weights[t] = torch.softmax(logits[t, units[t]], dim=-1)
    return units, weights


def routed_feed_forward(h, w, p, mlp, follow=None, close=0.0):
    top = mlp["router"]["top"]
    units, weights = route(h, w, p, top) if follow is None else route_following(h, w, p, top, follow, close)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for unit, weight in zip(units[t].tolist(), weights[t]):
            out[t] += weight * gated_unit(h[t : t + 1], w, f"{p}e{unit}.")[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, mlp, follow=None, close=0.0):
    return dense_feed_forward(h, w, p) if mlp["kind"] == "dense" else routed_feed_forward(h, w, p, mlp, follow, close)


def mixer(layer, h, w, p, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        return attention(h, w, p, m, eps)
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps)
    if kind == "retention":
        return retention(h, w, p, m, eps)[0]
    raise ValueError(kind)


def layer_order(config):
    """The layers' numbers in the order they run: a loop's span repeated in place."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    span = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + span * loop["times"] + list(range(loop["stop"], count))


def hyper_sublayer(streams, w, p, mult, eps, norm_weight, sublayer):
    """One sublayer on several residual streams ``[S, T, width]``: it reads a weighted sum of them, and every new
    stream is a mix of the old ones plus its share of the sublayer's output."""
    u = torch.einsum("s,stw->tw", w[p + "in"], streams)
    y = sublayer(rms_norm(u, norm_weight, eps))
    return torch.einsum("sr,stw->rtw", w[p + "mix"], streams) + mult * w[p + "out"].view(-1, 1, 1) * y


def forward(config, w, tokens, return_layers=False, follow=None, close=0.0):
    """Logits ``[T, vocab]`` of one whole sequence (and the stream after every layer run).  ``follow``: per layer run
    with routed units, another implementation's choices ``[T, top]``, taken where a decision was closer than ``close``."""
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    count = config.get("streams")
    streams = x.unsqueeze(0).repeat(count, 1, 1) if count else None
    after = []
    for run, index in enumerate(layer_order(config)):
        layer, name = config["layers"][index], f"l{index}."
        theirs = None if follow is None else follow.get(run)
        mix = lambda h: mixer(layer, h, w, name + "mix.", eps)  # noqa: E731
        ff = lambda h: feed_forward(h, w, name + "mlp.", layer["mlp"], theirs, close)  # noqa: E731
        if streams is None:
            x = x + mult * mix(rms_norm(x, w[name + "norm1"], eps))
            if layer.get("mlp") is not None:
                x = x + mult * ff(rms_norm(x, w[name + "norm2"], eps))
        else:
            streams = hyper_sublayer(streams, w, name + "hc1.", mult, eps, w[name + "norm1"], mix)
            if layer.get("mlp") is not None:
                streams = hyper_sublayer(streams, w, name + "hc2.", mult, eps, w[name + "norm2"], ff)
            x = streams.sum(0)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
