"""Plain implementation of the Botuvik decoder for the tests: whole sequences, no cache, float64 by default,
one function per mechanism, written from the design's equations. It shares no code with the library's parts.

Notation: x is the stream [T, d]; h a normed form of it; positions count from 0; matrices are stored [out, in]
and applied as h @ W.T.
"""
import json
import math
import os

import torch

from plain_llama import read_safetensors


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# --------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x divided by the root of (its mean square + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def rotate_neighbour_pairs(v, positions, base, dims):
    """Rotate the first ``dims`` features of the last axis: feature 2i pairs with 2i + 1, by the angle
    position * base^(-2i / dims); (u, w) -> (u cos - w sin, w cos + u sin). The rest pass unchanged.
    ``v``: [T, heads, n] with n >= dims."""
    if dims == 0:
        return v
    out = v.clone()
    for i in range(dims // 2):
        angle = positions.to(v.dtype) * (base ** (-2.0 * i / dims))
        cos, sin = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        u, w = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = u * cos - w * sin
        out[..., 2 * i + 1] = w * cos + u * sin
    return out


def capped_scores(q, k, scale, cap):
    """q [Tq, n], k [Tk, n] -> cap * tanh(scale * q k^T / cap)."""
    s = (q @ k.T) * scale
    return cap * torch.tanh(s / cap) if cap else s


def softmax_with_sink(scores, sink):
    """Row-wise softmax whose denominator also holds exp(sink): the weights of a row sum to less than one."""
    big = torch.maximum(scores.max(-1, keepdim=True).values, sink)
    e = torch.exp(scores - big)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - big))


# --------------------------------------------------------------------------- mixers
def capped_attention(h, w, p, m, eps, positions=None):
    """Grouped-query attention: biased projections, rotation of neighbouring pairs, queries and keys divided by
    their root mean square per head, scaled and capped scores, causal mask, a sink per head, output projection."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    q = unit_rms(rotate_neighbour_pairs(q, positions, m["rot"]["base"], m["rot"]["dims"]), eps)
    k = unit_rms(rotate_neighbour_pairs(k, positions, m["rot"]["base"], m["rot"]["dims"]), eps)
    seen = positions[None, :] <= positions[:, None]
    heads = []
    for head in range(H):
        g = head // (H // G)
        s = capped_scores(q[:, head], k[:, g], m["scale"], m["softcap"]).masked_fill(~seen, -math.inf)
        heads.append(softmax_with_sink(s, w[p + "sink"][head]) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[p + "o"].T


def log_sigmoid(z):
    return -(torch.clamp(-z, min=0) + torch.log1p(torch.exp(-z.abs())))


def matrix_memory(h, w, p, m, eps, state=None):
    """Per head: S <- exp(f + m_prev - m) S + exp(i - m) k v^T, n likewise with k alone, m = max(f + m_prev, i) with
    m starting at 0; o = S^T q / (max(|n . q|, exp(-m)) + 1e-6). ``state``: (S, n, m) to go on from, else zeros.
    Returns the mixer's output and the state it leaves."""
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    i_log = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    f_log = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    if state is None:
        S = torch.zeros(H, dk, dv, dtype=h.dtype)
        n = torch.zeros(H, dk, dtype=h.dtype)
        big = torch.zeros(H, dtype=h.dtype)
    else:
        S, n, big = state
    out = []
    for t in range(T):
        new_big = torch.maximum(f_log[t] + big, i_log[t])
        keep = torch.exp(f_log[t] + big - new_big)
        take = torch.exp(i_log[t] - new_big)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        big = new_big
        below = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-big)) + 1e-6
        out.append(torch.einsum("hkv,hk->hv", S, q[t]) / below[:, None])
    o = unit_rms(torch.stack(out), eps).reshape(T, H * dv) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, (S, n, big)


# --------------------------------------------------------------------------- feed-forwards
def squared_relu_ffn(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def gated_expert(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(scores, groups, keep, top):
    """scores [T, E] -> (chosen expert indices [T, top], their weights, the smallest gap that decided a choice).
    A group (E / groups neighbours) scores the sum of its two largest scores; the ``top`` largest scores within the
    ``keep`` best groups win; weights = scores / (their sum + 1e-20)."""
    T, E = scores.shape
    per = E // groups
    grouped = scores.view(T, groups, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    order = group_score.sort(dim=-1, descending=True)
    gap = torch.tensor(math.inf, dtype=scores.dtype)
    if keep < groups:
        gap = torch.minimum(gap, (order.values[:, keep - 1] - order.values[:, keep]).min())
    open_group = torch.zeros(T, groups, dtype=torch.bool)
    open_group.scatter_(1, order.indices[:, :keep], True)
    allowed = open_group[:, :, None].expand(T, groups, per).reshape(T, E)
    masked = torch.where(allowed, scores, torch.full_like(scores, -1.0))
    ranked = masked.sort(dim=-1, descending=True)
    if top < keep * per:
        gap = torch.minimum(gap, (ranked.values[:, top - 1] - ranked.values[:, top]).min())
    chosen = ranked.indices[:, :top]
    weights = scores.gather(1, chosen)
    return chosen, weights / (weights.sum(-1, keepdim=True) + 1e-20), float(gap)


def mixture_ffn(h, w, p, mlp, gaps=None):
    r = mlp["router"]
    scores = torch.sigmoid(h @ w[p + "router"].T)
    chosen, weights, gap = route(scores, r["groups"]["count"], r["groups"]["keep"], r["top"])
    if gaps is not None:
        gaps.append(gap)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        for slot in range(r["top"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += weights[rows, slot][:, None] * gated_expert(h[rows], w, f"{p}e{e}.")
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.")
    return out


# --------------------------------------------------------------------------- the model
def run_order(cfg):
    """(layer, pass number or None) for every run: the looped span ``times`` times in a row."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, dtype=torch.float64, rows=None, streams=None, gaps=None):
    """Logits [T (or len(rows)), vocab] of a whole sequence. ``streams``: a list that receives the stream after
    every run of a layer; ``gaps``: a list that receives the smallest deciding gap of every routing."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    first = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = first.clone()
    for i, number in run_order(cfg):
        if number is not None:
            if number > 0:
                x = x + first
            x = x + w["loop.step"][number]
        layer, p = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = capped_attention(h, w, p + "mix.", layer["mixer"], eps)
        else:
            y, _ = matrix_memory(h, w, p + "mix.", layer["mixer"], eps)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if layer["mlp"]["kind"] == "dense":
                y = squared_relu_ffn(h, w, p + "mlp.")
            else:
                y = mixture_ffn(h, w, p + "mlp.", layer["mlp"], gaps)
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
