"""Plain implementation of the Ramupel decoder for the tests: whole sequences, no cache, float64 by default,
one function per mechanism, written from the design's equations. It shares no code with the library's parts.

Notation: x is the stream [T, d]; h its normed form; positions count from 0; matrices are stored [out, in]
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
def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * gain."""
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * gain


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def softplus(z):
    return torch.clamp(z, min=0) + torch.log1p(torch.exp(-z.abs()))


def xielu(z, p, q):
    """softplus(p) z^2 + z/2 above zero; (1/2 + softplus(q)) (e^z - 1 - z) + z/2 at and below."""
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def rotate_half_pairs(v, positions, base, dims):
    """Rotate the first ``dims`` features of the last axis: feature i pairs with i + dims/2, angle p * base^(-2i/dims).
    ``v``: [T, ..., n] with n >= dims; the features beyond ``dims`` pass unchanged."""
    if dims == 0:
        return v
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


# --------------------------------------------------------------------------- mixers
def latent_attention_core(q, down, gate_logits, w, prefix, m, eps, positions=None):
    """From the projections: ``q`` [T, H, dim + rot_dim], ``down`` [T, kv_rank + rot_dim], ``gate_logits`` [T, H].
    Returns the heads' gated outputs [T, H * vdim] (before the output projection) and the softmax weights."""
    T = q.shape[0]
    H, dn, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    latent = rms_norm(down[:, :rank], w[prefix + "dkv.norm"], eps)
    shared = rotate_half_pairs(down[:, rank:], pos, base, dims)                       # [T, dr]
    q_plain, q_rot = q[..., :dn], rotate_half_pairs(q[..., dn:], pos, base, dims)
    k_plain = (latent @ w[prefix + "uk"].T).reshape(T, H, dn)
    values = (latent @ w[prefix + "uv"].T).reshape(T, H, dv)
    scores = torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, shared)
    scores = scores * m["scale"]
    visible = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hts,shd->thd", weights, values)
    out = out * torch.sigmoid(gate_logits)[:, :, None]
    return out.reshape(T, H * dv), weights


def latent_attention(h, w, prefix, m, eps, positions=None):
    """Keys and values of every head come from one normed latent per position plus one shared rotated key part."""
    T = h.shape[0]
    q = (h @ w[prefix + "q"].T).reshape(T, m["heads"], m["dim"] + m["rot_dim"])
    heads, _ = latent_attention_core(q, h @ w[prefix + "dkv"].T, h @ w[prefix + "g"].T, w, prefix, m, eps, positions)
    return heads @ w[prefix + "o"].T


def gla_decay(h, w, prefix, m):
    z = (h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "a2.b"]
    return torch.sigmoid(z) ** (1.0 / m["tau"])


def gla_core(q, k, v, a, gate, gain, eps, state=None):
    """Token by token: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t with q already scaled; ``q, k, a`` [T, H, dk],
    ``v`` [T, H, dv], ``gate`` [T, H * dv]. Returns the normed, gated heads [T, H * dv] and the final state."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, gain, eps).reshape(T, H * dv)
    return o * gate * torch.sigmoid(gate), S


def gated_linear_attention(h, w, prefix, m, eps, state=None):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[prefix + "k"].T).reshape(T, H, dk)
    v = (h @ w[prefix + "v"].T).reshape(T, H, dv)
    a = gla_decay(h, w, prefix, m).reshape(T, H, dk)
    heads, S = gla_core(q, k, v, a, h @ w[prefix + "g"].T, w[prefix + "norm"], eps, state)
    return heads @ w[prefix + "o"].T, S


def dense_ffn(h, w, prefix):
    act = w[prefix + "act"]
    return xielu(h @ w[prefix + "up"].T, act[0], act[1]) @ w[prefix + "down"].T


# --------------------------------------------------------------------------- the model
def forward(cfg, weights, tokens, dtype=torch.float64, rows=None, streams_out=None):
    """Logits [T, vocab] (or the given rows) of one whole sequence."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    results = [x]                                   # the embedding's output, then every layer's result
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            mixed = latent_attention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "gla":
            mixed, _ = gated_linear_attention(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        update = mixed * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
        if layer["mlp"] is not None:
            update = update + dense_ffn(h, w, p + "mlp.") * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
        results.append(x + update)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        if streams_out is not None:
            streams_out.append(x)
    x = layer_norm(x, w["final.norm"], eps)
    if rows is not None:
        x = x[torch.tensor(rows)]
    return x @ w["embed"].T


def greedy(cfg, weights, prompt, count):
    """``count`` tokens by argmax, each from a whole-sequence forward; also the margin between the best and the
    second-best logit at each step (a test may skip steps that rounding could flip)."""
    tokens, chosen, margins = list(prompt), [], []
    for _ in range(count):
        row = forward(cfg, weights, tokens, rows=[len(tokens) - 1])[0]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]) / float(row.abs().max()))
        chosen.append(int(row.argmax()))
        tokens.append(chosen[-1])
    return chosen, margins
