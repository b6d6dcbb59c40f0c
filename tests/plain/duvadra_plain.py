"""Plain, slow, whole-sequence implementation of the Duvadra decoder: the oracle of its tests.

Every mechanism is one function that walks a sequence in the precision it is given (float64 by default).
No cache, no batching, no kernels; nothing is shared with the ``return_b200`` package.  The configuration is
config.json as a plain dict, the weights a dict name -> tensor.

Notation.  a: a sublayer's input [T, width].  Linear maps are stored [out, in] and applied as ``a @ W.T``.
A recurrent state M of a head is a [key rows, value columns] matrix read out as ``M.T @ q``.  Positions start at 0.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        lo, hi = m["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=_DT[m["dtype"]]).reshape(m["shape"]).clone()
    return out


def read_model(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        c = json.load(f)
    w = {k: (v.to(dtype) if v.is_floating_point() else v)
         for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return c, w


# --------------------------------------------------------------------------- small pieces

def rms(x, eps):
    """x over the root of (its mean square plus eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def causal_conv(z, taps, bias=None):
    """z [T, C], taps [C, K] with the last column for the token itself; what lies before the sequence is zero."""
    T, C = z.shape
    K = taps.shape[1]
    padded = torch.cat([z.new_zeros(K - 1, C), z], 0)
    out = z.new_zeros(T, C)
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out if bias is None else out + bias


def visible(T, kind, size):
    """[T, T] bool: may row i look at column j.  kind "window": the last ``size`` positions, the row's own included;
    "chunk": the earlier positions of the row's own block of ``size``; None: every earlier position."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if kind == "window":
        ok = ok & (i - j < size)
    elif kind == "chunk":
        ok = ok & (i // size == j // size)
    return ok


def masked_softmax(scores, ok, sink=None):
    """Softmax over the allowed columns of every row; ``sink`` [heads] adds exp(sink) to a row's denominator and
    nothing else.  scores [heads, T, T]."""
    s = scores.masked_fill(~ok, float("-inf"))
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - top)
    return e / den


def rotate_interleaved(x, dims, base):
    """x [T, heads, dim]: elements (2i, 2i + 1), i < dims / 2, turn by the angle t * base^(-2i / dims)."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attend(q, k, v, scale, ok, sink=None, softcap=None, slopes=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap is not None:
        s = softcap * torch.tanh(s / softcap)
    if slopes is not None:
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(s.dtype)
        s = s - slopes[:, None, None] * dist
    p = masked_softmax(s, ok, sink)
    return torch.einsum("hij,jhd->ihd", p, vv)


# --------------------------------------------------------------------------- mixers with keys

def chunked_attention(w, p, m, a, shared=None):
    """Softly capped scores with a penalty per head that grows with the distance, inside blocks of ``mask.size``
    positions counted from the sequence's start; one gate per head.  ``shared``: (k, v) of the layer whose keys and
    values this layer reads instead of having its own.  Returns (output, (k, v))."""
    T = a.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T).view(T, H, d)
    if shared is None:
        k = (a @ w[p + "k"].T).view(T, G, d)
        v = (a @ w[p + "v"].T).view(T, G, dv)
    else:
        k, v = shared
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=a.dtype)
    mask = m.get("mask")
    ok = visible(T, "chunk" if mask else None, mask["size"] if mask else 0)
    o = attend(q, k, v, m["scale"], ok, softcap=m.get("softcap"), slopes=slopes)
    o = o * torch.sigmoid(a @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T, (k, v)


def sink_window_attention(w, p, m, a):
    """Biased projections, no positions, a sliding window, a sink per head in the denominator, a gate per element."""
    T = a.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (a @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (a @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    mask = m.get("mask")
    ok = visible(T, "window" if mask else None, mask["size"] if mask else 0)
    o = attend(q, k, v, m["scale"], ok, sink=w[p + "sink"]).reshape(T, H * dv)
    return (o * torch.sigmoid(a @ w[p + "g"].T)) @ w[p + "o"].T


def keys_as_values_attention(w, p, m, a, eps):
    """Values are the key projection as it comes out; queries and keys are normed over their whole projection and then
    turned by position (neighbouring pairs); sliding window; a gate per element."""
    T = a.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = a @ w[p + "q"].T
    k = a @ w[p + "k"].T
    v = k.view(T, G, d)
    q = (rms(q, eps) * w[p + "q.norm"]).view(T, H, d)
    k = (rms(k, eps) * w[p + "k.norm"]).view(T, G, d)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q = rotate_interleaved(q, rot["dims"], rot["base"])
        k = rotate_interleaved(k, rot["dims"], rot["base"])
    mask = m.get("mask")
    ok = visible(T, "window" if mask else None, mask["size"] if mask else 0)
    o = attend(q, k, v, m["scale"], ok).reshape(T, H * d)
    return (o * torch.sigmoid(a @ w[p + "g"].T)) @ w[p + "o"].T


# --------------------------------------------------------------------------- mixers with a state

def gated_delta(w, p, m, a, eps):
    """Delta rule with one decay per head and token.  M <- g M; e = beta (v - M^T k); M <- M + k e^T; o = M^T q."""
    T = a.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(causal_conv(a @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = F.silu(causal_conv(a @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = F.silu(causal_conv(a @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(a @ w[p + "b"].T)                                          # [T, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(a @ w[p + "a"].T + w[p + "dt_bias"]))
    out = a.new_zeros(T, H, dv)
    for h in range(H):
        kh = h // (H // G)
        M = a.new_zeros(d, dv)
        for t in range(T):
            M = g[t, h] * M
            e = beta[t, h] * (v[t, h] - M.T @ k[t, kh])
            M = M + torch.outer(k[t, kh], e)
            out[t, h] = M.T @ q[t, kh]
    out = rms(out, eps) * w[p + "norm"]
    out = out.reshape(T, H * dv) * F.silu(a @ w[p + "g"].T)
    return out @ w[p + "o"].T


def gated_linear_recurrence(w, p, m, a):
    """Two branches of ``width``: y = gelu(W_y a + b) and u = conv(W_x a + b).  Per channel, with gates from
    block-diagonal maps of u: r, i = sigmoid(.), log f = -8 r softplus(lam), s <- f s + sqrt(1 - f^2) i u from s = 0."""
    T = a.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(a @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(a @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    f = torch.exp(-8.0 * r * F.softplus(w[p + "lam"]))
    s = a.new_zeros(W)
    out = a.new_zeros(T, W)
    for t in range(T):
        s = f[t] * s + torch.sqrt(1.0 - f[t] ** 2) * i[t] * u[t]
        out[t] = s
    return (out * y) @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forwards

def capped_unit(w, p, mlp, a):
    lim = mlp["limit"]
    g = torch.clamp(a @ w[p + "gate"].T, max=lim)
    u = torch.clamp(a @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(z, r):
    """z [T, E] router outputs -> (chosen experts [T, top], their weights [T, top])."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        per = s.view(-1, n, E // n)
        rank = per.topk(min(2, E // n), dim=-1).values.sum(-1)                  # [T, n]
        best = rank.topk(keep, dim=-1).indices
        on = torch.zeros_like(rank, dtype=torch.bool).scatter_(1, best, True)
        allowed = on[:, :, None].expand(-1, -1, E // n).reshape(-1, E)
    picked = s.masked_fill(~allowed, float("-inf")).topk(top, dim=-1).indices
    wts = s.gather(1, picked)
    wts = wts / (wts.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return picked, wts


def experts(w, p, mlp, a, router_dtype=None):
    r = mlp["router"]
    z = a @ w[p + "router"].T
    picked, wts = route(z.to(router_dtype) if router_dtype is not None else z, r)
    out = torch.zeros_like(a)
    for t in range(a.shape[0]):
        for e, c in zip(picked[t].tolist(), wts[t]):
            q = f"{p}e{e}."
            out[t] += c.to(a.dtype) * ((F.silu(a[t] @ w[q + "gate"].T) * (a[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


# --------------------------------------------------------------------------- the model

def embed(c, w, ids):
    ids = torch.as_tensor(ids, dtype=torch.long)
    x = w["embed"][ids] * c.get("embedding", {}).get("scale", 1.0)
    bg = c.get("embedding", {}).get("bigram")
    if bg:
        n = bg["buckets"]
        rows = torch.full_like(ids, n)                                          # the row of a token with nothing before it
        rows[1:] = (ids[:-1] * bg["mul_prev"] + ids[1:] * bg["mul_cur"]) % n
        x = x + w["bigram"][rows]
    return x


def mixer(c, w, i, a, kept):
    layer = c["layers"][i]
    p, m, eps = f"l{i}.mix.", layer["mixer"], c["norm"]["eps"]
    kind = layer["type"]
    if kind == "attention":
        src = m.get("kv_from")
        y, kv = chunked_attention(w, p, m, a, kept[src] if src is not None else None)
        kept[i] = kv
        return y
    if kind == "parallel":
        left = sink_window_attention(w, p + "left.", m["left"], a)
        right = gated_delta(w, p + "right.", m["right"], a, eps)
    elif kind == "parallel_2":
        left = keys_as_values_attention(w, p + "left.", m["left"], a, eps)
        right = gated_linear_recurrence(w, p + "right.", m["right"], a)
    else:
        raise ValueError(kind)
    return m["left_scale"] * left + m["right_scale"] * right


def forward(c, w, ids, trace=None):
    """ids -> logits [T, vocab].  ``trace``: a list that receives the residual stream after every layer."""
    eps, mult = c["norm"]["eps"], c.get("residual_mult", 1.0)
    x = embed(c, w, ids)
    kept = {}
    for i, layer in enumerate(c["layers"]):
        x = x + mult * mixer(c, w, i, rms(x, eps) * w[f"l{i}.norm1"], kept)
        mlp = layer.get("mlp")
        if mlp:
            a = rms(x, eps) * w[f"l{i}.norm2"]
            y = capped_unit(w, f"l{i}.mlp.", mlp, a) if mlp["kind"] == "dense" else experts(w, f"l{i}.mlp.", mlp, a)
            x = x + mult * y
        if trace is not None:
            trace.append(x.clone())
    z = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = c.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
