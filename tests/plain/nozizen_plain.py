"""Plain, slow, whole-sequence implementation of the Nozizen decoder: the oracle of its tests.

Every mechanism is one function that walks a sequence in the precision it is given (float64 by default).
No cache, no batching, no kernels; nothing is shared with the ``return_b200`` package.  The configuration is
config.json as a plain dict, the weights a dict name -> tensor.

Notation.  a: a sublayer's input [T, width].  Linear maps are stored [out, in] and applied as ``a @ W.T``.
A recurrent state M of a head is a [key rows, value columns] matrix read out as ``M.T @ q``.
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


def relu_squared(z):
    return torch.relu(z) ** 2


# --------------------------------------------------------------------------- mixer: wkv

def wkv_mixer(w, p, m, a, eps):
    """Time mixing with a decay per head and key row that depends on the token, and a bonus for the token itself.

    b_t = a_(t-1) (zero before the first token).  Each of r, k, v, g, d reads a_t + (b_t - a_t) mu.  Per head:
    o_t = (M + diag(u) k_t v_t^T)^T r_t, then M <- diag(e_t) M + k_t v_t^T, with e_t = exp(-exp(W2 tanh(W1 x_d) + w0)).
    o over its root mean square per head, times a weight over all heads, times silu(W_g x_g), then W_o."""
    T = a.shape[0]
    H, D = m["heads"], m["dim"]
    before = torch.cat([torch.zeros_like(a[:1]), a[:-1]], 0)

    def shifted(name):
        return a + (before - a) * w[p + "mu." + name]

    r = (shifted("r") @ w[p + "r"].T).view(T, H, D)
    k = (shifted("k") @ w[p + "k"].T).view(T, H, D)
    v = (shifted("v") @ w[p + "v"].T).view(T, H, D)
    gate = F.silu(shifted("g") @ w[p + "g"].T)
    e = torch.exp(-torch.exp(torch.tanh(shifted("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, D)
    u = w[p + "u"]
    M = a.new_zeros(H, D, D)
    o = a.new_zeros(T, H, D)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", M + u[:, :, None] * kv, r[t])
        M = e[t][:, :, None] * M + kv
    o = rms(o, eps).reshape(T, H * D) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- mixer: mamba2

def mamba2_mixer(w, p, m, a, eps):
    """State-space mixer.  W_in a = [z | x | B | C | dt]; x, B, C pass a causal convolution per channel (the last tap
    is the token's own; zeros before the sequence) plus a bias, then silu.  dt <- softplus(dt + dt_bias).  Per head h
    with group g(h): M <- exp(-exp(A_log_h) dt) M + dt B_t x_t^T, y_t = M^T C_t + D_h x_t.  y times silu(z), normed in
    ``norm_groups`` equal parts, times a weight, then W_o."""
    T = a.shape[0]
    H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = a @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    taps, bias = w[p + "conv"], w[p + "conv.b"]
    padded = torch.cat([xbc.new_zeros(K - 1, xbc.shape[1]), xbc], 0)
    conv = sum(padded[j:j + T] * taps[:, j] for j in range(K)) + bias
    conv = F.silu(conv)
    x = conv[:, :inner].view(T, H, P)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = F.softplus(dt + w[p + "dt_bias"])
    rate = torch.exp(w[p + "A_log"])
    skip = w[p + "D"]
    M = a.new_zeros(H, N, P)
    y = a.new_zeros(T, H, P)
    per = H // G
    for t in range(T):
        for h in range(H):
            g = h // per
            M[h] = torch.exp(-rate[h] * dt[t, h]) * M[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = M[h].T @ C[t, g] + skip[h] * x[t, h]
    y = y.reshape(T, inner) * F.silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# --------------------------------------------------------------------------- mixer: attention

def rotary_tables(rot, positions, dtype):
    """cos and sin [T, dims/2] of the angles p f_i, f_i = base^(-2 i / dims); with ``scaling`` the frequencies are
    stretched along a ramp over i and both tables are multiplied by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    gain = 1.0
    sc = rot.get("scaling")
    if sc:
        def at(turns):
            return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(at(sc["fast"])), 0)
        hi = min(math.ceil(at(sc["slow"])), dims - 1)
        span = max(hi - lo, 0.001)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / span, 0.0), 1.0)
            f[i] = f[i] / sc["factor"] * ramp + f[i] * (1.0 - ramp)
        gain = 0.1 * math.log(sc["factor"]) + 1.0
    ang = torch.outer(torch.arange(positions, dtype=torch.float64), torch.tensor(f, dtype=torch.float64))
    return (ang.cos() * gain).to(dtype), (ang.sin() * gain).to(dtype)


def rotate(x, cos, sin, dims):
    """x [T, heads, dim]: element i of the first ``dims`` is paired with element i + dims/2."""
    half = dims // 2
    lo, hi, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s, rest], -1)


def attention_mixer(w, p, m, a, eps):
    """Grouped-query softmax attention with rotary positions on part of a head and a sliding window: token i sees
    token j when 0 <= i - j < size."""
    T = a.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (a @ w[p + "q"].T).view(T, H, D)
    k = (a @ w[p + "k"].T).view(T, G, D)
    v = (a @ w[p + "v"].T).view(T, G, V)
    rot = m.get("rot")
    if rot and rot["dims"]:
        cos, sin = rotary_tables(rot, T, a.dtype)
        q, k = rotate(q, cos, sin, rot["dims"]), rotate(k, cos, sin, rot["dims"])
    i = torch.arange(T)
    seen = i[None, :] <= i[:, None]
    mask = m.get("mask")
    if mask:
        seen = seen & (i[:, None] - i[None, :] < mask["size"])
    out = a.new_zeros(T, H, V)
    per = H // G
    for h in range(H):
        g = h // per
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


MIXERS = {"wkv": wkv_mixer, "mamba2": mamba2_mixer, "attention": attention_mixer}


# --------------------------------------------------------------------------- feed-forwards

def dense_ff(w, p, a):
    return relu_squared(a @ w[p + "up"].T) @ w[p + "down"].T


def router(w, p, mlp, a):
    """(chosen experts [T, top], their weights [T, top]): the largest logits W a + b, softmax over the chosen only."""
    logits = a @ w[p + "router"].T + w[p + "router.b"]
    top = logits.topk(mlp["router"]["top"], dim=-1)
    return top.indices, torch.softmax(top.values, -1)


def expert(w, p, a):
    return (F.silu(a @ w[p + "gate"].T) * (a @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(w, p, mlp, a):
    chosen, weight = router(w, p, mlp, a)
    y = torch.zeros_like(a)
    for t in range(a.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            y[t] += g * expert(w, f"{p}e{e}.", a[t:t + 1])[0]
    return y


def feed_forward(w, p, mlp, a):
    return dense_ff(w, p, a) if mlp["kind"] == "dense" else moe_ff(w, p, mlp, a)


# --------------------------------------------------------------------------- hyper-connections, layers, model

def hyper_sublayer(w, p, xs, sublayer, norm_w, eps):
    """xs [streams, T, width].  The sublayer reads sum_s in[s] xs[s]; then, all at once from the old streams,
    xs[t] <- sum_s mix[s, t] xs[s] + out[t] y."""
    read = torch.einsum("s,stw->tw", w[p + "in"], xs)
    y = sublayer(rms(read, eps) * norm_w)
    return torch.einsum("sr,stw->rtw", w[p + "mix"], xs) + w[p + "out"][:, None, None] * y[None]


def layer_order(c):
    """Indices of the layers in the order they run: layers start .. stop - 1 run ``times`` times in a row."""
    n = len(c["layers"])
    loop = c.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(c, w, ids, keep_layers=False):
    """(logits [T, vocab], the sum of the streams after every layer run or None)."""
    eps = c["norm"]["eps"]
    dtype = w["embed"].dtype
    x = w["embed"][torch.tensor(ids)] * (c.get("embedding") or {}).get("scale", 1.0)
    hyper = c.get("streams") is not None          # without the key: one stream and plain residual sums
    S = int(c["streams"]) if hyper else 1
    xs = x[None].repeat(S, 1, 1)
    after = []
    for i in layer_order(c):
        layer = c["layers"][i]
        p = f"l{i}."
        mixer = MIXERS[layer["type"]]

        def run_mixer(a):
            return mixer(w, p + "mix.", layer["mixer"], a, eps)

        def run_ff(a):
            return feed_forward(w, p + "mlp.", layer["mlp"], a)

        if hyper:
            xs = hyper_sublayer(w, p + "hc1.", xs, run_mixer, w[p + "norm1"], eps)
            if layer.get("mlp"):
                xs = hyper_sublayer(w, p + "hc2.", xs, run_ff, w[p + "norm2"], eps)
        else:
            xs = xs + run_mixer(rms(xs[0], eps) * w[p + "norm1"])[None]
            if layer.get("mlp"):
                xs = xs + run_ff(rms(xs[0], eps) * w[p + "norm2"])[None]
        if keep_layers:
            after.append(xs.sum(0))
    x = xs.sum(0)
    logits = (rms(x, eps) * w["final.norm"]) @ w["embed"].T
    return logits.to(dtype), (torch.stack(after) if keep_layers else None)
