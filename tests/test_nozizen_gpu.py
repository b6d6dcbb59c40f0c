"""The Nozizen decoder through the engine against the plain implementation (tests/plain/nozizen_plain.py).

Every test makes a small configuration of its own with random weights (written as a bfloat16 checkpoint, as a model
folder holds them), replays a trace through the engine's step function and compares every logits row with the plain
implementation's, which walks the whole sequence in float64, token by token where there is a recurrence.
float32 path: every row within 1e-4 of its size.  bfloat16 path: rows weighed together (see ``assert_close``).
Where random weights would hide a fault (a key just outside a window, a state that was lost far back) the scores are
made sharp and the decays slow, and the test first shows that the plain model itself moves by far more than the
tolerance when that key or state is lost.
"""
import json
import os
import types

import pytest
import torch

import helpers
from helpers import collect, mixed, pool_tokens, portions, random_ids, tail_decoded, whole
from plain import nozizen_plain as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 1.0 / 12}


# ------------------------------------------------------------------------------- configurations

def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def wkv_layer(heads=3, dim=8, rank=6, mlp="default"):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": dense() if mlp == "default" else mlp}


def ssm_layer(heads=4, vdim=6, state=10, groups=2, conv=4, norm_groups=3, mlp="default"):
    m = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "mamba2", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def attn_layer(heads=4, kv_heads=2, dim=12, vdim=20, window=19, rot=8, base=5000.0, scaling=True, scale=None, mlp="default"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
        if scaling:
            m["rot"]["scaling"] = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    return {"type": "attention", "mixer": m, "mlp": dense(40) if mlp == "default" else mlp}


def config(layers, vocab=97, width=40, eps=1e-5, streams=3, loop=None, scale=20.0):
    c = {"architecture": "Nozizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        c["streams"] = streams
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if scale:
        c["embedding"] = {"scale": scale}
    return c


def full_config():
    """All three mixers and both feed-forwards, a layer without a feed-forward, two windows (one shorter than a page, one
    that spans several), and a run of three layers that repeats: every pass has states and a cache of its own."""
    return config([wkv_layer(), ssm_layer(), attn_layer(window=5, mlp=None), attn_layer(heads=2, kv_heads=2, dim=16, vdim=8, rot=16, mlp=moe(5, 3, 16)),
                   wkv_layer(heads=2, dim=16, rank=4, mlp=moe(4, 1, 32)), ssm_layer(heads=2, vdim=16, state=8, groups=1, conv=2, norm_groups=1, mlp=dense(48))],
                  loop=(1, 4, 2))


def other_sizes_config():
    """The values one (one head, one group, one part, one tap, one expert chosen, as many chosen as there are, a window
    of one, one stream), sizes that fill no whole warp or vector, keys wider than 64 and than 128, state and value
    sizes that differ both ways, a rotation over the whole head and over two numbers of it, no window, a run that
    repeats three times from the first layer on."""
    return config([ssm_layer(heads=1, vdim=33, state=7, groups=1, conv=1, norm_groups=1, mlp=moe(3, 3, 9)),
                   wkv_layer(heads=1, dim=72, rank=1, mlp=None),
                   attn_layer(heads=1, kv_heads=1, dim=40, vdim=7, window=1, rot=2, scaling=False, mlp=moe(35, 4, 8)),
                   ssm_layer(heads=6, vdim=8, state=136, groups=3, conv=7, norm_groups=6, mlp=moe(2, 1, 40)),
                   attn_layer(heads=6, kv_heads=3, dim=8, vdim=24, window=None, rot=8, base=300.0, mlp=dense(9)),
                   wkv_layer(heads=5, dim=24, rank=11, mlp=dense(7))],
                  vocab=61, width=24, eps=1e-6, streams=1, loop=(0, 2, 3), scale=16.5)


_MODELS = {}


def model(tmp_path_factory, name, raw, seed=3, patch=None):
    """(model folder, (config, float64 weights), memo of plain logits), cached: the plain walk is slow.  config.json is
    written as a model folder holds it: a time mix's decay rank is not in it, only in its tensors' shapes.  ``patch``
    changes tensors (name -> tensor) before they are written."""
    if name not in _MODELS:
        from return_b200.config.nozizen_config import NozizenConfig
        from return_b200.weights import loader
        from return_b200.weights.safetensors_io import write_safetensors
        d = str(tmp_path_factory.mktemp(name))
        loader.write_random_model(d, NozizenConfig(raw), seed, torch.bfloat16)
        path = os.path.join(d, "config.json")
        c = json.load(open(path))
        for layer in c["layers"]:
            layer["mixer"].pop("decay_rank", None)
        json.dump(c, open(path, "w"))
        if patch is not None:
            tensors = plain.read_safetensors(os.path.join(d, "model.safetensors"))
            patch(tensors)
            write_safetensors(os.path.join(d, "model.safetensors"), [(n, t.bfloat16().contiguous()) for n, t in tensors.items()])
        _MODELS[name] = (d, plain.read_model(d), {})
    return _MODELS[name]


def plain_rows(entry, ids):
    d, (c, w), memo = entry
    key = tuple(ids)
    if key not in memo:
        memo[key] = plain.forward(c, w, list(ids))[0].float()
    return memo[key]


def requests_for(entry, lens, seed=10):
    return {f"r{i}": random_ids(entry[1][0]["vocab"], n, seed + i) for i, n in enumerate(lens)}


def run_trace(model_dir, dtype, steps, page_size=16, max_reside=4, graph=False):
    from return_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(model_dir, dtype, pool_tokens(steps), page_size=page_size, max_reside=max_reside, poison=True,
                       use_cuda_graph=graph)
    outs = []
    for st in steps:
        lg = rp.run_step(st)
        outs.append(None if lg is None else lg.float().cpu())
        rp.runner.manager.check()
    assert rp.runner.manager.num_requests == 0 and rp.runner.manager.pages_used() == [0] * len(rp.runner.manager.groups)
    return collect(steps, outs)


def row_errors(got, want):
    """The error of every row as a part of the row's size, both with their means taken off (as the softmax sees them)."""
    assert got.shape == want.shape and torch.isfinite(got).all()
    got, want = got - got.mean(1, keepdim=True), want - want.mean(1, keepdim=True)
    return (got - want).norm(dim=1) / want.norm(dim=1)


def worst(got, want):
    return float(row_errors(got, want).max())


def assert_close(got, want, dtype, what="", mean=0.03):
    """float32: every row within 1e-4 of its size.  bfloat16: rounding moves single rows far more than the rest (a
    router whose best candidates are nearly tied chooses another expert than the float64 walk does; a head's read-out
    near zero is divided by its own size), so the rows are weighed together: their mean within 3 %, at most one row in
    ten (or two) beyond a twelfth, none beyond six tenths.  A lost key, a wrong window, a stale page or a lost state
    moves every row behind it, and the tests that aim at single rows compare those rows with what the fault would give."""
    e = row_errors(got, want)
    if dtype == "float32":
        assert float(e.max()) < TOL[dtype], (what, dtype, float(e.max()), int(e.argmax()))
        return
    over = int((e > TOL[dtype]).sum())
    assert over <= max(2, e.numel() // 10) and float(e.max()) < 0.6 and float(e.mean()) < mean, \
        (what, dtype, over, float(e.max()), float(e.mean()), int(e.argmax()))


def compare(entry, dtype, steps, requests, **kw):
    got = run_trace(entry[0], dtype, steps, **kw)
    for rid, ids in requests.items():
        assert_close(got[rid], plain_rows(entry, ids), dtype, rid)


# ------------------------------------------------------------------------------- kernels of single mechanisms

def _segments(lens, slots):
    """The step tables the state kernels read, for segments of the given lengths in the given state slots."""
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    tok_seg = [i for i, n in enumerate(lens) for _ in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return types.SimpleNamespace(cu_q=i32(cu), tok_seg=i32(tok_seg), seg_slot=i32(slots), num_segments=len(lens), num_tokens=cu[-1])


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,H", [(1, 40), (3, 72), (4, 296), (8, 24), (2, 38), (3, 1026), (4, 4096), (8, 2048)])
def test_streams_read_and_write(S, H, dtype):
    """The read (weighted sum of the streams, normed), the write (all streams at once from the old ones), the write with
    the next read in the same kernel, and the plain sum that goes to the final norm, against the plain sublayer."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(S * 100 + H)
    T, eps = 7, 1e-5
    xs = torch.randn((S, T, H), generator=g, dtype=torch.float64) * 2.0
    w = {"c.in": torch.randn(S, generator=g, dtype=torch.float64), "c.out": torch.randn(S, generator=g, dtype=torch.float64),
         "c.mix": torch.randn((S, S), generator=g, dtype=torch.float64)}
    nw, nw2 = 1.0 + 0.1 * torch.randn(H, generator=g, dtype=torch.float64), 1.0 + 0.1 * torch.randn(H, generator=g, dtype=torch.float64)
    y = torch.randn((T, H), generator=g, dtype=torch.float64).to(dtype).double()
    seen = {}

    def sublayer(a):
        seen["read"] = a
        return y
    want = plain.hyper_sublayer(w, "c.", xs, sublayer, nw, eps)
    f32 = lambda t: t.float().cuda().contiguous()
    streams = f32(xs.permute(1, 0, 2))
    out = torch.empty((T, H), dtype=dtype, device="cuda")
    ops.hyper_read_norm(streams, f32(w["c.in"]), f32(nw), eps, out)
    assert torch.allclose(out.cpu().double(), seen["read"], **_tol(dtype))
    read2 = torch.randn(S, generator=g, dtype=torch.float64)
    nxt = torch.empty((T, H), dtype=dtype, device="cuda")
    ops.hyper_write(streams, y.to(dtype).cuda(), f32(w["c.mix"]), f32(w["c.out"]), nxt=(f32(read2), f32(nw2), eps, 0.0), out=nxt)
    assert torch.allclose(streams.cpu().double().permute(1, 0, 2), want, rtol=1e-5, atol=1e-5)
    assert torch.allclose(nxt.cpu().double(), plain.rms(torch.einsum("s,stw->tw", read2, want), eps) * nw2, **_tol(dtype))
    alone = f32(xs.permute(1, 0, 2))
    ops.hyper_write(alone, y.to(dtype).cuda(), f32(w["c.mix"]), f32(w["c.out"]))
    assert torch.equal(alone, streams)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    picked = torch.empty((3, H), dtype=dtype, device="cuda")
    ops.hyper_read_norm(streams, None, f32(nw), eps, picked, rows=rows)
    assert torch.allclose(picked.cpu().double(), (plain.rms(want.sum(0), eps) * nw)[[5, 0, 5]], **_tol(dtype))


def test_embedding_scaled_into_every_stream():
    from return_b200.ext import ops
    table = torch.randn((11, 24), generator=torch.Generator().manual_seed(0)).bfloat16()
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32)
    out = torch.empty((4, 3, 24), dtype=torch.float32, device="cuda")
    ops.embedding(table.cuda(), ids.cuda(), out, 2.5)
    assert torch.equal(out.cpu(), (table.float()[ids.long()] * 2.5)[:, None, :].expand(4, 3, 24))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations(dtype):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(1)
    x = (torch.randn((9, 37), generator=g) * 3.0).to(dtype)
    for kind, f in (("relu2", plain.relu_squared), ("tanh", torch.tanh), ("silu", torch.nn.functional.silu)):
        out = torch.empty_like(x, device="cuda")
        ops.activation(x.cuda(), out, kind)
        assert torch.allclose(out.cpu().double(), f(x.double()), **_tol(dtype)), kind
    bias = torch.randn(37, generator=g)
    out = torch.empty((9, 37), dtype=torch.float32, device="cuda")
    ops.activation(x.float().cuda(), out, "neg_exp_exp", bias=bias.cuda())
    assert torch.allclose(out.cpu().double(), torch.exp(-torch.exp(x.float().double() + bias.double())), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows", [1, 5, 8, 13, 40])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_product_with_an_activation_behind_it(rows, dtype):
    """``ops.linear(..., act=)``: few bfloat16 rows take the activation in the product's epilogue, more rows and float32
    in a launch of their own; both against the activation of the float64 product."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(rows)
    K, N = 72, 52
    x = (torch.randn((rows, K), generator=g)).to(dtype)
    w = (torch.randn((N, K), generator=g) * K ** -0.5).to(dtype)
    bias = torch.randn(N, generator=g)
    z = x.double() @ w.double().t()
    cases = (("relu2", plain.relu_squared(z), None), ("tanh", torch.tanh(z), None), ("silu", torch.nn.functional.silu(z), None),
             ("neg_exp_exp", torch.exp(-torch.exp(z + bias.double())), bias))
    for kind, want, b in cases:
        for out_dtype in (dtype, torch.float32):
            out = torch.empty((rows, N), dtype=out_dtype, device="cuda")
            ops.linear(x.cuda(), w.cuda(), out, act=kind, bias=None if b is None else b.cuda())
            tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else \
                (dict(rtol=2e-2, atol=2e-2) if out_dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5))
            assert torch.allclose(out.cpu().double(), want, **tol), (kind, rows, out_dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_blends_with_the_token_before(dtype):
    """Three segments: one from a request that kept a last input, one new (its slot holds zeros), one of a single token;
    afterwards every slot holds its segment's last input."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(2)
    W, off = 40, 16
    lens, slots = [5, 3, 1], [2, 0, 3]
    b = _segments(lens, slots)
    x = torch.randn((9, W), generator=g).to(dtype)
    mu = torch.rand((5, W), generator=g).to(dtype)
    state = torch.zeros((5, off + W), dtype=torch.float32)
    state[2, off:] = torch.randn(W, generator=g).to(dtype).float()
    state[3, off:] = torch.randn(W, generator=g).to(dtype).float()
    before = torch.cat([state[2:3, off:], x[:4].float(), state[0:1, off:], x[5:7].float(), state[3:4, off:]]).double()
    want = x.double()[None] + (before - x.double())[None] * mu.double()[:, None, :]
    dev_state = state.cuda()
    out = torch.empty((5, 9, W), dtype=dtype, device="cuda")
    ops.token_shift_mix(x.cuda(), mu.cuda(), dev_state, off, b, out)
    assert torch.allclose(out.cpu().double(), want, **_tol(dtype))
    ops.conv_state_update(x.cuda(), 2, dev_state, off, b, W)
    kept = dev_state.cpu()
    assert torch.equal(kept[2, off:], x[4].float()) and torch.equal(kept[0, off:], x[7].float()) and torch.equal(kept[3, off:], x[8].float())
    assert not kept[:, :off].any() and not kept[1].any() and not kept[4].any()


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_convolution_steps_and_decays_of_a_state_space_scan(taps):
    """The causal convolution across a segment's start (from the inputs the request kept, zeros for a new one), its bias
    and silu; softplus without a clamp, far into its linear part; the decay."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(3)
    H, C, lead = 3, 22, 5
    lens, slots = [6, 1, 2], [1, 3, 0]
    b = _segments(lens, slots)
    T = 9
    x = (torch.randn((T, lead + C + H), generator=g) * 1.5).bfloat16()
    x[2, lead + C] = 40.0                                           # a step far beyond where softplus is its argument
    w, bias = torch.randn((C, taps), generator=g).bfloat16(), torch.randn(C, generator=g).bfloat16()
    dt_bias, A_log = torch.randn(H, generator=g).bfloat16(), torch.randn(H, generator=g).bfloat16()
    off = 8
    state = torch.zeros((4, off + C * (taps - 1)), dtype=torch.float32)
    hist = torch.randn((C, taps - 1), generator=g).bfloat16().float()
    state[3, off:] = hist.reshape(-1)                               # [channel][taps - 1], oldest first
    xc = x[:, lead:lead + C].double()
    conv = torch.zeros((T, C), dtype=torch.float64)
    starts = {0: torch.zeros((taps - 1, C), dtype=torch.float64), 6: hist.double().T, 7: torch.zeros((taps - 1, C), dtype=torch.float64)}
    t = 0
    for n in lens:
        padded = torch.cat([starts[t], xc[t:t + n]], 0)
        conv[t:t + n] = sum(padded[j:j + n] * w.double()[:, j] for j in range(taps)) + bias.double()
        t += n
    want_dt = torch.nn.functional.softplus(x[:, lead + C:].double() + dt_bias.double(), threshold=1e9)
    dev_state = state.cuda()
    got, dt, decay = (torch.empty((T, n), dtype=torch.float32, device="cuda") for n in (C, H, H))
    ops.ssm_prep(x.cuda(), lead, C, w.cuda(), bias.cuda(), dev_state, off, b, got, lead + C, H, dt_bias.cuda(), A_log.cuda(), dt, decay)
    assert torch.allclose(got.cpu().double(), torch.nn.functional.silu(conv), rtol=1e-5, atol=1e-5)
    assert torch.allclose(dt.cpu().double(), want_dt, rtol=1e-5, atol=1e-6) and float(dt[2, 0]) > 38.0
    assert torch.allclose(decay.cpu().double(), torch.exp(-torch.exp(A_log.double()) * want_dt), rtol=1e-5, atol=1e-7)
    if taps > 1:
        ops.conv_state_update(x.cuda()[:, lead:], taps, dev_state, off, b, C)
        kept = dev_state.cpu()[:, off:].view(4, C, taps - 1)
        assert torch.equal(kept[1], xc[6 - (taps - 1):6].float().T.contiguous())
        assert torch.equal(kept[0][:, -1], xc[8].float()) and torch.equal(kept[3][:, -1], xc[6].float())
        if taps == 4:                                               # a segment shorter than the history keeps the older inputs' tail
            assert torch.equal(kept[3][:, :2], hist[:, 1:]) and torch.equal(kept[0][:, 0], torch.zeros(C))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("parts,n", [(1, 40), (3, 24), (6, 48), (2, 66), (2, 512), (3, 900), (1, 1500), (2, 2500)])
def test_gate_then_norm_over_equal_parts(parts, n, dtype):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(parts)
    y, z = torch.randn((5, n), generator=g) * 3.0, torch.randn((5, n + 3), generator=g).to(dtype)
    w = (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    out = torch.empty((5, n), dtype=dtype, device="cuda")
    ops.gated_part_norm(y.cuda(), z.cuda()[:, 3:], w.cuda(), parts, 1e-5, out)
    v = y.double() * torch.nn.functional.silu(z.double()[:, 3:])
    want = plain.rms(v.view(5, parts, n // parts), 1e-5).reshape(5, n) * w.double()
    assert torch.allclose(out.cpu().double(), want, **_tol(dtype))


def _scan_state(slots, heads, dim, vdim):
    return torch.zeros((slots, heads * ((dim + 7) // 8 * 8) * vdim), dtype=torch.float32, device="cuda")


@pytest.mark.parametrize("H,D", [(2, 8), (3, 24), (1, 72), (2, 136)])
def test_scan_with_row_decays_and_a_bonus(H, D):
    """o = (M + diag(u) k v^T)^T r, then M <- diag(e) M + k v^T, over a prompt and then token by token from the state
    it left, beside a second request; against the plain loop."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(D)
    T = 21
    r, k, v = (torch.randn((2, T, H, D), generator=g, dtype=torch.float64) * 0.5 for _ in range(3))
    e = torch.rand((2, T, H, D), generator=g, dtype=torch.float64) * 0.5 + 0.5
    u = torch.randn((H, D), generator=g, dtype=torch.float64)
    want = torch.zeros((2, T, H, D), dtype=torch.float64)
    for s in range(2):
        M = torch.zeros((H, D, D), dtype=torch.float64)
        for t in range(T):
            kv = k[s, t][:, :, None] * v[s, t][:, None, :]
            want[s, t] = torch.einsum("hij,hi->hj", M + u[:, :, None] * kv, r[s, t])
            M = e[s, t][:, :, None] * M + kv
    state = _scan_state(3, H, D, D)
    got = torch.zeros((2, T, H * D), dtype=torch.float32)
    cuts = [(0, 13, 0, 5), (13, 14, 5, 6)] + [(t, t + 1, t - 8, t - 7) for t in range(14, 21)] + [(21, 21, 13, 21)]
    for a0, a1, b0, b1 in cuts:                                     # request a in slot 2, request b in slot 0, uneven portions
        lens = [n for n in (a1 - a0, b1 - b0) if n]
        slots = [sl for sl, n in ((2, a1 - a0), (0, b1 - b0)) if n]
        b = _segments(lens, slots)
        cat = lambda x: torch.cat([x[0, a0:a1], x[1, b0:b1]]).reshape(sum(lens), H * D).float().cuda().contiguous()
        out = torch.empty((sum(lens), H * D), dtype=torch.float32, device="cuda")
        ops.linear_scan(ops.SCAN_BONUS, cat(r), cat(k), cat(v), cat(e), None, state, (0, 0, 0), b, out, H, H, D, D,
                        extra=u.float().cuda().contiguous())
        got[0, a0:a1], got[1, b0:b1] = out[:a1 - a0].cpu(), out[a1 - a0:].cpu()
    assert torch.allclose(got.double(), want.reshape(2, T, H * D), rtol=1e-4, atol=1e-4)
    assert not state[1].any()                                       # the slot of no request stayed as it was


@pytest.mark.parametrize("H,G,N,P", [(4, 2, 10, 6), (1, 1, 7, 33), (6, 3, 136, 8), (2, 2, 40, 40)])
def test_scan_of_a_state_space(H, G, N, P):
    """M <- a M + dt B x^T, y = M^T C + D x, heads sharing the maps of their group; a prompt, then token by token."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(N)
    T = 19
    x = torch.randn((T, H, P), generator=g, dtype=torch.float64)
    B, C = (torch.randn((T, G, N), generator=g, dtype=torch.float64) * 0.5 for _ in range(2))
    a = torch.rand((T, H), generator=g, dtype=torch.float64) * 0.5 + 0.5
    dt = torch.rand((T, H), generator=g, dtype=torch.float64) + 0.1
    skip = torch.randn(H, generator=g, dtype=torch.float64)
    want = torch.zeros((T, H, P), dtype=torch.float64)
    M = torch.zeros((H, N, P), dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            grp = h // (H // G)
            M[h] = a[t, h] * M[h] + dt[t, h] * torch.outer(B[t, grp], x[t, h])
            want[t, h] = M[h].T @ C[t, grp] + skip[h] * x[t, h]
    state = _scan_state(2, H, N, P)
    got = torch.zeros((T, H * P), dtype=torch.float32)
    f32 = lambda t_, lo, hi: t_[lo:hi].reshape(hi - lo, -1).float().cuda().contiguous()
    for lo, hi in [(0, 11)] + [(t, t + 1) for t in range(11, T)]:
        b = _segments([hi - lo], [1])
        out = torch.empty((hi - lo, H * P), dtype=torch.float32, device="cuda")
        ops.linear_scan(ops.SCAN_SSM, f32(C, lo, hi), f32(B, lo, hi), f32(x, lo, hi), f32(a, lo, hi), f32(dt, lo, hi), state,
                        (0, 0, 0), b, out, H, G, N, P, extra=skip.float().cuda().contiguous())
        got[lo:hi] = out.cpu()
    assert torch.allclose(got.double(), want.reshape(T, H * P), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("E,top", [(12, 4), (5, 2), (7, 1), (3, 3), (35, 4), (64, 8)])
def test_router_with_a_bias_weighs_the_chosen_logits_only(E, top):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    z, bias = torch.randn((50, E), generator=g) * 3.0, torch.randn(E, generator=g) * 2.0
    z[0] -= 60.0                                                    # far below zero: only the differences count
    w = {"r.router": torch.eye(E, dtype=torch.float64), "r.router.b": bias.double()}
    idx, wt = plain.router(w, "r.", {"router": {"experts": E, "top": top}}, z.double())
    expert_of = torch.empty((50, top), dtype=torch.int32, device="cuda")
    weight = torch.empty((50, top), dtype=torch.float32, device="cuda")
    ops.moe_route(z.cuda(), expert_of, weight, top, 1, 1, 0.0, bias=bias.cuda())
    assert torch.equal(expert_of.cpu().long(), idx)
    assert torch.allclose(weight.cpu().double(), wt, rtol=1e-5, atol=1e-7)
    without = torch.empty_like(expert_of)
    ops.moe_route(z.cuda(), without, weight, top, 1, 1, 0.0)
    assert not torch.equal(without, expert_of)                      # the bias does change who is chosen


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_gated_unit_of_an_expert(dtype):
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(5)
    x = (torch.randn((9, 2 * 37), generator=g) * 3.0).to(dtype)
    out = torch.empty((9, 37), dtype=dtype, device="cuda")
    ops.clamped_glu(x.cuda(), out, float("inf"), 1.0, 0.0)
    want = torch.nn.functional.silu(x.double()[:, :37]) * x.double()[:, 37:]
    assert torch.allclose(out.cpu().double(), want, **_tol(dtype))


# ------------------------------------------------------------------------------- each mechanism alone in a model

ALONE = {
    "time_mix": lambda: config([wkv_layer(mlp=None)]),
    "time_mix_one_stream": lambda: config([wkv_layer(heads=2, dim=40, rank=3, mlp=None)], streams=1),
    "state_space": lambda: config([ssm_layer(mlp=None)]),
    "state_space_one_group_two_taps": lambda: config([ssm_layer(heads=3, vdim=16, state=24, groups=1, conv=2, norm_groups=1, mlp=None)], streams=None),
    "attention": lambda: config([attn_layer(mlp=None)]),
    "attention_plain_frequencies_no_window": lambda: config([attn_layer(window=None, scaling=False, mlp=None)]),
    "attention_no_positions": lambda: config([attn_layer(rot=None, window=7, mlp=None)], streams=None),
    "attention_rotated_in_twos": lambda: config([attn_layer(dim=16, vdim=16, rot=6, mlp=None)]),
    "dense": lambda: config([attn_layer(window=500, mlp=dense())]),
    "experts": lambda: config([attn_layer(window=500, mlp=moe())]),
    "experts_top_one_no_streams": lambda: config([attn_layer(window=500, mlp=moe(4, 1, 40))], streams=None),
    "streams_alone_twice": lambda: config([attn_layer(window=500, mlp=dense(16))], streams=5, loop=(0, 1, 2), scale=None),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(tmp_path_factory, name, dtype):
    entry = model(tmp_path_factory, name, ALONE[name]())
    reqs = requests_for(entry, (70, 1, 33), seed=1)
    compare(entry, dtype, whole(reqs), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_residual_stream_after_every_layer_run(tmp_path_factory, dtype):
    """The sum of the streams behind every run of a layer (a repeated layer counts each time), not the logits alone."""
    from return_b200.engine.replay import TraceReplayer
    entry = model(tmp_path_factory, "full", full_config())
    ids = requests_for(entry, (37,), seed=3)["r0"]
    c, w = entry[1]
    _, want = plain.forward(c, w, ids, keep_layers=True)
    rp = TraceReplayer(entry[0], dtype, 64, max_reside=2)
    got = []
    rp.runner.model.after_block = lambda i, streams, delta: got.append(streams.sum(1).double().cpu())
    rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": ids, "want": [36]}], "end": ["a"]})
    assert len(got) == want.shape[0] == 9
    for i, (a, b) in enumerate(zip(got, want)):
        e = float((a - b).norm() / b.norm())
        assert e < (1e-4 if dtype == "float32" else 2e-2), (i, e)


# ------------------------------------------------------------------------------- the whole model under every schedule

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_against_decoding_token_by_token(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (90, 47, 16))
    compare(entry, dtype, tail_decoded(reqs, tail=40), reqs)
    first = {"t": reqs["r1"][:24]}                                     # from the very first token on, one by one
    compare(entry, dtype, tail_decoded(first, tail=24), first)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(2, 3, 17, 2, 5, 33, 7), (16, 16, 1, 15, 2, 30, 32, 1), (1, 2, 1, 64, 2)])
def test_portions_of_prompts(tmp_path_factory, dtype, sizes):
    """Portions down to two tokens (and one), cut on page borders and off them, shorter and longer than the windows,
    the conv taps and the scan's chunks of eight."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (101, 64, 31))
    compare(entry, dtype, portions(reqs, list(sizes)), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path_factory, dtype):
    """Seven requests through four slots and a pool that holds four of them: portions of some beside single tokens of
    others, each compared with the request alone (the plain walk).  Pages of 8: the windows give pages back."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 80, 17, 49, 2, 71), seed=40)
    for seed in (0, 1):
        compare(entry, dtype, mixed(reqs, max_live=4, portion=13, decode_tail=6, seed=seed), reqs, page_size=8)


def test_one_slot_and_few_pages_taken_again_and_again(tmp_path_factory):
    """Every request inherits the slot, the states and the pages of the one before it, and starts from nothing."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (40, 9, 40, 23), seed=70)
    compare(entry, "float32", tail_decoded(reqs, tail=5), reqs, max_reside=1, page_size=4)
    compare(entry, "bfloat16", tail_decoded(reqs, tail=5), reqs, max_reside=1, page_size=4)


def test_batching_and_cutting_do_not_change_float32_logits_at_all(tmp_path_factory):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (60, 33, 45), seed=90)
    a = run_trace(entry[0], "float32", whole(reqs))
    b = run_trace(entry[0], "float32", mixed(reqs, max_live=3, portion=9, decode_tail=8, seed=2))
    for rid in reqs:
        assert torch.equal(a[rid], b[rid]), rid


# ------------------------------------------------------------------------------- faults that random weights would hide

def _slow_decays(tensors):
    """States that hardly forget: a time mix whose decays stay near exp(-exp(-7)), a state space with a small rate; and
    mixers that add four times what they would to the streams, so that what they lose shows in the logits."""
    for n, t in tensors.items():
        if n.endswith("mix.o"):
            t.mul_(4.0)
        if n.endswith("mix.w0"):
            t.fill_(-7.0)
        elif n.endswith("mix.w2"):
            t.mul_(0.1)
        elif n.endswith("mix.A_log"):
            t.fill_(-6.0)
        elif n.endswith("mix.dt_bias"):
            t.fill_(0.0)


def sharp_config(window=37):
    """Attention whose scores are eight times larger than usual, so that single keys stand out (the first without
    positions and under a window, the second rotated and over all keys), beside states that hardly forget: a key lost
    far back, a window that is one token off or a state cut short moves the logits by far more than the tolerance."""
    return config([attn_layer(heads=2, kv_heads=1, dim=16, vdim=16, window=window, rot=None, scale=8 * 16 ** -0.5, mlp=None),
                   attn_layer(heads=2, kv_heads=2, dim=16, vdim=16, window=None, rot=16, scale=8 * 16 ** -0.5, mlp=None),
                   wkv_layer(heads=2, dim=16, rank=4, mlp=None), ssm_layer(heads=2, vdim=16, state=16, groups=1, conv=3, norm_groups=2, mlp=None)],
                  width=32, streams=2)


def slow_states_config():
    return config([wkv_layer(heads=2, dim=16, rank=4, mlp=None), ssm_layer(heads=2, vdim=16, state=16, groups=2, conv=3, norm_groups=1, mlp=None)],
                  width=32, streams=2)


def _changed(entry, change):
    """Plain logits of a model whose configuration or weights were changed by ``change(config, weights)``."""
    import copy
    c, w = copy.deepcopy(entry[1][0]), dict(entry[1][1])
    change(c, w)
    return lambda ids: plain.forward(c, w, list(ids))[0].float()


def _standing_out_pair(c, w):
    """(a, b, fillers): of all pairs of tokens, the one whose score in head 0 of the first layer (which has no positions:
    a token's query and key there depend on the token alone) is the largest, b asking and a answering, and tokens that
    b scores low."""
    m, eps = c["layers"][0]["mixer"], c["norm"]["eps"]
    D = m["dim"]
    h = plain.rms(w["embed"] * c["embedding"]["scale"] * w["l0.hc1.in"].sum(), eps) * w["l0.norm1"]
    q, k = (h @ w["l0.mix.q"].T)[:, :D], (h @ w["l0.mix.k"].T)[:, :D]
    s0 = (q @ k.T) * m["scale"]
    b, a = divmod(int(s0.argmax()), s0.shape[1])
    return a, b, [int(x) for x in s0[b].argsort()[:30] if int(x) not in (a, b)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_just_inside_and_outside_the_window(tmp_path_factory, dtype):
    """A key that one query scores far above all others is put at the window's last place for two queries and one
    place behind it for two more.  The plain model with a window one shorter (one longer) gives other logits there, so
    an engine whose window is one token off cannot pass: in whole prompts, when the window passes over decoded tokens,
    and when the asking token is the first of its portion."""
    entry = model(tmp_path_factory, "sharp", sharp_config(window=37), patch=_slow_decays)
    c, w = entry[1]
    a, b, fill = _standing_out_pair(c, w)
    g = torch.Generator().manual_seed(1)
    ids = [fill[int(i)] for i in torch.randint(0, len(fill), (170,), generator=g)]
    inside, outside = [40, 120], [80, 160]
    for p in inside:
        ids[p], ids[p - 36] = b, a
    for p in outside:
        ids[p], ids[p - 37] = b, a
    want = plain_rows(entry, ids)

    def set_window(n):
        return lambda c, w: c["layers"][0]["mixer"]["mask"].update(size=n)
    shorter = row_errors(_changed(entry, set_window(36))(ids), want)
    longer = row_errors(_changed(entry, set_window(38))(ids), want)
    assert float(shorter[inside].min()) > 2 * TOL[dtype] and float(longer[outside].min()) > 2 * TOL[dtype]
    reqs = {"edge": ids}
    for steps, page in ((whole(reqs), 16), (tail_decoded(reqs, tail=60), 8),
                        (portions(reqs, [36, 2, 37, 1, 38, 3, 33]), 4),
                        (portions(reqs, [119, 2, 38, 1, 2, 8]), 16)):
        got = run_trace(entry[0], dtype, steps, page_size=page)["edge"]
        assert_close(got, want, dtype, "edge", mean=0.06)
        e = row_errors(got, want)                        # at the aimed rows: far nearer the right window than either wrong one
        assert (e[inside] < 0.25 * shorter[inside]).all() and (e[outside] < 0.25 * longer[outside]).all(), (e[inside], e[outside])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["sharp", "slow_states"])
def test_keys_and_states_far_back_and_at_page_borders(tmp_path_factory, dtype, name):
    """The last rows lean on what the first two hundred tokens left (single far keys of the attention over all keys,
    states that hardly forget): without them the plain model gives other rows."""
    entry = model(tmp_path_factory, name, sharp_config() if name == "sharp" else slow_states_config(), patch=_slow_decays)
    ids = requests_for(entry, (330,), seed=6)["r0"]
    want = plain_rows(entry, ids)
    c, w = entry[1]
    short = plain.forward(c, w, ids[200:])[0].float()
    lost = row_errors(short[-20:], want[-20:])
    assert float(lost.min()) > TOL[dtype] and float(lost.mean()) > 4 * TOL[dtype]
    reqs = {"far": ids}
    for steps, page in ((tail_decoded(reqs, tail=36), 16),                           # decoding across two page borders
                        (portions(reqs, [250, 6, 10, 2, 62]), 8)):                   # portions behind a long prefix
        got = run_trace(entry[0], dtype, steps, page_size=page)["far"]
        assert_close(got, want, dtype, "far", mean=0.06)               # sharp scores multiply the rounding of a query
        assert float(row_errors(got[-20:], want[-20:]).mean()) < 0.25 * float(lost.mean())


def test_a_slot_taken_again_does_not_inherit_slow_states(tmp_path_factory):
    """Two requests one after the other through one slot: the second starts from zero states, zero conv inputs and no
    token before its first (the plain walk of the second alone), although the first left states that hardly decay."""
    entry = model(tmp_path_factory, "slow_states", slow_states_config(), patch=_slow_decays)
    reqs = requests_for(entry, (50, 30), seed=12)
    for dtype in ("float32", "bfloat16"):
        compare(entry, dtype, portions(reqs, [7, 1, 20]), reqs, max_reside=1)
    joined = plain_rows(entry, reqs["r0"] + reqs["r1"])[50:]
    assert float(row_errors(joined, plain_rows(entry, reqs["r1"])).min()) > 2 * TOL["bfloat16"]      # inheriting would show


@pytest.mark.parametrize("dtype,graph", [("float32", False), ("bfloat16", True)])
def test_long_decoding(tmp_path_factory, dtype, graph):
    """Up to 160 tokens decoded one by one behind a prompt of three; in bfloat16 through the captured graphs of generation."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = dict(zip("xy", requests_for(entry, (163, 150), seed=8).values()))
    steps = []
    for k in range(161):
        entries = [{"id": rid, "tokens": ids[:3] if k == 0 else [ids[2 + k]], "want": [2] if k == 0 else [0]}
                   for rid, ids in reqs.items() if 2 + k < len(ids)]
        ended = [rid for rid, ids in reqs.items() if 2 + k == len(ids) - 1]
        steps.append({"step": k, "entries": entries, "end": ended})
    got = run_trace(entry[0], dtype, steps, graph=graph)
    for rid, ids in reqs.items():
        assert_close(got[rid], plain_rows(entry, ids)[2:], dtype, rid)


def test_a_long_prompt_scanned_in_pieces_side_by_side(tmp_path_factory, monkeypatch):
    """On the bfloat16 path a time mix and a state-space mixer cut a portion of 1,024 tokens or more into pieces that
    are scanned at the same time, hand the states from piece to piece (a piece's transition is the product of its
    tokens' decays, per key row or per head) and scan again.  The outputs of every piece, the state that the tokens
    decoded afterwards start from, and a short request in the same step must all be right; the decays are slow, so a
    state handed on wrongly would show to the end.  The float32 path never cuts."""
    from return_b200.ext import ops
    raw = config([wkv_layer(heads=2, dim=24, rank=4, mlp=None), ssm_layer(heads=3, vdim=16, state=24, groups=1, conv=3, norm_groups=1, mlp=None),
                  wkv_layer(heads=1, dim=40, rank=2, mlp=dense(32)), ssm_layer(heads=2, vdim=40, state=8, groups=2, conv=2, norm_groups=2, mlp=None)],
                 width=32, streams=2)
    entry = model(tmp_path_factory, "pieces", raw, patch=_slow_decays)
    reqs = requests_for(entry, (1300, 40), seed=80)
    long_ids, short_ids = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": short_ids[:30], "want": list(range(30))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": long_ids[:100], "want": list(range(100))},
                                      {"id": "r1", "tokens": short_ids[30:31], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": short_ids[31:32], "want": [0]},
                                      {"id": "r0", "tokens": long_ids[100:1290], "want": list(range(1190))}], "end": []}]
    for k in range(8):
        steps.append({"step": 3 + k, "entries": [{"id": "r0", "tokens": [long_ids[1290 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [short_ids[32 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 7 else []})
    calls, combine = [], ops.scan_pieces_combine_sums
    monkeypatch.setattr(ops, "scan_pieces_combine_sums", lambda *a, **k: (calls.append(a[5]), combine(*a, **k))[1])
    got = run_trace(entry[0], "bfloat16", steps)
    assert calls == [True, False, True, False]                       # once a layer, in the step that holds the long portion
    assert_close(got["r0"][:1298], plain_rows(entry, long_ids)[:1298], "bfloat16", "long")
    assert_close(got["r1"], plain_rows(entry, short_ids), "bfloat16", "short")
    one = run_trace(entry[0], "bfloat16", tail_decoded({"r0": long_ids[:1000]}, tail=8))
    assert len(calls) == 4                                           # a portion of 992 tokens is walked in one go
    assert_close(got["r0"][:1000], one["r0"], "bfloat16", "pieces against one walk")
    exact = run_trace(entry[0], "float32", steps)
    assert len(calls) == 4
    assert_close(exact["r0"][:1298], plain_rows(entry, long_ids)[:1298], "float32", "long")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "other", other_sizes_config(), seed=11)
    reqs = requests_for(entry, (75, 20, 1), seed=20)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=11, decode_tail=9, seed=3), reqs, page_size=4, max_reside=2)


def wide_config():
    """Sizes that pick the tensor-core kernels of prompts in bfloat16: attention heads of 64 (keys of 64 beside values
    of 48) under a window and of 128 over all keys, experts with enough pairs for the grouped products."""
    return config([attn_layer(heads=4, kv_heads=2, dim=64, vdim=48, window=300, rot=32, mlp=moe(8, 2, 32)),
                   wkv_layer(heads=2, dim=64, rank=8, mlp=dense(96)),
                   attn_layer(heads=2, kv_heads=1, dim=96, vdim=128, window=None, rot=96, scaling=False, mlp=moe(4, 2, 64)),
                   ssm_layer(heads=4, vdim=32, state=64, groups=2, conv=4, norm_groups=2, mlp=None)], width=64, streams=2)


def test_a_prompt_of_many_rows(tmp_path_factory):
    """A portion long enough for the tensor-core kernels of prompts, beside a short request, then a shorter portion
    behind the long cached prefix beside a decoded token, then decoded tokens; in bfloat16 also through the graphs."""
    entry = model(tmp_path_factory, "wide", wide_config(), seed=5)
    reqs = requests_for(entry, (1200, 40), seed=33)
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": b[:20], "want": list(range(20))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": a[:1100], "want": [0, 500, 1099]},
                                      {"id": "r1", "tokens": b[20:21], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "r0", "tokens": a[1100:1190], "want": list(range(90))},
                                      {"id": "r1", "tokens": b[21:22], "want": [0]}], "end": []}]
    for k in range(10):
        steps.append({"step": 3 + k, "entries": [{"id": "r0", "tokens": [a[1190 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [b[22 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 9 else []})
    want0, want1 = plain_rows(entry, a)[[0, 500, 1099] + list(range(1100, 1200))], plain_rows(entry, b)[:32]
    for dtype, graph in (("bfloat16", False), ("float32", False), ("bfloat16", True)):
        got = run_trace(entry[0], dtype, steps, graph=graph)
        assert_close(got["r0"], want0, dtype, "long")
        assert_close(got["r1"], want1, dtype, "short")


# ------------------------------------------------------------------------------- generation through the engine

def _greedy_plain(entry, prompt, n):
    c, w = entry[1]
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(c, w, ids)[0][-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_scheduler(tmp_path_factory, graph):
    """Five prompts through three slots, portions of 24 beside decoded tokens: the scheduler admits, cuts, frees and
    hands slots on; the tokens are the plain model's."""
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    entry = model(tmp_path_factory, "full", full_config())
    prompts = list(requests_for(entry, (5, 29, 1, 40, 12), seed=30).values())
    eng = Engine(entry[0], EngineConfig(max_token=512, max_reside=3, page_size=16, prefill_chunk=24, dtype="float32",
                                        use_cuda_graph=graph))
    got = eng.generate(prompts, max_new_tokens=10, temperature=0.0)
    assert [r.output_ids for r in got] == [_greedy_plain(entry, p, 10) for p in prompts]
    assert eng.runner.manager.pages_used() == [0] * len(eng.runner.manager.groups)


def test_bfloat16_generation_picks_tokens_the_plain_model_rates_highest(tmp_path_factory):
    from return_b200.engine.config import EngineConfig
    from return_b200.engine.engine import Engine
    entry = model(tmp_path_factory, "full", full_config())
    c, w = entry[1]
    prompts = list(requests_for(entry, (7, 33, 20), seed=50).values())
    eng = Engine(entry[0], EngineConfig(max_token=512, max_reside=4, page_size=16, prefill_chunk=32, dtype="bfloat16"))
    for p, r in zip(prompts, eng.generate(prompts, max_new_tokens=8, temperature=0.0)):
        lg = plain.forward(c, w, p + r.output_ids)[0]
        for k, tok in enumerate(r.output_ids):
            row = lg[len(p) - 1 + k]
            assert row[tok] >= row.max() - 0.1 * row.std(), (k, tok)


def test_command_line_generates(tmp_path_factory):
    import subprocess
    import sys
    entry = model(tmp_path_factory, "full", full_config())
    prompt = requests_for(entry, (9,), seed=60)["r0"]
    out = subprocess.run([sys.executable, "-m", "return_b200", "generate", "--model", entry[0], "--prompt-ids",
                          ",".join(map(str, prompt)), "--new", "6", "--temperature", "0", "--dtype", "float32",
                          "--max-token", "256", "--max-reside", "2"], capture_output=True, text=True, timeout=600,
                         cwd=helpers.ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[0])["output_ids"] == _greedy_plain(entry, prompt, 6)


def test_command_line_replays_a_trace(tmp_path_factory):
    import subprocess
    import sys
    entry = model(tmp_path_factory, "full", full_config())
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [5, 6], "want": [0, 1]}], "end": ["a"]}]
    out = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", entry[0], "--dtype",
                          "float32", "--out", os.path.join(entry[0], "out"), "--max-tokens", "64"],
                         input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and all(f"done {i}" in out.stdout for i in range(3)), out.stderr[-2000:]
    assert not os.path.exists(os.path.join(entry[0], "out", "1.f32"))
    want = plain_rows(entry, [1, 2, 3, 4, 5, 6])
    for step, rows in ((0, [2]), (2, [4, 5])):
        got = torch.frombuffer(bytearray(open(os.path.join(entry[0], "out", f"{step}.f32"), "rb").read()), dtype=torch.float32)
        assert worst(got.view(len(rows), -1), want[rows]) < TOL["float32"]
