"""The Duvadra decoder through the engine against the plain implementation (tests/plain/duvadra_plain.py).

Every test makes a small configuration of its own with random weights (written as a bfloat16 checkpoint, as a model
folder holds them), replays a trace through the engine's step function and compares every logits row with the plain
implementation's, which walks the whole sequence in float64, token by token where there is a recurrence.
float32 path: every row within 1e-4 of its size.  bfloat16 path: rows weighed together (see ``assert_close``).
Where random weights would hide a fault (a key at a window's or a block's edge, a state that was lost far back) the
scores are made sharp and the decays slow, and the test first shows that the plain model itself moves by far more
than the tolerance when that key or state is lost.
"""
import copy
import json
import os
import types

import pytest
import torch

import helpers
from helpers import collect, mixed, pool_tokens, portions, random_ids, tail_decoded, whole
from plain import duvadra_plain as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 1.0 / 12}


# ------------------------------------------------------------------------------- configurations

def dense(ff=56, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=24, count=3, keep=2, scale=1.5):
    r = {"experts": experts, "top": top, "scale": scale}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def attn(heads=4, kv_heads=2, dim=12, vdim=20, size=19, scale=None, **more):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if size:
        m["mask"] = {"size": size}
    m.update(more)
    return m


def chunk_layer(mlp="default", kv_from=None, softcap=7.0, **a):
    m = attn(**a)
    m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": dense() if mlp == "default" else mlp}


def delta_layer(left=None, heads=4, kv_heads=2, dim=10, vdim=6, conv=4, scales=(0.7, 0.6), mlp="default"):
    m = {"left": left or attn(heads=3, kv_heads=1, dim=8, vdim=14, size=21),
         "right": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
         "left_scale": scales[0], "right_scale": scales[1]}
    return {"type": "parallel", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def lru_layer(left=None, width=24, blocks=3, conv=3, rot=6, base=3000.0, scales=(0.9, 0.4), mlp="default"):
    left = left or attn(heads=4, kv_heads=2, dim=10, vdim=10, size=26)
    if rot:
        left["rot"] = {"base": base, "dims": rot}
    m = {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": scales[0], "right_scale": scales[1]}
    return {"type": "parallel_2", "mixer": m, "mlp": dense(40, 0.8) if mlp == "default" else mlp}


def config(layers, vocab=97, width=40, eps=1e-5, mult=0.6, bigram=(53, 31, 7), scale=3.0, cap=12.0):
    c = {"architecture": "Duvadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    emb = {}
    if scale:
        emb["scale"] = scale
    if bigram:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    if emb:
        c["embedding"] = emb
    if mult is not None:
        c["residual_mult"] = mult
    if cap:
        c["logit_softcap"] = cap
    return c


def full_config():
    """All three mixers and both feed-forwards, a layer without a feed-forward, a layer that reads an earlier layer's
    keys under another block size, a window shorter than a page and windows that span several."""
    return config([chunk_layer(size=13), lru_layer(), delta_layer(mlp=None), chunk_layer(size=29, kv_from=0, mlp=moe(5, 3, 16, 1, 1)),
                   delta_layer(left=attn(heads=2, kv_heads=2, dim=16, vdim=8, size=5), heads=2, kv_heads=1, dim=16, vdim=12, conv=2,
                               mlp=dense(48)),
                   chunk_layer(heads=2, kv_heads=1, dim=16, vdim=16, size=40, softcap=3.0, mlp=moe(4, 1, 32, 2, 1))])


def other_sizes_config():
    """The values one (one head, one key head, one block, one tap, one group, as many experts chosen as there are, a
    window and a block of one position), sizes that fill no whole warp or vector, keys and values that differ both ways,
    a rotation over the whole head and over two numbers of it and none, no mask, no pair table, no factor, no caps."""
    return config([lru_layer(left=attn(heads=1, kv_heads=1, dim=40, vdim=40, size=1), width=33, blocks=1, conv=1, rot=2, mlp=moe(3, 3, 9, 1, 1, 1.0)),
                   chunk_layer(heads=1, kv_heads=1, dim=7, vdim=33, size=1, softcap=None, mlp=None),
                   delta_layer(left=attn(heads=6, kv_heads=3, dim=24, vdim=8, size=None), heads=1, kv_heads=1, dim=72, vdim=5, conv=7,
                               mlp=moe(35, 4, 8, 5, 2, 0.5)),
                   lru_layer(left=attn(heads=2, kv_heads=1, dim=18, vdim=18, size=300), width=36, blocks=36, conv=2, rot=18, base=200.0,
                             mlp=dense(9, 50.0)),
                   chunk_layer(heads=5, kv_heads=5, dim=24, vdim=16, size=None, kv_from=None, mlp=moe(2, 1, 40, 2, 2)),
                   lru_layer(left=attn(heads=3, kv_heads=3, dim=8, vdim=8, size=9), width=8, blocks=2, conv=5, rot=0, mlp=dense(7)),
                   chunk_layer(heads=10, kv_heads=5, dim=24, vdim=16, size=200, kv_from=4, mlp=None)],
                  vocab=61, width=36, eps=1e-6, mult=None, bigram=None, scale=None, cap=None)


def wide_config():
    """Sizes that pick the tensor-core kernels of prompts in bfloat16: windowed heads of 64 with a sink and of 128 with a
    rotation, block attention with heads of 96 and of 128, experts with enough pairs for the grouped products."""
    return config([delta_layer(left=attn(heads=4, kv_heads=2, dim=64, vdim=48, size=300), heads=2, kv_heads=1, dim=64, vdim=32, mlp=moe(8, 2, 32, 2, 1)),
                   chunk_layer(heads=8, kv_heads=4, dim=96, vdim=96, size=256, softcap=30.0, mlp=dense(96)),
                   lru_layer(left=attn(heads=2, kv_heads=1, dim=128, vdim=128, size=700), width=128, blocks=4, conv=4, rot=64, mlp=moe(4, 2, 64, 1, 1)),
                   chunk_layer(heads=8, kv_heads=1, dim=128, vdim=64, size=1000, mlp=None)], width=64, scale=6.0)


_MODELS = {}


def model(tmp_path_factory, name, raw, seed=3, patch=None):
    """(model folder, (config, float64 weights), memo of plain logits), cached: the plain walk is slow.  ``patch``
    changes tensors (name -> tensor) before they are written."""
    if name not in _MODELS:
        from return_b200.config.duvadra_config import DuvadraConfig
        from return_b200.weights import loader
        from return_b200.weights.safetensors_io import write_safetensors
        d = str(tmp_path_factory.mktemp(name))
        loader.write_random_model(d, DuvadraConfig(raw), seed, torch.bfloat16)
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
        memo[key] = plain.forward(c, w, list(ids)).float()
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


def assert_close(got, want, dtype, what="", mean=0.03, robust=False):
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
    if robust:            # configurations drawn at random: single rows may move by their own size (see below); the middle row may not
        assert over <= max(2, e.numel() // 10) and float(e.median()) < mean, (what, dtype, over, float(e.max()), float(e.median()))
        return
    assert over <= max(2, e.numel() // 10) and float(e.max()) < 0.6 and float(e.mean()) < mean, \
        (what, dtype, over, float(e.max()), float(e.mean()), int(e.argmax()))


def compare(entry, dtype, steps, requests, robust=False, **kw):
    got = run_trace(entry[0], dtype, steps, **kw)
    for rid, ids in requests.items():
        assert_close(got[rid], plain_rows(entry, ids), dtype, rid, robust=robust)


# ------------------------------------------------------------------------------- kernels of single mechanisms

def _segments(lens, slots, pos0=None):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    tok_seg = [i for i, n in enumerate(lens) for _ in range(n)]
    pos0 = pos0 or [0] * len(lens)
    pos = [pos0[i] + k for i, n in enumerate(lens) for k in range(n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return types.SimpleNamespace(cu_q=i32(cu), tok_seg=i32(tok_seg), seg_slot=i32(slots), pos=i32(pos), num_segments=len(lens),
                                 num_tokens=cu[-1])


@pytest.mark.parametrize("E,top,count,keep", [(15, 2, 3, 1), (6, 6, 1, 1), (35, 4, 5, 2), (8, 3, 8, 3), (40, 1, 4, 4)])
def test_router_choice(E, top, count, keep):
    """Logistic scores, groups ranked by their two best, the weights over their sum times a factor, against the plain
    router on logits far enough apart that no choice is a close call."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(E * 7 + top)
    z = torch.randn((50, E), generator=g) * 2.0
    r = {"experts": E, "top": top, "scale": 1.75, "groups": {"count": count, "keep": keep}}
    picked, wts = plain.route(z.double(), r)
    expert_of = torch.empty((50, top), dtype=torch.int32, device="cuda")
    weight = torch.empty((50, top), dtype=torch.float32, device="cuda")
    ops.moe_route(z.cuda(), expert_of, weight, top, count, keep, 1e-20, score="sigmoid", group_top=2, scale=1.75)
    got = {(t, int(e)): float(x) for t in range(50) for e, x in zip(expert_of[t].cpu(), weight[t].cpu())}
    want = {(t, int(e)): float(x) for t in range(50) for e, x in zip(picked[t], wts[t])}
    assert got.keys() == want.keys()
    assert max(abs(got[k] - want[k]) for k in want) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_token_pairs(dtype):
    """The pair row of a token in the middle of a step, of a step's first token (from the request's kept token), of a
    sequence's first token (the table's last row), and the kept token afterwards."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(4)
    V, H, buckets = 23, 20, 11
    table, pairs = torch.randn((V, H), generator=g).to(dtype), torch.randn((buckets + 1, H), generator=g).to(dtype)
    b = _segments([3, 1, 2], [2, 0, 1], pos0=[0, 5, 9])
    b.tokens = torch.tensor([4, 22, 7, 1, 9, 9], dtype=torch.int32, device="cuda")
    last = torch.tensor([13, 6, 99, 5], dtype=torch.int32, device="cuda")
    out = torch.empty((6, H), dtype=torch.float32, device="cuda")
    ops.embedding_pair(table.cuda(), pairs.cuda(), b, last, out, 1.5, buckets, 113, 29)
    ops.last_token_update(b, last)
    prev = [None, 4, 22, 13, 6, 9]
    rows = [buckets if p is None else (p * 113 + t * 29) % buckets for p, t in zip(prev, b.tokens.tolist())]
    want = table.double()[b.tokens.long().cpu()] * 1.5 + pairs.double()[rows]
    assert torch.allclose(out.cpu().double(), want, rtol=1e-6, atol=1e-6)
    assert last.tolist() == [1, 9, 7, 5]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,B,K", [(24, 3, 4), (33, 1, 1), (36, 36, 2), (256, 4, 7)])
def test_gated_linear_recurrence_kernels(W, B, K, dtype):
    """The convolution with held inputs and the channel recurrence, a sequence cut into two steps (the second beside
    another request), against the plain walk of the whole sequence."""
    from return_b200.ext import ops
    g = torch.Generator().manual_seed(W + K)
    T, bs = 19, W // B
    rnd = lambda *s: torch.randn(s, generator=g, dtype=torch.float64)
    proj = rnd(T, 2 * W).to(dtype)
    w = {"y.b": rnd(W) * 0.2, "x.b": rnd(W) * 0.2, "conv": rnd(W, K) * 0.5, "conv.b": rnd(W) * 0.2, "ra": rnd(B, bs, bs) * bs ** -0.5,
         "ri": rnd(B, bs, bs) * bs ** -0.5, "ra.b": rnd(B, bs), "ri.b": rnd(B, bs), "lam": rnd(W) - 2.0}
    w = {k: v.to(dtype) for k, v in w.items()}
    wd = {k: v.double() for k, v in w.items()}
    # the plain walk, from the projections on
    u = plain.causal_conv(proj.double()[:, W:] + wd["x.b"], wd["conv"], wd["conv.b"])
    ub = u.view(T, B, bs)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wd["ra"]) + wd["ra.b"]).reshape(T, W)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wd["ri"]) + wd["ri.b"]).reshape(T, W)
    f = torch.exp(-8.0 * r * torch.nn.functional.softplus(wd["lam"]))
    s, want = torch.zeros(W, dtype=torch.float64), []
    for t in range(T):
        s = f[t] * s + torch.sqrt(1 - f[t] ** 2) * i[t] * u[t]
        want.append(s * plain.gelu_tanh(proj.double()[t, :W] + wd["y.b"]))
    want = torch.stack(want)
    state = torch.zeros((3, W + W * (K - 1)), dtype=torch.float32, device="cuda")
    state[1] = 7.0                                               # another request's slot: must stay as it is
    cw = {k: v.cuda().contiguous() for k, v in w.items()}
    got = []
    for lo, hi, lens, slots, pos0 in ((0, 11, [11], [2], [0]), (11, T, [T - 11], [2], [11])):
        b = _segments(lens, slots, pos0)
        x = proj[lo:hi].cuda()
        n = hi - lo
        uu = torch.empty((n, W), dtype=dtype, device="cuda")
        ops.gated_conv(x[:, W:], cw["x.b"], cw["conv"], cw["conv.b"], state, W, b, uu)
        ops.conv_state_update(x[:, W:], K, state, W, b, W)
        gates = torch.empty((2, B, n, bs), dtype=torch.float32, device="cuda")
        ops.linear_heads(uu.view(n, B, bs).transpose(0, 1), cw["ra"], gates[0])
        ops.linear_heads(uu.view(n, B, bs).transpose(0, 1), cw["ri"], gates[1])
        out = torch.empty((n, W), dtype=dtype, device="cuda")
        ops.gated_recurrence(uu, gates, bs, cw["ra.b"], cw["ri.b"], cw["lam"], 8.0, x, cw["y.b"], state, 0, b, out)
        got.append(out.cpu().double())
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=5e-2, atol=5e-2)
    assert torch.allclose(torch.cat(got), want, **tol)
    assert bool((state[1] == 7.0).all())


# ------------------------------------------------------------------------------- each mechanism alone, as a one-layer model

ALONE = {
    "blocks": lambda: config([chunk_layer(mlp=None)]),
    "blocks_shared": lambda: config([chunk_layer(size=11, mlp=None), chunk_layer(size=17, kv_from=0, mlp=None)]),
    "window_sink_delta": lambda: config([delta_layer(mlp=None)]),
    "window_rot_lru": lambda: config([lru_layer(mlp=None)]),
    "capped_unit": lambda: config([chunk_layer(mlp=dense(48, 0.5))], bigram=None),
    "experts": lambda: config([chunk_layer(mlp=moe(10, 3, 16, 5, 2, 1.7))], bigram=None),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(tmp_path_factory, name, dtype):
    """A model of one layer (two where a layer reads another's keys): whole prompts, prompts against token-by-token
    decoding, and portions down to single first tokens."""
    entry = model(tmp_path_factory, "alone_" + name, ALONE[name](), seed=7)
    reqs = requests_for(entry, (70, 9), seed=40)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, tail_decoded(reqs, tail=40), reqs, page_size=8)
    compare(entry, dtype, portions(reqs, [1, 1, 2, 17, 3, 30]), reqs, page_size=4)


# ------------------------------------------------------------------------------- the whole model under every schedule

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_decoding(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (130, 37, 1, 64), seed=10)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, tail_decoded(reqs, tail=48), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_several_sizes(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (150, 33), seed=14)
    compare(entry, dtype, portions(reqs, [2, 29, 13, 2, 5, 40, 3]), reqs, page_size=8)
    compare(entry, dtype, portions(reqs, [64, 1, 2, 16]), reqs, page_size=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path_factory, dtype):
    """Six requests through two and three slots, portions beside decoded tokens, requests that sit out a step: every
    request's rows are those of the request alone."""
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (90, 41, 7, 66, 30, 2), seed=22)
    compare(entry, dtype, mixed(reqs, max_live=3, portion=19, decode_tail=12, seed=1), reqs, page_size=8, max_reside=3)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=7, decode_tail=25, seed=2), reqs, page_size=4, max_reside=2)


def test_batching_and_cutting_do_not_change_float32_logits_at_all(tmp_path_factory):
    entry = model(tmp_path_factory, "full", full_config())
    reqs = requests_for(entry, (80, 35, 12), seed=31)
    a = run_trace(entry[0], "float32", whole(reqs))
    b = run_trace(entry[0], "float32", mixed(reqs, max_live=3, portion=9, decode_tail=10, seed=5), page_size=4, max_reside=3)
    c = run_trace(entry[0], "float32", portions(reqs, [2, 31, 1, 7]), page_size=8)
    for rid in reqs:
        assert torch.equal(a[rid], b[rid]) and torch.equal(a[rid], c[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(tmp_path_factory, dtype):
    entry = model(tmp_path_factory, "other", other_sizes_config(), seed=11)
    reqs = requests_for(entry, (75, 20, 1), seed=20)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=11, decode_tail=9, seed=3), reqs, page_size=4, max_reside=2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_query_heads_on_one_key_head(tmp_path_factory, dtype):
    """Twenty and forty query heads a key head: the decode kernel packs a key head's query heads into tiles of 16 rows,
    and every row keeps its own head's slope, sink and gate."""
    raw = config([chunk_layer(heads=20, kv_heads=1, dim=16, vdim=16, size=23, mlp=None),
                  delta_layer(left=attn(heads=40, kv_heads=2, dim=8, vdim=12, size=17), heads=6, kv_heads=1, dim=8, vdim=8, mlp=None),
                  chunk_layer(heads=36, kv_heads=1, dim=16, vdim=16, size=31, kv_from=0, mlp=dense(24))], width=48)
    entry = model(tmp_path_factory, "many_heads", raw, seed=9)
    reqs = requests_for(entry, (70, 33), seed=44)
    compare(entry, dtype, tail_decoded(reqs, tail=45), reqs, page_size=8)
    compare(entry, dtype, mixed(reqs, max_live=2, portion=9, decode_tail=20, seed=7), reqs, page_size=4, max_reside=2)


def _random_config(rng):
    """A configuration no fixed case has: two to five layers of random kinds and sizes (head sizes that fill no vector,
    odd head counts, windows and blocks from one position to beyond the prompts, taps from one to six, any number of
    experts and groups), later block attentions reading an earlier one's keys."""
    width = rng.choice([24, 36, 40, 56, 64])
    layers, owners = [], []                                    # owners: (layer, kv_heads, dim, vdim) of block attentions with keys
    for i in range(rng.randint(2, 5)):
        kind = rng.choice(["attention", "parallel", "parallel_2"])
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 3, 5])
        size = rng.choice([None, 1, 3, 7, 16, 29, 64, 200])
        mlp = rng.choice([None, dense(rng.choice([7, 24, 40]), rng.choice([0.4, 2.0, 30.0])),
                          moe(*rng.choice([(4, 1, 16, 2, 1), (6, 2, 8, 3, 2), (9, 3, 12, 3, 3), (5, 5, 8, 1, 1), (16, 4, 8, 4, 2)]),
                              scale=rng.choice([0.7, 1.0, 3.0]))])
        if kind == "attention":
            if owners and rng.random() < 0.5:
                src, kv, dim, vdim = rng.choice(owners)
                heads = kv * rng.choice([1, 2, 4])
                layers.append(chunk_layer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, size=size, kv_from=src,
                                          softcap=rng.choice([None, 2.0, 25.0]), mlp=mlp))
            else:
                dim, vdim = rng.choice([7, 8, 16, 20, 48]), rng.choice([5, 8, 16, 24, 40])
                owners.append((i, kv, dim, vdim))
                layers.append(chunk_layer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, size=size,
                                          softcap=rng.choice([None, 2.0, 25.0]), mlp=mlp))
        elif kind == "parallel":
            rk = rng.choice([1, 2])
            layers.append(delta_layer(left=attn(heads=heads, kv_heads=kv, dim=rng.choice([6, 8, 16, 24]), vdim=rng.choice([4, 8, 16, 36]), size=size),
                                      heads=rk * rng.choice([1, 2, 3]), kv_heads=rk, dim=rng.choice([5, 8, 16, 40]),
                                      vdim=rng.choice([3, 8, 16, 33]), conv=rng.randint(1, 6),
                                      scales=(rng.choice([0.3, 1.0]), rng.choice([0.5, 1.2])), mlp=mlp))
        else:
            dim = rng.choice([6, 8, 16, 32])
            blocks = rng.choice([1, 2, 3, 6])
            layers.append(lru_layer(left=attn(heads=heads, kv_heads=kv, dim=dim, vdim=dim, size=size), width=blocks * rng.choice([1, 4, 7, 16]),
                                    blocks=blocks, conv=rng.randint(1, 6), rot=rng.choice([0, 2, dim // 2 // 2 * 2, dim]),
                                    base=rng.choice([50.0, 10000.0]), scales=(rng.choice([0.3, 1.0]), rng.choice([0.5, 1.2])), mlp=mlp))
    return config(layers, vocab=rng.randint(30, 200), width=width, eps=rng.choice([1e-6, 1e-5, 1e-3]),
                  mult=rng.choice([None, 0.4, 1.0, 1.3]), bigram=rng.choice([None, (31, 5, 3), (97, 1000003, 7919)]),
                  scale=rng.choice([None, 0.5, 4.0]), cap=rng.choice([None, 5.0, 40.0]))


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configurations_and_traces(tmp_path_factory, seed):
    import random
    rng = random.Random(500 + seed)
    raw = _random_config(rng)
    entry = model(tmp_path_factory, f"fuzz{seed}", raw, seed=seed)
    reqs = requests_for(entry, [rng.randint(1, 80) for _ in range(rng.randint(2, 4))], seed=100 + seed)
    steps = mixed(reqs, max_live=rng.randint(1, 3), portion=rng.randint(2, 30), decode_tail=rng.randint(0, 20), seed=seed)
    page = rng.choice([4, 8, 16, 32])
    for dtype in ("float32", "bfloat16"):
        try:
            # Where bfloat16 turns a router's choice among few experts with large weights, or the sign of the one product
            # q . k that a delta rule's first token is read out with (its read-out is then divided by its own size), a
            # single row moves by its own size.  Such rows stay as few as everywhere (two, or one in ten) and the middle
            # row within 3 %; the float32 rows hold each to 1e-4.
            compare(entry, dtype, steps, reqs, robust=True, page_size=page, max_reside=3)
        except AssertionError as e:
            raise AssertionError((raw, page, str(e)[:300]))


# ------------------------------------------------------------------------------- edges, far states, slots

def _slow_decays(tensors):
    """States that hardly forget: what a request saw far back still shows at its end."""
    for name, t in tensors.items():
        if name.endswith("right.A_log"):
            t.fill_(-6.0)
        if name.endswith("right.lam"):
            t.fill_(-7.0)


def sharp_config(kind, size=37):
    """One layer without a feed-forward whose attention scores are eight times larger than usual, so that single
    keys stand out; no pair table, so that a token's query and key depend on the token alone."""
    if kind == "block":
        first = chunk_layer(heads=2, kv_heads=1, dim=16, vdim=16, size=size, scale=8 * 16 ** -0.5, softcap=60.0, mlp=None)
    else:
        first = delta_layer(left=attn(heads=2, kv_heads=1, dim=16, vdim=16, size=size, scale=8 * 16 ** -0.5), heads=2, kv_heads=1,
                            dim=16, vdim=16, scales=(1.0, 0.2), mlp=None)
    return config([first], width=32, bigram=None, mult=1.0, cap=None, scale=0.25)


def slow_states_config():
    """Both state mixers, weighing far more than the windowed attentions beside them, with the pair table."""
    return config([delta_layer(scales=(0.2, 1.5), mlp=None), lru_layer(scales=(0.2, 1.5), mlp=None)], width=32, mult=1.0)


def _standing_out_pair(c, w, kind):
    """(a, b, fillers): of all pairs of tokens, the one whose score in head 0 of the first layer is the largest, b asking
    and a answering, and tokens that b scores low."""
    p = "l0.mix." if kind == "block" else "l0.mix.left."
    m = c["layers"][0]["mixer"] if kind == "block" else c["layers"][0]["mixer"]["left"]
    D = m["dim"]
    h = plain.rms(w["embed"] * c["embedding"]["scale"], c["norm"]["eps"]) * w["l0.norm1"]
    q, k = h @ w[p + "q"].T, h @ w[p + "k"].T
    if kind != "block":
        q, k = q + w[p + "q.b"], k + w[p + "k.b"]
    s0 = (q[:, :D] @ k[:, :D].T) * m["scale"]
    b, a = divmod(int(s0.argmax()), s0.shape[1])
    return a, b, [int(x) for x in s0[b].argsort()[:30] if int(x) not in (a, b)]


def _with_bound_moved(entry, by):
    """Plain logits of the model whose every row sees one key more below its lowest (by = -1) or loses its lowest
    (by = +1): what an engine whose window or block is one token off would compute."""
    c, w = entry[1]
    true_visible = plain.visible

    def moved(T, kind, size):
        ok = true_visible(T, kind, size)
        if kind is None:
            return ok
        for i in range(T):
            lo = int(ok[i].nonzero()[0])
            if by < 0 and lo > 0:
                ok[i, lo - 1] = True
            if by > 0 and lo < i:
                ok[i, lo] = False
        return ok

    def run(ids):
        plain.visible = moved
        try:
            return plain.forward(c, w, list(ids)).float()
        finally:
            plain.visible = true_visible
    return run


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["block", "window"])
def test_keys_just_inside_and_outside_a_window_and_a_block(tmp_path_factory, kind, dtype):
    """A key that one query scores far above all others is put at the lowest place two queries can see and one place
    below it for two more.  The plain model with that bound moved by one gives other logits there, so an engine whose
    window or block is one token off cannot pass: in whole prompts, when the edge passes over decoded tokens, and when
    the asking token is the first of its portion."""
    size = 37
    entry = model(tmp_path_factory, "sharp_" + kind, sharp_config(kind, size), patch=_slow_decays)
    c, w = entry[1]
    a, b, fill = _standing_out_pair(c, w, kind)
    g = torch.Generator().manual_seed(1)
    ids = [fill[int(i)] for i in torch.randint(0, len(fill), (170,), generator=g)]
    if kind == "window":                                         # the asking places, and how far below them the key sits
        inside, outside = {40: 36, 120: 36}, {80: 37, 160: 37}
    else:                                                        # blocks of 37 begin at 37, 74, 111, 148
        inside, outside = {60: 60 - 37, 140: 140 - 111}, {100: 100 - 73, 150: 150 - 147}
    for p, back in {**inside, **outside}.items():
        ids[p], ids[p - back] = b, a
    inside, outside = sorted(inside), sorted(outside)
    want = plain_rows(entry, ids)
    fewer = row_errors(_with_bound_moved(entry, +1)(ids), want)
    more = row_errors(_with_bound_moved(entry, -1)(ids), want)
    assert float(fewer[inside].min()) > 0.15 and float(more[outside].min()) > 0.15
    reqs = {"edge": ids}
    for steps, page in ((whole(reqs), 16), (tail_decoded(reqs, tail=130), 8),
                        (portions(reqs, [36, 2, 37, 1, 38, 3, 33]), 4),
                        (portions(reqs, [60, 2, 38, 20, 27, 3]), 16)):         # 60, 100, 120, 150 begin portions
        got = run_trace(entry[0], dtype, steps, page_size=page)["edge"]
        assert_close(got, want, dtype, "edge", mean=0.06)
        e = row_errors(got, want)                        # at the aimed rows: far nearer the right bound than either wrong one
        assert (e[inside] < 0.25 * fewer[inside]).all() and (e[outside] < 0.25 * more[outside]).all(), (e[inside], e[outside])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_states_far_back_and_at_page_borders(tmp_path_factory, dtype):
    """Every attention of the design forgets behind its window or block; what reaches further is the states.  With slow
    decays the last rows lean on the first two hundred tokens: without them the plain model gives other rows."""
    entry = model(tmp_path_factory, "slow_states", slow_states_config(), patch=_slow_decays)
    ids = requests_for(entry, (330,), seed=6)["r0"]
    want = plain_rows(entry, ids)
    c, w = entry[1]
    short = plain.forward(c, w, ids[200:]).float()
    lost = row_errors(short[-20:], want[-20:])
    assert float(lost.mean()) > 0.08
    reqs = {"far": ids}
    for steps, page in ((tail_decoded(reqs, tail=36), 16), (portions(reqs, [250, 6, 10, 2, 62]), 8)):
        got = run_trace(entry[0], dtype, steps, page_size=page)["far"]
        assert_close(got, want, dtype, "far", mean=0.06)
        assert float(row_errors(got[-20:], want[-20:]).mean()) < 0.25 * float(lost.mean())


def test_a_slot_taken_again_inherits_nothing(tmp_path_factory):
    """Two requests one after the other through one slot: the second starts from zero states, zero conv inputs and no
    token before its first (the plain walk of the second alone), although the first left states that hardly decay."""
    entry = model(tmp_path_factory, "slow_states", slow_states_config(), patch=_slow_decays)
    reqs = requests_for(entry, (50, 30), seed=12)
    for dtype in ("float32", "bfloat16"):
        compare(entry, dtype, portions(reqs, [7, 1, 20]), reqs, max_reside=1)
    joined = plain_rows(entry, reqs["r0"] + reqs["r1"])[50:]
    assert float(row_errors(joined, plain_rows(entry, reqs["r1"])).mean()) > 0.08                    # inheriting would show


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


def test_a_long_portion_of_the_channel_recurrence_walked_in_pieces(tmp_path_factory, monkeypatch):
    """On the bfloat16 path the gated linear recurrence cuts a portion of 256 tokens or more into pieces that are walked
    at the same time, hands the states from piece to piece and walks again.  The outputs of every piece, the state that
    the tokens decoded afterwards start from, and a short request in the same step must all be right; the decays are
    slow, so a state handed on wrongly would show to the end.  The float32 path never cuts."""
    from return_b200.ext import ops
    entry = model(tmp_path_factory, "slow_states", slow_states_config(), patch=_slow_decays)
    reqs = requests_for(entry, (700, 40), seed=80)
    long_ids, short_ids = reqs["r0"], reqs["r1"]
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": short_ids[:30], "want": list(range(30))}], "end": []},
             {"step": 1, "entries": [{"id": "r0", "tokens": long_ids[:100], "want": list(range(100))},
                                      {"id": "r1", "tokens": short_ids[30:31], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "r1", "tokens": short_ids[31:32], "want": [0]},
                                      {"id": "r0", "tokens": long_ids[100:690], "want": list(range(590))}], "end": []}]
    for k in range(8):
        steps.append({"step": 3 + k, "entries": [{"id": "r0", "tokens": [long_ids[690 + k]], "want": [0]},
                                                  {"id": "r1", "tokens": [short_ids[32 + k]], "want": [0]}],
                      "end": ["r0", "r1"] if k == 7 else []})
    calls, combine = [], ops.gated_pieces_combine
    monkeypatch.setattr(ops, "gated_pieces_combine", lambda *a, **k: (calls.append(a[0].shape[0]), combine(*a, **k))[1])
    got = run_trace(entry[0], "bfloat16", steps)
    assert calls == [10]                                              # once, in the step that holds the long portion: nine pieces and the short request
    assert_close(got["r0"][:698], plain_rows(entry, long_ids)[:698], "bfloat16", "long")
    assert_close(got["r1"], plain_rows(entry, short_ids), "bfloat16", "short")
    exact = run_trace(entry[0], "float32", steps)
    assert len(calls) == 1
    assert_close(exact["r0"][:698], plain_rows(entry, long_ids)[:698], "float32", "long")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_blocks_that_begin_inside_the_tensor_core_tiles(tmp_path_factory, dtype):
    """Block attentions with heads of 64 and 128 (in bfloat16 the tcgen05 kernel's rows of 256 queries and tiles of 64
    keys) under blocks of 37, 100 and 300 positions, so that every tile of rows holds several blocks' beginnings and whole
    key tiles that a row may not see; one layer reads another's keys under a larger block."""
    raw = config([chunk_layer(heads=8, kv_heads=2, dim=64, vdim=64, size=37, mlp=None),
                  chunk_layer(heads=8, kv_heads=1, dim=128, vdim=128, size=100, softcap=None, mlp=None),
                  chunk_layer(heads=16, kv_heads=2, dim=64, vdim=64, size=300, kv_from=0, softcap=20.0, mlp=dense(64))], width=64)
    entry = model(tmp_path_factory, "tile_blocks", raw, seed=13)
    reqs = requests_for(entry, (700, 90), seed=71)
    compare(entry, dtype, whole(reqs), reqs)
    compare(entry, dtype, portions(reqs, [300, 2, 257, 64, 70]), reqs, page_size=16)
    compare(entry, dtype, tail_decoded({"r0": reqs["r0"][:400]}, tail=40), {"r0": reqs["r0"][:400]}, page_size=8)


# ------------------------------------------------------------------------------- generation through the engine

def _greedy_plain(entry, prompt, n):
    c, w = entry[1]
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(c, w, ids)[-1].argmax()))
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
        lg = plain.forward(c, w, p + r.output_ids)
        for k, tok in enumerate(r.output_ids):
            row = lg[len(p) - 1 + k]
            assert row[tok] >= row.max() - 0.1 * row.std(), (k, tok)


def test_command_line_generates_and_replays(tmp_path_factory):
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
