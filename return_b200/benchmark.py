"""Throughput measurements of the engine: decode tokens/s at a batch size after prompts of a given
length, and prefill tokens/s, timed on the device with CUDA events.

After the reference's own definitions: decode tok/s = batch * steps / time over timed steps that
follow warm-up steps (rollout/utils/bench_sym.py:24-52), prefill tok/s = tokens / time for a whole
prompt including its one row of logits (rollout/utils/bench_prefill.py:22-43); token ids are
uniform over the vocabulary (rollout/utils/bench_sym.py:26).
"""
from __future__ import annotations

from typing import Dict, List

import torch


def _random_ids(vocab: int, n: int, gen: torch.Generator) -> List[int]:
    return torch.randint(0, vocab, (n,), generator=gen).tolist()


def fill_requests(runner, batch: int, ctx: int, seed: int = 1, chunk: int = 4096, prefix: str = "bench") -> List[str]:
    """``batch`` requests with ``ctx`` tokens each in the cache (run through the model, nothing wanted)."""
    gen = torch.Generator().manual_seed(seed)
    rids = []
    for i in range(batch):
        rid = f"{prefix}-{i}"
        runner.add_request(rid)
        ids = _random_ids(runner.vocab_size, ctx, gen)
        for a in range(0, ctx, chunk):
            runner.step([runner.reserve(rid, ids[a:a + chunk])])
        rids.append(rid)
    torch.cuda.synchronize()
    return rids


def decode_throughput(runner, batch: int, ctx: int, steps: int, warmup: int, seed: int = 1) -> Dict[str, float]:
    """Decode steps of ``batch`` requests that each hold ``ctx`` tokens: every step appends one token
    per request and computes its logits.  Device time by CUDA events around exactly ``steps`` steps."""
    rids = fill_requests(runner, batch, ctx, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    toks = [_random_ids(runner.vocab_size, batch, gen) for _ in range(steps + warmup)]

    def one(k):
        entries = [runner.reserve(rid, [toks[k][i]], [0]) for i, rid in enumerate(rids)]
        return runner.step(entries)

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for k in range(warmup, warmup + steps):
        one(k)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    for rid in rids:
        runner.free_request(rid)
    return {"tokens_per_s": batch * 1000.0 / ms, "ms_per_step": ms, "kv_tokens": batch * (ctx + warmup + steps // 2)}


def prefill_throughput(runner, tokens: int, iters: int, warmup: int, seed: int = 2) -> Dict[str, float]:
    """One prompt of ``tokens`` tokens in one step, with the logits of its last position."""
    gen = torch.Generator().manual_seed(seed)
    times = []
    for k in range(warmup + iters):
        ids = _random_ids(runner.vocab_size, tokens, gen)
        rid = f"prefill-{k}"
        runner.add_request(rid)
        entry = runner.reserve(rid, ids, [tokens - 1])
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([entry])
        end.record()
        torch.cuda.synchronize()
        if k >= warmup:
            times.append(start.elapsed_time(end))
        runner.free_request(rid)
    ms = sum(times) / len(times)
    return {"tokens_per_s": tokens * 1000.0 / ms, "ms": ms, "tokens": tokens}


# Kernel names of a decode step by kind, after the reference's table (rollout/utils/prof_graph.py:27-43): its
# kinds, the names of this engine's kernels (and of the library's matrix products).
PROFILE_BUCKETS = [
    ("decode_attn", ["attn_decode", "attn_combine"]),
    ("prefill_attn", ["attn_prefill", "attention_simt", "tc5_merge"]),
    ("gemm/matmul", ["gemm", "nvjet", "cutlass", "cublas", "matmul"]),
    ("rmsnorm", ["rmsnorm", "norm_rows"]),
    ("rope", ["rope"]),
    ("elementwise", ["swiglu", "embedding", "elementwise", "copy", "fill"]),
    ("softmax/sample", ["sample", "argmax"]),
]


def profile_bucket(kernel_name: str) -> str:
    low = kernel_name.lower()
    for label, keys in PROFILE_BUCKETS:
        if any(k in low for k in keys):
            return label
    return "other"


def profile_decode(runner, batch: int, ctx: int, steps: int, warmup: int, seed: int = 1) -> Dict[str, object]:
    """Where the device time of decode steps goes, by kind of kernel: the table that the reference prints with
    ``torch.profiler`` over graph-replayed decode steps (rollout/utils/prof_graph.py:76-107).  CUDA activity only;
    times are each kernel's own device time summed, so kernels that overlap count twice and the sum may exceed
    the step's wall time."""
    from collections import defaultdict
    from torch.profiler import ProfilerActivity, profile
    rids = fill_requests(runner, batch, ctx, seed, prefix="prof")
    gen = torch.Generator().manual_seed(seed + 1)
    toks = [_random_ids(runner.vocab_size, batch, gen) for _ in range(steps + warmup)]

    def one(k):
        return runner.step([runner.reserve(rid, [toks[k][i]], [0]) for i, rid in enumerate(rids)])

    for k in range(warmup):
        one(k)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA], record_shapes=False) as prof:
        for k in range(warmup, warmup + steps):
            one(k)
        torch.cuda.synchronize()
    for rid in rids:
        runner.free_request(rid)
    bucket, count, per_kernel = defaultdict(float), defaultdict(int), defaultdict(float)
    for e in prof.key_averages():
        us = getattr(e, "self_device_time_total", 0) or getattr(e, "self_cuda_time_total", 0)
        if us <= 0:
            continue
        b = profile_bucket(e.key)
        bucket[b] += us
        count[b] += e.count
        per_kernel[e.key] += us
    total = sum(bucket.values()) or 1.0
    return {"batch": batch, "ctx": ctx, "steps": steps, "gpu_ms_per_step": total / 1e3 / steps,
            "buckets": [{"bucket": b, "ms_per_step": us / 1e3 / steps, "share": us / total, "kernels_per_step": count[b] / steps}
                        for b, us in sorted(bucket.items(), key=lambda kv: -kv[1])],
            "top_kernels": [{"kernel": k[:80], "ms_per_step": us / 1e3 / steps, "share": us / total}
                            for k, us in sorted(per_kernel.items(), key=lambda kv: -kv[1])[:12]]}


def decode_step_bytes(cfg, batch: int, kv_tokens_total: int, dtype_bytes: int = 2) -> int:
    """Bytes a decode step has to read: every weight it uses once (the embedding rows it gathers
    are negligible and left out; a tied head is counted once, as the head), plus the cached keys and
    values of the live requests."""
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = (q + 2 * kv) * H + H * q + 2 * I * H + H * I + 2 * H + 2 * cfg.head_dim
    weights = (L * per_layer + H + cfg.vocab_size * H) * dtype_bytes
    cache = kv_tokens_total * L * 2 * kv * dtype_bytes
    return weights + cache


def prefill_flops(cfg, tokens: int, logit_rows: int = 1) -> float:
    """Floating-point operations of one whole-prompt step: matrix products of every layer, causal
    attention (half the square), and the head on ``logit_rows`` rows."""
    H, I, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    linear = 2.0 * tokens * ((q + 2 * kv) * H + H * q + 2 * I * H + H * I)
    attn = 4.0 * tokens * tokens * q / 2.0
    return L * (linear + attn) + 2.0 * logit_rows * cfg.vocab_size * H


# ------------------------------------------------------------------------------- single kernels

def _paged_case(batch: int, ctx: int, q_len: int, heads: int, kv_heads: int, head_dim: int, page: int, device):
    """Random bfloat16 pools and the tables of ``batch`` requests that hold ``ctx`` keys each and
    bring ``q_len`` new tokens (already in the cache)."""
    blocks = (ctx + page - 1) // page
    n_pages = batch * blocks
    g = torch.Generator(device=device).manual_seed(0)
    k_pool = torch.randn((n_pages, kv_heads, page, head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    v_pool = torch.randn((n_pages, kv_heads, page, head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    perm = torch.randperm(n_pages, generator=g, device=device).to(torch.int32).view(batch, blocks)
    T = batch * q_len
    qkv = torch.randn((T, (heads + 2 * kv_heads) * head_dim), generator=g, device=device, dtype=torch.float32).bfloat16()
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=device)
    cu_q = i32([i * q_len for i in range(batch + 1)])
    seg_pos0 = i32([ctx - q_len] * batch)
    seg_kv_len = i32([ctx] * batch)
    return qkv, k_pool, v_pool, perm.contiguous(), cu_q, seg_pos0, seg_kv_len


def _time_kernels(fns, iters: int, warmup: int) -> float:
    """Mean device milliseconds of one launch: every pass runs all of ``fns`` back to back between two
    CUDA events, so launch overhead is hidden behind the queue as in a real step.  The callers make
    ``fns`` read different buffers whose total size exceeds L2, so every launch reads from HBM."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()            # one pass as a graph: no host time between the launches
    with torch.cuda.graph(graph):
        for fn in fns:
            fn()
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / (iters * len(fns))


def _copies_beyond_l2(nbytes: int, l2_bytes: int = 126 << 20) -> int:
    return max(2, min(64, (2 * l2_bytes + nbytes - 1) // max(1, nbytes)))


def kernel_attention_decode(batch=64, ctx=2048, heads=32, kv_heads=8, head_dim=128, page=16, splits=0,
                            iters=10, warmup=3) -> Dict[str, float]:
    """The split-KV decode attention kernel alone: device time and the bandwidth of the keys and values it reads."""
    from .ext import ops
    dev = torch.device("cuda:0")
    nbytes = 2 * batch * ctx * kv_heads * head_dim * 2
    group = heads // kv_heads
    n = splits or ops.decode_splits(batch * kv_heads * ((group + 15) // 16), ctx)
    segs = torch.arange(batch, dtype=torch.int32, device=dev)
    fns = []
    for _ in range(_copies_beyond_l2(nbytes)):
        qkv, k_pool, v_pool, bt, cu_q, _, seg_kv_len = _paged_case(batch, ctx, 1, heads, kv_heads, head_dim, page, dev)
        out = torch.empty((batch, heads * head_dim), dtype=torch.bfloat16, device=dev)
        fns.append(lambda a=(qkv, k_pool, v_pool, cu_q, seg_kv_len, bt, out): ops.attention_decode_mma(
            a[0], a[1], a[2], segs, a[3], a[4], a[5], page, a[6], heads, kv_heads, head_dim, head_dim ** -0.5, 0, n))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": "attention_decode", "batch": batch, "ctx": ctx, "splits": n, "ms": ms,
            "GBps": nbytes / ms / 1e6}


def kernel_attention_prefill(batch=1, ctx=2048, q_len=2048, heads=32, kv_heads=8, head_dim=128, page=16,
                             iters=10, warmup=3, impl=0, splits=0) -> Dict[str, float]:
    """The prefill attention kernel alone: device time and causal TFLOP/s.
    ``impl`` 0: the tcgen05 kernel (head sizes 64 and 128); 1: the mma.sync kernel.
    ``splits``: ways the tcgen05 kernel splits the keys (0: the engine's choice for this many CTAs)."""
    from .ext import ops
    dev = torch.device("cuda:0")
    qkv, k_pool, v_pool, bt, cu_q, seg_pos0, _ = _paged_case(batch, ctx, q_len, heads, kv_heads, head_dim, page, dev)
    out = torch.empty((batch * q_len, heads * head_dim), dtype=torch.bfloat16, device=dev)
    rows = 64 if impl else ops.TC5_TILE_ROWS
    tiles = torch.tensor([(i, r) for i in range(batch) for r in range(0, q_len, rows)], dtype=torch.int32, device=dev)
    kernel = ops.attention_prefill_mma if impl else ops.attention_prefill_tc5
    splits = splits or ops.prefill_splits(int(tiles.shape[0]) * heads, ctx)
    more = {} if impl else {"num_splits": splits, "held": {}}
    fn = lambda: kernel(qkv, k_pool, v_pool, tiles, cu_q, seg_pos0, bt, page, out, heads,
                        kv_heads, head_dim, head_dim ** -0.5, 0, **more)
    ms = _time_kernels([fn], iters, warmup)
    flops = 4.0 * batch * heads * head_dim * (q_len * (ctx - q_len) + q_len * q_len / 2.0)
    return {"kernel": "attention_prefill_mma" if impl else "attention_prefill_tc5", "batch": batch, "ctx": ctx, "q_len": q_len, "splits": 1 if impl else splits,
            "ctas": int(tiles.shape[0]) * heads, "ms": ms, "TFLOPs": flops / ms / 1e9}


def kernel_gemm(M=8, N=4096, K=4096, iters=10, warmup=3, out_f32=0, impl=0) -> Dict[str, float]:
    """A bfloat16 matrix product alone: device time, weight bandwidth and TFLOP/s.
    ``impl`` 0: ``ops.linear`` (the engine's choice); 1: the tcgen05 kernel; 2: cuBLAS (``torch.mm``);
    3: the tcgen05 weight-streaming kernel; 4: the mma.sync weight-streaming kernel; 5: the tcgen05 kernel on
    256 x 256 tiles by pairs of CTAs."""
    from .ext import ops
    dev = torch.device("cuda:0")
    fns = []
    for _ in range(_copies_beyond_l2(N * K * 2)):
        x = torch.randn((M, K), device=dev).bfloat16()
        w = torch.randn((N, K), device=dev).bfloat16()
        out = torch.empty((M, N), dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
        if impl == 1:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(*a))
        elif impl == 2:
            fns.append(lambda a=(x, w, out): torch.mm(a[0], a[1].t(), out=a[2]))
        elif impl == 3:
            fns.append(lambda a=(x, w, out): ops.gemm_stream(*a))
        elif impl == 4:
            fns.append(lambda a=(x, w, out): ops.gemm_skinny(*a))
        elif impl == 5:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(*a, pair=True))
        else:
            fns.append(lambda a=(x, w, out): ops.linear(*a))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": ("linear", "gemm_tc5", "cublas", "gemm_stream", "gemm_skinny", "gemm_tc5_pair")[impl], "M": M, "N": N, "K": K, "ms": ms, "GBps": N * K * 2 / ms / 1e6,
            "TFLOPs": 2.0 * M * N * K / ms / 1e9}


def kernel_experts(tokens=2048, top=4, experts=32, N=3072, K=2048, iters=10, warmup=3, impl=0, pairs=0) -> Dict[str, object]:
    """The experts' product alone over (token, expert) pairs sorted by expert, the tokens choosing evenly at random:
    ``impl`` 0: the tcgen05 kernel; 1: the mma.sync tiles; 2: a pair streams its expert's rows (decoded tokens; give
    ``pairs``).  Device time, TFLOP/s, and the bandwidth of the experts' weights that the pairs reach."""
    from .ext import ops
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(3)
    n_pairs = pairs or tokens * top
    expert_of = torch.randint(0, experts, (n_pairs,), generator=g).int()
    offsets = torch.tensor([0] + torch.bincount(expert_of.long(), minlength=experts).cumsum(0).tolist(), dtype=torch.int32).to(dev)
    order = expert_of.sort(stable=True).indices.int().to(dev)
    expert_dev = expert_of.to(dev)
    reached = int(expert_of.unique().numel())
    fns = []
    for _ in range(_copies_beyond_l2(experts * N * K * 2)):
        x = torch.randn((n_pairs, K), device=dev).bfloat16()
        w = (torch.randn((experts, N, K), device=dev) * K ** -0.5).bfloat16()
        out = torch.empty((n_pairs, N), dtype=torch.bfloat16, device=dev)
        if impl == 0:
            fns.append(lambda a=(x, w, out): ops.moe_tc5_gemm(a[0], a[1], offsets, a[2]))
        elif impl == 1:
            fns.append(lambda a=(x, w, out): ops.moe_grouped_gemm(a[0], order, 1, a[1], offsets, a[2]))
        else:
            fns.append(lambda a=(x, w, out): ops.moe_pair_linear(a[0], 1, a[1], expert_dev, a[2]))
    ms = _time_kernels(fns, iters, warmup)
    ops.check_status(dev)
    return {"kernel": ("moe_tc5", "moe_grouped_mma", "moe_pair_linear")[impl], "pairs": n_pairs, "experts": experts,
            "experts_reached": reached, "N": N, "K": K, "ms": ms, "TFLOPs": 2.0 * n_pairs * N * K / ms / 1e9,
            "GBps_of_reached_weights": reached * N * K * 2 / ms / 1e6}


def kernel_elementwise(rows=2048, hidden=4096, intermediate=12288, iters=10, warmup=3) -> Dict[str, object]:
    """The residual add + RMSNorm kernel and the SwiGLU kernel alone, over buffers larger than L2: device time and
    the bandwidth of what each must read and write (norm: stream in and out in float32, delta in, normed rows out;
    SwiGLU: [rows, 2 I] in, [rows, I] out)."""
    from .ext import ops
    dev = torch.device("cuda:0")
    w = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    norm_bytes = rows * hidden * (4 + 4 + 2 + 2)
    fns = []
    for _ in range(_copies_beyond_l2(norm_bytes)):
        stream = torch.randn(rows, hidden, device=dev)
        delta = torch.randn(rows, hidden, device=dev).bfloat16()
        out = torch.empty(rows, hidden, device=dev, dtype=torch.bfloat16)
        fns.append(lambda a=(stream, delta, out): ops.add_rmsnorm(a[0], a[1], w, 1e-6, a[2]))
    ms_norm = _time_kernels(fns, iters, warmup)
    act_bytes = rows * intermediate * 3 * 2
    fns = []
    for _ in range(_copies_beyond_l2(act_bytes)):
        gu = torch.randn(rows, 2 * intermediate, device=dev).bfloat16()
        out = torch.empty(rows, intermediate, device=dev, dtype=torch.bfloat16)
        fns.append(lambda a=(gu, out): ops.swiglu(a[0], a[1], 8))
    ms_act = _time_kernels(fns, iters, warmup)
    return {"rows": rows, "add_rmsnorm": {"ms": ms_norm, "GBps": norm_bytes / ms_norm / 1e6},
            "swiglu": {"ms": ms_act, "GBps": act_bytes / ms_act / 1e6}}


def kernel_gated(M=2048, I=12288, K=4096, iters=10, warmup=3, impl=0) -> Dict[str, float]:
    """The gated feed-forward product out = silu(x Wg^T) * (x Wu^T) alone.  ``impl`` 0: the engine's
    choice (``ops.gated_linear``); 1: the tcgen05 kernel with the SwiGLU epilogue; 2: cuBLAS + the SwiGLU kernel;
    3: the tcgen05 kernel by pairs of CTAs with the SwiGLU epilogue."""
    from .ext import ops
    dev = torch.device("cuda:0")
    fns = []
    for _ in range(_copies_beyond_l2(2 * I * K * 2)):
        x = torch.randn((M, K), device=dev).bfloat16()
        w = torch.randn((2 * I, K), device=dev).bfloat16()
        out = torch.empty((M, I), dtype=torch.bfloat16, device=dev)
        gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device=dev)
        if impl == 1:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(a[0], a[1], a[2], gated=True))
        elif impl == 3:
            fns.append(lambda a=(x, w, out): ops.gemm_tc5(a[0], a[1], a[2], gated=True, pair=True))
        elif impl == 2:
            def two(a=(x, w, out, gu)):
                torch.mm(a[0], a[1].t(), out=a[3])
                ops.swiglu(a[3], a[2], 8)
            fns.append(two)
        else:
            fns.append(lambda a=(x, w, out): ops.gated_linear(a[0], a[1], a[2], 8))
    ms = _time_kernels(fns, iters, warmup)
    return {"kernel": ("gated_linear", "gemm_tc5_gated", "cublas+swiglu", "gemm_tc5_pair_gated")[impl], "M": M, "I": I, "K": K, "ms": ms,
            "TFLOPs": 4.0 * M * I * K / ms / 1e9}


# ------------------------------------------------------------------------------- named workloads through the engine

WORKLOADS = {
    # 64 requests with prompt lengths uniform in [16, 4096], prompts in portions of 512 tokens beside decodes
    "0.6b-mixed": dict(
        model=dict(vocab_size=151936, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28,
                   num_attention_heads=16, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=40960),
        seed=5, requests=64, prompt=(16, 4096), new=128, chunk=512, max_reside=64, ctx=8192),
    # 16 requests with 2,048-token prompts, then 256 decoded tokens each
    "32b": dict(
        model=dict(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                   num_attention_heads=64, num_key_value_heads=8, head_dim=128, rope_theta=1000000.0,
                   rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960),
        seed=6, requests=16, prompt=(2048, 2048), new=256, chunk=8192, max_reside=16, ctx=8192),
}


def run_workload(name: str, layers: int = 0, new: int = 0) -> Dict[str, object]:
    """One of the named workloads through ``Engine.generate`` (scheduler, portions, decode, sampling off: greedy):
    wall time, tokens per second of the whole job and of its decode steps.  ``layers`` / ``new``: fewer layers or
    fewer new tokens than the workload names, where time needs it (both are reported)."""
    import time
    from .config.model_config import Qwen3Config
    from .engine.config import EngineConfig
    from .engine.engine import Engine
    from .engine.request import Request
    from .engine.runner import ModelRunner
    w = WORKLOADS[name]
    raw = dict(w["model"])
    full_layers = raw["num_hidden_layers"]
    if layers:
        raw["num_hidden_layers"] = layers
    cfg = Qwen3Config.from_dict(raw)
    n_new = new or w["new"]
    gen = torch.Generator().manual_seed(w["seed"])
    lo, hi = w["prompt"]
    lens = [int(torch.randint(lo, hi + 1, (1,), generator=gen)) for _ in range(w["requests"])]
    pool = sum((n + n_new + 63) // 64 * 64 for n in lens) + 1024
    ecfg = EngineConfig(max_token=pool, max_reside=w["max_reside"], page_size=16, prefill_chunk=w["chunk"], dtype="bfloat16",
                        max_model_len=w["ctx"], use_cuda_graph=True, capture_at_start=True, seed=w["seed"])
    runner = ModelRunner.from_random(cfg, ecfg, seed=w["seed"])
    engine = Engine(runner)
    reqs = [Request(f"w{i}", _random_ids(cfg.vocab_size, n, gen), max_new_tokens=n_new, temperature=0.0) for i, n in enumerate(lens)]
    # start-up, untimed: the engine has captured its decode graphs (as the reference's build_graph does);
    # one short request goes through prefill and a few decode steps
    engine.generate([_random_ids(cfg.vocab_size, 64, gen)], max_new_tokens=4, temperature=0.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = engine.generate(reqs)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = engine.stats()
    return {"workload": name, "layers": cfg.num_hidden_layers, "full_layers": full_layers, "requests": len(reqs),
            "prompt_tokens": sum(lens), "new_tokens": sum(r.num_tokens for r in out), "seconds": round(dt, 3),
            "tokens_per_s": round((sum(lens) + sum(r.num_tokens for r in out)) / dt, 1),
            "generated_per_s": round(sum(r.num_tokens for r in out) / dt, 1),
            "steps": st["steps"], "preemptions": st["preemptions"], "decode_tps": st.get("decode_tps"),
            "prefill_tps": st.get("prefill_tps"), "decode_graphs": len(runner._graphs)}


def kernel_scan(mode=0, batch=1, tokens=2048, heads=16, kv_heads=0, dim=128, vdim=128, iters=10, warmup=3) -> Dict[str, object]:
    """The recurrence kernel of the mixers with a matrix state alone: ``batch`` segments of ``tokens`` tokens each
    (tokens = 1: a decode step).  mode 0: fixed decay, 1: matrix memory, 2: delta rule, 3: row decays with a bonus, 4: state
    space.  Reports the time of a launch,
    the float32 operations per second, and the bandwidth on the states (each read and written once)."""
    from types import SimpleNamespace
    from .ext import ops
    dev = torch.device("cuda:0")
    G = kv_heads or heads
    T = batch * tokens
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
    unit = lambda x, n: torch.nn.functional.normalize(x.view(T, -1, n), dim=-1).reshape(T, -1)
    q, k, v = unit(rnd(T, G * dim), dim), unit(rnd(T, G * dim), dim), rnd(T, heads * vdim)
    pad = (dim + 7) // 8 * 8
    s_floats = heads * pad * vdim
    n_off, m_off = s_floats, s_floats + heads * pad
    copies = max(1, _copies_beyond_l2(batch * (m_off + heads) * 4)) if tokens == 1 else 1
    states = [torch.zeros((batch, m_off + heads), device=dev) for _ in range(copies)]
    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)
    b = SimpleNamespace(cu_q=i32([i * tokens for i in range(batch + 1)]), seg_slot=i32(list(range(batch))), num_segments=batch)
    if mode == ops.SCAN_DECAY:
        ga, gb = torch.linspace(0.97, 0.999, heads, device=dev), None
    elif mode == ops.SCAN_MEMORY:
        ga, gb = rnd(T, 2 * heads), torch.zeros(2 * heads, device=dev)
    elif mode == ops.SCAN_SSM:
        ga, gb = torch.sigmoid(rnd(T, heads) + 3.0).contiguous(), torch.sigmoid(rnd(T, heads)).contiguous()
    else:
        ga, gb = torch.sigmoid(rnd(T, heads * dim) + 3.0).contiguous(), torch.sigmoid(rnd(T, heads)).contiguous()
    extra = None
    if mode == ops.SCAN_BONUS:
        gb, extra = None, rnd(heads * dim)
    elif mode == ops.SCAN_SSM:
        extra = rnd(heads)
    out = torch.empty((T, heads * vdim), device=dev)
    fns = [(lambda st=st: ops.linear_scan(mode, q, k, v, ga, gb, st, (0, n_off, m_off), b, out, heads, G, dim, vdim,
                                          q_scale=dim ** -0.5 if mode < ops.SCAN_BONUS else 1.0, cap=15.0, extra=extra))
           for st in states]
    ms = _time_kernels(fns, iters, warmup)
    flops = T * heads * dim * vdim * (6.0 if mode == ops.SCAN_DELTA else 4.0)
    return {"kernel": "linear_scan", "mode": mode, "batch": batch, "tokens": tokens, "heads": heads, "dim": dim, "vdim": vdim,
            "ms": round(ms, 4), "ns_per_token": round(ms * 1e6 / tokens, 1), "tflops_f32": round(flops / ms / 1e9, 3),
            "state_gbs": round(2.0 * batch * s_floats * 4 / ms / 1e6, 1)}


# ------------------------------------------------------------------------------- two designs at equal layer sizes

# Layer sizes that resemble real models: (width, feed-forward, heads of 128).  Every fourth layer of the Pisatar model
# is the sum of attention and matrix memory, the one before it the delta rule, the others retention.
DESIGN_SIZES = {
    "1k": dict(width=1024, ff=3072, heads=8, kv_heads=2, layers=8, vocab=32768),
    "2k": dict(width=2048, ff=6144, heads=16, kv_heads=4, layers=8, vocab=32768),
    "4k": dict(width=4096, ff=12288, heads=32, kv_heads=8, layers=4, vocab=32768),
}


def pisatar_raw_config(width: int, ff: int, heads: int, kv_heads: int, layers: int, vocab: int) -> dict:
    """A Pisatar configuration whose mixers carry as many heads of 128 as the attention of a Qwen3 model of this width."""
    mlp = {"kind": "dense", "ff": ff}
    retention = {"type": "retention", "mlp": mlp,
                 "mixer": {"heads": heads, "dim": 128, "vdim": 128, "rot": {"base": 1e6, "dims": 128},
                           "decay": [1.0 - 2.0 ** -(5 + 4 * i / max(1, heads - 1)) for i in range(heads)]}}
    delta = {"type": "channel_delta", "mlp": mlp,
             "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}}
    both = {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                               "rot": {"base": 1e4, "dims": 64,
                                       "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 2048}}},
                      "right": {"heads": heads // 2, "dim": 128, "vdim": 256, "gate_cap": 15.0},
                      "left_scale": 1.0, "right_scale": 1.0}}
    pattern = [retention, retention, delta, both]
    return {"architecture": "Pisatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [pattern[i % 4] for i in range(layers)]}


def step_kernel_times(fn, steps: int) -> Dict[str, float]:
    """Device milliseconds per call of ``fn`` by kernel name (torch.profiler, CUDA activity only)."""
    from collections import defaultdict
    from torch.profiler import ProfilerActivity, profile
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA], record_shapes=False) as prof:
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
    out = defaultdict(float)
    for e in prof.key_averages():
        us = getattr(e, "self_device_time_total", 0) or getattr(e, "self_cuda_time_total", 0)
        if us > 0:
            out[e.key] += us / 1e3 / steps
    return dict(out)


def _kernel_ms(times: Dict[str, float], *needles: str) -> float:
    return sum(ms for name, ms in times.items() if any(n in name for n in needles))


def measure_design(cfg, tokens: int, batch: int, steps: int, warmup: int, page: int = 16) -> Dict[str, object]:
    """Prefill of one prompt of ``tokens`` and decode steps of ``batch`` requests behind prompts of ``tokens``, with the
    device time of each by kernel."""
    from .engine.config import EngineConfig
    from .engine.runner import ModelRunner
    pool = batch * ((tokens + 2 * (warmup + steps) + 64 + 63) // 64 * 64) + 2 * tokens
    ecfg = EngineConfig(max_token=pool, max_reside=batch + 1, page_size=page, prefill_chunk=8192, dtype="bfloat16",
                        max_model_len=tokens + 2 * (warmup + steps) + 64, use_cuda_graph=True, seed=4)
    runner = ModelRunner.from_random(cfg, ecfg, seed=4)
    pf = prefill_throughput(runner, tokens, iters=max(3, steps // 8), warmup=3)
    gen = torch.Generator().manual_seed(7)

    def one_prefill():
        runner.add_request("p")
        runner.step([runner.reserve("p", _random_ids(runner.vocab_size, tokens, gen), [tokens - 1])])
        runner.free_request("p")
    pf_kernels = step_kernel_times(one_prefill, 2)
    dec = decode_throughput(runner, batch, tokens, steps, warmup)
    rids = fill_requests(runner, batch, tokens, prefix="k")
    toks = _random_ids(runner.vocab_size, batch, gen)

    def one_decode():
        runner.step([runner.reserve(rid, [toks[i]], [0]) for i, rid in enumerate(rids)])
    for _ in range(3):
        one_decode()
    dec_kernels = step_kernel_times(one_decode, 8)
    for rid in rids:
        runner.free_request(rid)
    del runner
    torch.cuda.empty_cache()
    top = lambda d: {k[:60]: round(v, 4) for k, v in sorted(d.items(), key=lambda kv: -kv[1])[:8]}
    return {"prefill_tokens_per_s": round(pf["tokens_per_s"], 1), "prefill_ms": round(pf["ms"], 3),
            "decode_tokens_per_s": round(dec["tokens_per_s"], 1), "decode_ms": round(dec["ms_per_step"], 4),
            "prefill_kernels": pf_kernels, "decode_kernels": dec_kernels,
            "prefill_top": top(pf_kernels), "decode_top": top(dec_kernels)}


def compare_designs(size: str, tokens: int, batch: int, steps: int, warmup: int, hbm_gbs: float, bf16_tflops: float):
    """The Pisatar design beside the Qwen3 decoder at equal width, feed-forward, layer count and heads: throughput of
    both, and how far the kernel that mixes tokens is from its roofline in each (the scan over matrix states against
    the attention over cached keys).  Rooflines: decode kernels against the copy bandwidth (the state read and written
    once, the keys and values read once); prefill kernels against the tensor peak for the attention (causal half of
    4 T^2 heads dim) and against the same peak for the scan (4 to 6 T heads dim vdim, which the scan runs in float32
    on the CUDA cores)."""
    from .config.model_config import Qwen3Config
    from .config.pisatar_config import PisatarConfig
    sz = DESIGN_SIZES[size]
    W, ff, H, G, L, V = sz["width"], sz["ff"], sz["heads"], sz["kv_heads"], sz["layers"], sz["vocab"]
    new = measure_design(PisatarConfig(pisatar_raw_config(W, ff, H, G, L, V)), tokens, batch, steps, warmup)
    old = measure_design(Qwen3Config.from_dict(dict(vocab_size=V, hidden_size=W, intermediate_size=ff, num_hidden_layers=L,
                                                    num_attention_heads=H, num_key_value_heads=G, head_dim=128,
                                                    rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                                    max_position_embeddings=32768)), tokens, batch, steps, warmup)
    D = 128
    n_ret, n_delta, n_both = (L + 3) // 4 + (L + 2) // 4, (L + 1) // 4, L // 4
    state_bytes = 4 * D * (n_ret * H * 128 + n_delta * H * 128 + n_both * (H // 2) * 256)      # per request, all layers
    scan_flops = tokens * D * (4.0 * n_ret * H * 128 + 6.0 * n_delta * H * 128 + 4.0 * n_both * (H // 2) * 256)
    kv_bytes = lambda layers: 2 * 2 * G * D * tokens * batch * layers
    attn_flops = lambda layers: 4.0 * tokens * tokens * H * D / 2 * layers
    scan_dec = _kernel_ms(new["decode_kernels"], "linear_scan")
    scan_pf = _kernel_ms(new["prefill_kernels"], "linear_scan")
    att_dec_new = _kernel_ms(new["decode_kernels"], "attn_decode", "attn_combine")
    att_dec_old = _kernel_ms(old["decode_kernels"], "attn_decode", "attn_combine")
    att_pf_new = _kernel_ms(new["prefill_kernels"], "attn_prefill", "attention_tc5", "tc5_merge")
    att_pf_old = _kernel_ms(old["prefill_kernels"], "attn_prefill", "attention_tc5", "tc5_merge")
    frac = lambda work, ms, peak: round(work / (ms * 1e-3) / peak, 4) if ms > 0 else None
    kernels = {
        "decode_scan": {"ms": round(scan_dec, 4), "of_hbm": frac(2.0 * state_bytes * batch, scan_dec, hbm_gbs * 1e9)},
        "decode_attention_pisatar": {"ms": round(att_dec_new, 4), "of_hbm": frac(kv_bytes(n_both), att_dec_new, hbm_gbs * 1e9)},
        "decode_attention_qwen3": {"ms": round(att_dec_old, 4), "of_hbm": frac(kv_bytes(L), att_dec_old, hbm_gbs * 1e9)},
        "prefill_scan": {"ms": round(scan_pf, 4), "of_bf16_peak": frac(scan_flops, scan_pf, bf16_tflops * 1e12)},
        "prefill_attention_pisatar": {"ms": round(att_pf_new, 4), "of_bf16_peak": frac(attn_flops(n_both), att_pf_new, bf16_tflops * 1e12)},
        "prefill_attention_qwen3": {"ms": round(att_pf_old, 4), "of_bf16_peak": frac(attn_flops(L), att_pf_old, bf16_tflops * 1e12)},
    }
    for r in (new, old):
        del r["prefill_kernels"], r["decode_kernels"]
    return {"size": size, "width": W, "ff": ff, "heads": H, "kv_heads": G, "layers": L, "tokens": tokens, "batch": batch,
            "pisatar": new, "qwen3": old, "kernels": kernels}


def gonozen_raw_config(width: int, ff: int, heads: int, layers: int, vocab: int, window: int = 1024) -> dict:
    """A Gonozen configuration at the layer sizes of a Qwen3 model of this width: heads of 128, every third layer windowed
    (latent of 128 numbers, no positions), the others with a latent of 192 and a rotated part of 64; 32 experts of a
    quarter of the dense feed-forward each, four of them a token (of the four best of eight groups), so that a token's
    experts do the work of the dense feed-forward, and a shared expert of the same size beside them."""
    mlp = {"kind": "moe", "router": {"experts": 32, "top": 4, "groups": {"count": 8, "keep": 4}},
           "expert": {"ff": ff // 4, "limit": 7.0}, "shared": {"ff": ff // 4, "limit": 7.0}}
    rotated = {"type": "latent_attention", "mlp": mlp,
               "mixer": {"heads": heads, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 192, "scale": 128 ** -0.5,
                         "rot": {"base": 1e4, "dims": 64, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
    windowed = {"type": "latent_attention_2", "mlp": mlp,
                "mixer": {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": 128, "q_rank": max(128, width // 4),
                          "scale": 128 ** -0.5, "mask": {"size": window}}}
    pattern = [windowed, rotated, rotated]
    return {"architecture": "Gonozen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [pattern[i % 3] for i in range(layers)]}


def compare_gonozen(size: str, tokens: int, batch: int, steps: int, warmup: int, hbm_gbs: float, bf16_tflops: float):
    """The Gonozen design beside the Qwen3 decoder at equal width, layer count and heads, the experts that a token uses
    as large together as the dense feed-forward: throughput of both, and how far the kernels of the new mechanisms are
    from their rooflines beside the like kernels of the Qwen3 model.  Rooflines: attention over decoded tokens against
    the copy bandwidth (every cached vector of the visible keys read once); attention over a prompt against the tensor
    peak, counting what the kernel computes (scores and weighted means over the cached vector's width for the latents,
    over the head size for Qwen3; the causal half, or the window's band); the experts' products of a prompt against the
    tensor peak beside the dense gated product and its down projection; the experts' products of decoded tokens against
    the copy bandwidth (each pair's expert read once) beside the dense feed-forward's weights read once."""
    from .config.gonozen_config import GonozenConfig
    from .config.model_config import Qwen3Config
    sz = DESIGN_SIZES[size]
    W, ff, H, G, L, V = sz["width"], sz["ff"], sz["heads"], sz["kv_heads"], sz["layers"], sz["vocab"]
    raw = gonozen_raw_config(W, ff, H, L, V)
    new = measure_design(GonozenConfig(raw), tokens, batch, steps, warmup)
    old = measure_design(Qwen3Config.from_dict(dict(vocab_size=V, hidden_size=W, intermediate_size=ff, num_hidden_layers=L,
                                                    num_attention_heads=H, num_key_value_heads=G, head_dim=128,
                                                    rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False,
                                                    max_position_embeddings=32768)), tokens, batch, steps, warmup)
    frac = lambda work, ms, peak: round(work / (ms * 1e-3) / peak, 4) if ms > 0 else None
    lat_bytes = 0.0
    lat_flops = {"tcgen05": 0.0, "mma_sync": 0.0}          # by the kernel that a cached vector's width runs on
    for layer in raw["layers"]:
        m = layer["mixer"]
        width = (m["kv_rank"] + m.get("rot_dim", 0) + 15) // 16 * 16
        window = m.get("mask", {}).get("size")
        seen = min(tokens, window) if window else tokens
        lat_bytes += 2.0 * width * seen * batch
        keys = tokens * tokens / 2 if not window or window >= tokens else tokens * window - window * window / 2
        head = (max(m["dim"] + m.get("rot_dim", 0), m["vdim"]) + 15) // 16 * 16
        if head in (64, 128) and head < width:             # a prompt runs with keys and values written out per head
            lat_flops["tcgen05"] += 4.0 * keys * H * head
        else:
            lat_flops["tcgen05" if width in (64, 128) else "mma_sync"] += 4.0 * keys * H * width
    mlp = raw["layers"][0]["mlp"]
    F, top = mlp["expert"]["ff"], mlp["router"]["top"]
    moe_flops = L * 2.0 * tokens * top * 3 * F * W
    E = mlp["router"]["experts"]
    distinct = E * (1.0 - (1.0 - 1.0 / E) ** (batch * top))     # experts that a step's pairs reach, if they chose evenly
    moe_bytes = L * 2.0 * distinct * 3 * F * W
    dense_flops, dense_bytes = L * 2.0 * tokens * 3 * ff * W, L * 2.0 * 3 * ff * W
    D = 128
    k_new, k_old = new["prefill_kernels"], old["prefill_kernels"]
    d_new, d_old = new["decode_kernels"], old["decode_kernels"]
    att = ("attn_prefill", "merge_key_splits")
    att_tc5, att_mma = ("attn_prefill_tc5", "merge_key_splits"), ("attn_prefill_kernel",)
    dec = ("attn_decode", "attn_combine")
    ff_old_pf = sum(ms for name, ms in k_old.items() if ms >= sorted(k_old.values())[-3] and not any(n in name for n in att))
    kernels = {
        "decode_attention_latents": {"ms": round(_kernel_ms(d_new, *dec), 4), "of_hbm": frac(lat_bytes, _kernel_ms(d_new, *dec), hbm_gbs * 1e9)},
        "decode_attention_qwen3": {"ms": round(_kernel_ms(d_old, *dec), 4),
                                   "of_hbm": frac(2.0 * 2 * G * D * tokens * batch * L, _kernel_ms(d_old, *dec), hbm_gbs * 1e9)},
        "prefill_attention_written_out": {"ms": round(_kernel_ms(k_new, "latent_expand", "latent_gather", "latent_take"), 4),
                                          "note": "gather, scatter and take-values kernels of the expanded form; its product is a library kernel"},
        "prefill_attention_latents_of_128_tcgen05": {"ms": round(_kernel_ms(k_new, *att_tc5), 4),
                                                     "of_bf16_peak": frac(lat_flops["tcgen05"], _kernel_ms(k_new, *att_tc5), bf16_tflops * 1e12)},
        "prefill_attention_latents_of_256_mma_sync": {"ms": round(_kernel_ms(k_new, *att_mma), 4),
                                                      "of_bf16_peak": frac(lat_flops["mma_sync"], _kernel_ms(k_new, *att_mma), bf16_tflops * 1e12)},
        "prefill_attention_qwen3": {"ms": round(_kernel_ms(k_old, *att), 4),
                                    "of_bf16_peak": frac(4.0 * tokens * tokens / 2 * H * D * L, _kernel_ms(k_old, *att), bf16_tflops * 1e12)},
        "prefill_experts": {"ms": round(_kernel_ms(k_new, "moe_grouped_gemm", "moe_tc5"), 4),
                            "of_bf16_peak": frac(moe_flops, _kernel_ms(k_new, "moe_grouped_gemm", "moe_tc5"), bf16_tflops * 1e12)},
        "prefill_dense_feed_forward_qwen3": {"ms": round(ff_old_pf, 4), "of_bf16_peak": frac(dense_flops, ff_old_pf, bf16_tflops * 1e12),
                                             "note": "the three largest kernels of the step beside the attention: the gated product and the down projection among them"},
        "decode_experts": {"ms": round(_kernel_ms(d_new, "moe_pair_linear", "moe_grouped_gemm"), 4),
                           "of_hbm": frac(moe_bytes, _kernel_ms(d_new, "moe_pair_linear", "moe_grouped_gemm"), hbm_gbs * 1e9)},
        "decode_weight_streaming_qwen3": {"ms": round(_kernel_ms(d_old, "gemm_skinny"), 4),
                                          "of_hbm": frac(dense_bytes + L * 2.0 * W * (H + 2 * G + H) * D, _kernel_ms(d_old, "gemm_skinny"), hbm_gbs * 1e9)},
    }
    for r in (new, old):
        del r["prefill_kernels"], r["decode_kernels"]
    return {"size": size, "width": W, "ff": ff, "heads": H, "layers": L, "tokens": tokens, "batch": batch,
            "experts": mlp["router"], "expert_ff": F, "gonozen": new, "qwen3": old, "kernels": kernels}


def nozizen_raw_config(width: int, ff: int, heads: int, kv_heads: int, layers: int, vocab: int, window: int = 1024,
                       streams: int = 4) -> dict:
    """A Nozizen configuration whose mixers carry as many heads of 128 as the attention of a Qwen3 model of this width:
    of every four layers the first is a time mix (states of 128 x 128), the next two state-space mixers (a state of 128
    rows for a head's 128 values, ``kv_heads`` groups, four taps), the fourth a windowed attention (rotation over half a
    head, stretched); the first and third feed-forwards are dense, the others 32 experts of a quarter of the dense size
    each, four of them a token, so that a token's experts do the dense feed-forward's work."""
    dense = {"kind": "dense", "ff": ff}
    experts = {"kind": "moe", "router": {"experts": 32, "top": 4}, "expert": {"ff": ff // 4}}
    time_mix = {"type": "wkv", "mixer": {"heads": heads, "dim": 128, "decay_rank": 64}}
    space = {"type": "mamba2", "mixer": {"heads": heads, "vdim": 128, "state": 128, "groups": kv_heads, "conv": 4,
                                         "norm_groups": kv_heads}}
    attention = {"type": "attention",
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                           "mask": {"size": window},
                           "rot": {"base": 1e4, "dims": 64, "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}}
    pattern = [(time_mix, dense), (space, experts), (space, dense), (attention, experts)]
    return {"architecture": "Nozizen", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": float(width) ** 0.5}, "streams": streams,
            "layers": [dict(pattern[i % 4][0], mlp=pattern[i % 4][1]) for i in range(layers)]}


def compare_nozizen(size: str, tokens: int, batch: int, steps: int, warmup: int, hbm_gbs: float, bf16_tflops: float):
    """The Nozizen design beside the Pisatar decoder (the nearest the engine has: state mixers on the same scan kernel,
    a softmax attention, dense feed-forwards) at equal width, feed-forward, layer count and heads: throughput of both,
    and how far the kernels of each mechanism are from their rooflines beside the like kernels of the other model.
    Rooflines: the scan over decoded tokens against the copy bandwidth (every state read and written once); the scan
    over a prompt against the tensor peak (4 T heads dim vdim operations, as for the Pisatar row, although the scan
    runs in float32 on the CUDA cores); attention over decoded tokens against the copy bandwidth (the keys and values
    the window shows read once); attention over a prompt against the tensor peak (the causal half, or the window's
    band); the kernels that read and write the residual streams against the copy bandwidth (each stream read and
    written once a sublayer, beside Pisatar's add-and-norm kernel over its one stream); the experts' products of a
    prompt against the tensor peak and of decoded tokens against the copy bandwidth (each reached expert read once)."""
    from .config.nozizen_config import NozizenConfig
    from .config.pisatar_config import PisatarConfig
    sz = DESIGN_SIZES[size]
    W, ff, H, G, L, V = sz["width"], sz["ff"], sz["heads"], sz["kv_heads"], sz["layers"], sz["vocab"]
    raw = nozizen_raw_config(W, ff, H, G, L, V)
    new = measure_design(NozizenConfig(raw), tokens, batch, steps, warmup)
    old = measure_design(PisatarConfig(pisatar_raw_config(W, ff, H, G, L, V)), tokens, batch, steps, warmup)
    D, S = 128, raw["streams"]
    kinds = [layer["type"] for layer in raw["layers"]]
    n_state, n_att = kinds.count("wkv") + kinds.count("mamba2"), kinds.count("attention")
    n_moe = sum(1 for layer in raw["layers"] if layer["mlp"]["kind"] == "moe")
    window = raw["layers"][3]["mixer"]["mask"]["size"] if L > 3 else tokens
    seen = min(tokens, window)
    frac = lambda work, ms, peak: round(work / (ms * 1e-3) / peak, 4) if ms > 0 else None
    state_bytes_new = 4.0 * D * D * H * n_state
    scan_flops_new = 4.0 * tokens * D * D * H * n_state
    o_ret, o_delta, o_both = (L + 3) // 4 + (L + 2) // 4, (L + 1) // 4, L // 4
    state_bytes_old = 4.0 * D * (o_ret * H * 128 + o_delta * H * 128 + o_both * (H // 2) * 256)
    scan_flops_old = tokens * D * (4.0 * o_ret * H * 128 + 6.0 * o_delta * H * 128 + 4.0 * o_both * (H // 2) * 256)
    band = tokens * tokens / 2 if window >= tokens else tokens * window - window * window / 2
    F, top, E = ff // 4, 4, 32
    distinct = E * (1.0 - (1.0 - 1.0 / E) ** (batch * top))
    k_new, k_old, d_new, d_old = new["prefill_kernels"], old["prefill_kernels"], new["decode_kernels"], old["decode_kernels"]
    att_pf, att_dec = ("attn_prefill", "attention_tc5", "merge_key_splits", "tc5_merge"), ("attn_decode", "attn_combine")
    hyper = ("hyper_read_norm", "hyper_write")
    moe_pf, moe_dec = ("moe_grouped_gemm", "moe_tc5"), ("moe_pair_linear", "moe_grouped_gemm")
    small = ("token_shift_mix", "ssm_prep", "conv_state_update", "gated_part_norm", "head_norm_gate", "activation_kernel",
             "clamped_glu", "moe_combine", "moe_route", "moe_sort", "moe_gather")
    hbm, peak = hbm_gbs * 1e9, bf16_tflops * 1e12
    row = lambda times, names, work, roof, key: {"ms": round(_kernel_ms(times, *names), 4), key: frac(work, _kernel_ms(times, *names), roof)}
    kernels = {
        "decode_scan_nozizen": row(d_new, ("linear_scan",), 2.0 * state_bytes_new * batch, hbm, "of_hbm"),
        "decode_scan_pisatar": row(d_old, ("linear_scan",), 2.0 * state_bytes_old * batch, hbm, "of_hbm"),
        "prefill_scan_nozizen": row(k_new, ("linear_scan",), scan_flops_new, peak, "of_bf16_peak"),
        "prefill_scan_pisatar": row(k_old, ("linear_scan",), scan_flops_old, peak, "of_bf16_peak"),
        "decode_attention_nozizen": row(d_new, att_dec, 2.0 * 2 * G * D * seen * batch * n_att, hbm, "of_hbm"),
        "decode_attention_pisatar": row(d_old, att_dec, 2.0 * 2 * G * D * tokens * batch * o_both, hbm, "of_hbm"),
        "prefill_attention_nozizen": row(k_new, att_pf, 4.0 * band * H * D * n_att, peak, "of_bf16_peak"),
        "prefill_attention_pisatar": row(k_old, att_pf, 4.0 * tokens * tokens / 2 * H * D * o_both, peak, "of_bf16_peak"),
        # a sublayer's write does the next read as well: S streams of float32 read and written once, the sublayer's
        # output read and the next normed rows written (the first layer's own read comes to one sublayer in 2 L)
        "prefill_streams_nozizen": row(k_new, hyper, 2 * L * tokens * W * (2.0 * S * 4 + 2 * 2), hbm, "of_hbm"),
        "prefill_add_norm_pisatar": row(k_old, ("add_dual_norm",), L * tokens * W * (2.0 * 4 + 2 * 2 + 2 * 2), hbm, "of_hbm"),
        "prefill_experts_nozizen": row(k_new, moe_pf, n_moe * 2.0 * tokens * top * 3 * F * W, peak, "of_bf16_peak"),
        "decode_experts_nozizen": row(d_new, moe_dec, n_moe * 2.0 * distinct * 3 * F * W, hbm, "of_hbm"),
        "prefill_small_kernels_nozizen": {"ms": round(_kernel_ms(k_new, *small), 4),
                                          "note": "blends, convolution, gates and norms around the scans, the activation, the experts' helpers"},
        "decode_streams_nozizen": {"ms": round(_kernel_ms(d_new, *hyper), 4)},
        "decode_small_kernels_nozizen": {"ms": round(_kernel_ms(d_new, *small), 4)},
    }
    for r in (new, old):
        del r["prefill_kernels"], r["decode_kernels"]
    return {"size": size, "width": W, "ff": ff, "heads": H, "kv_heads": G, "layers": L, "tokens": tokens, "batch": batch,
            "streams": S, "window": window, "nozizen": new, "pisatar": old, "kernels": kernels}


def duvadra_raw_config(width: int, ff: int, heads: int, kv_heads: int, layers: int, vocab: int, window: int = 1024,
                       block: int = 8192) -> dict:
    """A Duvadra configuration whose mixers carry as many heads of 128 as the attention of a Qwen3 model of this width: of
    every four layers the first is an attention inside blocks of ``block`` positions (soft cap, distance slopes, a gate a
    head), the second a windowed attention whose values are its keys (rotation over half a head) beside a gated linear
    recurrence as wide as the model in blocks of 128, the third a block attention on the first layer's keys and values,
    the fourth a windowed attention with a sink beside a gated delta rule (states of 128 x 128, four taps); the first and
    fourth feed-forwards are capped gated units, the others 32 experts of a quarter of the dense size each in 8 groups of
    which 4 are kept, four experts a token, so that a token's experts do the dense feed-forward's work."""
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    experts = {"kind": "moe", "router": {"experts": 32, "top": 4, "scale": 2.0, "groups": {"count": 8, "keep": 4}},
               "expert": {"ff": ff // 4}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5}
    blocks = {"type": "attention", "mixer": dict(att, softcap=40.0, mask={"size": block})}
    lru = {"type": "parallel_2", "mixer": {"left": dict(att, mask={"size": window}, rot={"base": 1e4, "dims": 64}),
                                           "right": {"width": width, "blocks": max(1, width // 128), "conv": 4},
                                           "left_scale": 0.6, "right_scale": 0.9}}
    delta = {"type": "parallel", "mixer": {"left": dict(att, mask={"size": window}),
                                           "right": {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "conv": 4},
                                           "left_scale": 0.9, "right_scale": 0.6}}
    out = []
    for i in range(layers):
        k = i % 4
        if k == 0:
            out.append(dict(blocks, mlp=dense))
        elif k == 1:
            out.append(dict(lru, mlp=experts))
        elif k == 2:
            out.append({"type": "attention", "mixer": dict(blocks["mixer"], kv_from=i - 2), "mlp": experts})
        else:
            out.append(dict(delta, mlp=dense))
    return {"architecture": "Duvadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "logit_softcap": 20.0, "embedding": {"scale": 2.0, "bigram": {"buckets": 65521, "mul_prev": 1009, "mul_cur": 31}},
            "layers": out}


def compare_duvadra(size: str, tokens: int, batch: int, steps: int, warmup: int, hbm_gbs: float, bf16_tflops: float):
    """The Duvadra design beside the Nozizen decoder (the nearest the engine has: a windowed attention, state mixers on
    the scan kernel, capped or plain gated units beside experts) at equal width, feed-forward, layer count and heads:
    throughput of both, and how far the kernels of each mechanism are from their rooflines beside the like kernels of the
    other model.  Rooflines: the scan and the channel recurrence over decoded tokens against the copy bandwidth (every
    state read and written once); the scan over a prompt against the tensor peak (6 T heads dim vdim operations for the
    delta rule, 4 for Nozizen's, although the scans run in float32 on the CUDA cores); the channel recurrence over a
    prompt against the copy bandwidth (inputs, two gate rows in float32 and the gate branch read, the output written);
    attention over decoded tokens against the copy bandwidth (the keys and values a query sees read once); attention over
    a prompt against the tensor peak (the causal half, or the window's band), the block attention (the kernels with the
    score options) and the windowed ones (the plain kernel) apart; the kernels that add to the residual stream and norm it against the copy
    bandwidth; the experts' products of a prompt against the tensor peak and of decoded tokens against the copy bandwidth
    (each reached expert read once)."""
    from .config.duvadra_config import DuvadraConfig
    from .config.nozizen_config import NozizenConfig
    sz = DESIGN_SIZES[size]
    W, ff, H, G, L, V = sz["width"], sz["ff"], sz["heads"], sz["kv_heads"], sz["layers"], sz["vocab"]
    raw = duvadra_raw_config(W, ff, H, G, L, V)
    new = measure_design(DuvadraConfig(raw), tokens, batch, steps, warmup)
    old_raw = nozizen_raw_config(W, ff, H, G, L, V)
    old = measure_design(NozizenConfig(old_raw), tokens, batch, steps, warmup)
    D = 128
    kinds = [layer["type"] for layer in raw["layers"]]
    n_blocks, n_lru, n_delta = kinds.count("attention"), kinds.count("parallel_2"), kinds.count("parallel")
    n_moe = sum(1 for layer in raw["layers"] if layer["mlp"]["kind"] == "moe")
    window = 1024
    seen = min(tokens, window)
    band = tokens * tokens / 2 if window >= tokens else tokens * window - window * window / 2
    o_kinds = [layer["type"] for layer in old_raw["layers"]]
    o_state, o_att = o_kinds.count("wkv") + o_kinds.count("mamba2"), o_kinds.count("attention")
    o_moe = sum(1 for layer in old_raw["layers"] if layer["mlp"]["kind"] == "moe")
    S = old_raw["streams"]
    F, top, E = ff // 4, 4, 32
    distinct = E * (1.0 - (1.0 - 1.0 / E) ** (batch * top))
    frac = lambda work, ms, peak: round(work / (ms * 1e-3) / peak, 4) if ms > 0 else None
    k_new, k_old, d_new, d_old = new["prefill_kernels"], old["prefill_kernels"], new["decode_kernels"], old["decode_kernels"]
    att_dec = ("attn_decode", "attn_combine")
    moe_pf, moe_dec = ("moe_grouped_gemm", "moe_tc5"), ("moe_pair_linear", "moe_grouped_gemm")
    small = ("attn_prep", "attn_gate", "gated_conv", "conv_state_update", "delta_prep", "head_norm_gate", "scaled_sum",
             "clamped_glu", "moe_combine", "moe_route", "moe_sort", "moe_gather", "embedding_pair", "last_token")
    hbm, peak = hbm_gbs * 1e9, bf16_tflops * 1e12
    row = lambda times, names, work, roof, key: {"ms": round(_kernel_ms(times, *names), 4), key: frac(work, _kernel_ms(times, *names), roof)}
    kernels = {
        "decode_scan_duvadra": row(d_new, ("linear_scan",), 2.0 * 4 * D * D * H * n_delta * batch, hbm, "of_hbm"),
        "decode_scan_nozizen": row(d_old, ("linear_scan",), 2.0 * 4 * D * D * H * o_state * batch, hbm, "of_hbm"),
        "prefill_scan_duvadra": row(k_new, ("linear_scan",), 6.0 * tokens * D * D * H * n_delta, peak, "of_bf16_peak"),
        "prefill_scan_nozizen": row(k_old, ("linear_scan",), 4.0 * tokens * D * D * H * o_state, peak, "of_bf16_peak"),
        "decode_recurrence_duvadra": row(d_new, ("gated_recurrence",), n_lru * batch * W * (2.0 * 4 + 2 + 8 + 2 + 2), hbm, "of_hbm"),
        "prefill_recurrence_duvadra": row(k_new, ("gated_recurrence", "gated_pieces_combine"), n_lru * tokens * W * (2.0 + 8 + 2 + 2), hbm, "of_hbm"),
        "decode_attention_duvadra": row(d_new, att_dec, 2.0 * 2 * G * D * batch * (tokens * n_blocks + seen * (n_lru + n_delta)), hbm, "of_hbm"),
        "decode_attention_nozizen": row(d_old, att_dec, 2.0 * 2 * G * D * seen * batch * o_att, hbm, "of_hbm"),
        "prefill_attention_blocks_duvadra": row(k_new, ("attn_prefill_kernel", "attn_prefill_tc5_kernel<true>"), 4.0 * tokens * tokens / 2 * H * D * n_blocks, peak, "of_bf16_peak"),
        "prefill_attention_window_duvadra": row(k_new, ("attn_prefill_tc5_kernel<false>", "merge_key_splits", "tc5_merge"), 4.0 * band * H * D * (n_lru + n_delta), peak, "of_bf16_peak"),
        "prefill_attention_nozizen": row(k_old, ("attn_prefill", "attention_tc5", "merge_key_splits", "tc5_merge"), 4.0 * band * H * D * o_att, peak, "of_bf16_peak"),
        # every sublayer: the float32 stream read and written, the sublayer's output read (float32 from the mixers,
        # bfloat16 from the feed-forwards), the normed rows written
        "prefill_add_norm_duvadra": row(k_new, ("add_dual_norm",), L * tokens * W * (2.0 * 2 * 4 + 4 + 2 + 2 * 2), hbm, "of_hbm"),
        "prefill_streams_nozizen": row(k_old, ("hyper_read_norm", "hyper_write"), 2 * L * tokens * W * (2.0 * S * 4 + 2 * 2), hbm, "of_hbm"),
        "prefill_experts_duvadra": row(k_new, moe_pf, n_moe * 2.0 * tokens * top * 3 * F * W, peak, "of_bf16_peak"),
        "prefill_experts_nozizen": row(k_old, moe_pf, o_moe * 2.0 * tokens * top * 3 * F * W, peak, "of_bf16_peak"),
        "decode_experts_duvadra": row(d_new, moe_dec, n_moe * 2.0 * distinct * 3 * F * W, hbm, "of_hbm"),
        "decode_experts_nozizen": row(d_old, moe_dec, o_moe * 2.0 * distinct * 3 * F * W, hbm, "of_hbm"),
        "prefill_small_kernels_duvadra": {"ms": round(_kernel_ms(k_new, *small), 4),
                                          "note": "row preparation and gates of the attentions, convolutions, the delta rule's "
                                                  "preparation, norms behind the scans, the experts' helpers, the embedding"},
        "decode_small_kernels_duvadra": {"ms": round(_kernel_ms(d_new, *small), 4)},
        "decode_add_norm_duvadra": {"ms": round(_kernel_ms(d_new, "add_dual_norm"), 4)},
    }
    for r in (new, old):
        del r["prefill_kernels"], r["decode_kernels"]
    return {"size": size, "width": W, "ff": ff, "heads": H, "kv_heads": G, "layers": L, "tokens": tokens, "batch": batch,
            "window": window, "block": 8192, "duvadra": new, "nozizen": old, "kernels": kernels}
