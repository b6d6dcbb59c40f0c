"""Mixers that keep a matrix state per head and request instead of cached keys: retention (a fixed decay a
head), the gated delta rule with a decay per key channel, and the matrix memory with exponential gates.

All three are "product, recurrence, product": the input projections are one matrix product (their weights
concatenated at load), the recurrence runs in float32 whatever the activation type (``csrc/recurrent.cu``: one
kernel walks every segment of the step token by token, so prompts, portions and single tokens are one path and a
token's result does not depend on the cutting), the read-out is normed per head, gated and projected out.

A request's state is one float32 row of its slot (``StateNeed``): the matrices S [heads, key rows in groups of 8,
value dim, 8] first, then what else the mixer carries (conv inputs; normaliser and running maximum).  A slot is
zeroed when a request takes it, which is every part's starting state.
"""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import torch

from ..ext import ops
from .base import MIXERS, POSITION_ENCODINGS, Mixer, ParamSpec, StateNeed


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class _StateMixer(Mixer):
    """What the three share: sizes, the state row's layout, buffers."""

    def _sizes(self):
        s = self.spec
        self.H, self.D, self.V = s.num_heads, s.key_dim, s.value_dim
        if self.D > ops.SCAN_MAX_KEY_DIM:
            raise ValueError(f"key_dim={self.D}: the scan kernel holds up to {ops.SCAN_MAX_KEY_DIM} key rows a head")
        self.s_floats = self.H * _pad8(self.D) * self.V

    def out_projection(self):
        return self.p_o

    # A segment of at least this many tokens is cut into pieces that are scanned side by side (bfloat16 path only:
    # the sums then take another order than token by token, which the float32 path never does).
    PIECES_MIN_TOKENS = 1024
    PIECE_MIN_TOKENS = 128

    def _pieces(self, batch):
        """None, or (a batch whose segments are the pieces, first piece of every segment, number of pieces) when the
        step holds a long segment and its CTAs alone would leave most SMs idle.  Worked out once per step."""
        host = getattr(batch, "host", None)
        if host is None or not getattr(host, "num_multi", 0):
            return None
        memo = getattr(batch, "scratch", None)
        key = ("state_mixer.pieces.plan", self.H, self.V)
        if memo is not None and key in memo:
            return memo[key]
        plan = None
        lens = np.diff(host.cu_q).astype(np.int64)
        if int(lens.max()) >= self.PIECES_MIN_TOKENS:
            ctas = self.H * ((self.V + 31) // 32)
            want = (2 * ops.num_sms()) // max(1, ctas * int((lens >= self.PIECES_MIN_TOKENS).sum()))
            if want >= 3:                                   # two passes over the tokens: fewer pieces would not pay
                cuts, first = [0], [0]
                for start, n in zip(host.cu_q[:-1], lens):
                    k = int(min(want, max(1, n // self.PIECE_MIN_TOKENS))) if n >= self.PIECES_MIN_TOKENS else 1
                    edges = [int(start) + (int(n) * i) // k for i in range(1, k + 1)]
                    cuts.extend(edges)
                    first.append(first[-1] + k)
                n_pieces = len(cuts) - 1
                tables = torch.from_numpy(np.asarray(cuts + first + list(range(n_pieces)), np.int32)).to(
                    self.env.device, non_blocking=True)
                a, c = len(cuts), len(cuts) + len(first)
                virtual = SimpleNamespace(cu_q=tables[:a], seg_slot=tables[c:], num_segments=n_pieces)
                plan = (virtual, tables[a:c], n_pieces)
        if memo is not None:
            memo[key] = plan
        return plan


    def _scan(self, mode, q, k, v, decay, step, ctx, out, groups, extra, by_row, pieces):
        """The scan of a mixer whose decays differ from token to token (per head, or per head and key row with
        ``by_row``).  With ``pieces`` the long segments are scanned in pieces side by side: every piece from zero, the
        states handed on in order (a piece's transition is the product of its tokens' decays), every piece again."""
        b = ctx.batch
        if pieces is None:
            ops.linear_scan(mode, q, k, v, decay, step, ctx.state, (0, 0, 0), b, out, self.H, groups, self.D, self.V, extra=extra)
            return
        virtual, seg_first, n_pieces = pieces
        dev = out.device
        held = ctx.buffer(self.spec.kind + ".pieces", (n_pieces, self.s_floats), torch.float32, dev)
        sums = ctx.buffer(self.spec.kind + ".piece_decays", (n_pieces, decay.shape[1]), torch.float32, dev)
        held.zero_()
        for again in (False, True):
            ops.linear_scan(mode, q, k, v, decay, step, held, (0, 0, 0), virtual, out, self.H, groups, self.D, self.V, extra=extra)
            if not again:
                ops.scan_pieces_combine_sums(held, ctx.state, 0, decay, sums, by_row, self.D, self.V, virtual.cu_q, seg_first,
                                             b.seg_slot, _pad8(self.D) * self.V, self.s_floats, b.num_segments)

    def _project_out(self, mixed, ctx):
        y = ctx.buffer(self.spec.kind + ".y", (mixed.shape[0], self.spec.hidden_size), torch.float32, mixed.device)
        ops.linear(mixed, self.p_o, y)
        return y


@MIXERS.register("retention")
class Retention(_StateMixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self._sizes()
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        self.position = POSITION_ENCODINGS.build(spec.position, env) if spec.position is not None else None
        if self.position is not None and not hasattr(self.position, "tables"):
            raise ValueError("retention rotates pairs of a head: the position encoding must give rotary tables")
        self._decay = None

    def params(self):
        s = self.spec
        return {"in": ParamSpec((2 * self.H * self.D + 2 * self.H * self.V, s.hidden_size)),
                "o": ParamSpec((s.hidden_size, self.H * self.V))}

    def cache_need(self):
        return StateNeed((self.s_floats,), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev = x.shape[0], x.device
        HD, HV = self.H * self.D, self.H * self.V
        proj = ctx.buffer("retention.in", (T, 2 * HD + 2 * HV), x.dtype, dev)
        ops.linear(x, self.p_in, proj)
        q32 = ctx.buffer("retention.q", (T, HD), torch.float32, dev)
        k32 = ctx.buffer("retention.k", (T, HD), torch.float32, dev)
        cos, sin, rot = self.position.tables() if self.position is not None else (None, None, 0)
        ops.rotary_to_f32(proj, 0, HD, cos, sin, rot, b.pos, q32, k32, self.H, self.D, 1.0, self.D ** -0.5)
        if self._decay is None:
            self._decay = torch.tensor(s.decay, dtype=torch.float32, device=dev)
        o = ctx.buffer("retention.o", (T, HV), torch.float32, dev)
        v = proj[:, 2 * HD:2 * HD + HV]
        pieces = self._pieces(b) if x.dtype != torch.float32 else None
        if pieces is None:
            ops.linear_scan(ops.SCAN_DECAY, q32, k32, v, self._decay, None, ctx.state, (0, 0, 0), b, o,
                            self.H, self.H, self.D, self.V)
        else:
            # long segments in pieces side by side: scan every piece from zero, hand the states on in order, scan again
            virtual, seg_first, n_pieces = pieces
            held = ctx.buffer("retention.pieces", (n_pieces, self.s_floats), torch.float32, dev)
            held.zero_()
            for _ in range(2):
                ops.linear_scan(ops.SCAN_DECAY, q32, k32, v, self._decay, None, held, (0, 0, 0), virtual, o,
                                self.H, self.H, self.D, self.V)
                if _ == 0:
                    ops.scan_pieces_combine(held, ctx.state, 0, self._decay, virtual.cu_q, seg_first, b.seg_slot,
                                            _pad8(self.D) * self.V, self.s_floats, b.num_segments)
        mixed = ctx.buffer("retention.mixed", (T, HV), x.dtype, dev)
        ops.head_norm_gate(o, proj[:, 2 * HD + HV:], None, 0, 0, s.eps, mixed, self.H, self.V)
        return self._project_out(mixed, ctx)


@MIXERS.register("channel_delta")
class ChannelDelta(_StateMixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self._sizes()
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads={s.num_heads} is not a multiple of num_kv_heads={s.num_kv_heads}")
        if not (1 <= s.conv_taps <= 33):
            raise ValueError("conv_taps: 1 to 33")
        if s.unit_eps != 1e-6:
            raise ValueError("the kernel's unit vectors use 1e-6 under the root")
        self.G = s.num_kv_heads
        self.channels = 2 * self.G * self.D + self.H * self.V
        self.conv_off = self.s_floats

    def params(self):
        s = self.spec
        C, HD, HV = self.channels, self.H * self.D, self.H * self.V
        return {"in": ParamSpec((C + s.decay_rank + s.gate_rank, s.hidden_size)),          # q, k, v, decay low rank, gate low rank
                "conv": ParamSpec((C, s.conv_taps), role="vector", init="normal:0.5"),
                "beta": ParamSpec((self.H, s.hidden_size)),
                "decay_up": ParamSpec((HD, s.decay_rank), init="normal:0.2"),
                "gate_up": ParamSpec((HV, s.gate_rank), init="normal:0.2"),
                "A_log": ParamSpec((self.H,), role="vector", init="normal:0.5"),
                "dt_bias": ParamSpec((HD,), role="vector", init="normal:0.5"),
                "norm": ParamSpec((self.V,), role="vector", init="ones_normal"),
                "o": ParamSpec((s.hidden_size, HV))}

    def cache_need(self):
        return StateNeed((self.s_floats + self.channels * (self.spec.conv_taps - 1),), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev = x.shape[0], x.device
        C, GD, HD, HV = self.channels, self.G * self.D, self.H * self.D, self.H * self.V
        proj = ctx.buffer("channel_delta.in", (T, C + s.decay_rank + s.gate_rank), x.dtype, dev)
        ops.linear(x, self.p_in, proj)
        beta = ctx.buffer("channel_delta.beta", (T, self.H), torch.float32, dev)
        ops.linear(x, self.p_beta, beta)
        decay = ctx.buffer("channel_delta.decay", (T, HD), torch.float32, dev)
        ops.linear(proj[:, C:C + s.decay_rank], self.p_decay_up, decay)
        gate = ctx.buffer("channel_delta.gate", (T, HV), x.dtype, dev)
        ops.linear(proj[:, C + s.decay_rank:], self.p_gate_up, gate)
        q32 = ctx.buffer("channel_delta.q", (T, GD), torch.float32, dev)
        k32 = ctx.buffer("channel_delta.k", (T, GD), torch.float32, dev)
        v32 = ctx.buffer("channel_delta.v", (T, HV), torch.float32, dev)
        ops.delta_prep(proj, self.p_conv, ctx.state, self.conv_off, b, q32, k32, v32, decay, self.p_A_log,
                       self.p_dt_bias, beta, self.H, self.G, self.D, self.V, self.D ** -0.5)
        ops.conv_state_update(proj, s.conv_taps, ctx.state, self.conv_off, b, C)      # after every token read the old one
        o = ctx.buffer("channel_delta.o", (T, HV), torch.float32, dev)
        ops.linear_scan(ops.SCAN_DELTA, q32, k32, v32, decay, beta, ctx.state, (0, 0, 0), b, o,
                        self.H, self.G, self.D, self.V)
        mixed = ctx.buffer("channel_delta.mixed", (T, HV), x.dtype, dev)
        ops.head_norm_gate(o, gate, self.p_norm, 1, 1, s.eps, mixed, self.H, self.V)
        return self._project_out(mixed, ctx)


@MIXERS.register("matrix_memory")
class MatrixMemory(_StateMixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self._sizes()
        if spec.gate_cap <= 0:
            raise ValueError("gate_cap must be positive")
        self.n_off = self.s_floats
        self.m_off = self.n_off + self.H * _pad8(self.D)

    def params(self):
        s = self.spec
        HD, HV = self.H * self.D, self.H * self.V
        return {"in": ParamSpec((2 * HD + 2 * HV, s.hidden_size)),                       # q, k, v, output gate
                "gates": ParamSpec((2 * self.H, s.hidden_size)),                         # input gate rows, forget gate rows
                "gate_bias": ParamSpec((2 * self.H,), role="vector", init="normal:0.5"),
                "norm": ParamSpec((HV,), role="vector", init="ones_normal"),
                "o": ParamSpec((s.hidden_size, HV))}

    def bind(self, tensors):
        super().bind(tensors)
        self._bias32 = self.p_gate_bias.float().contiguous()

    def cache_need(self):
        return StateNeed((self.m_off + self.H,), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev = x.shape[0], x.device
        HD, HV = self.H * self.D, self.H * self.V
        proj = ctx.buffer("matrix_memory.in", (T, 2 * HD + 2 * HV), x.dtype, dev)
        ops.linear(x, self.p_in, proj)
        gates = ctx.buffer("matrix_memory.gates", (T, 2 * self.H), torch.float32, dev)
        ops.linear(x, self.p_gates, gates)
        o = ctx.buffer("matrix_memory.o", (T, HV), torch.float32, dev)
        q, k, v = proj[:, :HD], proj[:, HD:2 * HD], proj[:, 2 * HD:2 * HD + HV]
        offsets = (0, self.n_off, self.m_off)
        pieces = self._pieces(b) if x.dtype != torch.float32 else None
        if pieces is None:
            ops.linear_scan(ops.SCAN_MEMORY, q, k, v, gates, self._bias32, ctx.state, offsets, b, o, self.H, self.H,
                            self.D, self.V, q_scale=self.D ** -0.5, cap=s.gate_cap)
        else:
            # long segments in pieces side by side (see Retention.forward); a piece starts from nothing, which for the
            # running maximum is minus infinity, and also leaves the sum of its log forget gates behind the maxima
            virtual, seg_first, n_pieces = pieces
            f_off = self.m_off + self.H
            held = ctx.buffer("matrix_memory.pieces", (n_pieces, f_off + self.H), torch.float32, dev)
            held.zero_()
            held[:, self.m_off:f_off].fill_(float("-inf"))
            ops.linear_scan(ops.SCAN_MEMORY, q, k, v, gates, self._bias32, held, offsets, virtual, o, self.H, self.H,
                            self.D, self.V, q_scale=self.D ** -0.5, cap=s.gate_cap, forgot_offset=f_off)
            ops.memory_pieces_combine(held, ctx.state, offsets, f_off, seg_first, b.seg_slot, _pad8(self.D) * self.V,
                                      _pad8(self.D), self.H, b.num_segments)
            ops.linear_scan(ops.SCAN_MEMORY, q, k, v, gates, self._bias32, held, offsets, virtual, o, self.H, self.H,
                            self.D, self.V, q_scale=self.D ** -0.5, cap=s.gate_cap)
        mixed = ctx.buffer("matrix_memory.mixed", (T, HV), x.dtype, dev)
        ops.head_norm_gate(o, proj[:, 2 * HD + HV:], self.p_norm, 2, 1, s.eps, mixed, self.H, self.V)
        return self._project_out(mixed, ctx)


@MIXERS.register("time_mix")
class TimeMix(_StateMixer):
    """``TimeMixSpec``: five projections of five blends of a token's input with its predecessor's, a decay per token,
    head and key row through a low rank, the scan with a bonus for the token's own pair, per-head norm, gate, output
    projection.  The request's state row holds S and then the last input it saw (zero for a new request)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        self.H, self.D, self.V = s.num_heads, s.key_dim, s.key_dim
        if self.D > ops.SCAN_MAX_KEY_DIM:
            raise ValueError(f"key_dim={self.D}: the scan kernel holds up to {ops.SCAN_MAX_KEY_DIM} key rows a head")
        if s.decay_rank <= 0:
            raise ValueError("decay_rank must be positive")
        self.s_floats = self.H * _pad8(self.D) * self.V
        self.shift_off = self.s_floats

    def params(self):
        s = self.spec
        W, HD = s.hidden_size, self.H * self.D
        return {"mu": ParamSpec((5, W), role="vector", init="uniform01"),                  # rows: r, k, v, gate, decay
                "r": ParamSpec((HD, W)), "k": ParamSpec((HD, W)), "v": ParamSpec((HD, W)), "g": ParamSpec((HD, W)),
                "decay_down": ParamSpec((s.decay_rank, W)),
                "decay_up": ParamSpec((HD, s.decay_rank), init="normal:0.2"),
                "decay_bias": ParamSpec((HD,), role="vector", init="normal:0.5"),
                "bonus": ParamSpec((self.H, self.D), role="vector", init="normal:0.5"),
                "norm": ParamSpec((HD,), role="vector", init="ones_normal"),
                "o": ParamSpec((s.hidden_size, HD))}

    def bind(self, tensors):
        super().bind(tensors)
        self._bonus32 = self.p_bonus.float().contiguous()

    def cache_need(self):
        return StateNeed((self.s_floats + self.spec.hidden_size,), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev, dt = x.shape[0], x.device, x.dtype
        W, HD = s.hidden_size, self.H * self.D
        mixes = ctx.buffer("time_mix.mixes", (5, T, W), dt, dev)
        ops.token_shift_mix(x, self.p_mu, ctx.state, self.shift_off, b, mixes)
        ops.conv_state_update(x, 2, ctx.state, self.shift_off, b, W)           # the last input, after every token read the old one
        proj = ctx.buffer("time_mix.rkvg", (4, T, HD), dt, dev)
        for i, w in enumerate((self.p_r, self.p_k, self.p_v, self.p_g)):
            ops.linear(mixes[i], w, proj[i])
        low = ctx.buffer("time_mix.low", (T, s.decay_rank), dt, dev)
        ops.linear(mixes[4], self.p_decay_down, low, act="tanh")
        decay = ctx.buffer("time_mix.decay", (T, HD), torch.float32, dev)
        ops.linear(low, self.p_decay_up, decay, act="neg_exp_exp", bias=self.p_decay_bias)
        o = ctx.buffer("time_mix.o", (T, HD), torch.float32, dev)
        self._scan(ops.SCAN_BONUS, proj[0], proj[1], proj[2], decay, None, ctx, o, self.H, self._bonus32, True,
                   self._pieces(b) if dt != torch.float32 else None)
        mixed = ctx.buffer("time_mix.mixed", (T, HD), dt, dev)
        ops.head_norm_gate(o, proj[3], self.p_norm, 2, 0, s.eps, mixed, self.H, self.V)
        return self._project_out(mixed, ctx)


@MIXERS.register("state_space")
class StateSpace(_StateMixer):
    """``StateSpaceSpec``: one projection, the convolution of its x, B and C channels, the scan with a scalar decay per
    token and head, gate, norm over equal parts, output projection.  The request's state row holds S (the state size
    as key rows, the head's values as columns) and then the last ``conv_taps - 1`` inputs of every convolved channel."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        self.H, self.D, self.V = s.num_heads, s.state_dim, s.value_dim
        if self.D > ops.SCAN_MAX_KEY_DIM:
            raise ValueError(f"state_dim={self.D}: the scan kernel holds up to {ops.SCAN_MAX_KEY_DIM} state rows a head")
        if s.groups < 1 or s.num_heads % s.groups:
            raise ValueError(f"num_heads={s.num_heads} is not a multiple of groups={s.groups}")
        self.inner = self.H * self.V
        if s.norm_groups < 1 or self.inner % s.norm_groups:
            raise ValueError(f"{self.inner} values do not form {s.norm_groups} equal parts")
        if not (1 <= s.conv_taps <= 33):
            raise ValueError("conv_taps: 1 to 33")
        self.GN = s.groups * self.D
        self.channels = self.inner + 2 * self.GN
        self.s_floats = self.H * _pad8(self.D) * self.V
        self.conv_off = self.s_floats

    def params(self):
        s = self.spec
        return {"in": ParamSpec((2 * self.inner + 2 * self.GN + self.H, s.hidden_size)),       # z, x, B, C, dt
                "conv": ParamSpec((self.channels, s.conv_taps), role="vector", init="normal:0.5"),
                "conv_bias": ParamSpec((self.channels,), role="vector", init="normal:0.2"),
                "dt_bias": ParamSpec((self.H,), role="vector", init="normal:0.5"),
                "A_log": ParamSpec((self.H,), role="vector", init="normal:0.5"),
                "D": ParamSpec((self.H,), role="vector", init="ones_normal"),
                "norm": ParamSpec((self.inner,), role="vector", init="ones_normal"),
                "o": ParamSpec((s.hidden_size, self.inner))}

    def bind(self, tensors):
        super().bind(tensors)
        self._skip32 = self.p_D.float().contiguous()

    def cache_need(self):
        return StateNeed((self.s_floats + self.channels * (self.spec.conv_taps - 1),), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev = x.shape[0], x.device
        inner, GN, C = self.inner, self.GN, self.channels
        proj = ctx.buffer("state_space.in", (T, 2 * inner + 2 * GN + self.H), x.dtype, dev)
        ops.linear(x, self.p_in, proj)
        conv = ctx.buffer("state_space.conv", (T, C), torch.float32, dev)
        step = ctx.buffer("state_space.dt", (T, self.H), torch.float32, dev)
        decay = ctx.buffer("state_space.decay", (T, self.H), torch.float32, dev)
        ops.ssm_prep(proj, inner, C, self.p_conv, self.p_conv_bias, ctx.state, self.conv_off, b, conv, inner + C, self.H,
                     self.p_dt_bias, self.p_A_log, step, decay)
        ops.conv_state_update(proj[:, inner:], s.conv_taps, ctx.state, self.conv_off, b, C)   # after every token read the old one
        y = ctx.buffer("state_space.y", (T, inner), torch.float32, dev)
        self._scan(ops.SCAN_SSM, conv[:, inner + GN:], conv[:, inner:inner + GN], conv[:, :inner], decay, step, ctx, y,
                   s.groups, self._skip32, False, self._pieces(b) if x.dtype != torch.float32 else None)
        mixed = ctx.buffer("state_space.mixed", (T, inner), x.dtype, dev)
        ops.gated_part_norm(y, proj[:, :inner], self.p_norm, s.norm_groups, s.eps, mixed)
        return self._project_out(mixed, ctx)


@MIXERS.register("gated_delta")
class GatedDelta(_StateMixer):
    """``GatedDeltaSpec``: the delta rule with one decay a head.  The request's state row holds S and then the last
    ``conv_taps - 1`` inputs of every convolved channel."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self._sizes()
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads={s.num_heads} is not a multiple of num_kv_heads={s.num_kv_heads}")
        if not (1 <= s.conv_taps <= 33):
            raise ValueError("conv_taps: 1 to 33")
        if s.unit_eps != 1e-6:
            raise ValueError("the kernel's unit vectors use 1e-6 under the root")
        self.G = s.num_kv_heads
        self.channels = 2 * self.G * self.D + self.H * self.V
        self.conv_off = self.s_floats

    def params(self):
        s = self.spec
        C, HV = self.channels, self.H * self.V
        return {"in": ParamSpec((C + HV, s.hidden_size)),                                 # q, k, v, output gate
                "conv": ParamSpec((C, s.conv_taps), role="vector", init="normal:0.5"),
                "beta": ParamSpec((self.H, s.hidden_size)),
                "decay": ParamSpec((self.H, s.hidden_size)),
                "A_log": ParamSpec((self.H,), role="vector", init="normal:0.5"),
                "dt_bias": ParamSpec((self.H,), role="vector", init="normal:0.5"),
                "norm": ParamSpec((self.V,), role="vector", init="ones_normal"),
                "o": ParamSpec((s.hidden_size, HV))}

    def cache_need(self):
        return StateNeed((self.s_floats + self.channels * (self.spec.conv_taps - 1),), torch.float32)

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev = x.shape[0], x.device
        C, GD, HV = self.channels, self.G * self.D, self.H * self.V
        proj = ctx.buffer("gated_delta.in", (T, C + HV), x.dtype, dev)
        ops.linear(x, self.p_in, proj)
        beta = ctx.buffer("gated_delta.beta", (T, self.H), torch.float32, dev)
        ops.linear(x, self.p_beta, beta)
        decay = ctx.buffer("gated_delta.decay", (T, self.H), torch.float32, dev)
        ops.linear(x, self.p_decay, decay)
        q32 = ctx.buffer("gated_delta.q", (T, GD), torch.float32, dev)
        k32 = ctx.buffer("gated_delta.k", (T, GD), torch.float32, dev)
        v32 = ctx.buffer("gated_delta.v", (T, HV), torch.float32, dev)
        ops.delta_prep(proj, self.p_conv, ctx.state, self.conv_off, b, q32, k32, v32, decay, self.p_A_log,
                       self.p_dt_bias, beta, self.H, self.G, self.D, self.V, self.D ** -0.5, head_decay=True)
        ops.conv_state_update(proj, s.conv_taps, ctx.state, self.conv_off, b, C)      # after every token read the old one
        o = ctx.buffer("gated_delta.o", (T, HV), torch.float32, dev)
        ops.linear_scan(ops.SCAN_DELTA_HEAD, q32, k32, v32, decay, beta, ctx.state, (0, 0, 0), b, o,
                        self.H, self.G, self.D, self.V)
        mixed = ctx.buffer("gated_delta.mixed", (T, HV), x.dtype, dev)
        ops.head_norm_gate(o, proj[:, C:], self.p_norm, 1, 0, s.eps, mixed, self.H, self.V)
        return self._project_out(mixed, ctx)


@MIXERS.register("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """``GatedLinearRecurrenceSpec``: one product gives [y | x]; a kernel convolves x over time (reading the request's
    held inputs before the step's first token); two batched products over the blocks give the gates' pre-activations in
    float32; a kernel walks every segment token by token, one thread a channel, and leaves s * gelu_tanh(y); the
    output projection follows.  The request's state row holds s [width] and then the last ``conv_taps - 1`` inputs of
    every channel (kept without their bias)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.blocks < 1 or s.width % s.blocks:
            raise ValueError(f"width={s.width} does not form {s.blocks} equal blocks")
        if not (1 <= s.conv_taps <= 33):
            raise ValueError("conv_taps: 1 to 33")
        self.W, self.bs = s.width, s.width // s.blocks
        self.conv_off = self.W

    def params(self):
        s = self.spec
        W, B, bs = self.W, s.blocks, self.bs
        return {"in": ParamSpec((2 * W, s.hidden_size)),                                  # y rows, then x rows
                "in_bias": ParamSpec((2 * W,), role="vector", init="normal:0.2"),
                "conv": ParamSpec((W, s.conv_taps), role="vector", init="normal:0.5"),
                "conv_bias": ParamSpec((W,), role="vector", init="normal:0.2"),
                "gate_r": ParamSpec((B, bs, bs), init="fan_in"), "gate_i": ParamSpec((B, bs, bs), init="fan_in"),
                "gate_r_bias": ParamSpec((B, bs), role="vector", init="normal:0.5"),
                "gate_i_bias": ParamSpec((B, bs), role="vector", init="normal:0.5"),
                "lam": ParamSpec((W,), role="vector", init="normal:0.5"),
                "o": ParamSpec((s.hidden_size, W))}

    def bind(self, tensors):
        super().bind(tensors)
        # the small vectors share one type, whatever the file stores each in
        dt = torch.float32 if any(tensors[n].dtype == torch.float32 for n in
                                  ("in_bias", "conv", "conv_bias", "gate_r_bias", "gate_i_bias", "lam")) else self.env.act_dtype
        for n in ("in_bias", "conv", "conv_bias", "gate_r_bias", "gate_i_bias", "lam"):
            setattr(self, "p_" + n, tensors[n].to(dt).contiguous())

    def cache_need(self):
        return StateNeed((self.W + self.W * (self.spec.conv_taps - 1),), torch.float32)

    def out_projection(self):
        return self.p_o

    # A segment of at least PIECES_MIN_TOKENS tokens is cut into pieces of about PIECE_TOKENS that are walked side by
    # side (bfloat16 path only: the sums then take another order than token by token, which the float32 path never does).
    PIECES_MIN_TOKENS = 256
    PIECE_TOKENS = 64

    def _pieces(self, batch):
        """None, or (a batch whose segments are the pieces, first piece of every segment, number of pieces) when the step
        holds a long segment.  Worked out once per step from the host tables."""
        host = getattr(batch, "host", None)
        if host is None or not getattr(host, "num_multi", 0):
            return None
        memo = getattr(batch, "scratch", None)
        key = "gated_linear_recurrence.pieces.plan"
        if memo is not None and key in memo:
            return memo[key]
        plan = None
        lens = np.diff(host.cu_q).astype(np.int64)
        if int(lens.max()) >= self.PIECES_MIN_TOKENS:
            cuts, first = [0], [0]
            for start, n in zip(host.cu_q[:-1], lens):
                k = int(max(1, n // self.PIECE_TOKENS)) if n >= self.PIECES_MIN_TOKENS else 1
                cuts.extend(int(start) + (int(n) * i) // k for i in range(1, k + 1))
                first.append(first[-1] + k)
            n_pieces = len(cuts) - 1
            tables = torch.from_numpy(np.asarray(cuts + first + list(range(n_pieces)), np.int32)).to(self.env.device, non_blocking=True)
            a, c = len(cuts), len(cuts) + len(first)
            plan = (SimpleNamespace(cu_q=tables[:a], seg_slot=tables[c:], num_segments=n_pieces), tables[a:c], n_pieces)
        if memo is not None:
            memo[key] = plan
        return plan

    def forward(self, x, ctx):
        s, b = self.spec, ctx.batch
        T, dev, dt = x.shape[0], x.device, x.dtype
        W, B, bs = self.W, s.blocks, self.bs
        proj = ctx.buffer("gated_linear_recurrence.in", (T, 2 * W), dt, dev)
        ops.linear(x, self.p_in, proj)
        u = ctx.buffer("gated_linear_recurrence.u", (T, W), dt, dev)
        ops.gated_conv(proj[:, W:], self.p_in_bias[W:], self.p_conv, self.p_conv_bias, ctx.state, self.conv_off, b, u)
        ops.conv_state_update(proj[:, W:], s.conv_taps, ctx.state, self.conv_off, b, W)  # after every token read the old one
        gates = ctx.buffer("gated_linear_recurrence.gates", (2, B, T, bs), torch.float32, dev)
        ub = u.view(T, B, bs).transpose(0, 1)
        ops.linear_heads(ub, self.p_gate_r, gates[0])
        ops.linear_heads(ub, self.p_gate_i, gates[1])
        mixed = ctx.buffer("gated_linear_recurrence.mixed", (T, W), dt, dev)
        args = (u, gates, bs, self.p_gate_r_bias, self.p_gate_i_bias, self.p_lam, float(s.decay_scale), proj, self.p_in_bias[:W])
        pieces = self._pieces(b) if dt != torch.float32 else None
        if pieces is None:
            ops.gated_recurrence(*args, ctx.state, 0, b, mixed)
        else:
            # every piece from zero, the states handed on in order (a piece's transition is the product of its tokens'
            # factors), every piece again from the state it starts with
            virtual, seg_first, n_pieces = pieces
            held = ctx.buffer("gated_linear_recurrence.pieces", (n_pieces, W), torch.float32, dev)
            sums = ctx.buffer("gated_linear_recurrence.piece_decays", (n_pieces, W), torch.float32, dev)
            held.zero_()
            ops.gated_recurrence(*args, held, 0, virtual, mixed, log_decay=sums)
            ops.gated_pieces_combine(held, sums, ctx.state, 0, seg_first, b.seg_slot, b.num_segments)
            ops.gated_recurrence(*args, held, 0, virtual, mixed)
        y = ctx.buffer("gated_linear_recurrence.y", (T, s.hidden_size), torch.float32, dev)
        ops.linear(mixed, self.p_o, y)
        return y
