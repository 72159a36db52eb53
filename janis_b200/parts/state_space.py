"""State-space mixers: the selective scan with a state per channel, and its state-space-duality form with a
scalar decay per head.

Both run the same recurrence over C channels with N states each, per sequence and token t:

    S[c, n] <- exp(delta[c] A[c, n]) S[c, n] + delta[c] u[c] B[n],      o[c] = sum_n S[c, n] C[n] + D[c] u[c]

`SelectiveScanMixer` (y is the mixer's input, `inner` channels):
    [u | z] = W_in y;  u = silu(conv(u));  [lo | B | C] = W_x u;  delta = softplus(W_dt lo + b_dt) per channel;
    A = -exp(A_log) [inner, N];  out = W_o (o * silu(z)).

`DualityMixer` (H heads of P channels, G groups of B and C; a head uses group h // (H / G)):
    [z | u | B | C | dt] = W_in y;  (u, B, C) = silu(conv(u | B | C));  delta = softplus(dt + dt_bias) per head;
    A = -exp(A_log) per head;  D per head;  out = W_o (rms_parts(o * silu(z)) * w_norm), the RMS norm taken over
    `norm_groups` equal parts of the H P channels, after the gate.

The convolution is causal and per channel (`taps` weights, the last one the current token's, zeros before the
sequence's start).  A cache line holds two fixed-size parts per sequence: the state S [C, N] in float32 and the
last taps - 1 inputs of the convolution; a step loads them, runs its tokens in order and writes them back, so a
prompt, a prompt that continues and a decode step are one code path.  delta, the decays, the state and o are
float32 whatever the projections are stored in.
"""
from __future__ import annotations

import torch

from ..cache.cache import StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext


def _conv_need(taps: int, channels: int) -> StateNeed:
    return StateNeed((max(taps - 1, 1), channels), torch.float32)


class SelectiveScanMixer(Mixer):
    NAMES = ("in", "conv", "conv_bias", "x", "dt", "dt_bias", "A_log", "D", "o")

    def __init__(self, hidden: int, inner: int, state: int, dt_rank: int, taps: int, names: dict[str, str],
                 init_std: float = 0.02):
        for k in self.NAMES:
            if k not in names:
                raise ValueError(f"the selective scan needs the checkpoint name of its {k!r} tensor")
        if not 1 <= taps <= 16:
            raise ValueError(f"the convolution kernel takes 1 to 16 taps, found {taps}")
        if state > 512:
            raise ValueError(f"the scan kernel takes up to 512 states a channel, found {state}")
        self.hidden, self.inner, self.state, self.dt_rank, self.taps = hidden, inner, state, dt_rank, taps
        self.names = dict(names)
        self.init_std = init_std
        self.w_in = self.w_conv = self.b_conv = self.w_x = self.w_dt = self.b_dt = None
        self.A = self.D = self.w_o = None

    def tensor_specs(self):
        W, C, N, R, s, n = self.hidden, self.inner, self.state, self.dt_rank, self.init_std, self.names
        return {n["in"]: TensorSpec((2 * C, W), init_std=s), n["conv"]: TensorSpec((C, self.taps), init_std=0.3),
                n["conv_bias"]: TensorSpec((C,), init_std=0.1), n["x"]: TensorSpec((R + 2 * N, C), init_std=s),
                n["dt"]: TensorSpec((C, R), init_std=R ** -0.5), n["dt_bias"]: TensorSpec((C,), init_std=1.0, init_mean=-2.0),
                n["A_log"]: TensorSpec((C, N), init_std=0.5), n["D"]: TensorSpec((C,), init_std=0.5, init_mean=1.0),
                n["o"]: TensorSpec((W, C), init_std=s)}

    def cache_needs(self):
        return {"state": StateNeed((self.inner, self.state), torch.float32), "conv": _conv_need(self.taps, self.inner)}

    def prompt_flops(self, n_tokens: int) -> float:
        return 6.0 * self.inner * self.state * n_tokens + 2.0 * self.inner * self.taps * n_tokens

    def load(self, store, rt: Runtime):
        n, R = self.names, self.dt_rank
        f32 = lambda k: store.get(n[k]).to(torch.float32).contiguous()
        self.w_in = store.get(n["in"], rt.dtype).contiguous()
        self.w_conv, self.b_conv = f32("conv"), f32("conv_bias")
        self.w_x = store.get(n["x"], rt.dtype).contiguous()                    # rows lo | B | C
        # W_dt reads the first R columns of W_x's output; widened with zero columns it reads the whole row, so that
        # the row needs no copy (a product with zero adds exactly nothing)
        w_dt = store.get(n["dt"], rt.dtype)
        self.w_dt = torch.cat([w_dt, torch.zeros((self.inner, 2 * self.state), dtype=w_dt.dtype, device=w_dt.device)],
                              dim=1).contiguous()
        del w_dt
        store.drop(n["dt"])
        self.b_dt = f32("dt_bias")
        self.A = (-torch.exp(f32("A_log"))).contiguous()
        self.D = f32("D")
        self.w_o = store.get(n["o"], rt.dtype).contiguous()

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        st, cv = line["state"], line["conv"]
        if not st.write:
            raise ValueError("a recurrent state has one writer: a scan layer cannot read another's line")
        T, C, N, R = ctx.n_tok, self.inner, self.state, self.dt_rank
        uz = rt.linear(x, self.w_in, ws.buf("ssm.in", (T, 2 * C), rt.dtype))
        u = ws.buf("ssm.u", (T, C), rt.dtype)
        ops.causal_conv_silu(uz, 0, C, self.w_conv, self.b_conv, cv.data, ctx.tok_seq, ctx.seq_slot, ctx.seq_first_row,
                             ctx.seq_start, ctx.seq_end, ctx.n_seq, u, one_token=ctx.mode == "decode")
        xp = rt.linear(u, self.w_x, ws.buf("ssm.x", (T, R + 2 * N), rt.dtype))          # lo | B | C
        dt = rt.linear(xp, self.w_dt, ws.buf("ssm.dt", (T, C), rt.dtype))
        y = ws.buf("ssm.y", (T, C), rt.dtype)
        ops.selective_scan(u, 0, dt, 0, self.b_dt, self.A, True, xp, R, R + N, self.D, uz, C, ctx.seq_slot,
                           ctx.seq_first_row, ctx.seq_start, ctx.seq_end, ctx.n_seq, st.data, y, C, N, 1, C,
                           scratch=ws.buf("scan.steps", (ops.selective_scan_scratch_floats(T, C),), torch.float32))
        return rt.linear(y, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))


class DualityMixer(Mixer):
    NAMES = ("in", "conv", "conv_bias", "dt_bias", "A_log", "D", "norm", "o")

    def __init__(self, hidden: int, n_heads: int, head_dim: int, state: int, groups: int, norm_groups: int, taps: int,
                 norm_eps: float, names: dict[str, str], init_std: float = 0.02):
        for k in self.NAMES:
            if k not in names:
                raise ValueError(f"the state-space-duality mixer needs the checkpoint name of its {k!r} tensor")
        if n_heads % groups:
            raise ValueError(f"{n_heads} heads do not divide over {groups} groups")
        if (n_heads * head_dim) % norm_groups:
            raise ValueError(f"{n_heads * head_dim} channels do not divide into {norm_groups} parts")
        if not 1 <= taps <= 16:
            raise ValueError(f"the convolution kernel takes 1 to 16 taps, found {taps}")
        if state > 512:
            raise ValueError(f"the scan kernel takes up to 512 states a channel, found {state}")
        self.hidden, self.n_heads, self.head_dim, self.state = hidden, n_heads, head_dim, state
        self.groups, self.norm_groups, self.taps, self.norm_eps = groups, norm_groups, taps, float(norm_eps)
        self.inner = n_heads * head_dim
        self.conv_channels = self.inner + 2 * groups * state
        self.names = dict(names)
        self.init_std = init_std
        self.w_in = self.w_conv = self.b_conv = self.b_dt = self.A = self.D = self.w_norm = self.w_o = None

    def tensor_specs(self):
        W, C, H, s, n = self.hidden, self.inner, self.n_heads, self.init_std, self.names
        return {n["in"]: TensorSpec((C + self.conv_channels + H, W), init_std=s),
                n["conv"]: TensorSpec((self.conv_channels, self.taps), init_std=0.3),
                n["conv_bias"]: TensorSpec((self.conv_channels,), init_std=0.1),
                n["dt_bias"]: TensorSpec((H,), init_std=1.0, init_mean=-1.0), n["A_log"]: TensorSpec((H,), init_std=0.5),
                n["D"]: TensorSpec((H,), init_std=0.5, init_mean=1.0), n["norm"]: TensorSpec((C,), init_std=0.1, init_mean=1.0),
                n["o"]: TensorSpec((W, C), init_std=s)}

    def cache_needs(self):
        return {"state": StateNeed((self.inner, self.state), torch.float32),
                "conv": _conv_need(self.taps, self.conv_channels)}

    def prompt_flops(self, n_tokens: int) -> float:
        return 6.0 * self.inner * self.state * n_tokens + 2.0 * self.conv_channels * self.taps * n_tokens

    def load(self, store, rt: Runtime):
        n = self.names
        f32 = lambda k: store.get(n[k]).to(torch.float32).contiguous()
        self.w_in = store.get(n["in"], rt.dtype).contiguous()
        self.w_conv, self.b_conv = f32("conv"), f32("conv_bias")
        self.b_dt = f32("dt_bias")
        self.A = (-torch.exp(f32("A_log"))).contiguous()
        self.D = f32("D")
        self.w_norm = f32("norm")
        self.w_o = store.get(n["o"], rt.dtype).contiguous()

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        st, cv = line["state"], line["conv"]
        if not st.write:
            raise ValueError("a recurrent state has one writer: a scan layer cannot read another's line")
        T, C, N, H, P, G = ctx.n_tok, self.inner, self.state, self.n_heads, self.head_dim, self.groups
        CC = self.conv_channels
        rows = rt.linear(x, self.w_in, ws.buf("ssd.in", (T, C + CC + H), rt.dtype))        # z | u | B | C | dt
        ubc = ws.buf("ssd.ubc", (T, CC), rt.dtype)
        ops.causal_conv_silu(rows, C, CC, self.w_conv, self.b_conv, cv.data, ctx.tok_seq, ctx.seq_slot,
                             ctx.seq_first_row, ctx.seq_start, ctx.seq_end, ctx.n_seq, ubc, one_token=ctx.mode == "decode")
        o = ws.buf("ssd.o", (T, C), torch.float32)
        ops.selective_scan(ubc, 0, rows, C + CC, self.b_dt, self.A, False, ubc, C, C + G * N, self.D, None, 0,
                           ctx.seq_slot, ctx.seq_first_row, ctx.seq_start, ctx.seq_end, ctx.n_seq, st.data, o, C, N, P,
                           (H // G) * P, scratch=ws.buf("scan.steps", (ops.selective_scan_scratch_floats(T, H),), torch.float32))
        y = ws.buf("ssd.y", (T, C), rt.dtype)
        ops.gate_group_norm(o, rows, 0, self.w_norm, self.norm_eps, self.norm_groups, y)
        return rt.linear(y, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
