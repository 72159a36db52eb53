"""Gated linear attention: a recurrent mixer whose state is a matrix per head.

With y the mixer's input, per head (d key channels, dv value channels):

    q = Wq y * q_scale,   k = Wk y,   v = Wv y
    a = sigmoid(Wa2 (Wa1 y) + b)^(1/tau)              a decay per key channel, through a low-rank projection
    S <- diag(a) S + k v^T,   o = S^T q               S starts at zero and lives in the cache, in float32

then each head's o is RMS-normed over its dv channels (one weight vector for all heads), the heads are put side by
side, multiplied by silu(Wg y) and projected by Wo.  Four projections of y are one product over the rows
q | k | v | g concatenated at load; the decay logits are two small products of their own.  Decays (from the
logits on), the state and o are float32 whatever the activations are.

The state is a fixed-size part of a cache line (`StateNeed`, stored as S^T: [heads, dv, d]): a step loads it, runs its tokens in order and
writes it back, so a prompt, a prompt that continues and a decode step are one code path; sequences without a
slot (padding) start from zero and store nothing.
"""
from __future__ import annotations

import torch

from ..cache.cache import StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext


class GatedLinearAttention(Mixer):
    NAMES = ("q", "k", "v", "g", "o", "a1", "a2", "a2_bias", "norm")

    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, tau: float, norm_eps: float,
                 names: dict[str, str], rank: int | None = None, q_scale: float | None = None, init_std: float = 0.02):
        for k in self.NAMES:
            if k not in names:
                raise ValueError(f"gated linear attention needs the checkpoint name of its {k!r} tensor")
        if key_dim > 256:
            raise ValueError(f"the recurrence kernel takes up to 256 key channels a head, found {key_dim}")
        if not tau > 0:
            raise ValueError("tau must be positive")
        self.hidden, self.n_heads, self.key_dim, self.value_dim = hidden, n_heads, key_dim, value_dim
        self.tau, self.norm_eps = float(tau), float(norm_eps)
        self.rank = int(rank) if rank else None          # None: the stored tensor decides
        self.q_scale = float(q_scale) if q_scale is not None else key_dim ** -0.5
        self.names = dict(names)
        self.init_std = init_std
        self.w_in = self.w_a1 = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def tensor_specs(self):
        H, d, dv, W, s, n = self.n_heads, self.key_dim, self.value_dim, self.hidden, self.init_std, self.names
        return {n["q"]: TensorSpec((H * d, W), init_std=s), n["k"]: TensorSpec((H * d, W), init_std=s),
                n["v"]: TensorSpec((H * dv, W), init_std=s), n["g"]: TensorSpec((H * dv, W), init_std=s),
                n["o"]: TensorSpec((W, H * dv), init_std=s), n["a1"]: TensorSpec((self.rank, W), init_std=s),
                n["a2"]: TensorSpec((H * d, self.rank), init_std=0.2), n["a2_bias"]: TensorSpec((H * d,), init_std=1.0),
                n["norm"]: TensorSpec((dv,), init_std=0.1)}

    def cache_needs(self):
        return {"state": StateNeed((self.n_heads, self.value_dim, self.key_dim), torch.float32)}     # S^T per head

    def prompt_flops(self, n_tokens: int) -> float:
        return 5.0 * self.n_heads * self.key_dim * self.value_dim * n_tokens      # decay, outer product, read-out

    def load(self, store, rt: Runtime):
        n = self.names
        parts = [store.get(n[k], rt.dtype) for k in ("q", "k", "v", "g")]
        self.w_in = torch.cat(parts, dim=0).contiguous()
        del parts
        store.drop(*(n[k] for k in ("q", "k", "v", "g")))
        self.w_a1 = store.get(n["a1"], rt.dtype).contiguous()
        self.rank = int(self.w_a1.shape[0])
        self.w_a2 = store.get(n["a2"], rt.dtype).contiguous()
        if tuple(self.w_a2.shape) != (self.n_heads * self.key_dim, self.rank):
            raise ValueError(f"{n['a2']}: shape {tuple(self.w_a2.shape)} does not continue the rank {self.rank} of {n['a1']}")
        self.b_a2 = store.get(n["a2_bias"], rt.dtype).contiguous()
        self.w_norm = store.get(n["norm"]).to(torch.float32).contiguous()
        self.w_o = store.get(n["o"], rt.dtype).contiguous()

    def forward(self, x, ctx: StepContext, line):
        rt, ws, ops = ctx.rt, ctx.ws, ctx.rt.ops
        st = line["state"]
        if not st.write:
            raise ValueError("a recurrent state has one writer: a gated-linear-attention layer cannot read another's line")
        T, H, d, dv, r = ctx.n_tok, self.n_heads, self.key_dim, self.value_dim, self.rank
        q_off, k_off, v_off, g_off = 0, H * d, 2 * H * d, 2 * H * d + H * dv
        rows = ws.buf("gla.rows", (T, g_off + H * dv), rt.dtype)
        rt.linear(x, self.w_in, rows)
        z = rt.linear(rt.linear(x, self.w_a1, ws.buf("gla.a1", (T, r), rt.dtype)), self.w_a2,
                      ws.buf("gla.z", (T, H * d), rt.dtype))
        o = ws.buf("gla.o", (T, H * dv), torch.float32)
        ops.gla_scan(rows, q_off, k_off, v_off, z, self.b_a2, ctx.seq_slot, ctx.seq_first_row, ctx.seq_start,
                     ctx.seq_end, st.data, o, ctx.n_seq, H, d, dv, self.q_scale, self.tau,
                     decay=ws.buf("gla.decay", (T, H * d), torch.float32))
        y = ws.buf("gla.y", (T, H * dv), rt.dtype)
        ops.head_norm_gate(o, rows, g_off, self.w_norm, self.norm_eps, y, H, dv)
        return rt.linear(y, self.w_o, ws.buf("mixer.out", (T, self.hidden), rt.dtype))
