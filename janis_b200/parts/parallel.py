"""Mixers side by side: several mixers read the same input and their outputs are averaged.

    out = (1 / n) sum_i  rms(mixer_i(y)) * w_i          rms(x) = x / sqrt(mean(x^2) + eps) over the model width

Each branch's output is normed with a weight vector of its own (plain, no offset) before the mean, so that
branches of different scale count alike.  The norms and the sum are float32; the result is handed to the block
as float32 and enters the residual sum unrounded.

The branches keep what they need in the same cache line, under their own names (`left.kv`, `right.state`, ...):
the line a branch sees holds its parts alone.
"""
from __future__ import annotations

import torch

from ..cache.cache import CacheLine
from ..weights.loader import TensorSpec
from .base import Mixer, Runtime, StepContext


class ParallelMixers(Mixer):
    def __init__(self, hidden: int, branches: dict[str, Mixer], out_norm_names: dict[str, str], eps: float,
                 init_std: float = 0.1):
        if not branches:
            raise ValueError("parallel mixers need at least one branch")
        for k in branches:
            if k not in out_norm_names:
                raise ValueError(f"branch {k!r} needs the checkpoint name of its output norm's weight")
        self.hidden = hidden
        self.branches = dict(branches)
        self.out_norm_names = dict(out_norm_names)
        self.eps = float(eps)
        self.init_std = init_std
        self.out_weights: dict[str, torch.Tensor] = {}

    def tensor_specs(self):
        return {self.out_norm_names[k]: TensorSpec((self.hidden,), init_std=self.init_std, init_mean=1.0)
                for k in self.branches}

    def sub_parts(self):
        return list(self.branches.values())

    def cache_needs(self):
        return {f"{k}.{name}": need for k, m in self.branches.items() for name, need in m.cache_needs().items()}

    def prompt_flops(self, n_tokens: int) -> float:
        return sum(m.prompt_flops(n_tokens) for m in self.branches.values())

    def load(self, store, rt: Runtime):
        for k in self.branches:
            self.out_weights[k] = store.get(self.out_norm_names[k]).to(torch.float32).contiguous()

    def forward(self, x, ctx: StepContext, line):
        ws, ops = ctx.ws, ctx.rt.ops
        acc = ws.buf("parallel.sum", (ctx.n_tok, self.hidden), torch.float32)
        share = 1.0 / len(self.branches)
        for i, (k, mixer) in enumerate(self.branches.items()):
            own = CacheLine(line.index, line.write, {name[len(k) + 1:]: part for name, part in line.parts.items()
                                                     if name.startswith(k + ".")}, line.has_readers)
            r = mixer.forward(x, ctx, own)
            ops.rmsnorm_accumulate(r, self.out_weights[k], self.eps, share, acc, first=i == 0)
        return acc
