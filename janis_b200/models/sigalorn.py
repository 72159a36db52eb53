"""Sigalorn as an arrangement of parts.

A decoder whose layers are listed in the configuration, each with one of two mixers and an optional dense
feed-forward, in the arrangement with a norm before and after each sublayer (`SandwichBlock`):

* "attention": `TalkingHeadsAttention` with a sink, a block mask, rotated values and a stored head-mixing matrix;
  a layer with `kv_from` reads the cache line of the layer it names (schedule entry with write=False).
* "gla": `GatedLinearAttention`.

Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
The embedding constant multiplies in float32; the head is a table of its own, capped.
"""
from __future__ import annotations

from ..config.sigalorn import SigalornConfig
from ..engine.model import DecoderModel, LayerCall
from ..parts import registry as parts
from ..registry import register_architecture


def build_sigalorn(cfg: SigalornConfig) -> DecoderModel:
    W = cfg.width

    def norm(name):
        return parts.make("norm", "rms_norm", width=W, eps=cfg.norm_eps, weight_name=name, offset=0.0, init_std=0.3, init_mean=1.0)

    blocks, schedule, line_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        if layer.type == "attention":
            own = m.kv_from is None
            names = {k: f"{p}.mix.{k}" for k in (("q", "k", "v", "o", "talk") if own else ("q", "o", "talk"))}
            mixer = parts.make(
                "mixer", "talking_heads_attention", hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, key_dim=m.dim,
                value_dim=m.vdim, scale=m.scale, block=m.block, sink=True, own_kv=own, names=names,
                position=parts.make("position", "rotary", head_dim=m.dim, base=m.rot_base, rotary_dims=m.rot_dims),
                value_position=parts.make("position", "rotary", head_dim=m.vdim, base=m.rot_base))
            if own:
                line_of[i] = len(line_of)
                schedule.append(LayerCall(i, line_of[i]))
            else:
                schedule.append(LayerCall(i, line_of[m.kv_from], write=False))
        else:
            mixer = parts.make(
                "mixer", "gated_linear_attention", hidden=W, n_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                tau=m.tau, norm_eps=cfg.norm_eps, rank=m.rank,
                names={"q": f"{p}.mix.q", "k": f"{p}.mix.k", "v": f"{p}.mix.v", "g": f"{p}.mix.g", "o": f"{p}.mix.o",
                       "a1": f"{p}.mix.a1", "a2": f"{p}.mix.a2", "a2_bias": f"{p}.mix.a2.b", "norm": f"{p}.mix.norm"})
            line_of[i] = len(line_of)
            schedule.append(LayerCall(i, line_of[i]))
        ff = None
        if layer.mlp is not None:
            ff = parts.make("feed_forward", "dense_mlp", hidden=W, intermediate=layer.mlp.ff, act="xielu",
                            names={"up": f"{p}.mlp.up", "up_bias": f"{p}.mlp.up.b", "down": f"{p}.mlp.down",
                                   "down_bias": f"{p}.mlp.down.b", "act": f"{p}.mlp.act"})
        blocks.append(parts.make(
            "block", "sandwich", mixer=mixer, feed_forward=ff, input_norm=norm(f"{p}.norm1"),
            post_mixer_norm=norm(f"{p}.norm1b"), pre_ff_norm=norm(f"{p}.norm2") if ff is not None else None,
            post_ff_norm=norm(f"{p}.norm2b") if ff is not None else None))
    return DecoderModel(
        cfg,
        embedding=parts.make("embedding", "scaled_table", vocab=cfg.vocab, hidden=W, table_name="embed",
                             scale=cfg.embedding_scale, round_scale=False, init_std=1.0),
        blocks=blocks,
        final_norm=norm("final.norm"),
        head=parts.make("head", "capped_linear", vocab=cfg.vocab, hidden=W, table_name="head",
                        softcap=cfg.logit_softcap, init_std=W ** -0.5),
        schedule=schedule,
        max_context=1 << 20)


register_architecture("Sigalorn", SigalornConfig, build_sigalorn, model_types=("sigalorn",), replace=True)
