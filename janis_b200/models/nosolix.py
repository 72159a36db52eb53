"""Nosolix as an arrangement of parts.

A decoder whose layers are listed in the configuration, in the pre-norm arrangement (`PreNormBlock`) with Dynamic
Tanh norms, each with one of two mixers and a dense feed-forward, a mixture of experts, or none:

* "mamba1": `SelectiveScanMixer`.
* "parallel": `ParallelMixers` over `left`, `TalkingHeadsAttention` without head mixing or sink, over a sliding
  window, with band-scaled rotary frequencies and an output gate, and `right`, `DualityMixer`.

Tensor names: `embed`, `l<i>.norm1|norm2` (each with `.b` and `.alpha`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`,
`head`.  The embedding constant multiplies in float32; the head is a table of its own, without a cap.
"""
from __future__ import annotations

from ..config.nosolix import MoeSpec, NosolixConfig
from ..engine.model import DecoderModel, LayerCall
from ..parts import registry as parts
from ..registry import register_architecture


def _selective(W, p, m):
    return parts.make("mixer", "selective_scan", hidden=W, inner=m.inner, state=m.state, dt_rank=m.dt_rank, taps=m.conv,
                      names={"in": f"{p}.in", "conv": f"{p}.conv", "conv_bias": f"{p}.conv.b", "x": f"{p}.x",
                             "dt": f"{p}.dt", "dt_bias": f"{p}.dt.b", "A_log": f"{p}.A_log", "D": f"{p}.D", "o": f"{p}.o"})


def _parallel(W, p, m, eps):
    a, d = m.left, m.right
    scaling = a.rot_scaling.to_dict() if a.rot_scaling is not None else None
    left = parts.make(
        "mixer", "talking_heads_attention", hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, key_dim=a.dim,
        value_dim=a.vdim, scale=a.scale, window=a.window, sink=False,
        names={k: f"{p}.left.{k}" for k in ("q", "k", "v", "g", "o")},
        position=parts.make("position", "rotary", head_dim=a.dim, base=a.rot_base, rotary_dims=a.rot_dims,
                            band_scaling=scaling))
    right = parts.make(
        "mixer", "state_space_duality", hidden=W, n_heads=d.heads, head_dim=d.vdim, state=d.state, groups=d.groups,
        norm_groups=d.norm_groups, taps=d.conv, norm_eps=eps,
        names={"in": f"{p}.right.in", "conv": f"{p}.right.conv", "conv_bias": f"{p}.right.conv.b",
               "dt_bias": f"{p}.right.dt_bias", "A_log": f"{p}.right.A_log", "D": f"{p}.right.D",
               "norm": f"{p}.right.norm", "o": f"{p}.right.o"})
    return parts.make("mixer", "parallel", hidden=W, branches={"left": left, "right": right},
                      out_norm_names={"left": f"{p}.left.out", "right": f"{p}.right.out"}, eps=eps)


def _feed_forward(W, p, f):
    if isinstance(f, MoeSpec):
        names = {"router": f"{p}.router", "correction": f"{p}.correction", "expert": p + ".e{e}.{w}"}
        if f.shared is not None:
            names.update(shared=p + ".shared.{w}", shared_gate=f"{p}.shared.sg")
        return parts.make("feed_forward", "routed_experts", hidden=W, n_experts=f.experts, top=f.top,
                          expert_ff=f.expert.ff, limit=f.expert.limit, scale=f.scale, group_count=f.group_count,
                          group_keep=f.group_keep, shared_ff=f.shared.ff if f.shared is not None else 0,
                          shared_limit=f.shared.limit if f.shared is not None else 0.0, names=names)
    return parts.make("feed_forward", "dense_mlp", hidden=W, intermediate=f.ff, act="relu2",
                      names={"up": f"{p}.up", "down": f"{p}.down"})


def build_nosolix(cfg: NosolixConfig) -> DecoderModel:
    W = cfg.width

    def norm(name):
        return parts.make("norm", "dynamic_tanh", width=W, weight_name=name)

    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        if layer.type == "mamba1":
            mixer = _selective(W, f"{p}.mix", layer.mixer)
        else:
            mixer = _parallel(W, f"{p}.mix", layer.mixer, cfg.norm_eps)
        ff = _feed_forward(W, f"{p}.mlp", layer.mlp) if layer.mlp is not None else None
        blocks.append(parts.make("block", "pre_norm", mixer=mixer, feed_forward=ff, input_norm=norm(f"{p}.norm1"),
                                 pre_ff_norm=norm(f"{p}.norm2") if ff is not None else None))
    return DecoderModel(
        cfg,
        embedding=parts.make("embedding", "scaled_table", vocab=cfg.vocab, hidden=W, table_name="embed",
                             scale=cfg.embedding_scale, round_scale=False, init_std=1.0),
        blocks=blocks,
        final_norm=norm("final.norm"),
        head=parts.make("head", "capped_linear", vocab=cfg.vocab, hidden=W, table_name="head", softcap=0.0,
                        init_std=W ** -0.5),
        schedule=[LayerCall(i, i) for i in range(len(blocks))],
        max_context=1 << 20)


register_architecture("Nosolix", NosolixConfig, build_nosolix, model_types=("nosolix",), replace=True)
