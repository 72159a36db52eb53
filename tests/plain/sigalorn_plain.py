"""Plain, slow Sigalorn: whole sequences, no cache, one function per mechanism.

It is the oracle of the Sigalorn tests and shares no code with the package under
test (the container reader is the other oracle's).  Everything runs in float64
torch operations on whatever device the weights are on.

The design, in this file's notation.  x is the residual stream [T, width].

* embedding:      x = E[token] * s_e
* layer:          x += N1b(mixer(N1(x)));  x += N2b(ff(N2(x)))   (the second line only with a feed-forward)
* norm:           N(x) = x / sqrt(mean(x^2) + eps) * w
* feed-forward:   D act(U y + b_u) + b_d with act = xIELU(p, q):
                  z > 0: softplus(p) z^2 + z/2;   z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2
* 'gla' mixer:    per head q = (Wq y) / sqrt(dim), k = Wk y, v = Wv y, a = sigmoid(Wa2 Wa1 y + b)^(1/tau);
                  S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; o normed per head over vdim (one weight for
                  all heads), times silu(Wg y), then Wo
* 'attention':    grouped heads; rotary on the first rot.dims of q and k (pairs i, i + dims/2); values rotated by their
                  own position over all of vdim and the head's output turned back by the query's position; raw scores
                  scaled, then mixed over heads by a matrix; a key is seen when it is not later than the query and
                  lies in the same block of mask.size positions; softmax with 1 added to the denominator; Wo.
                  A layer with kv_from takes keys and values from that layer.
* output:         final norm, head, cap * tanh(logits / cap)
"""
from __future__ import annotations

import math

import torch

from .gemma2_plain import load_folder  # noqa: F401  (the folder reader: config dict and float64 tensors)

F = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def softplus(x):
    return torch.logaddexp(x, torch.zeros_like(x))


def xielu(z, p, q):
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def dense_ff(y, w, pre):
    act = w[pre + "act"]
    z = y @ w[pre + "up"].T + w[pre + "up.b"]
    return xielu(z, act[0], act[1]) @ w[pre + "down"].T + w[pre + "down.b"]


def turn(x, pos, base, dims):
    """Rotate the first `dims` features of x [T, heads, n] by pos * base^(-2i/dims), pairs (i, i + dims/2)."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F, device=x.device)
    a = pos.to(F)[:, None, None] * f[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def gla_mixer(y, w, pre, m, eps):
    T = y.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (y @ w[pre + "q"].T).view(T, H, d) / math.sqrt(d)
    k = (y @ w[pre + "k"].T).view(T, H, d)
    v = (y @ w[pre + "v"].T).view(T, H, dv)
    z = (y @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = torch.exp(-softplus(-z) / tau).view(T, H, d)          # sigmoid(z)^(1/tau)
    S = torch.zeros(H, d, dv, dtype=F, device=y.device)
    o = torch.empty(T, H, dv, dtype=F, device=y.device)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w[pre + "norm"], eps)
    g = y @ w[pre + "g"].T
    return (o.reshape(T, H * dv) * (g * torch.sigmoid(g))) @ w[pre + "o"].T


def attention_keys_values(y, w, pre, m):
    """Keys (rotated over rot.dims) and values (rotated over vdim) of a layer that has projections of its own."""
    T = y.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T, device=y.device)
    k = turn((y @ w[pre + "k"].T).view(T, G, d), pos, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    v = turn((y @ w[pre + "v"].T).view(T, G, dv), pos, float(m["rot"]["base"]), dv)
    return k, v


def attention_mixer(y, w, pre, m, k, v):
    T = y.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    base, size = float(m["rot"]["base"]), int(m["mask"]["size"])
    pos = torch.arange(T, device=y.device)
    q = turn((y @ w[pre + "q"].T).view(T, H, d), pos, base, int(m["rot"]["dims"]))
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)                          # query head h uses key/value head h // rep
    vh = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * float(m["scale"])
    s = torch.einsum("hg,gij->hij", w[pre + "talk"], s)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[None, :] // size) == (pos[:, None] // size))
    e = torch.where(seen[None], torch.exp(s), torch.zeros_like(s))
    p = e / (1.0 + e.sum(-1, keepdim=True))
    o = torch.einsum("hij,jhv->ihv", p, vh)
    o = turn(o, -pos, base, dv)
    return o.reshape(T, H * dv) @ w[pre + "o"].T


def forward(cfg, w, tokens, layers_out=None):
    """float64 logits [T, vocab]; `layers_out`, a list, receives the residual stream after every layer."""
    dev = w["embed"].device
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), device=dev)] * float(cfg["embedding"]["scale"])
    kv = {}
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        y = rms_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "gla":
            r = gla_mixer(y, w, pre + "mix.", m, eps)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kv[i] = attention_keys_values(y, w, pre + "mix.", m)
                src = i
            r = attention_mixer(y, w, pre + "mix.", m, *kv[src])
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + rms_norm(r, w[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            y = rms_norm(x, w[pre + "norm2"], eps)
            x = x + rms_norm(dense_ff(y, w, pre + "mlp."), w[pre + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    y = rms_norm(x, w["final.norm"], eps)
    logits = y @ w["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap > 0 else logits
