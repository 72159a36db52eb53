"""Plain, slow Nosolix: whole sequences, no cache, one function per mechanism.

It is the oracle of the Nosolix tests and shares no code with the package under
test (the container reader is the other oracle's).  Everything runs in float64
torch operations.

The design, in this file's notation.  r is the residual stream [T, width], y a sublayer's input.

* embedding:     r = E[token] * s_e
* layer:         r += mixer(N1(r));  r += ff(N2(r))         (the second line only with a feed-forward)
* norm:          N(r) = tanh(alpha r) * w + b                with a scalar alpha: no mean, no variance
* 'mamba1':      [u | z] = W_in y;  u = silu(conv(u));  [lo | B | C] = W_x u;  delta = softplus(W_dt lo + b_dt);
                 S_t[c, n] = exp(delta_c A[c, n]) S_{t-1}[c, n] + delta_c u_c B_n,  A = -exp(A_log);
                 o_c = sum_n S_t[c, n] C_n + D_c u_c;  out = W_o (o * silu(z))
* 'parallel':    out = (rms(left(y)) * w_l + rms(right(y)) * w_r) / 2 with
   left:         grouped softmax attention over a sliding window (query i sees keys i - size < j <= i), rotary on
                 the first rot.dims features (pairs i, i + dims/2) with frequencies rescaled by wavelength bands,
                 values of their own size, heads gated by sigmoid(W_g y) before W_o
   right:        [z | u | B | C | dt] = W_in y;  (u, B, C) = silu(conv(u, B, C));  delta = softplus(dt + dt_bias) per head;
                 S_t = exp(-exp(A_log_h) delta) S_{t-1} + delta B_t u_t^T;  o_t = S_t^T C_t + D_h u_t;
                 out = W_o (rms_parts(o * silu(z)) * w_norm)
* feed-forward:  dense: W_down relu(W_up y)^2;  moe: routed experts + gated shared expert (see `moe_ff`)
* output:        final norm, head
"""
from __future__ import annotations

import math

import torch

from .gemma2_plain import load_folder  # noqa: F401  (the folder reader: config dict and float64 tensors)

F = torch.float64


def dyt_norm(x, w, pre):
    return torch.tanh(w[pre + ".alpha"] * x) * w[pre] + w[pre + ".b"]


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def softplus(x):
    return torch.logaddexp(x, torch.zeros_like(x))


def silu(x):
    return x * torch.sigmoid(x)


def causal_conv(x, kernel, bias):
    """x [T, C], kernel [C, taps]: out[t, c] = bias[c] + sum_j kernel[c, taps - 1 - j] x[t - j, c], zeros before t = 0."""
    T, C = x.shape
    taps = kernel.shape[1]
    out = bias.expand(T, C).clone()
    for j in range(taps):
        if j < T:
            out[j:] += kernel[:, taps - 1 - j] * x[:T - j]
    return out


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------

def selective_scan_mixer(y, w, pre, m):
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    T = y.shape[0]
    uz = y @ w[pre + "in"].T
    u, z = uz[:, :inner], uz[:, inner:]
    u = silu(causal_conv(u, w[pre + "conv"], w[pre + "conv.b"]))
    p = u @ w[pre + "x"].T
    lo, B, C = p[:, :R], p[:, R:R + N], p[:, R + N:R + 2 * N]
    delta = softplus(lo @ w[pre + "dt"].T + w[pre + "dt.b"])            # [T, inner]
    A = -torch.exp(w[pre + "A_log"])                                   # [inner, N]
    S = torch.zeros(inner, N, dtype=F)
    o = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(delta[t][:, None] * A) * S + (delta[t] * u[t])[:, None] * B[t][None, :]
        o[t] = S @ C[t] + w[pre + "D"] * u[t]
    return (o * silu(z)) @ w[pre + "o"].T


def scaled_frequencies(rot):
    """base^(-2i/dims), rescaled by wavelength: short waves kept, long ones divided by `factor`, a blend between."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F)
    factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
    out = []
    for v in f:
        wave = 2.0 * math.pi / v
        if wave < orig / high:
            out.append(v)
        elif wave > orig / low:
            out.append(v / factor)
        else:
            s = (orig / wave - low) / (high - low)
            out.append((1.0 - s) * v / factor + s * v)
    return torch.tensor(out, dtype=F)


def turn(x, pos, freq):
    """x [T, heads, n]: the first 2 len(freq) features rotated by pos * freq, pairs (i, i + len(freq))."""
    h = freq.numel()
    if h == 0:
        return x
    ang = pos.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :h], x[..., h:2 * h]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., 2 * h:]], dim=-1)


def window_attention(y, w, pre, m):
    T = y.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    freq = scaled_frequencies(m["rot"])
    q = turn((y @ w[pre + "q"].T).view(T, H, d), pos, freq)
    k = turn((y @ w[pre + "k"].T).view(T, G, d), pos, freq)
    v = (y @ w[pre + "v"].T).view(T, G, dv)
    size = m["mask"]["size"]
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i) & (i - j < size)
    out = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(y @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def duality_mixer(y, w, pre, m, eps):
    T = y.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    p = y @ w[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + "conv"], w[pre + "conv.b"]))
    u = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    delta = softplus(dt + w[pre + "dt_bias"])                          # [T, H]
    a = -torch.exp(w[pre + "A_log"])                                   # [H]
    S = torch.zeros(H, N, P, dtype=F)
    o = torch.zeros(T, H, P, dtype=F)
    per = H // G
    for t in range(T):
        Bh = B[t].repeat_interleave(per, dim=0)                        # [H, N]
        Ch = C[t].repeat_interleave(per, dim=0)
        S = torch.exp(a * delta[t])[:, None, None] * S + delta[t][:, None, None] * Bh[:, :, None] * u[t][:, None, :]
        o[t] = torch.einsum("hnp,hn->hp", S, Ch) + w[pre + "D"][:, None] * u[t]
    g = o.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    g = rms(g.view(T, parts, inner // parts), eps).reshape(T, inner) * w[pre + "norm"]
    return g @ w[pre + "o"].T


def parallel_mixer(y, w, pre, m, eps):
    left = window_attention(y, w, pre + "left.", m["left"])
    right = duality_mixer(y, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[pre + "left.out"] + rms(right, eps) * w[pre + "right.out"])


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------

def dense_ff(y, w, pre):
    return torch.relu(y @ w[pre + "up"].T) ** 2 @ w[pre + "down"].T


def expert(y, w, pre, limit):
    g = torch.clamp(y @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(y @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def route(y, w, pre, router):
    """(chosen experts [T, top], their weights [T, top])."""
    E, top = router["experts"], router["top"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(y @ w[pre + "router"].T)                        # [T, E]
    choice = s + w[pre + "correction"]
    n_g, keep = groups["count"], groups["keep"]
    per = E // n_g
    grouped = choice.view(-1, n_g, per)
    g_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)        # [T, n_g]
    best = g_score.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(g_score, dtype=torch.bool).scatter_(1, best, True)
    masked = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), choice,
                         torch.full_like(choice, -math.inf))
    idx = masked.topk(top, dim=-1).indices
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * router["scale"]


def moe_ff(y, w, pre, mlp):
    idx, wts = route(y, w, pre, mlp["router"])
    out = torch.zeros(y.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for t in range(y.shape[0]):
        for e, a in zip(idx[t].tolist(), wts[t]):
            out[t] += a * expert(y[t:t + 1], w, f"{pre}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        sg = torch.sigmoid(y @ w[pre + "shared.sg"].T)                # [T, 1]
        out = out + sg * expert(y, w, pre + "shared.", mlp["shared"]["limit"])
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """float64 logits [T, vocab] of a whole sequence from position 0 (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    r = w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = dyt_norm(r, w, p + "norm1")
        if layer["type"] == "mamba1":
            r = r + selective_scan_mixer(y, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "parallel":
            r = r + parallel_mixer(y, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp:
            y = dyt_norm(r, w, p + "norm2")
            r = r + (dense_ff(y, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(y, w, p + "mlp.", mlp))
        after.append(r.clone())
    logits = dyt_norm(r, w, "final.norm") @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
