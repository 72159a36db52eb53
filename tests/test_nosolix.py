"""Nosolix: each mechanism against its plain statement, and the engine against the plain model.

The configurations are small and differ from each other in every size and option: state counts that are no power
of two, one and several groups of B and C, one and several parts of the gated norm, grouped and ungrouped attention
heads, values wider and narrower than keys, rotary widths below the key size and none at all, windows that are no
multiple of a cache page (and a window of one position), with and without frequency scaling, dense feed-forwards,
mixtures with one and several expert groups, with and without a shared expert, layers without a feed-forward, both
layer orders.  Weights are seeded random ones with the query/key projections scaled up, so that the attention weights
are far from uniform and a key that is wrongly seen or missed changes the logits.

Engine cases run on the GPU (`-m gpu`, float32 and bfloat16) and, as a check of the host side alone, on the CPU
over the plain kernel statements (float32, shorter requests).  The bfloat16 cases use folders whose routers are
steep (scores at 0 or 1 for all but a token in a hundred) and whose corrections are well apart: the rounding of the
router's input then seldom changes which experts are chosen, which in the soft-router folders it does for a token
in a hundred, and a changed choice is a changed row of logits, not a rounding.
"""
from __future__ import annotations

import copy
import math

import pytest
import torch

from tests.conftest import random_tokens
from tests.helpers import assert_logits as _assert_exact, make_engine, run_in_pieces, run_requests

GPU = pytest.mark.gpu
CASES = [pytest.param("cuda", "float32", marks=GPU), pytest.param("cuda", "bfloat16", marks=GPU),
         pytest.param("refs", "float32")]


def assert_logits(got, want, dtype, what):
    """float32: every logit within 1e-4 of the largest one.  bfloat16: rows are judged by the root mean square of
    their difference against that of the logits: 98 in 100 (or all but two) within 4 %, at most two beyond 10 % (a
    router's close call that the rounding decides the other way), half of them within 1 %."""
    if dtype in ("float32", torch.float32):
        return _assert_exact(got, want, dtype, what)
    got, want = got.detach().double().cpu(), want.double().cpu()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    rows = (got - want).pow(2).mean(1).sqrt() / want.pow(2).mean().sqrt()
    over = int((rows > 4e-2).sum())
    assert int((rows > 1e-1).sum()) <= 2 and over <= max(2, rows.numel() // 50) and rows.median().item() < 1e-2, \
        (f"{what}: worst row {rows.max().item():.3f} at {int(rows.argmax())}, {over} of {rows.numel()} rows over 4 %: "
         f"{(rows > 4e-2).nonzero().flatten().tolist()[:12]}, median {rows.median().item():.4f}")


def _scan(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def _par(heads, kv, dim, vdim, rot, window, scale, ssd, base=10000.0, scaling=None):
    rotd = {"base": base, "dims": rot}
    if scaling:
        rotd["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    h, p, n, g, parts, conv = ssd
    return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
                     "rot": rotd},
            "right": {"heads": h, "vdim": p, "state": n, "groups": g, "norm_groups": parts, "conv": conv}}


def _moe(experts, top, ff, limit, scale, count, keep, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}},
            "shared": {"ff": shared[0], "limit": shared[1]} if shared else None}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


DENSE = lambda ff: {"kind": "dense", "ff": ff}

NOS_A = {"architecture": "Nosolix", "vocab": 200, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6}, "layers": [
    _layer("parallel", _par(4, 2, 32, 16, 16, 24, 0.2, (4, 8, 12, 2, 2, 3), scaling=(8.0, 1.0, 4.0, 64)), DENSE(96)),
    _layer("mamba1", _scan(96, 12, 5, 4), _moe(8, 2, 24, 1.5, 2.0, 4, 2, shared=(40, 0.7))),
    _layer("mamba1", _scan(72, 8, 8, 2), None),
    _layer("parallel", _par(2, 2, 16, 24, 16, 1, 0.3, (2, 16, 8, 1, 1, 4), base=500.0), _moe(6, 3, 16, 0.8, 1.0, 1, 1))]}

NOS_B = {"architecture": "Nosolix", "vocab": 333, "width": 96, "embedding": {"scale": 1.4}, "norm": {"eps": 1e-5}, "layers": [
    _layer("mamba1", _scan(160, 24, 6, 4), DENSE(128)),
    _layer("parallel", _par(6, 1, 24, 8, 8, 70, 0.25, (3, 16, 40, 3, 1, 2), base=1000.0, scaling=(2.0, 2.0, 8.0, 32)),
           _moe(12, 4, 32, 1.0, 2.5, 3, 1, shared=(48, 1.2))),
    _layer("parallel", _par(3, 3, 48, 40, 0, 130, 0.1, (8, 4, 33, 4, 4, 4)), None)]}

# sizes a tensor-core kernel takes; a window of two whole pages; one expert chosen; experts in groups of one
NOS_C = {"architecture": "Nosolix", "vocab": 512, "width": 128, "embedding": {"scale": 11.3}, "norm": {"eps": 1e-6}, "layers": [
    _layer("parallel", _par(8, 2, 64, 64, 64, 128, 0.11, (4, 32, 64, 1, 1, 4), base=300000.0, scaling=(4.0, 1.0, 4.0, 256)),
           _moe(16, 1, 64, 2.0, 1.0, 16, 4)),
    _layer("mamba1", _scan(256, 16, 8, 4), _moe(4, 4, 32, 1.0, 3.0, 2, 2, shared=(32, 1.0))),
    _layer("parallel", _par(16, 16, 16, 32, 8, 100, 0.2, (2, 64, 128, 2, 8, 4), base=300000.0), DENSE(256))]}

# sizes that are multiples of nothing useful
NOS_D = {"architecture": "Nosolix", "vocab": 301, "width": 70, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-4}, "layers": [
    _layer("mamba1", _scan(50, 3, 3, 1), DENSE(50)),
    _layer("parallel", _par(5, 5, 10, 6, 6, 33, 0.3, (5, 6, 7, 5, 3, 3), base=100.0), _moe(9, 2, 11, 0.5, 1.7, 3, 2, shared=(13, 0.9))),
    _layer("mamba1", _scan(34, 37, 1, 5), None),
    _layer("parallel", _par(3, 1, 12, 14, 12, 5, 0.4, (1, 22, 5, 1, 2, 2), base=100.0, scaling=(3.0, 1.0, 2.0, 16)), DENSE(22))]}

NOS = {"A": NOS_A, "B": NOS_B, "C": NOS_C, "D": NOS_D}


def write_nosolix(model_dir: str, raw: dict, seed: int, steep_router: bool = False, gain: float = 4.0,
                  qk_gain: float = 6.0, router_gain: float = 20.0) -> None:
    """A folder of seeded random weights: query and key projections scaled up; step-size biases spread, so that
    some channels forget within a few tokens and others remember hundreds; with steep_router the routers' rows are
    scaled up (scores near 0 or 1) and the corrections are distinct steps with a jitter.  The gains suit widths of
    a hundred; a model of real width takes smaller ones."""
    from janis_b200 import build_model
    from janis_b200.weights.loader import random_tensors, write_model_folder
    _, cfg, model = build_model(raw)
    tensors = random_tensors(model.tensor_specs(), seed, "cpu")
    for name, t in list(tensors.items()):
        if name.endswith(".left.q") or name.endswith(".left.k"):
            tensors[name] = (t.float() * qk_gain).to(torch.bfloat16)
        elif name.endswith(".dt.b") or name.endswith(".dt_bias"):
            tensors[name] = (t.float() * 2.0 - 1.0).to(torch.bfloat16)
        elif name.endswith(".mlp.router"):
            tensors[name] = (t.float() * router_gain * (200.0 if steep_router else 1.0)).to(torch.bfloat16)
        elif name.endswith(".mlp.correction") and steep_router:
            g = torch.Generator().manual_seed(seed)
            n = t.numel()       # distinct steps with a jitter, so that sums of two do not tie between groups
            tensors[name] = (0.07 * torch.randperm(n, generator=g).float() + 0.03 * torch.rand(n, generator=g)).to(torch.bfloat16)
        elif any(name.endswith(x) for x in (".o", ".down", ".up", ".gate", ".in", ".left.v", ".left.g", ".mix.x")):
            tensors[name] = (t.float() * gain).to(torch.bfloat16)
    write_model_folder(model_dir, cfg.to_dict(), tensors, {"seed": str(seed)})


@pytest.fixture(scope="module")
def nos_dirs(tmp_path_factory):
    out = {}
    for i, (key, raw) in enumerate(NOS.items()):
        for steep in (False, True):
            d = tmp_path_factory.mktemp(f"nosolix_{key}{'_steep' if steep else ''}")
            write_nosolix(str(d), raw, 300 + i, steep)
            out[(key, steep)] = str(d)
    return out


@pytest.fixture(scope="module")
def plain(nos_dirs):
    from tests.plain import nosolix_plain as P
    loaded, memo = {}, {}

    def logits(key, steep, tokens):
        if (key, steep) not in loaded:
            loaded[(key, steep)] = P.load_folder(nos_dirs[(key, steep)])
        k = (key, steep, tuple(tokens))
        if k not in memo:
            cfg, w = loaded[(key, steep)]
            memo[k] = P.forward(cfg, w, list(tokens))
        return memo[k]

    return logits


@pytest.fixture(scope="module")
def engines(nos_dirs):
    made = {}

    def get(key, dtype, on, **kw):
        steep = dtype == "bfloat16"
        k = (key, dtype, on, tuple(sorted(kw.items())))
        if k not in made:
            made[k] = make_engine(nos_dirs[(key, steep)], dtype, on, **kw)
        return made[k], steep

    yield get
    for e in made.values():
        e.close()


def keys_for(on):
    return ["A", "B", "C", "D"] if on == "cuda" else ["A", "B", "D"]


# ---------------------------------------------------------------------------
# configuration and registry
# ---------------------------------------------------------------------------

def test_configuration_reads_back_and_guards():
    from janis_b200 import ConfigError, NosolixConfig, build_model, resolve
    cfg = NosolixConfig.from_dict(NOS_A)
    assert NosolixConfig.from_dict(cfg.to_dict()) == cfg
    assert resolve(NOS_A).name == "Nosolix"
    assert cfg.layers[0].mixer.left.window == 24 and cfg.layers[0].mixer.left.rot_scaling.factor == 8.0
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp.group_keep == 2 and cfg.layers[3].mlp.shared is None
    _, _, model = build_model(NOS_A)
    specs = model.tensor_specs()
    assert "l2.norm2" not in specs and "l2.mlp.up" not in specs and "l3.mlp.shared.sg" not in specs
    assert specs["l1.mlp.shared.sg"].shape == (1, 64) and specs["l0.mix.right.in"].shape == (2 * 32 + 2 * 2 * 12 + 4, 64)
    assert specs["l0.norm1.alpha"].shape == () and specs["l1.mix.x"].shape == (5 + 2 * 12, 96)
    needs = model.cache_line_needs()
    assert set(needs[0]) == {"left.kv", "right.state", "right.conv"} and set(needs[1]) == {"state", "conv"}
    for bad in ({**NOS_A, "layers": [{"type": "conv", "mixer": {}, "mlp": None}]},
                {**NOS_A, "layers": [_layer("parallel", _par(4, 3, 32, 16, 16, 24, 0.2, (4, 8, 12, 2, 2, 3)), None)]},
                {**NOS_A, "layers": [_layer("parallel", _par(4, 2, 32, 16, 16, 24, 0.2, (4, 8, 12, 3, 2, 3)), None)]},
                {**NOS_A, "layers": [_layer("mamba1", _scan(96, 12, 5, 4), _moe(8, 5, 24, 1.5, 2.0, 4, 2))]},
                {**NOS_A, "layers": [_layer("mamba1", _scan(96, 12, 5, 4), {"kind": "sparse", "ff": 3})]}):
        with pytest.raises(ConfigError):
            NosolixConfig.from_dict(bad)


# ---------------------------------------------------------------------------
# the plain oracle's functions against hand-made cases (CPU)
# ---------------------------------------------------------------------------

def test_plain_router_by_hand():
    from tests.plain import nosolix_plain as P
    F = torch.float64
    # six experts in three groups; logits chosen so that sigmoid gives round scores
    s = torch.tensor([[0.9, 0.1, 0.5, 0.6, 0.2, 0.8]], dtype=F)
    z = torch.log(s / (1 - s))
    w = {"r.router": torch.eye(6, dtype=F), "r.correction": torch.tensor([0.0, 0.0, 0.3, 0.3, 0.0, -0.5], dtype=F)}
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    # choice scores: .9 .1 | .8 .9 | .2 .3 -> group scores 1.0, 1.7, 0.5: groups 1 and 0 stay; best two: experts 0 and 3 (.9, .9)
    idx, wts = P.route(z, w, "r.", router)
    assert sorted(idx[0].tolist()) == [0, 3]
    got = dict(zip(idx[0].tolist(), wts[0].tolist()))
    assert abs(got[0] - 0.9 / 1.5 * 2.0) < 1e-12 and abs(got[3] - 0.6 / 1.5 * 2.0) < 1e-12
    # a negative choice score inside a kept group still beats any score outside it
    w["r.correction"] = torch.tensor([-5.0, -5.0, 0.0, 0.0, 0.0, 0.0], dtype=F)
    router["groups"]["keep"] = 1
    router["top"] = 2
    idx, _ = P.route(z, w, "r.", router)          # group scores -9, 1.1, 1.0 -> group 1 alone
    assert sorted(idx[0].tolist()) == [2, 3]


def test_plain_conv_window_and_expert_by_hand():
    from tests.plain import nosolix_plain as P
    F = torch.float64
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=F)
    out = P.causal_conv(x, torch.tensor([[100.0, 10.0, 1.0]], dtype=F), torch.tensor([0.5], dtype=F))
    assert out[:, 0].tolist() == [1.5, 12.5, 124.5]            # the last tap is the current token's
    g = P.expert(torch.tensor([[3.0, -3.0]], dtype=F), {"e.gate": torch.tensor([[1.0, 0.0]], dtype=F),
                                                       "e.up": torch.tensor([[0.0, 1.0]], dtype=F),
                                                       "e.down": torch.ones(1, 1, dtype=F)}, "e.", 2.0)
    want = 2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0)  # gate capped from above only, up from both sides
    assert abs(g.item() - want) < 1e-12
    # a window of 2: token 2 sees tokens 1 and 2, not token 0
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0, "rot": {"base": 10.0, "dims": 0}, "mask": {"size": 2}}
    eye = torch.eye(2, dtype=F)
    w = {"q": eye, "k": eye, "v": eye, "o": eye, "g": torch.zeros(2, 2, dtype=F)}
    y = torch.tensor([[50.0, 0.0], [0.0, 1.0], [1.0, 0.0]], dtype=F)
    o = P.window_attention(y, w, "", m)
    p = math.exp(1.0) / (math.exp(1.0) + 1.0)
    assert torch.allclose(o[2], 0.5 * torch.tensor([p, 1 - p], dtype=F), atol=1e-12)      # gate sigmoid(0) = 1/2
    f = P.scaled_frequencies({"dims": 8, "base": 10.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}})
    # wavelengths 6.28, 11.2, 19.9, 35.3: kept below 10; blended between 10 and 40
    assert abs(f[0] - 1.0) < 1e-15 and f[3] < 10 ** -0.75 and f[3] > 10 ** -0.75 / 4.0


# ---------------------------------------------------------------------------
# each kernel against its statement in tests/kernel_refs.py (GPU)
# ---------------------------------------------------------------------------

def _tables(lens, starts, slots):
    first, rows = [], 0
    for n in lens:
        first.append(rows)
        rows += n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    tok_seq = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in enumerate(lens)])
    return tok_seq, i32(slots), i32(first), i32(starts), i32([a + n for a, n in zip(starts, lens)]), rows


def _close(got, want, dtype, what, f32=2e-5, bf16=2e-2):
    got, want = got.detach().double().cpu(), want.double().cpu()
    assert torch.isfinite(got).all(), what
    tol = f32 if dtype == torch.float32 else bf16
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), (what, err)


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,K,off,width", [(96, 4, 0, 96), (50, 1, 3, 60), (33, 2, 7, 40), (300, 7, 16, 400), (8, 16, 0, 8)])
def test_conv_kernel_against_its_statement(dtype, C, K, off, width):
    """Sequences that start, that go on from a stored state with fewer tokens than taps and with many, and a
    padding sequence; the state that the step leaves is compared too."""
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    lens, starts, slots = [5, 1, 2, 40, 3], [0, 7, 3, 11, 0], [2, 0, 4, 1, -1]
    tok_seq, seq_slot, first, seq_start, seq_end, T = _tables(lens, starts, slots)
    g = torch.Generator().manual_seed(C + K)
    rows = torch.randn(T, width, generator=g).to(dtype)
    w, b = torch.randn(C, K, generator=g), torch.randn(C, generator=g)
    state = torch.randn(6, max(K - 1, 1), C, generator=g)
    state[2] = 0
    want, want_state = torch.zeros(T, C, dtype=dtype), state.clone()
    R.causal_conv_silu(rows, off, C, w, b, want_state, tok_seq, seq_slot, first, seq_start, seq_end, len(lens), want)
    got, got_state = torch.full((T, C), float("nan"), dtype=dtype, device="cuda"), state.clone().cuda()
    ops.causal_conv_silu(rows.cuda(), off, C, w.cuda(), b.cuda(), got_state, tok_seq.cuda(), seq_slot.cuda(), first.cuda(),
                         seq_start.cuda(), seq_end.cuda(), len(lens), got)
    _close(got, want, dtype, "conv")
    assert torch.equal(got_state.cpu(), want_state), "the inputs kept for the next step"
    # a decode step: one token a sequence, the kept inputs shifted by the convolution's own kernel
    lens, starts, slots = [1, 1, 1, 1], [0, 9, 2, 5], [5, 3, -1, 0]
    tok_seq, seq_slot, first, seq_start, seq_end, T = _tables(lens, starts, slots)
    rows = torch.randn(T, width, generator=g).to(dtype)
    want, want_state = torch.zeros(T, C, dtype=dtype), state.clone()
    R.causal_conv_silu(rows, off, C, w, b, want_state, tok_seq, seq_slot, first, seq_start, seq_end, len(lens), want)
    got, got_state = torch.full((T, C), float("nan"), dtype=dtype, device="cuda"), state.clone().cuda()
    ops.causal_conv_silu(rows.cuda(), off, C, w.cuda(), b.cuda(), got_state, tok_seq.cuda(), seq_slot.cuda(), first.cuda(),
                         seq_start.cuda(), seq_end.cuda(), len(lens), got, one_token=True)
    _close(got, want, dtype, "conv, one token a sequence")
    assert torch.equal(got_state.cpu(), want_state), "the inputs kept after a decode step"


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,N,cph,cpg,per_state,gated", [
    (96, 12, 1, 96, True, True), (50, 3, 1, 50, True, True), (34, 37, 1, 34, True, True), (64, 128, 1, 64, True, True),
    (32, 12, 8, 16, False, False), (30, 7, 6, 6, False, False), (128, 128, 64, 64, False, False), (22, 5, 22, 22, False, False),
    (256, 16, 1, 256, True, True), (40, 300, 8, 20, False, False), (16, 48, 4, 16, False, True)])
@pytest.mark.parametrize("aligned", [False, True])
def test_scan_kernel_against_its_statement(dtype, C, N, cph, cpg, per_state, gated, aligned):
    """Sequences from zero, from a stored state, of one token and of many, and a padding sequence; the state left
    behind is compared too.  Step sizes are spread so that some channels forget at once and others keep all.
    `aligned` puts B and C at 16-byte offsets in rows of whole 16-byte pieces, which the form with tiles in shared
    memory wants (it then runs where the state count allows it, and the register form is run beside it)."""
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    lens, starts, slots = [9, 1, 70, 2], [0, 30, 5, 0], [3, 0, 1, -1]
    _, seq_slot, first, seq_start, seq_end, T = _tables(lens, starts, slots)
    heads, groups = C // cph, C // cpg
    g = torch.Generator().manual_seed(C * N)
    u = torch.randn(T, C + 5, generator=g).to(dtype)
    dt = (torch.randn(T, heads + 3, generator=g) * 2.0).to(dtype)
    pad = 16 if aligned else 4                     # where B starts in its rows
    bc = torch.randn(T, (2 * groups * N + pad + 7) // 8 * 8 if aligned else 2 * groups * N + pad, generator=g).to(dtype)
    z = torch.randn(T, C + 2, generator=g).to(dtype) if gated else None
    dt_bias, D = torch.randn(heads, generator=g) - 1.0, torch.randn(heads, generator=g)
    A = -torch.exp(torch.randn(heads, N, generator=g)) if per_state else -torch.exp(torch.randn(heads, generator=g))
    state = torch.randn(4, C, N, generator=g)
    out_dtype = dtype if gated else torch.float32
    want, want_state = torch.zeros(T, C, dtype=out_dtype), state.clone()
    args = lambda dev, st, out: (dev(u), 5, dev(dt), 3, dev(dt_bias), dev(A), per_state, dev(bc), pad, pad + groups * N, dev(D),
                                 dev(z) if gated else None, 2, dev(seq_slot), dev(first), dev(seq_start), dev(seq_end),
                                 len(lens), st, out, C, N, cph, cpg)
    R.selective_scan(*args(lambda x: x, want_state, want))
    for lanes, form in [(n, f) for n in (0, 4, 8, 16, 32) for f in ((2, 1) if aligned else (0,))]:
        if lanes and lanes * 16 < N:                   # (0: chosen by the launch; then every count that holds the states)
            continue
        ops.selective_scan_set_lanes(lanes)
        ops.selective_scan_set_form(form)
        try:
            got, got_state = torch.full((T, C), float("nan"), dtype=out_dtype, device="cuda"), state.clone().cuda()
            ops.selective_scan(*args(lambda x: x.cuda(), got_state, got))
        finally:
            ops.selective_scan_set_lanes(0)
            ops.selective_scan_set_form(0)
        _close(got, want, out_dtype, f"scan, {lanes} lanes, form {form}", f32=5e-5)
        _close(got_state, want_state, torch.float32, "the state left behind", f32=5e-5)
        assert torch.equal(got_state[2].cpu(), state[2]), "a slot that is not in the step keeps its state"


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels_against_their_statements(dtype):
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    g = torch.Generator().manual_seed(5)
    dev = lambda x: x.cuda() if x is not None else None
    for T, H in ((7, 70), (3, 1024), (40, 192)):
        h, res = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g).to(dtype)
        w, b = torch.randn(H, generator=g), torch.randn(H, generator=g)
        rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32)
        for r, sel in ((res, None), (None, None), (None, rows), (res.float(), None)):
            R_out = torch.zeros(3 if sel is not None else T, H, dtype=dtype)
            hw, hg = h.clone(), h.clone().cuda()
            R.dyt_norm(hw, r, 0.7, w, b, R_out, sel)
            got = torch.full(R_out.shape, float("nan"), dtype=dtype, device="cuda")
            ops.dyt_norm(hg, dev(r), 0.7, dev(w), dev(b), got, dev(sel))
            _close(got, R_out, dtype, "dyt_norm")
            _close(hg, hw, torch.float32, "the stream after the sum", f32=1e-6)
        acc_w, acc_g = torch.randn(T, H, generator=g), None
        acc_g = acc_w.clone().cuda()
        for first in (True, False):
            x = (torch.randn(T, H, generator=g) * 3.0).to(dtype)
            R.rmsnorm_accumulate(x, w, 1e-5, 0.5, acc_w, first)
            ops.rmsnorm_accumulate(x.cuda(), w.cuda(), 1e-5, 0.5, acc_g, first)
            _close(acc_g, acc_w, torch.float32, "rmsnorm_accumulate", f32=1e-5)
    for T, C, parts, off, width in ((5, 96, 1, 0, 100), (9, 120, 3, 7, 140), (2, 4096, 2, 0, 4096), (4, 30, 30, 2, 40)):
        o, rows, w = torch.randn(T, C, generator=g), torch.randn(T, width, generator=g).to(dtype), torch.randn(C, generator=g)
        want, got = torch.zeros(T, C, dtype=dtype), torch.full((T, C), float("nan"), dtype=dtype, device="cuda")
        R.gate_group_norm(o, rows, off, w, 1e-5, parts, want)
        ops.gate_group_norm(o.cuda(), rows.cuda(), off, w.cuda(), 1e-5, parts, got)
        _close(got, want, dtype, "gate_group_norm")
        x = torch.randn(T, C, generator=g).to(dtype)
        xw, xg = x.clone(), x.clone().cuda()
        R.sigmoid_gate(xw, rows, min(off, width - C))
        ops.sigmoid_gate(xg, rows.cuda(), min(off, width - C))
        _close(xg, xw, dtype, "sigmoid_gate")


@GPU
@pytest.mark.parametrize("E,count,keep,top,shared", [(8, 4, 2, 2, True), (6, 1, 1, 3, False), (16, 16, 4, 1, False),
                                                     (4, 2, 2, 4, True), (9, 3, 2, 2, True), (64, 8, 3, 6, True),
                                                     (256, 8, 4, 8, False), (40, 2, 1, 20, False)])
def test_router_and_expert_kernels_against_their_statements(E, count, keep, top, shared):
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    g = torch.Generator().manual_seed(E)
    T = 37
    z = torch.randn(T, E + (1 if shared else 0), generator=g) * 2.0
    corr = torch.randn(E, generator=g) * 0.5
    want, got = torch.zeros_like(z), torch.full(z.shape, float("nan"), device="cuda")
    R.moe_route(z, corr, E, count, keep, top, 2.5, shared, want)
    ops.moe_route(z.cuda(), corr.cuda(), E, count, keep, top, 2.5, shared, got)
    assert ((want[:, :E] > 0).sum(1) == top).all()
    assert torch.equal(got[:, :E].cpu() > 0, want[:, :E] > 0), "the experts chosen"
    _close(got, want, torch.float32, "router weights", f32=1e-5)
    ff, sff = 24, 40 if shared else 0
    for dtype in (torch.float32, torch.bfloat16):
        gu = (torch.randn(T, 2 * (E * ff + sff), generator=g) * 2.0).to(dtype)
        a_want = torch.zeros(T, E * ff + sff, dtype=dtype)
        a_got = torch.full(a_want.shape, float("nan"), dtype=dtype, device="cuda")
        R.moe_expert_act(gu, want, E, ff, 1.5, sff, 0.7, 1.702, a_want)
        ops.moe_expert_act(gu.cuda(), want.cuda(), E, ff, 1.5, sff, 0.7, 1.702, a_got)
        _close(a_got, a_want, dtype, "expert activation")


def _paged(n_seq, lens, G, d, dv, dtype, seed, spare=3):
    from janis_b200.kernels.ops import PAGE
    g = torch.Generator().manual_seed(seed)
    per = [(n + PAGE - 1) // PAGE for n in lens]
    n_pages = sum(per) + spare
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(n_seq + 2, max(per), dtype=torch.int32)
    slots = torch.randperm(n_seq + 2, generator=g)[:n_seq].to(torch.int32)
    at = 0
    for s in range(n_seq):
        for j in range(per[s]):
            table[int(slots[s]), j] = order[at]
            at += 1
    k = torch.randn(n_pages, G, PAGE, d, generator=g).to(dtype)
    v = torch.randn(n_pages, G, PAGE, dv, generator=g).to(dtype)
    return k, v, table, slots


@GPU
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,window", [(4, 2, 32, 16, 24), (8, 2, 64, 96, 150), (3, 1, 24, 40, 1), (8, 8, 64, 64, 128),
                                             (5, 5, 8, 6, 7), (16, 4, 128, 64, 65), (2, 1, 16, 8, 300), (6, 3, 48, 48, 64)])
def test_windowed_attention_kernel_against_its_statement(dtype, H, G, d, dv, window):
    """Queries at the window's edges, at page borders and far into sequences over scattered pages.  For every query
    the oldest key inside its window and the newest key outside it both get a large score under head 0: the first
    must count, the second must not."""
    from janis_b200.kernels import ops
    from tests import kernel_refs as R
    lens = [1, 70, 129, 300]
    kp, vp, table, slots = _paged(len(lens), lens, G, d, dv, dtype, 3)
    pos, seq = [], []
    for s, n in enumerate(lens):
        for p in sorted({0, n - 1, n // 2, min(n - 1, 63), min(n - 1, 64), min(n - 1, window - 1), min(n - 1, window),
                         min(n - 1, window + 1), min(n - 1, 2 * window)}):
            pos.append(p)
            seq.append(s)
    T = len(pos)
    g = torch.Generator().manual_seed(9)
    q = torch.randn(T, H * d + 5, generator=g).to(dtype)
    # (queries of one sequence share its keys: the planted keys serve the last query of each sequence that reaches them)
    for t in range(T):
        hot = (q[t, :d].float() * (3.0 / max(q[t, :d].float().norm().item(), 1e-3))).to(dtype)
        for j in (pos[t] - window + 1, pos[t] - window):
            if j >= 0:
                kp[int(table[int(slots[seq[t]]), j // ops.PAGE]), 0, j % ops.PAGE] = hot
    tok_pos, tok_seq = torch.tensor(pos, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32)
    want = torch.zeros(T, H * dv, dtype=dtype)
    R.talk_attention(q, tok_pos, tok_seq, slots, kp, vp, table, None, None, want, H, G, d, dv, 0.4, 0, False, window=window)
    dev = lambda x: x.cuda() if x is not None else None
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for which, one_row, chunks in ((1, False, 1), (1, True, 1), (1, True, 3), (1, True, 7), (0, False, 1)):
        ops.talk_attention_set_kernel(which)
        try:
            got = torch.full((T, H * dv), float("nan"), dtype=dtype, device="cuda")
            n = ops.talk_attention_scratch_floats(T, chunks, H, dv)
            scratch = torch.full((n,), float("nan"), device="cuda") if n else None
            ops.talk_attention(dev(q), dev(tok_pos), dev(tok_seq), dev(slots), dev(kp), dev(vp), dev(table), None, None,
                               got, H, G, d, dv, 0.4, 0, False, one_row=one_row, max_keys=min(window, 300),
                               n_chunks=chunks, scratch=scratch, window=window)
        finally:
            ops.talk_attention_set_kernel(1)
        err = (got.cpu().double() - want.double()).abs().max().item()
        assert err <= tol * max(1.0, want.double().abs().max().item()), (which, one_row, chunks, err)


# ---------------------------------------------------------------------------
# the engine against the plain model
# ---------------------------------------------------------------------------

def _requests(vocab, lens, seed):
    return [random_tokens(vocab, n, seed + i) for i, n in enumerate(lens)]


@pytest.mark.parametrize("on,dtype", CASES)
def test_whole_prompts_and_decoding(engines, plain, on, dtype):
    """Prompts of unequal lengths in one batch, then decoded together token by token past every window; a second
    round of batches uses the freed slots and pages again."""
    for key in keys_for(on):
        eng, steep = engines(key, dtype, on, max_tokens=2048)
        V = NOS[key]["vocab"]
        lens = [1, 40, 150, 9, 77] if on == "cuda" else [1, 30, 9]
        extra = 80 if on == "cuda" else 12
        reqs = _requests(V, [n + extra for n in lens], 40)
        got = run_requests(eng, reqs, lens, max_live=3)
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, steep, r), dtype, f"{key} request {i} ({lens[i]} + {extra})")


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_request_alone_equals_the_request_in_a_batch(engines, on, dtype):
    """What else is in the step changes nothing beyond rounding: each request alone against the same in a batch."""
    key = "B"
    eng, _ = engines(key, dtype, on, max_tokens=2048)
    lens = [3, 90, 31] if on == "cuda" else [3, 20, 11]
    reqs = _requests(NOS[key]["vocab"], [n + 6 for n in lens], 70)
    together = run_requests(eng, reqs, lens)
    for i, r in enumerate(reqs):
        alone = run_requests(eng, [r], [lens[i]])[0]
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert (alone - together[i]).abs().max().item() <= tol * together[i].abs().max().item(), (key, i)


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("chunk", [2, 3, 16, 64, 65])
def test_prompts_in_pieces(engines, plain, on, dtype, chunk):
    """A prompt that comes in pieces (down to two tokens) onto what the pieces before left: the convolution's
    inputs, both states and the window's keys carry over."""
    if on == "refs" and chunk in (16, 65):
        pytest.skip("the CPU cases run two sizes")
    for key in (["A", "D"] if on == "refs" or chunk < 16 else keys_for(on)):
        eng, steep = engines(key, dtype, on, max_tokens=2048)
        lens = [70, 5, 141] if on == "cuda" and chunk >= 16 else [23, 5, 40]
        reqs = _requests(NOS[key]["vocab"], lens, 90 + chunk)
        got = run_in_pieces(eng, reqs, chunk)
        for i, r in enumerate(reqs):
            assert_logits(got[i], plain(key, steep, r), dtype, f"{key} request {i} in pieces of {chunk}")


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_graphs(engines, plain, dtype):
    """Hundreds of decode steps from a short prompt: replayed graphs, growing length buckets, windows that slide off
    the prompt, states that integrate every token."""
    key = "C"
    eng, steep = engines(key, dtype, "cuda", max_tokens=2048)
    reqs = _requests(NOS[key]["vocab"], [420, 300], 7)
    got = run_requests(eng, reqs, [4, 2])
    for i, r in enumerate(reqs):
        assert_logits(got[i], plain(key, steep, r), dtype, f"{key} long decoding {i}")


@pytest.mark.parametrize("on,dtype", [pytest.param("cuda", "float32", marks=GPU), pytest.param("refs", "float32")])
def test_greedy_generation_through_the_engine(engines, nos_dirs, on, dtype):
    """`generate` (scheduler, sampler, stop handling) against greedy decoding of the plain model."""
    from tests.plain import nosolix_plain as P
    key = "A"
    eng, steep = engines(key, dtype, on, max_tokens=1024)
    cfg, w = P.load_folder(nos_dirs[(key, steep)])
    prompts = _requests(NOS[key]["vocab"], [5, 17, 2], 11)
    n_new = 12 if on == "cuda" else 6
    replies = eng.generate(prompts, temp=0.0, max_tokens=n_new, stop=[])
    for p, r in zip(prompts, replies):
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(P.forward(cfg, w, seq)[-1].argmax()))
        assert r == seq[len(p):], (p, r, seq[len(p):])


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_command_line(nos_dirs, plain, dtype, tmp_path):
    """`bin/trace_run` as a user runs it: the model class comes from config.json; prompts in one batch, decoded
    together, a second batch on the freed slots; and `bin/janis generate` on the same folder."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    from tests.test_generation import ROOT, _trace
    key, steep = "D", dtype == "bfloat16"
    V = NOS[key]["vocab"]
    lens = [40, 9, 75, 1, 23, 130]
    reqs = [random_tokens(V, n, 210 + n) for n in lens]
    steps, peak = _trace(reqs, [max(1, n - 32) for n in lens], batch_of=3)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", nos_dirs[(key, steep)], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(peak)],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    got = {f"r{i}": [] for i in range(len(reqs))}
    for s in steps:
        arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V)
        o = 0
        for e in s["entries"]:
            got[e["id"]].append(torch.from_numpy(arr[o:o + len(e["want"])].copy()))
            o += len(e["want"])
        assert o == arr.shape[0]
    for i, r in enumerate(reqs):
        assert_logits(torch.cat(got[f"r{i}"]), plain(key, steep, r), dtype, f"trace request {i}")
    if dtype == "float32":
        from tests.plain import nosolix_plain as P
        cfg, w = P.load_folder(nos_dirs[(key, steep)])
        prompt = reqs[1]
        g = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janis"), "generate", "--model", nos_dirs[(key, steep)],
                            "--dtype", "float32", "--ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temp", "0", "--stop", ""],
                           capture_output=True, text=True, timeout=900)
        assert g.returncode == 0, g.stderr[-2000:]
        seq = list(prompt)
        for _ in range(5):
            seq.append(int(P.forward(cfg, w, seq)[-1].argmax()))
        assert ",".join(map(str, seq[len(prompt):])) in g.stdout.replace(" ", ""), g.stdout


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_shapes_of_a_real_model(tmp_path, dtype):
    """Two layers at the layer sizes of a 2-billion-parameter model (width 2304; 8 heads over 4 of 256; 72 state-space
    heads of 64 channels with 128 states; 4,608 scan channels with 16 states; 8 experts of 1,152), vocabulary cut to
    2,048: the kernels' launch shapes, vector loads and staged tiles at sizes the small models do not reach.  A prompt
    longer than the window, then decoded; beside it a short prompt."""
    from tests.plain import nosolix_plain as P
    raw = {"architecture": "Nosolix", "vocab": 2048, "width": 2304, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "layers": [
        _layer("parallel", _par(8, 4, 256, 256, 256, 200, 256 ** -0.5, (72, 64, 128, 1, 1, 4), scaling=(8.0, 1.0, 4.0, 128)),
               _moe(8, 2, 1152, 7.0, 1.5, 2, 1, shared=(1152, 7.0))),
        _layer("mamba1", _scan(4608, 16, 144, 4), DENSE(9216))]}
    steep = dtype == "bfloat16"
    write_nosolix(str(tmp_path), raw, 77, steep, gain=1.0, qk_gain=2.0, router_gain=2.0)
    cfg, w = P.load_folder(str(tmp_path))
    eng = make_engine(str(tmp_path), dtype, "cuda", max_tokens=1024)
    try:
        reqs = _requests(2048, [300 + 8, 5 + 8], 3)
        got = run_requests(eng, reqs, [300, 5])
        for i, r in enumerate(reqs):
            assert_logits(got[i], P.forward(cfg, w, r), dtype, f"real layer shapes, request {i}")
    finally:
        eng.close()
