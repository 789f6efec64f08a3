"""The mechanisms of the Pulenex design one by one, each built from its own parameters with weights of its own, against the
plain functions: the layer norm in its four forms, the normed sum of branches, the clamped gated feed-forward, rotary
positions in both pairings, the convolution with SiLU and filters side by side, retention with rotated q and k, the gated
delta rule, the chunked attention whose heads talk, and latent attention that reads another layer's rows."""
import numpy as np
import pytest
import torch

import helpers
from plain import pulenex_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _name(dtype):
    return "float32" if dtype == torch.float32 else "bfloat16"


def _context(cache, slot_tokens, dtype):
    from hymt2sharp_b200.engine.engine import StepEntry, make_context
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    entries = [StepEntry(s, [0] * n, []) for s, n in slot_tokens]
    ctx, _, _, plan = make_context(cache, entries, 10, dtype, DEV, status)
    return ctx, plan


def _cache_for(mixers, dtype, tokens=4096, slots=4):
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    from hymt2sharp_b200.parts import MixerSlot
    groups, mslots, offset = [], [], 0
    for m in mixers:
        n, sb = m.cache_need(), int(m.state_bytes())
        s = MixerSlot()
        if n is not None:
            groups.append(GroupSpec(n.kind, n.kv_heads, n.head_dim, 1, n.window, n.streams, n.value_dim))
            s.group, s.plane = len(groups) - 1, 0
        if sb:
            s.state_offset, s.state_bytes = offset, sb
            offset += -(-sb // 16) * 16
        mslots.append(s)
    return PagedCache(groups, dtype, DEV, tokens, max_slots=slots, state_bytes=offset), mslots


def _weights(part, scale=0.1, ranks=3):
    out = {}
    for n, s in part.tensors().items():
        shape = tuple(ranks if d == -1 else d for d in s.shape)
        base = torch.eye(*shape) if s.init == "identity" else (1.0 if s.init == "gain" else 0.0)
        out[n] = (torch.randn(shape) * (scale if len(shape) == 2 else 0.1) + base).to(torch.bfloat16)
    return out


def _run_mixer(part, cache, mslot, schedule, xs, dtype, poison=False):
    """schedule: [[(sequence index, tokens), ...], ...]; xs[i] [T_i, hidden]; returns per sequence what the mixer wrote."""
    slots = {}
    at = {i: 0 for i in range(len(xs))}
    outs = {i: [] for i in range(len(xs))}
    for step in schedule:
        for i, _ in step:
            if i not in slots:
                slots[i] = cache.alloc_slots(1)[0]
        ctx, plan = _context(cache, [(slots[i], n) for i, n in step], dtype)
        x = torch.cat([xs[i][at[i]:at[i] + n] for i, n in step]).to(DEV).to(dtype)
        res = torch.full((x.shape[0], xs[0].shape[1]), float("nan"), dtype=torch.float32, device=DEV)
        part.forward(x, res, ctx, mslot, store=True)
        cache.end_step(plan)
        o = 0
        for i, n in step:
            outs[i].append(res[o:o + n].cpu()); o += n; at[i] += n
    cache.free_slots(list(slots.values()))
    return [torch.cat(outs[i]) if outs[i] else torch.empty(0, xs[0].shape[1]) for i in range(len(xs))]


def _w64(w):
    return {k: v.to(F64) for k, v in w.items()}


SCHEDULES = {
    "whole": lambda n, m: [[(0, n), (1, m)]],
    "portions down to two tokens": lambda n, m: [[(0, 2), (1, 3)], [(0, 67), (1, 2)], [(0, n - 69), (1, m - 5)]],
    "a prompt and single tokens": lambda n, m: [[(0, n - 40), (1, m - 10)]] + [[(0, 1), (1, 1)]] * 10 + [[(0, 1)]] * 30,
}


# -- norms ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, W", [(5, 46), (130, 256), (3, 2050)])
def test_layer_norm_stored_added_and_followed_by_the_next(dtype, T, W):
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(T + W)
    a = build_part("norm", PartSpec("layernorm", dict(dim=W, eps=1e-5, weight="a")))
    b = build_part("norm", PartSpec("layernorm", dict(dim=W, eps=1e-6, weight="b")))
    w = {"a": (1 + 0.2 * torch.randn(W)).to(torch.bfloat16), "b": (1 + 0.2 * torch.randn(W)).to(torch.bfloat16)}
    a.load(w, DEV, dtype); b.load(w, DEV, dtype)
    x = torch.randn(T, W) * 3 + 2.0                      # a mean far from zero: an RMS norm in its place would show
    res = torch.randn(T, W)
    ref = plain.layer_norm(x.to(F64), w["a"].to(F64), 1e-5)
    out = a.forward(x.to(DEV), None, dtype, fresh=True)
    helpers.assert_close(out.float().cpu().numpy(), ref.numpy(), _name(dtype), "stored", factor=0.5)
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out = a.forward(x.to(DEV), None, torch.float32, rows_index=rows, rows=2, scale=0.25)
    helpers.assert_close(out.cpu().numpy(), 0.25 * ref[[T - 1, 0]].numpy(), "float32", "gathered and scaled")
    r1 = res.to(DEV).clone()
    a.add_into(x.to(DEV), r1)
    helpers.assert_close(r1.cpu().numpy(), (res.to(F64) + ref).numpy(), "float32", "added")
    r2 = res.to(DEV).clone()
    nxt = a.add_into_then(x.to(DEV), r2, b, dtype)
    helpers.assert_close(r2.cpu().numpy(), r1.cpu().numpy(), "float32", "the residual of the fused form", factor=0.1)
    ref2 = plain.layer_norm(res.to(F64) + ref, w["b"].to(F64), 1e-6)
    helpers.assert_close(nxt.float().cpu().numpy(), ref2.numpy(), _name(dtype), "added, then the next norm", factor=0.5)
    r3 = res.to(DEV).clone()
    rows_ = a.add_into_then_rows(x.to(DEV), r3, dtype)
    helpers.assert_close(r3.cpu().numpy(), r1.cpu().numpy(), "float32", "the residual of the rows form", factor=0.1)
    helpers.assert_close(rows_.float().cpu().numpy(), r1.cpu().numpy(), _name(dtype), "added, then the rows", factor=0.5)


@pytest.mark.parametrize("T, W, B", [(7, 46, 2), (65, 256, 1), (3, 1030, 4)])
def test_branches_normed_each_by_its_own_root_mean_square_and_summed(T, W, B):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(W)
    xs = [torch.randn(T, W) * (10.0 ** b) for b in range(B)]          # branches of very different size count alike
    gains = [(1 + 0.3 * torch.randn(W)) for _ in range(B)]
    scales = [0.5, 0.5, -1.0, 2.0][:B]
    out = torch.empty(T, W, device=DEV)
    ops.rmsnorm_sum(out, [x.to(DEV) for x in xs], [g.to(DEV) for g in gains], scales, 1e-5)
    ref = sum(s * plain.unit_rms(x.to(F64), 1e-5) * g.to(F64) for s, x, g in zip(scales, xs, gains))
    helpers.assert_close(out.cpu().numpy(), ref.numpy(), "float32", "normed sum")


# -- feed-forward --------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, W, F, limit", [(9, 46, 21, 0.3), (140, 128, 256, 1.0), (2, 64, 40, 7.0)])
def test_clamped_gated_feed_forward(dtype, T, W, F, limit):
    """With weights large enough that both clamps bite on many entries (and, at a limit of 7, on none)."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(F)
    ff = build_part("feed_forward", PartSpec("clamped_glu", dict(hidden=W, intermediate=F, limit=limit, alpha=1.702, gate_proj="gate",
                                                                 up_proj="up", down_proj="down", gate_bias="gate.b", up_bias="up.b",
                                                                 down_bias="down.b")))
    w = _weights(ff, 0.15)
    for k in ("gate.b", "up.b", "down.b"):
        w[k] = (torch.randn(w[k].shape) * 0.4).to(torch.bfloat16)
    ff.load(w, DEV, dtype)
    x = torch.randn(T, W).to(torch.bfloat16).float()
    cache, _ = _cache_for([], dtype)
    slot = cache.alloc_slots(1)[0]
    ctx, _ = _context(cache, [(slot, T)], dtype)
    ref = plain.clamped_glu(x.to(F64), _w64(w), "", limit)
    out = torch.full((T, W), float("nan"), device=DEV)
    ff.forward(x.to(DEV).to(dtype), out, ctx, store=True)
    helpers.assert_close(out.cpu().numpy(), ref.numpy(), _name(dtype), "stored", factor=2.0)
    acc = torch.ones((T, W), device=DEV)
    ff.forward(x.to(DEV).to(dtype), acc, ctx)
    helpers.assert_close(acc.cpu().numpy(), 1.0 + ref.numpy(), _name(dtype), "added", factor=2.0)
    g = x.to(F64) @ w["gate"].to(F64).T + w["gate.b"].to(F64)
    assert (float((g > limit).double().mean()) > 0.05) == (limit < 5)


# -- rotary positions ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("heads, d, dims, tail", [(3, 10, 6, 5), (4, 64, 64, 0), (2, 32, 16, 64), (1, 8, 0, 3)])
def test_rotation_of_heads_side_by_side(pairing, heads, d, dims, tail):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(d)
    T = 40
    pos = torch.randint(0, 300, (T,), dtype=torch.int32)     # (the angle is a float32 product: its error grows with the position)
    x = torch.randn(T, heads * d + tail)
    f = torch.tensor([100.0 ** (-2.0 * i / max(dims, 1)) for i in range(dims // 2)], dtype=F64).float()
    turn = plain.rotate_half if pairing == "half" else plain.rotate_pairs
    ref = torch.cat([turn(x[:, :heads * d].to(F64).reshape(T, heads, d), pos.long(), dims, 100.0).reshape(T, heads * d), x[:, heads * d:].to(F64)], 1)
    for dtype in (torch.float32, torch.bfloat16):
        xin = x.to(DEV).to(dtype)
        want = ref if dtype == torch.float32 else torch.cat([turn(xin.cpu().to(F64)[:, :heads * d].reshape(T, heads, d), pos.long(), dims, 100.0).reshape(T, -1),
                                                             xin.cpu().to(F64)[:, heads * d:]], 1)
        out = torch.full((T, heads * d + tail), float("nan"), device=DEV)
        ops.rotate_heads(out, xin, pos.to(DEV), f.to(DEV) if dims else None, heads, d, dims, pairing)
        helpers.assert_close(out.cpu().numpy(), want.numpy(), "float32", f"{pairing} into float32", factor=4.0)      # 32-bit out of either type
        ops.rotate_heads(xin, xin, pos.to(DEV), f.to(DEV) if dims else None, heads, d, dims, pairing)    # in place
        helpers.assert_close(xin.float().cpu().numpy(), want.numpy(), _name(dtype), f"{pairing} in place", factor=4.0 if dtype == torch.float32 else 0.5)


# -- the convolution with SiLU and several filters side by side ----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps, pieces", [(4, (12, 6)), (2, (7,)), (1, (8, 8, 3)), (3, (64, 64, 32))])
def test_convolution_with_silu_over_cuts(dtype, taps, pieces):
    from hymt2sharp_b200.parts import MixerSlot
    from hymt2sharp_b200.parts.conv import ShortConv
    torch.manual_seed(taps)
    C = sum(pieces)
    conv = ShortConv(C, taps, [(f"w{i}", c) for i, c in enumerate(pieces)], activation="silu")
    w = {f"w{i}": torch.randn(c, taps).to(torch.bfloat16) for i, c in enumerate(pieces)}
    assert set(conv.tensors()) == set(w)
    conv.load(w, DEV, dtype)

    class Holder:   # the convolution's state as a mixer would hold it
        def cache_need(self): return None
        def state_bytes(self): return conv.state_bytes()
    cache, (mslot,) = _cache_for([Holder()], dtype)
    cache.state.fill_(255)
    xs = [torch.randn(n, C + 5).to(torch.bfloat16).float() for n in (90, 21)]
    full = torch.cat([w[f"w{i}"] for i in range(len(pieces))]).to(F64)
    refs = [plain.silu(plain.short_conv(x[:, :C].to(F64), full)) for x in xs]
    for what, cuts in SCHEDULES.items():
        slots, at, outs = {}, [0, 0], [[], []]
        for step in cuts(90, 21):
            for i, _ in step:
                slots.setdefault(i, None)
                if slots[i] is None:
                    slots[i] = cache.alloc_slots(1)[0]
            ctx, plan = _context(cache, [(slots[i], n) for i, n in step], dtype)
            x = torch.cat([xs[i][at[i]:at[i] + n] for i, n in step]).to(DEV).to(dtype)
            y = conv.forward(x[:, :C], ctx, mslot)           # columns of a wider matrix
            cache.end_step(plan)
            o = 0
            for i, n in step:
                outs[i].append(y[o:o + n].float().cpu()); o += n; at[i] += n
        cache.free_slots(list(slots.values()))
        for i in range(2):
            helpers.assert_close(torch.cat(outs[i]).numpy(), refs[i].numpy(), _name(dtype), f"{what}, sequence {i}", factor=0.5)


# -- retention with rotated q and k ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, dim, vdim, dims", [(46, 3, 6, 10, 4), (64, 2, 64, 32, 64), (64, 1, 32, 40, 16), (48, 2, 24, 8, 0)])
def test_retention_with_rotary_positions(dtype, hidden, heads, dim, vdim, dims):
    """Whole prompts long enough for the passes over chunks, portions, single tokens, a second sequence beside the first: the
    rotation follows a token's position in its sequence, not its place in the step."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(hidden + dim)
    decay = [0.9, 0.97, 0.999][:heads]
    pos = PartSpec("neox_rope", dict(head_dim=dim, rope_dim=dims, base=300.0)) if dims else None
    part = build_part("mixer", PartSpec("retention", dict(hidden=hidden, heads=heads, dim=dim, vdim=vdim, decay=decay, eps=1e-5, q_proj="q",
                                                          k_proj="k", v_proj="v", g_proj="g", o_proj="o", position=pos)))
    w = _weights(part, 0.15)
    part.load(w, DEV, dtype)
    cache, (mslot,) = _cache_for([part], dtype)
    cache.state.fill_(255)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (330, 70)]
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(dims=dims, base=300.0))
    refs = [plain.retention(x.to(F64), _w64(w), "", m, 1e-5, torch.arange(x.shape[0])) for x in xs]
    for what, cuts in SCHEDULES.items():
        outs = _run_mixer(part, cache, mslot, cuts(330, 70), xs, dtype)
        for i in range(2):
            helpers.assert_close(outs[i].numpy(), refs[i].numpy(), _name(dtype), f"{what}, sequence {i}", factor=3.0 if dtype == torch.float32 else 6.0)


# -- the gated delta rule --------------------------------------------------------------------------------------------------------
def _delta(hidden, heads, kv_heads, dim, vdim, taps, ranks=(3, 5)):
    from hymt2sharp_b200.parts import PartSpec, build_part
    return build_part("mixer", PartSpec("gated_delta", dict(
        hidden=hidden, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, taps=taps, eps=1e-5, q_proj="q", k_proj="k", v_proj="v",
        q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", b_proj="b", a_log="A_log", a1_proj="a1", a2_proj="a2", dt_bias="dt_bias",
        g1_proj="g1", g2_proj="g2", norm="norm", o_proj="o", decay_rank=ranks[0], gate_rank=ranks[1])))


def _delta_weights(part, seed, a_log=None):
    torch.manual_seed(seed)
    w = _weights(part, 0.2)
    for k in ("q.conv", "k.conv", "v.conv"):
        w[k] = torch.randn(w[k].shape).to(torch.bfloat16)
    w["A_log"] = (torch.rand(w["A_log"].shape) * 4 - 3 if a_log is None else torch.full(w["A_log"].shape, a_log)).to(torch.bfloat16)
    w["dt_bias"] = torch.randn(w["dt_bias"].shape).to(torch.bfloat16)
    w["a2"] = (torch.randn(w["a2"].shape) * 2).to(torch.bfloat16)
    return w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, kv_heads, dim, vdim, taps", [(46, 4, 2, 6, 5, 2), (64, 2, 2, 16, 40, 4), (64, 3, 1, 32, 8, 3),
                                                                      (128, 2, 1, 64, 128, 4), (64, 1, 1, 128, 20, 1), (48, 1, 1, 160, 70, 4)])
def test_gated_delta_rule_in_prompts_portions_decoding_and_batches(dtype, hidden, heads, kv_heads, dim, vdim, taps):
    """Rows of a state column on 4 lanes (up to 16, 32, 64, 128 key channels) and on 8 (160); more value columns than a block
    holds; fewer q/k heads than value heads; whole prompts, portions, single tokens, a second sequence beside the first, in a
    state area that was poisoned."""
    part = _delta(hidden, heads, kv_heads, dim, vdim, taps)
    w = _delta_weights(part, hidden + dim)
    part.load(w, DEV, dtype)
    cache, (mslot,) = _cache_for([part], dtype)
    cache.state.fill_(255)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (150, 40)]
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim)
    refs = [plain.gated_delta(x.to(F64), _w64(w), "", m, 1e-5) for x in xs]
    for what, cuts in SCHEDULES.items():
        outs = _run_mixer(part, cache, mslot, cuts(150, 40), xs, dtype)
        for i in range(2):
            helpers.assert_close(outs[i].numpy(), refs[i].numpy(), _name(dtype), f"{what}, sequence {i}", factor=3.0 if dtype == torch.float32 else 8.0)


def test_gated_delta_rule_keeps_a_far_token_under_a_slow_decay_and_forgets_it_under_a_fast_one():
    """ONE token 600 places back differs between two sequences; with decays near one the last token's output still differs,
    with fast decays it does not; both as the plain recurrence says.  Prompt and decoded steps."""
    for a_log, kept in ((-9.0, True), (1.5, False)):
        part = _delta(32, 2, 1, 16, 8, 2)
        w = _delta_weights(part, 5, a_log=a_log)
        part.load(w, DEV, torch.float32)
        cache, (mslot,) = _cache_for([part], torch.float32)
        base = torch.randn(640, 32).to(torch.bfloat16).float()
        other = base.clone()
        other[20] = torch.randn(32) * 3
        m = dict(heads=2, kv_heads=1, dim=16, vdim=8)
        refs = [plain.gated_delta(x.to(F64), _w64(w), "", m, 1e-5) for x in (base, other)]
        outs = _run_mixer(part, cache, mslot, [[(0, 600), (1, 600)]] + [[(0, 1), (1, 1)]] * 40, [base, other], torch.float32)
        for i in range(2):
            helpers.assert_close(outs[i].numpy(), refs[i].numpy(), "float32", f"A_log {a_log}, sequence {i}", factor=3.0)
        gap = float((outs[0][-1] - outs[1][-1]).abs().max()) / float(outs[0][-1].abs().max())
        assert (gap > 1e-3) == kept, f"A_log {a_log}: the far token moves the last output by {gap:.2e}"


# -- the attention whose heads talk ----------------------------------------------------------------------------------------------
def _talk(hidden, heads, kv_heads, dim, scale, taps, mask, size, dims, sink=True, gate=True):
    from hymt2sharp_b200.parts import PartSpec, build_part
    pos = PartSpec("yarn_interleaved", dict(dims=dims, base=200.0, scaling=None)) if dims else None
    return build_part("mixer", PartSpec("talking_attention", dict(
        hidden=hidden, heads=heads, kv_heads=kv_heads, dim=dim, scale=scale, position=pos, q_proj="q", k_proj="k", o_proj="o", talk="talk",
        temp="temp", sink="sink" if sink else None, g_proj="g" if gate else None, mask=mask, mask_size=size, taps=taps,
        q_conv="q.conv" if taps else None, k_conv="k.conv" if taps else None)))


def _talk_weights(part, seed, heads):
    torch.manual_seed(seed)
    w = _weights(part, 0.3)
    w["talk"] = (torch.eye(heads) + 0.5 * torch.randn(heads, heads)).to(torch.bfloat16)
    w["temp"] = (0.5 + 1.5 * torch.rand(heads)).to(torch.bfloat16)
    if "sink" in w:
        w["sink"] = (torch.randn(heads) * 1.5).to(torch.bfloat16)
    for k in ("q.conv", "k.conv"):
        if k in w:
            w[k] = torch.randn(w[k].shape).to(torch.bfloat16)
    return w


def _talk_reference(x, w, heads, kv_heads, dim, scale, size, dims):
    w = dict(_w64(w))
    T = x.shape[0]
    if "q.conv" not in w:      # no convolution: a filter of one tap of ones
        w["q.conv"], w["k.conv"] = torch.ones(heads * dim, 1, dtype=F64), torch.ones(kv_heads * dim, 1, dtype=F64)
    if "sink" not in w:        # no sink: one that weighs nothing
        w["sink"] = torch.full((heads,), -1e30, dtype=F64)
    if "g" not in w:
        w["g"] = torch.zeros(heads * dim, x.shape[1], dtype=F64)
        w["o"] = w["o"] * 2.0          # (sigmoid(0) = 1/2)
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, scale=scale, rot=dict(dims=dims, base=200.0))
    if size:
        m["mask"] = dict(size=size)
    return plain.talking_attention(x.to(F64), w, "", m, torch.arange(T))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, kv_heads, dim, taps, size, dims, sink, gate", [
    (46, 4, 2, 10, 3, 7, 6, True, True),            # odd sizes: one entry an access; chunks shorter than a tile of keys
    (64, 6, 6, 16, 4, 64, 16, True, True),          # chunks as long as a cache block
    (64, 4, 1, 32, 4, 100, 32, True, False),        # one key head for all heads; chunks that straddle blocks; no gate
    (128, 2, 2, 64, 2, None, 32, False, True),      # no mask, no sink: plain causal softmax with mixed scores
    (64, 1, 1, 8, 0, 33, 0, True, True),            # one head (nothing to mix), no convolution, no rotation
    (64, 4, 2, 16, 2, 200, 8, True, True),          # chunks long enough that a decode step cuts its keys into splits
    (128, 16, 4, 128, 4, 48, 64, True, True),       # wide: fewer queries a block
])
def test_talking_attention_in_prompts_portions_decoding_and_batches(dtype, hidden, heads, kv_heads, dim, taps, size, dims, sink, gate):
    part = _talk(hidden, heads, kv_heads, dim, 0.3 * dim ** -0.5 * 4, taps, "chunk" if size else None, size or 0, dims, sink, gate)
    w = _talk_weights(part, hidden + dim, heads)
    part.load(w, DEV, dtype)
    cache, (mslot,) = _cache_for([part], dtype)
    for s in cache.storage:
        s.fill_(float("nan"))
    cache.state.fill_(255)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (210, 40)]
    refs = [_talk_reference(x, w, heads, kv_heads, dim, part.scale, size, dims) for x in xs]
    for what, cuts in SCHEDULES.items():
        outs = _run_mixer(part, cache, mslot, cuts(210, 40), xs, dtype)
        for i in range(2):
            helpers.assert_close(outs[i].numpy(), refs[i].numpy(), _name(dtype), f"{what}, sequence {i}", factor=3.0 if dtype == torch.float32 else 6.0)


@pytest.mark.parametrize("size", [7, 64, 100])
def test_a_loud_token_is_heard_to_the_end_of_its_chunk_and_not_beyond(size):
    """One input row eight times as loud as the others, placed at a chunk's last place, at the next chunk's first place and one
    behind: tokens of the same chunk differ from the quiet run, tokens of the next chunk do not (no filter here, which would
    carry an input a few places on); in a prompt, in portions that cut the chunk, and in decoded steps, each against
    the plain attention in 32-bit, where a mask that is one place off shows as a whole key's weight."""
    heads, kv_heads, dim, hidden, taps = 3, 1, 16, 48, 0
    part = _talk(hidden, heads, kv_heads, dim, 0.5, taps, "chunk", size, 8)
    w = _talk_weights(part, size, heads)
    part.load(w, DEV, torch.float32)
    cache, (mslot,) = _cache_for([part], torch.float32)
    T = 2 * size + 9
    torch.manual_seed(size)
    quiet = torch.randn(T, hidden).to(torch.bfloat16).float()
    for place in (size - 1, size, size + 1, 2 * size - 1):
        loud = quiet.clone()
        loud[place] *= 8.0
        ref_q, ref_l = (_talk_reference(x, w, heads, kv_heads, dim, 0.5, size, 8) for x in (quiet, loud))
        for what, cuts in {"prompt": [[(0, T)]], "portions": [[(0, size - 2)], [(0, 3)], [(0, T - size - 1)]],
                           "decoded": [[(0, size - 3)]] + [[(0, 1)]] * (T - size + 3)}.items():
            out = _run_mixer(part, cache, mslot, cuts, [loud], torch.float32)[0]
            helpers.assert_close(out.numpy(), ref_l.numpy(), "float32", f"size {size}, loud at {place}, {what}", factor=3.0)
        moved = (ref_l - ref_q).abs().amax(1) > 1e-6
        last = (place // size + 1) * size                      # first position of the chunk behind the loud token's
        # (a loud key may also score far below the others and weigh nothing for some query: most, not all, hear it)
        assert moved[place] and moved[place:min(last, T)].float().mean() > 0.5 and not moved[:place].any()
        assert not moved[min(T, last):].any()


# -- latent attention that reads another layer's rows ---------------------------------------------------------------------------------
def _latent(hidden, heads, dim, rot, vdim, rank, window, own, keep):
    from hymt2sharp_b200.parts import PartSpec, build_part
    pos = PartSpec("yarn_interleaved", dict(dims=rot, base=100.0, scaling=None))
    return build_part("mixer", PartSpec("latent_attention", dict(
        hidden=hidden, heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=0.3, eps=1e-5, position=pos, gate="head",
        q_proj="q", dkv_proj="dkv", dkv_norm="dkv.norm", uk_proj="uk", uv_proj="uv", o_proj="o", g_proj="g", window=window, own_kv=own,
        cache_window=keep)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, dim, rot, vdim, rank, w_src, w_rd", [(46, 3, 5, 4, 7, 9, 5, 11), (128, 2, 32, 16, 32, 64, 70, 33),
                                                                              (64, 4, 16, 16, 16, 64, 20, None)])
def test_latent_attention_reads_the_rows_of_another_layer(dtype, hidden, heads, dim, rot, vdim, rank, w_src, w_rd):
    """The writer caches its rows, the reader (other queries, up-projections, window and heads) attends over them: in whole
    prompts (the per-head form where the engine takes it), in portions and in decoded steps past both windows."""
    from hymt2sharp_b200.parts import MixerSlot
    keep = 0 if w_rd is None else max(w_src, w_rd)
    src = _latent(hidden, heads, dim, rot, vdim, rank, w_src, True, keep)
    rd = _latent(hidden, heads + 1, dim + 2, rot, vdim + 1, rank, w_rd, False, keep)
    assert "dkv" not in rd.tensors() and "dkv.norm" not in rd.tensors()
    torch.manual_seed(hidden)
    ws, wr = _weights(src, 0.3), _weights(rd, 0.3)
    src.load(ws, DEV, dtype); rd.load(wr, DEV, dtype)
    cache, (mslot,) = _cache_for([src], dtype)
    for s in cache.storage:
        s.fill_(float("nan"))
    reader = MixerSlot(group=mslot.group, plane=mslot.plane, writes=False)
    T = 150
    xa, xb = (torch.randn(T, hidden).to(torch.bfloat16).float() for _ in range(2))       # the two layers read different inputs
    pos = torch.arange(T)
    m_src = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=rank, scale=0.3, rot=dict(dims=rot, base=100.0), mask=dict(size=w_src))
    m_rd = dict(heads=heads + 1, dim=dim + 2, rot_dim=rot, vdim=vdim + 1, kv_rank=rank, scale=0.3, rot=dict(dims=rot, base=100.0))
    if w_rd:
        m_rd["mask"] = dict(size=w_rd)
    c, kr = plain.latent_rows(xa.to(F64), _w64(ws), "", m_src, 1e-5, pos)
    ref_src = plain.latent_attention(xa.to(F64), _w64(ws), "", m_src, pos, c, kr)
    ref_rd = plain.latent_attention(xb.to(F64), _w64(wr), "", m_rd, pos, c, kr)
    for what, cuts in {"whole": [T], "portions": [2, 70, 3, 75], "a prompt and single tokens": [100] + [1] * 50}.items():
        slot = cache.alloc_slots(1)[0]
        got_s, got_r, at = [], [], 0
        for n in cuts:
            ctx, plan = _context(cache, [(slot, n)], dtype)
            for part, ms, x, got in ((src, mslot, xa, got_s), (rd, reader, xb, got_r)):
                res = torch.full((n, hidden), float("nan"), dtype=torch.float32, device=DEV)
                part.forward(x[at:at + n].to(DEV).to(dtype), res, ctx, ms, store=True)
                got.append(res.cpu())
            cache.end_step(plan)
            at += n
        cache.free_slots([slot])
        f = 3.0 if dtype == torch.float32 else 6.0
        helpers.assert_close(torch.cat(got_s).numpy(), ref_src.numpy(), _name(dtype), f"{what}: the writer", factor=f)
        helpers.assert_close(torch.cat(got_r).numpy(), ref_rd.numpy(), _name(dtype), f"{what}: the reader", factor=f)


# -- two mixers side by side in a sandwich of layer norms ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_with_two_normed_mixers_side_by_side(dtype):
    from hymt2sharp_b200.parts import PartSpec, build_part
    W = 48
    norm = lambda n: PartSpec("layernorm", dict(dim=W, eps=1e-5, weight=n))
    left = PartSpec("talking_attention", dict(hidden=W, heads=2, kv_heads=1, dim=8, scale=0.4, position=None, q_proj="mix.left.q", k_proj="mix.left.k",
                                              o_proj="mix.left.o", talk="mix.left.talk", temp="mix.left.temp", sink="mix.left.sink", g_proj="mix.left.g",
                                              mask="chunk", mask_size=9, taps=2, q_conv="mix.left.q.conv", k_conv="mix.left.k.conv"))
    r = "mix.right."
    right = PartSpec("gated_delta", dict(hidden=W, heads=2, kv_heads=2, dim=8, vdim=6, taps=3, eps=1e-5, q_proj=r + "q", k_proj=r + "k", v_proj=r + "v",
                                         q_conv=r + "q.conv", k_conv=r + "k.conv", v_conv=r + "v.conv", b_proj=r + "b", a_log=r + "A_log", a1_proj=r + "a1",
                                         a2_proj=r + "a2", dt_bias=r + "dt_bias", g1_proj=r + "g1", g2_proj=r + "g2", norm=r + "norm", o_proj=r + "o",
                                         decay_rank=3, gate_rank=3))
    ff = PartSpec("clamped_glu", dict(hidden=W, intermediate=20, limit=1.0, alpha=1.702, gate_proj="mlp.gate", up_proj="mlp.up", down_proj="mlp.down",
                                      gate_bias="mlp.gate.b", up_bias="mlp.up.b", down_bias="mlp.down.b"))
    block = build_part("block", PartSpec("sandwich", dict(norm1=norm("norm1"), mixer=None, norm1_after=norm("norm1b"), norm2=norm("norm2"),
                                                          feed_forward=ff, norm2_after=norm("norm2b"),
                                                          mixers=[(left, "mix.left.out", 0.5), (right, "mix.right.out", 0.5)], mixers_eps=1e-5)))
    torch.manual_seed(3)
    w = _weights(block, 0.3)
    block.load(w, DEV, dtype)
    needs, states = block.cache_needs(), block.state_bytes()
    assert len(needs) == 2 and needs[0] is not None and needs[1] is None and states[0] > 0 and states[1] > 0

    class One:
        def __init__(self, i): self.i = i
        def cache_need(self): return needs[self.i]
        def state_bytes(self): return states[self.i]
    cache, mslots = _cache_for([One(0), One(1)], dtype)
    T = 40
    x = torch.randn(T, W)
    layer = dict(type="parallel", mixer=dict(left=dict(heads=2, kv_heads=1, dim=8, scale=0.4, mask=dict(size=9)),
                                             right=dict(heads=2, kv_heads=2, dim=8, vdim=6)), mlp=dict(limit=1.0))
    W64 = {"l0." + k: v for k, v in _w64(w).items()}
    h = plain.layer_norm(x.to(F64), W64["l0.norm1"], 1e-5)
    ref = x.to(F64) + plain.layer_norm(plain.parallel(h, W64, "l0.mix.", layer["mixer"], 1e-5, torch.arange(T)), W64["l0.norm1b"], 1e-5)
    ref = ref + plain.layer_norm(plain.clamped_glu(plain.layer_norm(ref, W64["l0.norm2"], 1e-5), W64, "l0.mlp.", 1.0), W64["l0.norm2b"], 1e-5)
    slot = cache.alloc_slots(1)[0]
    res = x.to(DEV).clone()
    for n, at in ((25, 0), (15, 25)):
        ctx, plan = _context(cache, [(slot, n)], dtype)
        piece = res[at:at + n].clone()
        block.forward(piece, ctx, mslots)
        res[at:at + n] = piece
        cache.end_step(plan)
    helpers.assert_close(res.cpu().numpy(), ref.numpy(), _name(dtype), "two portions", factor=3.0 if dtype == torch.float32 else 6.0)
