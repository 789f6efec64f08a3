"""The mechanisms of the Rutetar design one by one, each built from its own parameters with weights of its own, against the
plain functions: the residual in streams, the norm with a weight around zero, retention, time mixing with its token shift,
the attention with biases, a window and a gate per head, the gated feed-forward, the mixture with a router bias and weights
over the chosen outputs, and the block that holds two mixers side by side."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain import rutetar_plain as plain

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
    """A cache with one plane for every mixer that keeps keys and the state bytes of all of them; returns (cache, slots of the mixers)."""
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


def _weights(part, scale=0.1):
    out = {}
    for n, s in part.tensors().items():
        shape = tuple(3 if d == -1 else d for d in s.shape)
        base = torch.eye(*shape) if s.init == "identity" else (1.0 if s.init == "gain" else 0.0)
        out[n] = (torch.randn(shape) * (scale if len(shape) == 2 else 0.1) + base).to(torch.bfloat16)
    return out


def _run_mixer(part, cache, mslot, schedule, xs, dtype):
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


# -- the residual in streams ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S, T, W, B", [(1, 5, 44, 1), (2, 130, 256, 2), (3, 7, 37, 1), (8, 3, 1030, 4)])
def test_streams_read_write_and_both_at_once(dtype, S, T, W, B):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(S * T)
    X = torch.randn(S, T, W)
    w_in, w_out, mix = torch.randn(S), torch.randn(S), torch.eye(S) + 0.3 * torch.randn(S, S)
    gain = (1.0 + 0.1 * torch.randn(W))
    ys, scales = [torch.randn(T, W) for _ in range(B)], [0.6, 0.9, -1.5, 2.0][:B]
    Xd = X.to(DEV)
    first = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.streams_step(Xd, read=(w_in.to(DEV), gain.to(DEV), 1e-5, first))
    ref = plain.unit_rms(plain.streams_read(X.to(F64), w_in.to(F64)), 1e-5) * gain.to(F64)
    helpers.assert_close(first.float().cpu().numpy(), ref.numpy(), _name(dtype), "read", factor=0.5)
    y = sum(s * b.to(F64) for s, b in zip(scales, ys))
    Xn = plain.streams_write(X.to(F64), y, mix.to(F64), w_out.to(F64))
    two = Xd.clone()
    ops.streams_step(two, write=(mix.to(DEV).reshape(-1), w_out.to(DEV), [b.to(DEV) for b in ys], scales))
    helpers.assert_close(two.cpu().numpy(), Xn.numpy(), "float32", "write")
    out = torch.empty(T, W, dtype=dtype, device=DEV)
    ops.streams_step(Xd, write=(mix.to(DEV).reshape(-1), w_out.to(DEV), [b.to(DEV) for b in ys], scales), read=(w_in.to(DEV), gain.to(DEV), 1e-5, out))
    assert torch.equal(Xd, two)
    ref = plain.unit_rms(plain.streams_read(Xn, w_in.to(F64)), 1e-5) * gain.to(F64)
    helpers.assert_close(out.float().cpu().numpy(), ref.numpy(), _name(dtype), "write and read", factor=0.5)
    total = torch.empty(T, W, dtype=torch.float32, device=DEV)
    ops.streams_step(Xd, read=(torch.ones(S, device=DEV), None, 0.0, total))
    helpers.assert_close(total.cpu().numpy(), Xn.sum(0).numpy(), "float32", "sum")
    Xd[1:] = float("nan")
    ops.streams_fill(Xd)
    assert all(torch.equal(Xd[s], Xd[0]) for s in range(S))


def test_norm_with_a_weight_around_zero_keeps_the_weight_in_bfloat16():
    from hymt2sharp_b200.parts import PartSpec, build_part
    norm = build_part("norm", PartSpec("rmsnorm", dict(dim=40, eps=1e-6, weight="w", offset=1.0)))
    w = (torch.randn(40) * 0.01).to(torch.bfloat16)        # 1 + w rounded to bfloat16 would lose all of it
    norm.load({"w": w}, DEV, torch.bfloat16)
    x = torch.randn(9, 40)
    out = norm.forward(x.to(DEV), None, torch.float32, fresh=True)
    helpers.assert_close(out.cpu().numpy(), plain.offset_norm(x.to(F64), w.to(F64), 1e-6).numpy(), "float32", "offset norm")


# -- retention ---------------------------------------------------------------------------------------------------------------
def _retention(hidden, heads, dim, vdim, decay):
    from hymt2sharp_b200.parts import PartSpec, build_part
    return build_part("mixer", PartSpec("retention", dict(hidden=hidden, heads=heads, dim=dim, vdim=vdim, decay=decay, eps=1e-5, q_proj="q",
                                                          k_proj="k", v_proj="v", g_proj="g", o_proj="o")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, dim, vdim", [(44, 3, 6, 10), (64, 2, 16, 40), (64, 1, 32, 8), (128, 2, 64, 128), (64, 1, 128, 64), (48, 2, 24, 100)])
def test_retention_in_prompts_portions_decoding_and_batches(dtype, hidden, heads, dim, vdim):
    """State columns in registers (16, 32, 64, 128 key entries) and in shared memory (6, 24); more value columns than a block
    holds; a whole prompt long enough for the three passes over chunks, the same serially in portions, and single tokens;
    a second, shorter sequence beside it; then the slots used again by other sequences."""
    torch.manual_seed(hidden + dim)
    decay = [0.9, 0.97, 0.999][:heads]
    part = _retention(hidden, heads, dim, vdim, decay)
    w = _weights(part, 0.15)
    part.load(w, DEV, dtype)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (330, 70)]
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay)
    w64 = {k: v.to(F64) for k, v in w.items()}
    refs = [plain.retention_mixer(x.to(F64), w64, "", m, 1e-5).numpy() for x in xs]
    cache, (mslot,) = _cache_for([part], dtype)
    cache.state.fill_(255)                     # a slot's row is zeroed when it is handed out, and ignored at position 0
    schedules = {
        "whole, in one batch": [[(0, 330), (1, 70)]],
        "portions down to two tokens": [[(0, 2), (1, 2)], [(0, 3), (1, 64)], [(0, 191), (1, 4)], [(0, 64)], [(0, 70)]],
        "a prompt, then single tokens": [[(0, 300), (1, 40)]] + [[(0, 1), (1, 1)]] * 30,
        "one token at a time from the start": [[(1, 1)]] * 70,
    }
    for what, schedule in schedules.items():
        got = _run_mixer(part, cache, mslot, schedule, xs, dtype)
        for i, g in enumerate(got):
            if g.shape[0]:
                helpers.assert_close(g.numpy(), refs[i][:g.shape[0]], _name(dtype), f"retention {what}, sequence {i}", factor=2.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, dv, shift", [(3, 4, 0), (2, 36, 0), (2, 128, 0), (1, 132, 0), (2, 256, 4), (1, 300, 0), (2, 512, 0), (1, 516, 0),
                                              (3, 7, 0), (2, 64, 3), (2, 10, 0)])
def test_head_norm_with_gain_and_gate_at_every_width(dtype, heads, dv, shift):
    """A head's output over its root mean square, times a gain, times silu(gate): heads that a lane holds in one, two and four
    16-byte pieces, heads wider than that, widths that are no multiple of 4, and a gate that is a column range of a wider
    matrix starting at an aligned or an odd column."""
    from hymt2sharp_b200.kernels import ops
    g = torch.Generator().manual_seed(dv * 7 + heads)
    T, D = 37, heads * dv
    o = torch.randn(T, D, generator=g) * torch.rand(T, 1, generator=g) * 5
    wide = torch.randn(T, shift + D + (4 if shift == 4 else 5), generator=g).to(dtype)   # rows of 4 k entries keep the wide form
    gain = 1 + 0.3 * torch.randn(D, generator=g)
    for use_gain, use_gate in ((True, True), (False, True), (True, False), (False, False)):
        want = plain.unit_rms(o.to(F64).reshape(T, heads, dv), 1e-5).reshape(T, D)
        if use_gain:
            want = want * gain.to(F64)
        if use_gate:
            want = want * plain.silu(wide[:, shift:shift + D].to(F64))
        out = torch.full((T, D), float("nan"), dtype=dtype, device=DEV)
        gate = wide.to(DEV)[:, shift:shift + D] if use_gate else None
        ops.head_norm_gate(out, o.to(DEV), gate, gain.to(DEV) if use_gain else None, heads, dv, 1e-5)
        helpers.assert_close(out.double().cpu(), want, _name(dtype), f"head norm heads={heads} dv={dv} gain={use_gain} gate={use_gate}")


def test_retention_remembers_a_far_token_and_forgets_at_its_rate():
    """One token's key and value stand out among hundreds; with a decay of 1 - 2^-10 it is still there 600 tokens on (in the
    prompt's chunks and in decoded steps), with 0.9 it is gone: queries that point at the key read decay^distance * value."""
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.cache import PagedCache
    torch.manual_seed(5)
    heads, dim, vdim, T, at = 2, 16, 32, 640, 17
    direction = torch.nn.functional.normalize(torch.randn(heads, dim), dim=-1)
    q = direction.reshape(1, -1).repeat(T, 1)
    k = torch.randn(T, heads * dim) * 1e-3
    v = torch.randn(T, heads * vdim)
    k[at] = (direction * 50.0).reshape(-1)
    decay = torch.tensor([1.0 - 2.0 ** -10, 0.9])
    cache = PagedCache([], torch.float32, DEV, 1024, max_slots=2, state_bytes=4 * heads * dim * vdim)
    for steps in ([T], [600] + [1] * 40):
        slot = cache.alloc_slots(1)[0]
        outs, pos = [], 0
        for n in steps:
            ctx, plan = _context(cache, [(slot, n)], torch.float32)
            o = torch.empty(n, heads * vdim, device=DEV)
            sl = slice(pos, pos + n)
            from hymt2sharp_b200.parts.state_scan import chunk_plan
            ops.linear_scan(o, q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), ops.SCAN_FIXED_DECAY, cache.state, 0, ctx.cu_seqlens, ctx.slot_ids,
                            ctx.kv_lens, 1, heads, dim, vdim, decay=decay.to(DEV), k_scale=1.0, chunks=chunk_plan(ctx))
            cache.end_step(plan)
            outs.append(o.cpu()); pos += n
        o = torch.cat(outs).reshape(T, heads, vdim)
        cache.free_slots([slot])
        for t in (at, at + 1, 300, T - 1):
            want = 50.0 * float(decay[0]) ** (t - at) * v[at].reshape(heads, vdim)[0]
            assert torch.allclose(o[t, 0], want, atol=0.05), (steps[:2], t)
        assert o[at - 1, 0].abs().max() < 0.05 and o[T - 1, 1].abs().max() < 0.05


# -- time mixing ---------------------------------------------------------------------------------------------------------------
def _time_mix(hidden, heads, dim, rank):
    from hymt2sharp_b200.parts import PartSpec, build_part
    return build_part("mixer", PartSpec("time_mix", dict(hidden=hidden, heads=heads, dim=dim, eps=1e-5, decay_rank=rank, mu="mu.{}", r_proj="r",
                                                         k_proj="k", v_proj="v", g_proj="g", w1_proj="w1", w2_proj="w2", w0="w0", bonus="u",
                                                         norm="norm", o_proj="o")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, dim, rank", [(44, 3, 5, 3), (64, 2, 32, 16), (128, 2, 64, 8), (96, 1, 16, 1), (256, 2, 128, 32), (40, 1, 24, None),
                                                      (512, 8, 64, 16)])
def test_time_mixing_in_prompts_portions_decoding_and_batches(dtype, hidden, heads, dim, rank):
    """(The last shape's four projections are large enough for the tensor-core kernel at every number of tokens.)"""
    torch.manual_seed(hidden + dim)
    part = _time_mix(hidden, heads, dim, rank)
    w = _weights(part, 0.15)
    w["w0"] = (torch.randn(heads * dim) - 1.0).to(torch.bfloat16)      # decays from nearly 1 down to 0.1 a token
    w["w2"] = (w["w2"].float() * 5).to(torch.bfloat16)
    for s in "rkvgw":
        w[f"mu.{s}"] = torch.rand(hidden).to(torch.bfloat16)
    part.load(w, DEV, dtype)
    xs = [torch.randn(n, hidden).to(torch.bfloat16).float() for n in (330, 70)]
    m = dict(heads=heads, dim=dim)
    w64 = {k: v.to(F64) for k, v in w.items()}
    refs = [plain.time_mixer(x.to(F64), w64, "", m, 1e-5).numpy() for x in xs]
    cache, (mslot,) = _cache_for([part], dtype)
    cache.state.fill_(255)
    schedules = {
        "whole, in one batch": [[(0, 330), (1, 70)]],
        "portions down to two tokens": [[(0, 2), (1, 2)], [(0, 3), (1, 64)], [(0, 191), (1, 4)], [(0, 64)], [(0, 70)]],
        "a prompt, then single tokens": [[(0, 300), (1, 40)]] + [[(0, 1), (1, 1)]] * 30,
        "one token at a time from the start": [[(1, 1)]] * 70,
    }
    for what, schedule in schedules.items():
        got = _run_mixer(part, cache, mslot, schedule, xs, dtype)
        for i, g in enumerate(got):
            if g.shape[0]:
                helpers.assert_close(g.numpy(), refs[i][:g.shape[0]], _name(dtype), f"time mixing {what}, sequence {i}", factor=2.0)


def test_token_shift_takes_the_row_before_across_steps():
    """The first token of a step reads the last row of the step before from the state, a sequence's first token reads zeros
    whatever the slot held, and a padding row (slot -1) reads zeros and leaves nothing behind."""
    from hymt2sharp_b200.cache import PagedCache
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(1)
    W = 20
    cache = PagedCache([], torch.float32, DEV, 256, max_slots=3, state_bytes=4 * W + 16)
    cache.state.fill_(77)
    a, b = cache.alloc_slots(2)
    cache.state.fill_(77)
    mu = torch.rand(2, W)
    h = [torch.randn(9, W), torch.randn(4, W)]
    ref = [torch.cat([plain.token_shift(x.to(F64), mu[s].to(F64)) for s in range(2)], dim=1) for x in h]
    got = [[], []]
    for step in ([(a, 0, 3), (b, 1, 1)], [(a, 0, 1), (b, 1, 1)], [(a, 0, 5), (b, 1, 2)]):
        ctx, plan = _context(cache, [(s, n) for s, _, n in step], torch.float32)
        at = [sum(g.shape[0] for g in got[i]) for i in range(2)]
        x = torch.cat([h[i][at[i]:at[i] + n] for _, i, n in step]).to(DEV)
        out = torch.empty(x.shape[0], 2 * W, device=DEV)
        ops.token_shift(out, x, mu.to(DEV), cache.state, 16, ctx.token_seq, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens)
        cache.end_step(plan)
        o = 0
        for _, i, n in step:
            got[i].append(out[o:o + n].cpu()); o += n
    for i in range(2):
        helpers.assert_close(torch.cat(got[i]).numpy(), ref[i].numpy(), "float32", f"token shift, sequence {i}")


# -- the attention with biases, a window and a gate per head ----------------------------------------------------------------
def _window_attention(hidden, heads, kv, d, dv, dims, window, scale):
    from hymt2sharp_b200.parts import PartSpec, build_part
    return build_part("mixer", PartSpec("gqa_attention", dict(
        hidden=hidden, heads=heads, kv_heads=kv, head_dim=d, value_dim=dv, scale=scale, eps=1e-5, qk_norm=False, window=window,
        position=PartSpec("wavelength_scaled_rope", dict(dims=dims, base=1000.0, scaling=None)), q_proj="q", k_proj="k", v_proj="v",
        o_proj="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", head_gate="g")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, heads, kv, d, dv, dims, window", [
    (44, 3, 1, 10, 6, 4, 7),               # odd sizes, a window shorter than a block, part of a head rotated
    (64, 4, 4, 16, 16, 16, 70),            # as many kv heads as heads, the whole head rotated, a window longer than a block
    (64, 2, 1, 24, 40, 0, None),           # no rotation, no window
    (128, 4, 2, 64, 128, 32, 100),         # from here on the bfloat16 engine runs its tensor-core prompt kernel and its streaming
    (128, 2, 2, 128, 64, 128, 130),        # decode kernel
    (128, 8, 2, 64, 64, 48, 300),          # a window that the sequence never fills
])
def test_gated_window_attention_in_prompts_portions_and_decoding(dtype, hidden, heads, kv, d, dv, dims, window):
    torch.manual_seed(hidden + d + (window or 0))
    scale = 0.7 / math.sqrt(d)
    part = _window_attention(hidden, heads, kv, d, dv, dims, window, scale)
    w = _weights(part)
    for n in ("q.b", "k.b", "v.b"):
        w[n] = (torch.randn(w[n].shape) * 0.5).to(torch.bfloat16)
    w["g"] = (w["g"].float() * 5).to(torch.bfloat16)
    part.load(w, DEV, dtype)
    T = 290
    xs = [torch.randn(T, hidden).to(torch.bfloat16).float()]
    m = dict(heads=heads, kv_heads=kv, dim=d, vdim=dv, scale=scale, rot=dict(dims=dims, base=1000.0), mask=dict(size=window or 10 ** 6))
    ref = plain.gated_window_mixer(xs[0].to(F64), {k: v.to(F64) for k, v in w.items()}, "", m, torch.arange(T)).numpy()
    for steps in ([T], [2, 3, 59, 1, 63, 130, 32], [258] + [1] * 32):
        cache, (mslot,) = _cache_for([part], dtype)
        got = _run_mixer(part, cache, mslot, [[(0, n)] for n in steps], xs, dtype)[0]
        helpers.assert_close(got.numpy(), ref, _name(dtype), f"attention d={d} dv={dv} window={window} steps {steps[:3]}", factor=2.0)
        cache.book.audit()


def _planted_in_window(dtype, d, dv, window, key_at, length, decode_from):
    """Keys of small random entries except ONE, which is the query's direction made long, in a cache group that hands blocks
    back as the window moves on: a row's output is that key's value exactly as long as the key is among the row's last
    `window` positions.  Written through the appending kernel, read by the engine's own choice of attention kernel."""
    from hymt2sharp_b200.cache import GroupSpec, PagedCache
    from hymt2sharp_b200.kernels import fast, ops
    torch.manual_seed(key_at + window)
    nkv, g = 2, 2
    nh = nkv * g
    cache = PagedCache([GroupSpec("window", nkv, d, 1, window, 2, 0 if dv == d else dv)], dtype, DEV, 4096, max_slots=4)
    slots = cache.alloc_slots(2)
    lens = [length, 30]
    direction = torch.nn.functional.normalize(torch.randn(nkv, d), dim=-1)
    ks = [torch.randn(n, nkv, d) * 0.05 for n in lens]
    vs = [torch.randn(n, nkv, dv) for n in lens]
    ks[0][key_at] = direction * 4.0
    qs = [direction[:, None, :].expand(nkv, g, d).reshape(1, nh * d).repeat(n, 1) * 4.0 for n in lens]
    steps = [[min(decode_from, n) for n in lens]] + [[1 if decode_from + i < n else 0 for n in lens] for i in range(max(lens) - decode_from)]
    k_plane, v_plane = cache.plane(0, 0)
    outs, at = {}, [0, 0]
    for step in steps:
        idx = [i for i, n in enumerate(step) if n]
        ctx, plan = _context(cache, [(slots[i], step[i]) for i in idx], dtype)
        proj = torch.cat([torch.cat([qs[i][at[i]:at[i] + step[i]], ks[i][at[i]:at[i] + step[i]].reshape(step[i], -1),
                                     vs[i][at[i]:at[i] + step[i]].reshape(step[i], -1)], dim=1) for i in idx]).to(DEV).to(dtype)
        T = proj.shape[0]
        q = torch.empty(T, nh * d, dtype=dtype, device=DEV)
        ops.rope_kv_general(proj, q, k_plane, v_plane, cache.tables[0], cache.block_tokens, ctx.token_seq, ctx.token_pos, ctx.slot_ids,
                            None, 0, None, None, ops.NORM_NONE, 1e-5, nh, nkv, d, dv, True)
        out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
        if not fast.try_attention_kv(out, q, k_plane, v_plane, cache.tables[0], ctx, nh, nkv, d, dv, 1.0, window, False):
            split, ms, acc, ml = 0, 0, None, None
            if ctx.decode and ctx.max_kv_len > 256:
                split, ms = 256, -(-ctx.max_kv_len // 256)
                na, nm = ops.attention_simt_scratch(T, nh, dv, ms)
                acc, ml = torch.empty(na, device=DEV), torch.empty(nm, device=DEV)
            ops.attention_simt_kv(out, q, k_plane, v_plane, cache.tables[0], ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs,
                                  ctx.max_new_tokens, nh, nkv, d, dv, 1.0, window, False, split, ms, acc, ml)
        cache.end_step(plan)
        o = 0
        for i in idx:
            for j in range(step[i]):
                outs[(i, at[i] + j)] = out[o + j].float().cpu().reshape(nkv, g, dv)
            o += step[i]; at[i] += step[i]
    return outs, vs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, dv", [(16, 24), (64, 128)])
@pytest.mark.parametrize("window, key_at", [(40, 3), (40, 100), (64, 63), (65, 192), (1, 70), (200, 0), (130, 127)])
def test_a_key_is_seen_up_to_the_windows_edge_and_not_beyond(dtype, d, dv, window, key_at):
    """The last row that sees the key (window - 1 positions on) and the first that does not, as a prompt's rows and as decoded
    steps, beside a second sequence; with windows around a block's size and a key at a block's first and last place."""
    length = key_at + window + 12
    tol = 0.05 if dtype == torch.bfloat16 else 2e-3
    for decode_from in (length, max(1, key_at + window - 3)):
        outs, vs = _planted_in_window(dtype, d, dv, window, key_at, length, decode_from)
        want = vs[0][key_at][:, None, :]
        for t in (key_at, key_at + window // 2, key_at + window - 1):
            assert torch.allclose(outs[(0, t)], want.expand_as(outs[(0, t)]), atol=tol), (t, decode_from)
        for t in (key_at + window, key_at + window + 1, length - 1):
            assert not torch.allclose(outs[(0, t)], want.expand_as(outs[(0, t)]), atol=0.3), (t, decode_from)
        if key_at > 0:
            assert not torch.allclose(outs[(0, key_at - 1)], want.expand_as(outs[(0, key_at - 1)]), atol=0.3)


# -- feed-forwards -------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, ff, tokens", [(44, 13, 5), (128, 256, 200)])
def test_gated_feed_forward_with_the_tanh_form_of_gelu(dtype, hidden, ff, tokens):
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(ff)
    part = build_part("feed_forward", PartSpec("swiglu", dict(hidden=hidden, intermediate=ff, activation="gelu_tanh", gate_proj="gate",
                                                              up_proj="up", down_proj="down")))
    w = _weights(part, 0.3)
    part.load(w, DEV, dtype)
    x = torch.randn(tokens, hidden).to(torch.bfloat16).float()
    cache, _ = _cache_for([], dtype)
    ctx, plan = _context(cache, [(cache.alloc_slots(1)[0], tokens)], dtype)
    ref = plain.gated_feed_forward(x.to(F64), w["gate"].to(F64), w["up"].to(F64), w["down"].to(F64), plain.gelu_tanh).numpy()
    stored = torch.full((tokens, hidden), float("nan"), device=DEV)
    part.forward(x.to(DEV).to(dtype), stored, ctx, store=True)
    helpers.assert_close(stored.cpu().numpy(), ref, _name(dtype), "stored", factor=2.0)
    added = torch.ones(tokens, hidden, device=DEV)
    part.forward(x.to(DEV).to(dtype), added, ctx)
    helpers.assert_close(added.cpu().numpy() - 1.0, ref, _name(dtype), "added", factor=2.0)


@pytest.mark.parametrize("outputs, top", [(5, 1), (16, 4), (3, 3), (70, 8)])
def test_routing_with_a_bias_and_weights_over_the_chosen(outputs, top):
    from hymt2sharp_b200.kernels import ops
    torch.manual_seed(outputs)
    for T in (3, 200):                          # the one-launch form for few pairs, and the three kernels
        z = torch.randn(T, outputs) * 2
        z[0, : min(3, outputs)] = 1.5           # ties: the lower index wins
        bias = torch.randn(outputs)
        bias[: min(3, outputs)] = 0.25
        chosen = torch.empty(T, top, dtype=torch.int32, device=DEV)
        weight = torch.empty(T, top, device=DEV)
        ops.moe_route(chosen, weight, z.to(DEV), None, bias.to(DEV), True)
        eye_router = torch.eye(outputs, dtype=F64)
        for t in range(T):
            want, ww = plain.route(z[t].to(F64), eye_router, bias.to(F64), top)
            assert chosen[t].tolist() == want, t
            assert torch.allclose(weight[t].cpu().double(), ww, atol=1e-6)
        if T * top <= ops.MOE_SMALL_PAIRS:
            tile = ops.gemm_group_tile("skinny")
            tiles = ops.moe_tiles(T, top, outputs, tile)
            c2, w2 = torch.empty_like(chosen), torch.empty_like(weight)
            pair_row = torch.empty(T, top, dtype=torch.int32, device=DEV)
            row_token = torch.empty(tiles * tile, dtype=torch.int32, device=DEV)
            tile_group = torch.empty(tiles + 1, dtype=torch.int32, device=DEV)
            ops.moe_route_place(c2, w2, pair_row, row_token, tile_group, z.to(DEV), None, outputs, tile, bias.to(DEV), True)
            assert torch.equal(c2, chosen) and torch.equal(w2, weight)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden, experts, top, ff, tokens", [(44, 5, 1, 9, 7), (44, 3, 3, 5, 40), (128, 16, 4, 64, 3), (128, 16, 4, 64, 300), (64, 2, 1, 24, 1)])
def test_mixture_of_gated_experts_against_plain(dtype, hidden, experts, top, ff, tokens):
    """Every grouped kernel by the step's size (few rows, tensor cores, general), one token alone and a whole step."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(hidden + experts + tokens)
    part = build_part("feed_forward", PartSpec("routed_experts", dict(
        hidden=hidden, experts=experts, identity=0, top=top, intermediate=ff, activation="silu", router="router", router_bias="router.b",
        weights="chosen_softmax", gate_proj="e{}.gate", up_proj="e{}.up", down_proj="e{}.down")))
    w = _weights(part, 0.3)
    # router outputs a whole unit apart for every token: the choice never rests on rounding, the weights still differ by token
    w["router"] = (torch.randn(experts, hidden) * 0.02).to(torch.bfloat16)
    w["router.b"] = torch.randperm(experts).float().to(torch.bfloat16)
    part.load(w, DEV, dtype)
    x = torch.randn(tokens, hidden).to(torch.bfloat16).float()
    mlp = dict(router=dict(top=top, experts=experts))
    ref = plain.mixture(x.to(F64), {k: v.to(F64) for k, v in w.items()}, "", mlp).numpy()
    cache, _ = _cache_for([], dtype)
    ctx, plan = _context(cache, [(cache.alloc_slots(1)[0], tokens)], dtype)
    out = torch.full((tokens, hidden), float("nan"), device=DEV)
    part.forward(x.to(DEV).to(dtype), out, ctx, store=True)
    helpers.assert_close(out.cpu().numpy(), ref, _name(dtype), "mixture", factor=2.0)
    ctx1, _ = _context(cache, [(cache.alloc_slots(1)[0], 1)], dtype)
    one = torch.zeros((1, hidden), device=DEV)
    part.forward(x[-1:].to(DEV).to(dtype), one, ctx1)
    helpers.assert_close(one.cpu().numpy(), ref[-1:], _name(dtype), "one token alone", factor=2.0)


# -- the block ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams, with_ff", [(3, True), (1, True), (2, False), (None, True)])
def test_block_with_two_mixers_side_by_side_over_streams(dtype, streams, with_ff):
    """Two blocks in a row (the second one's input is prepared by the first one's last kernel), in a prompt and in
    single-token steps: attention and time mixing side by side with two scales, then a retention block."""
    from hymt2sharp_b200.parts import PartSpec, build_part
    torch.manual_seed(11 + (streams or 0))
    H, S = 48, streams or 1
    def norm(n):
        return PartSpec("rmsnorm", dict(dim=H, eps=1e-5, weight=n, offset=1.0))
    def tables(p, q):
        return None if streams is None else {k: f"{p}hc{q}.{k}" for k in ("in", "out", "mix")}
    left = PartSpec("gqa_attention", dict(hidden=H, heads=2, kv_heads=1, head_dim=8, value_dim=12, scale=0.3, eps=1e-5, qk_norm=False, window=9,
                                          position=PartSpec("wavelength_scaled_rope", dict(dims=4, base=100.0, scaling=None)),
                                          q_proj="a.mix.left.q", k_proj="a.mix.left.k", v_proj="a.mix.left.v", o_proj="a.mix.left.o",
                                          q_bias="a.mix.left.q.b", k_bias="a.mix.left.k.b", v_bias="a.mix.left.v.b", head_gate="a.mix.left.g"))
    r = "a.mix.right."
    right = PartSpec("time_mix", dict(hidden=H, heads=2, dim=8, eps=1e-5, decay_rank=4, mu=r + "mu.{}", r_proj=r + "r", k_proj=r + "k", v_proj=r + "v",
                                      g_proj=r + "g", w1_proj=r + "w1", w2_proj=r + "w2", w0=r + "w0", bonus=r + "u", norm=r + "norm", o_proj=r + "o"))
    ff = PartSpec("swiglu", dict(hidden=H, intermediate=40, activation="gelu_tanh", gate_proj="a.mlp.gate", up_proj="a.mlp.up", down_proj="a.mlp.down"))
    a = build_part("block", PartSpec("streams", dict(streams=S, norm1=norm("a.norm1"), mixers=[(left, 0.6), (right, -1.3)], hyper1=tables("a.", 1),
                                                      **(dict(norm2=norm("a.norm2"), feed_forward=ff, hyper2=tables("a.", 2)) if with_ff else {}))))
    ret = PartSpec("retention", dict(hidden=H, heads=2, dim=6, vdim=10, decay=[0.9, 0.99], eps=1e-5, q_proj="b.mix.q", k_proj="b.mix.k",
                                     v_proj="b.mix.v", g_proj="b.mix.g", o_proj="b.mix.o"))
    b = build_part("block", PartSpec("streams", dict(streams=S, norm1=norm("b.norm1"), mixers=[(ret, 1.0)], hyper1=tables("b.", 1))))
    w = {**_weights(a, 0.2), **_weights(b, 0.2)}
    a.load(w, DEV, dtype); b.load(w, DEV, dtype)
    w64 = {k: v.to(F64) for k, v in w.items()}
    T = 40
    x0 = torch.randn(T, H)
    # plain: the two layers by the plain model's own loop
    cfg = dict(norm=dict(eps=1e-5), layers=[
        dict(type="parallel", mixer=dict(left=dict(heads=2, kv_heads=1, dim=8, vdim=12, scale=0.3, rot=dict(dims=4, base=100.0), mask=dict(size=9)),
                                         right=dict(heads=2, dim=8), left_scale=0.6, right_scale=-1.3), mlp=dict(kind="dense", ff=40) if with_ff else None),
        dict(type="retention", mixer=dict(heads=2, dim=6, vdim=10, decay=[0.9, 0.99]), mlp=None)])
    if streams is not None:
        cfg["streams"] = streams
    names = {"a.": "l0.", "b.": "l1."}
    wp = {names[k[:2]] + k[2:]: v for k, v in w64.items()}
    wp.update({"embed": x0.to(F64), "final.norm": torch.zeros(H, dtype=F64), "head": torch.eye(H, dtype=F64)})
    _, seen = plain.forward(cfg, wp, list(range(T)), layers_out=True)
    cache, mslots = _cache_for(a.mixers + b.mixers, dtype)
    slot = cache.alloc_slots(1)[0]
    got, at = [], 0
    for n in [25] + [1] * 15:
        ctx, plan = _context(cache, [(slot, n)], dtype)
        X = x0[at:at + n].to(DEV)[None].repeat(S, 1, 1).contiguous()
        ctx.block_ahead = b
        a.forward(X, ctx, mslots[:2])
        assert ("stream_rows" in ctx.shared)
        ctx.block_ahead = None
        b.forward(X, ctx, mslots[2:])
        assert "stream_rows" not in ctx.shared
        cache.end_step(plan)
        got.append(X.sum(0).cpu()); at += n
    # a sequence's first tokens divide heads' outputs that are sums of a few terms by their root mean square, twice in a row
    # (time mixing, then retention): the rounding of bfloat16 products shows there enlarged, while the 32-bit run is held to
    # the shared limit
    helpers.assert_close(torch.cat(got).numpy(), seen[1].numpy(), _name(dtype), "two blocks over streams",
                         factor=2.0 if dtype == torch.float32 else 3.0)
