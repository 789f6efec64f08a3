"""The Rutetar design without a GPU: its configuration (every size read, errors that name their key), the registry, the
tensor list, the memory plan of a looped order, and the plain implementation's mechanisms against values worked out by hand."""
import copy
import math

import pytest
import torch

import rutetar_models
from plain import rutetar_plain as plain


def _cfg(name="odd"):
    return copy.deepcopy(rutetar_models.CONFIGS[name]["config"])


def test_every_size_is_read_and_written_back():
    from hymt2sharp_b200.config import RutetarConfig
    for name in rutetar_models.CONFIGS:
        raw = _cfg(name)
        cfg = RutetarConfig.from_dict(raw)
        assert cfg.to_dict() == raw
        assert RutetarConfig.from_dict(cfg.to_dict()) == cfg
    cfg = RutetarConfig.from_dict(_cfg("odd"))
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.norm_eps) == (101, 44, 3, 1e-5)
    a = cfg.layers[0].mixer
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim, a.left.window, a.left.rot_dims, a.left.rot_base) == (3, 1, 10, 6, 7, 4, 1000.0)
    assert (a.right.heads, a.right.dim, a.right.rank, a.left_scale, a.right_scale) == (3, 5, 3, 0.7, 1.2)
    assert cfg.layers[1].mixer.decay == (0.9, 0.97, 0.995) and cfg.layers[1].mlp is None
    assert (cfg.layers[0].mlp.kind, cfg.layers[0].mlp.experts, cfg.layers[0].mlp.top, cfg.layers[0].mlp.ff) == ("moe", 5, 1, 9)
    assert cfg.order() == [0, 1, 0, 1, 0, 1, 2, 3]
    bare = RutetarConfig.from_dict(_cfg("bare"))
    assert bare.streams is None and bare.loop is None and bare.order() == [0, 1]
    assert RutetarConfig.from_dict(_cfg("even")).layers[2].mixer.left.window is None


@pytest.mark.parametrize("change, key", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="conv"), "type 'conv'"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.9]), "mixer.decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=2), "mixer.left.kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "mixer.left.rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "mixer.left.scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "mixer.right_scale"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "mlp.router.top"),
    (lambda c: c["layers"][2]["mlp"].update(kind="glu"), "mlp.kind 'glu'"),
    (lambda c: c["loop"].update(stop=9), "loop.stop"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_errors_name_their_key(change, key):
    from hymt2sharp_b200.config import ConfigError, RutetarConfig
    raw = _cfg("odd")
    change(raw)
    with pytest.raises(ConfigError, match=key.replace(".", r"\.")):
        RutetarConfig.from_dict(raw)


def test_registry_tensor_list_and_memory_plan():
    from hymt2sharp_b200.config import RutetarConfig, get_architecture
    from hymt2sharp_b200.engine.model import DecoderModel
    arch = get_architecture("Rutetar")
    cfg = RutetarConfig.from_dict(_cfg("odd"))
    shapes = arch.tensor_shapes(cfg)
    assert shapes["l0.mix.left.q"].shape == (30, 44) and shapes["l0.mix.left.q.b"].shape == (30,)
    assert shapes["l0.mix.left.v"].shape == (6, 44) and shapes["l0.mix.left.g"].shape == (3, 44) and shapes["l0.mix.left.o"].shape == (44, 18)
    assert shapes["l0.mix.right.w1"].shape == (3, 44) and shapes["l0.mix.right.w2"].shape == (15, 3) and shapes["l0.mix.right.u"].shape == (3, 5)
    assert shapes["l0.mix.right.mu.w"].shape == (44,) and shapes["l0.mix.right.norm"].shape == (15,)
    assert shapes["l1.mix.g"].shape == (30, 44) and shapes["l1.mix.o"].shape == (44, 30) and "l1.mlp.gate" not in shapes and "l1.hc2.in" not in shapes
    assert shapes["l0.hc1.mix"].shape == (3, 3) and shapes["l0.hc2.out"].shape == (3,)
    assert shapes["l0.mlp.router.b"].shape == (5,) and shapes["l0.mlp.e4.gate"].shape == (9, 44) and shapes["l2.mlp.down"].shape == (44, 13)
    # a checkpoint's own width of the decay's inner projection
    raw = _cfg("odd")
    raw["layers"][0]["mixer"]["right"].pop("rank")
    open_rank = arch.tensor_shapes(RutetarConfig.from_dict(raw))
    assert open_rank["l0.mix.right.w1"].shape == (-1, 44) and open_rank["l0.mix.right.w2"].shape == (15, -1)
    bare = arch.tensor_shapes(RutetarConfig.from_dict(_cfg("bare")))
    assert not [n for n in bare if ".hc" in n]
    # three runs of layers 0 and 1: three cache planes of the window of 7, three states of each; the other window has its own group
    model = DecoderModel(arch.build_spec(cfg))
    assert [(g.kind, g.window, g.planes, g.kv_heads, g.head_dim, g.value_width) for g in model.groups] == [("window", 7, 3, 1, 10, 6), ("window", 90, 1, 4, 6, 6)]
    assert model.spec.residual_streams == 3 and [r.layer for r in model.spec.order] == [0, 1, 0, 1, 0, 1, 2, 3]
    states = [[s.state_bytes for s in row] for row in model.slots]
    assert states[0] == [0, 4 * (3 * 5 * 5 + 44)] and states[1] == [4 * 3 * 6 * 10] and states[6] == [4 * 12 * 4]
    offsets = [s.state_offset for row in model.slots for s in row if s.state_bytes]
    assert len(set(offsets)) == len(offsets) and model.state_bytes >= sum(sum(r) for r in states)
    assert [s.plane for row in model.slots for s in row if s.group == 0] == [0, 1, 2]


def test_step_chunks_of_a_long_portion():
    from types import SimpleNamespace
    from hymt2sharp_b200.kernels import ops
    from hymt2sharp_b200.parts.state_scan import chunk_plan
    chunk, minimum = ops.linear_scan_chunking()
    short = SimpleNamespace(shared={}, max_new_tokens=minimum - 1, host_new_tokens=[minimum - 1, 3], device=torch.device("cpu"))
    assert chunk_plan(short) is None
    news = [2 * chunk + 5, 1, chunk, minimum]
    ctx = SimpleNamespace(shared={}, max_new_tokens=max(news), host_new_tokens=news, device=torch.device("cpu"))
    count, cseq, cfirst, clen, seq0 = chunk_plan(ctx)
    per = [-(-n // chunk) for n in news]
    assert count == sum(per) and seq0.tolist() == [0] + [sum(per[:i + 1]) for i in range(len(per))]
    covered = []
    for s, f, l in zip(cseq.tolist(), cfirst.tolist(), clen.tolist()):
        assert 0 < l <= chunk
        covered += [(s, t) for t in range(f, f + l)]
    starts = [0, news[0], news[0] + news[1], news[0] + news[1] + news[2]]
    assert covered == [(s, starts[s] + t) for s, n in enumerate(news) for t in range(n)]
    assert chunk_plan(ctx) is ctx.shared["linear_scan_chunks"]


# -- the plain implementation against values worked out by hand ------------------------------------------------------------
def test_plain_norm_and_streams():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.offset_norm(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0), torch.tensor([[3.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))
    X = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=torch.float64)          # two streams, one token
    assert plain.streams_read(X, torch.tensor([2.0, 0.5], dtype=torch.float64)).tolist() == [[7.0, 14.0]]
    mix = torch.tensor([[1.0, 2.0], [0.0, 3.0]], dtype=torch.float64)                # [from, to]
    new = plain.streams_write(X, torch.tensor([[1.0, 1.0]], dtype=torch.float64), mix, torch.tensor([100.0, -1.0], dtype=torch.float64))
    assert new.tolist() == [[[101.0, 102.0]], [[31.0, 63.0]]]                       # to 0: 1*x0 + 0*x1 + 100 y; to 1: 2*x0 + 3*x1 - y


def test_plain_rotation_and_window():
    v = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 5.0]]], dtype=torch.float64).repeat(3, 1, 1)
    out = plain.rotate(v, torch.arange(3), 4, 100.0)
    for p in range(3):
        a0, a1 = p * 1.0, p * 100.0 ** -0.5
        want = [math.cos(a0), -math.sin(a1), math.sin(a0), math.cos(a1), 5.0]       # pairs (0, 2) and (1, 3); entry 4 stays
        assert torch.allclose(out[p, 0], torch.tensor(want, dtype=torch.float64))
    # one key/value head, values that name their position: with equal scores a token's output is the mean of what it sees
    T = 6
    q = torch.zeros(T, 2, 3, dtype=torch.float64)
    k = torch.zeros(T, 1, 3, dtype=torch.float64)
    val = torch.arange(T, dtype=torch.float64).reshape(T, 1, 1)
    o = plain.window_attention(q, k, val, 1.0, 3)
    assert torch.allclose(o[:, 0, 0], torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=torch.float64)) and torch.equal(o[:, 0], o[:, 1])


def test_plain_recurrences():
    one = torch.ones(3, 1, 1, dtype=torch.float64)
    o = plain.fixed_decay_recurrence(one, one * 2, torch.tensor([1.0, 10.0, 100.0], dtype=torch.float64).reshape(3, 1, 1), [0.5])
    assert o.flatten().tolist() == [2.0, 21.0, 210.5]                                # S: 2; 1 + 20; 10.5 + 200
    r = torch.ones(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([1.0, 10.0, 100.0], dtype=torch.float64).reshape(3, 1, 1)
    w = torch.full((3, 1, 1), 0.5, dtype=torch.float64)
    o = plain.bonus_recurrence(r, r.clone(), v, w, torch.tensor([[3.0]], dtype=torch.float64))
    assert o.flatten().tolist() == [3.0, 31.0, 310.5]                                # S before: 0, 1, 10.5; plus 3 * k v
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0]], dtype=torch.float64)
    assert plain.token_shift(h, torch.tensor([0.5, 0.0], dtype=torch.float64)).tolist() == [[0.5, 2.0], [2.0, 6.0]]


def test_plain_routing_and_order():
    h = torch.tensor([1.0, 0.0], dtype=torch.float64)
    router = torch.tensor([[1.0, 0.0], [3.0, 0.0], [3.0, 0.0], [0.0, 9.0]], dtype=torch.float64)
    chosen, weight = plain.route(h, router, torch.tensor([0.0, 0.0, 0.0, 2.0], dtype=torch.float64), 3)
    assert chosen == [1, 2, 3]                                                       # ties go to the lower index, the bias counts
    e = [math.exp(3), math.exp(3), math.exp(2)]
    assert torch.allclose(weight, torch.tensor([x / sum(e) for x in e], dtype=torch.float64))
    assert plain.layer_order(dict(layers=[0] * 5, loop=dict(start=1, stop=3, times=2))) == [0, 1, 2, 1, 2, 3, 4]
    assert plain.layer_order(dict(layers=[0] * 3)) == [0, 1, 2]
    z = torch.tensor([-1.0, 0.0, 2.0], dtype=torch.float64)
    assert torch.allclose(plain.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
