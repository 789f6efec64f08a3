"""The Pulenex design without a GPU: its configuration (every size read and written back, errors that name their key), the
registry, the tensor list, the memory plan (shared planes, windows kept for the widest reader, state offsets), and the plain
implementation's mechanisms against values worked out by hand."""
import copy
import math

import pytest
import torch

import pulenex_models
from plain import pulenex_plain as plain


def _cfg(name="odd"):
    return copy.deepcopy(pulenex_models.CONFIGS[name]["config"])


def test_configuration_reads_every_size_and_writes_it_back():
    from hymt2sharp_b200.config.pulenex import PulenexConfig
    from hymt2sharp_b200.config.registry import get_architecture
    for name in pulenex_models.CONFIGS:
        data = _cfg(name)
        cfg = PulenexConfig.from_dict(data)
        again = PulenexConfig.from_dict(cfg.to_dict())
        assert again == cfg and get_architecture("Pulenex").config_class is PulenexConfig
    cfg = PulenexConfig.from_dict(_cfg("odd"))
    left, right = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.conv, left.chunk, left.rot.dims, left.rot.base) == (4, 2, 10, 3, 7, 6, 100.0)
    assert (right.heads, right.kv_heads, right.dim, right.vdim, right.conv) == (4, 2, 6, 5, 2)
    assert cfg.layers[3].mixer.kv_from == 1 and cfg.layers[1].mixer.window == 5 and cfg.layers[2].mixer.decay == (0.9, 0.97, 0.995)
    assert cfg.logit_scale == 0.5 and cfg.layers[1].mlp is None and cfg.layers[0].mlp.limit == 0.3
    bare = PulenexConfig.from_dict(_cfg("bare"))
    assert bare.logit_scale is None and bare.layers[1].mixer.left.chunk is None and bare.layers[2].mixer.window is None
    assert bare.layers[0].mixer.rot.dims == 0


@pytest.mark.parametrize("change, key", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "mixer.left.heads"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=4), "mixer.left.vdim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["right"].pop("conv"), "mixer.right.conv"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "mixer.decay"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=8), "kv_from"),
    (lambda c: c["layers"][0]["mlp"].pop("limit"), "mlp.limit"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_configuration_errors_name_their_key(change, key):
    from hymt2sharp_b200.config.base import ConfigError
    from hymt2sharp_b200.config.pulenex import PulenexConfig
    data = _cfg("odd")
    change(data)
    with pytest.raises(ConfigError, match=key.replace(".", r"\.")):
        PulenexConfig.from_dict(data)


def test_tensor_list_and_memory_plan():
    from hymt2sharp_b200.config.pulenex import PulenexConfig
    from hymt2sharp_b200.engine.model import DecoderModel
    from hymt2sharp_b200.engine.pulenex import build_spec
    cfg = PulenexConfig.from_dict(_cfg("odd"))
    model = DecoderModel(build_spec(cfg))
    t = model.tensors()
    assert t["l0.mix.left.q.conv"].shape == (40, 3) and t["l0.mix.left.talk"].shape == (4, 4) and t["l0.mix.right.a2"].shape == (24, 3)
    assert t["l0.mix.right.g2"].shape == (20, 5) and t["l0.mix.left.out"].shape == (46,) and t["l0.mix.right.norm"].shape == (5,)
    assert "l3.mix.dkv" not in t and "l3.mix.dkv.norm" not in t and t["l3.mix.uk"].shape == (12, 9) and t["l1.mix.g"].shape == (3, 46)
    assert "l1.mlp.gate" not in t and "l1.norm2" not in t and t["l2.mlp.gate.b"].shape == (13,) and t["final.norm"].shape == (46,)
    # the reader of layer 1's rows looks back 11 positions, the writer 5: the plane keeps 11
    assert cfg.cache_windows() == {1: 11, 3: 11}
    kinds = {(g.kind, g.kv_heads, g.head_dim, g.window, g.streams): g.planes for g in model.groups}
    assert kinds == {("window", 2, 10, 7, 2): 1, ("window", 1, 13, 11, 1): 1, ("window", 3, 6, 90, 2): 1}
    reader, writer = model.slots[3][0], model.slots[1][0]
    assert (reader.group, reader.plane, reader.writes) == (writer.group, writer.plane, False)
    # state: per parallel layer the left's filter inputs, then the right's matrix and filter inputs; retention's matrix
    left0, right0 = model.slots[0]
    assert left0.state_bytes == 4 * 2 * 60 and right0.state_bytes == 4 * (4 * 6 * 5) + 4 * 1 * (12 + 12 + 20)
    assert model.slots[2][0].state_bytes == 4 * 3 * 6 * 10 and model.state_bytes >= right0.state_offset + right0.state_bytes
    even = PulenexConfig.from_dict(_cfg("even"))
    assert even.cache_windows() == {0: 0, 3: 0, 4: 0}        # one reader without a window: everything is kept
    assert DecoderModel(build_spec(even)).graph_safe


def test_plain_layer_norm_takes_the_mean_off():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    d = x - 3.0
    want = d / math.sqrt(float((d * d).mean()) + 0.1) * w
    assert torch.allclose(plain.layer_norm(x, w, 0.1), want)


def test_plain_rotations_pair_their_entries_as_named():
    v = torch.arange(1.0, 7.0, dtype=torch.float64).reshape(1, 1, 6)
    pos = torch.tensor([3])
    a0 = 3.0
    half = plain.rotate_half(v, pos, 4, 100.0)[0, 0]
    assert math.isclose(float(half[0]), 1 * math.cos(a0) - 3 * math.sin(a0)) and math.isclose(float(half[2]), 3 * math.cos(a0) + 1 * math.sin(a0))
    pairs = plain.rotate_pairs(v, pos, 4, 100.0)[0, 0]
    assert math.isclose(float(pairs[0]), 1 * math.cos(a0) - 2 * math.sin(a0)) and math.isclose(float(pairs[1]), 2 * math.cos(a0) + 1 * math.sin(a0))
    a1 = 3.0 * 100.0 ** -0.5
    assert math.isclose(float(pairs[2]), 3 * math.cos(a1) - 4 * math.sin(a1)) and float(pairs[4]) == 5.0 and float(half[5]) == 6.0


def test_plain_delta_rule_overwrites_what_a_key_holds():
    """With no decay and beta one, writing a second value under the same unit key replaces the first: the read gives the second."""
    S = torch.zeros(2, 1, dtype=torch.float64)
    k = torch.tensor([1.0, 0.0], dtype=torch.float64)
    for v in (5.0, -2.0):
        u = 1.0 * (torch.tensor([v], dtype=torch.float64) - S.T @ k)
        S = S + torch.outer(k, u)
    assert float((S.T @ k)[0]) == -2.0


def test_plain_sink_takes_its_share_and_chunks_cut_the_past():
    h = torch.eye(4, dtype=torch.float64)
    W = {"q": torch.zeros(2, 4, dtype=torch.float64), "k": torch.zeros(2, 4, dtype=torch.float64), "q.conv": torch.ones(2, 1, dtype=torch.float64),
         "k.conv": torch.ones(2, 1, dtype=torch.float64), "temp": torch.ones(1, dtype=torch.float64), "talk": torch.ones(1, 1, dtype=torch.float64),
         "sink": torch.zeros(1, dtype=torch.float64), "g": torch.zeros(2, 4, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64).repeat(2, 1)[:4]}
    W["k"][0] = torch.tensor([1.0, 2.0, 3.0, 4.0])           # token t's value is (t + 1, 0); all scores are zero
    m = dict(heads=1, kv_heads=1, dim=2, scale=1.0, mask=dict(size=2))
    out = plain.talking_attention(h, W, "", m, torch.arange(4))
    # weights 1 / (1 + seen keys): the sink counts once; chunks are {0, 1} and {2, 3}; sigmoid(0) = 1/2
    want = [1 / 2, (1 + 2) / 3, 3 / 2, (3 + 4) / 3]
    assert torch.allclose(out[:, 0], 0.5 * torch.tensor(want, dtype=torch.float64))
