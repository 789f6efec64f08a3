"""Tiny Pulenex configurations for the tests, and their model folders with random weights."""
from __future__ import annotations

ARCH = "Pulenex"


def _rot(dims, base):
    return dict(dims=dims, base=base)


def _retention(heads, dim, vdim, decay, rot=None, mlp=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, decay=decay)
    if rot is not None:
        m["rot"] = rot
    return dict(type="retention", mixer=m, mlp=mlp)


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, window, base, kv_from=None, mlp=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=_rot(rot_dim, base))
    if window is not None:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def _parallel(left, right, mlp=None):
    heads, kv_heads, dim, scale, conv, chunk, rot = left
    l = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, conv=conv, rot=rot)
    if chunk is not None:
        l["mask"] = dict(size=chunk)
    r_heads, r_kv, r_dim, r_vdim, r_conv, ranks = right
    r = dict(heads=r_heads, kv_heads=r_kv, dim=r_dim, vdim=r_vdim, conv=r_conv, decay_rank=ranks[0], gate_rank=ranks[1])
    return dict(type="parallel", mixer=dict(left=l, right=r), mlp=mlp)


def _dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


CONFIGS = {
    # odd sizes all round, nothing a multiple of 8; a parallel layer first; fewer key heads than heads on both sides; heads rotated
    # in part; chunks of 7 and windows of 5 and 11 on ONE cached plane (the reader looks back further than the writer); filters of 3
    # and 2 taps; a latent layer without a feed-forward, a retention layer with one; a clamp that bites (limit 0.3)
    "odd": dict(config=dict(architecture=ARCH, vocab=103, width=46, norm=dict(eps=1e-5), logit_scale=0.5, layers=[
        _parallel((4, 2, 10, 0.3, 3, 7, _rot(6, 100.0)), (4, 2, 6, 5, 2, (3, 5)), mlp=_dense(21, 0.3)),
        _latent(3, 5, 4, 7, 9, 0.3, 5, 50.0),
        _retention(3, 6, 10, [0.9, 0.97, 0.995], rot=_rot(4, 30.0), mlp=_dense(13, 1.0)),
        _latent(2, 6, 4, 3, 9, 0.4, 11, 50.0, kv_from=1, mlp=_dense(11, 2.0)),
        _parallel((3, 3, 6, 0.5, 2, 90, _rot(6, 1000.0)), (1, 1, 7, 9, 4, (2, 2))),
    ]), seed=41, sigma=0.1),
    # sizes in multiples of 16, on which the bfloat16 engine takes its tensor-core kernels; chunks as long as a cache block; one
    # key head for four heads; state columns of 32 and 64 in registers; two readers of one plane, one of them without a window
    "even": dict(config=dict(architecture=ARCH, vocab=512, width=128, norm=dict(eps=1e-6), logit_scale=0.25, layers=[
        _latent(2, 32, 16, 32, 64, 0.14, 70, 10000.0, mlp=_dense(192, 2.0)),
        _retention(2, 64, 32, [0.96875, 0.998], rot=_rot(32, 10000.0)),
        _parallel((4, 1, 32, 0.18, 4, 64, _rot(32, 10000.0)), (4, 2, 32, 64, 4, (16, 16)), mlp=_dense(160, 1.5)),
        _latent(4, 16, 16, 16, 64, 0.2, None, 10000.0, kv_from=0, mlp=_dense(96, 2.0)),
        _latent(2, 32, 16, 64, 64, 0.14, 33, 10000.0, kv_from=0),
        _parallel((2, 2, 64, 0.125, 4, 100, _rot(64, 500000.0)), (2, 1, 64, 32, 3, (8, 24)), mlp=_dense(160, 2.0)),
    ]), seed=42, sigma=0.08),
    # what a model may leave out: no masks (every token sees all before it), no rotation in retention, no logit scale; one head
    # everywhere; filters of one tap (no state of their own); state columns of 128 on the wide kernel
    "bare": dict(config=dict(architecture=ARCH, vocab=200, width=64, norm=dict(eps=1e-5), layers=[
        _retention(1, 128, 32, [0.99], mlp=_dense(96, 2.0)),
        _parallel((1, 1, 16, 0.25, 1, None, _rot(0, 10000.0)), (1, 1, 128, 16, 1, (4, 4)), mlp=_dense(48, 2.0)),
        _latent(1, 8, 8, 24, 16, 0.25, None, 10000.0, mlp=_dense(32, 2.0)),
        _latent(1, 8, 8, 8, 16, 0.25, None, 10000.0, kv_from=2),
    ]), seed=43, sigma=0.1),
}


def make_model_dir(folder: str, name: str) -> str:
    import os
    import torch
    from safetensors.torch import load_file, save_file
    from hymt2sharp_b200.config.pulenex import PulenexConfig
    from hymt2sharp_b200.weights import write_random_model
    spec = CONFIGS[name]
    write_random_model(folder, PulenexConfig.from_dict(spec["config"]), spec["seed"], spec["sigma"])
    # numbers that random matrices would leave without effect: sinks that take a real share of the softmax, head temperatures
    # and a mixing matrix far from the identity, decays of the delta rule between fast and slow
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(spec["seed"])
    for k in sorted(tensors):
        t = tensors[k]
        if k.endswith(".sink"):
            tensors[k] = (torch.randn(t.shape, generator=gen) * 1.5).to(t.dtype)
        elif k.endswith(".temp"):
            tensors[k] = (0.5 + 1.5 * torch.rand(t.shape, generator=gen)).to(t.dtype)
        elif k.endswith(".talk"):
            tensors[k] = (torch.eye(t.shape[0]) + 0.4 * torch.randn(t.shape, generator=gen)).to(t.dtype)
        elif k.endswith(".A_log"):
            tensors[k] = (torch.rand(t.shape, generator=gen) * 4.0 - 3.0).to(t.dtype)
        elif k.endswith(".dt_bias"):
            tensors[k] = (torch.randn(t.shape, generator=gen)).to(t.dtype)
        elif k.endswith(".mlp.gate.b") or k.endswith(".mlp.up.b") or k.endswith(".mlp.down.b"):
            tensors[k] = (torch.randn(t.shape, generator=gen) * 0.3).to(t.dtype)
    save_file(tensors, path)
    return folder
