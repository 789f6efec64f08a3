"""Tiny Rutetar configurations for the tests, and their model folders with random weights."""
from __future__ import annotations

ARCH = "Rutetar"


def _retention(heads, dim, vdim, decay, mlp=None):
    return dict(type="retention", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay), mlp=mlp)


def _parallel(heads, kv_heads, dim, vdim, scale, window, rot_dims, base, r_heads, r_dim, rank, left_scale, right_scale, mlp=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(dims=rot_dims, base=base))
    if window is not None:
        left["mask"] = dict(size=window)
    return dict(type="parallel", mixer=dict(left=left, right=dict(heads=r_heads, dim=r_dim, rank=rank), left_scale=left_scale,
                                            right_scale=right_scale), mlp=mlp)


def _dense(ff):
    return dict(kind="dense", ff=ff)


def _moe(experts, top, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


CONFIGS = {
    # odd sizes all round, nothing a multiple of 8: three streams; a loop over the first two layers, three times; one kv head
    # and as many kv heads as heads; a window of 7 and one wider than any test sequence's block; heads rotated in part and in
    # whole; time mixing whose heads do not fill the width; one chosen expert and all experts chosen; a layer without feed-forward
    "odd": dict(config=dict(architecture=ARCH, vocab=101, width=44, streams=3, norm=dict(eps=1e-5),
                            loop=dict(start=0, stop=2, times=3), layers=[
        _parallel(3, 1, 10, 6, 0.4, 7, 4, 1000.0, 3, 5, 3, 0.7, 1.2, mlp=_moe(5, 1, 9)),
        _retention(3, 6, 10, [0.9, 0.97, 0.995]),
        _retention(1, 12, 4, [0.98], mlp=_dense(13)),
        _parallel(4, 4, 6, 6, 0.5, 90, 6, 300.0, 1, 7, 2, 1.0, 0.5, mlp=_moe(3, 3, 5)),
    ]), seed=31, sigma=0.1),
    # sizes in multiples of 16: one stream with its tables; heads of 64 and 128 for keys and values, on which the bfloat16
    # engine takes its tensor-core attention; state columns held in registers (16, 64) ; a loop over the two middle layers;
    # an attention without a window; 12 experts of which 3 are chosen
    "even": dict(config=dict(architecture=ARCH, vocab=512, width=128, streams=1, norm=dict(eps=1e-6),
                             loop=dict(start=1, stop=3, times=2), layers=[
        _retention(2, 64, 128, [0.96875, 0.998], mlp=_moe(12, 3, 48)),
        _parallel(4, 2, 64, 128, 0.125, 100, 32, 10000.0, 2, 64, 16, 0.7, 0.8, mlp=_dense(320)),
        _parallel(2, 1, 128, 64, 0.09, None, 128, 50000.0, 4, 16, 8, 1.5, 1.0),
        _retention(4, 16, 32, [0.9, 0.95, 0.99, 0.999], mlp=_dense(192)),
    ]), seed=32, sigma=0.08),
    # no `streams` key and no loop: the plain residual sum; state columns of 128 and 32 in registers
    "bare": dict(config=dict(architecture=ARCH, vocab=200, width=64, norm=dict(eps=1e-5), layers=[
        _retention(1, 128, 32, [0.99], mlp=_dense(96)),
        _parallel(2, 2, 16, 24, 0.25, 20, 8, 10000.0, 2, 32, 4, 1.0, 1.0, mlp=_moe(4, 2, 24)),
    ]), seed=33, sigma=0.1),
}

ROUTER_SPREAD = 2.0
# Which experts a token gets is a discontinuous function of the router's input, and a recurrent state carries one token's
# other expert into every token behind it.  For the bfloat16 engine the models named here get routers whose choice rests on
# the bias (outputs a unit and a half apart, the input's share a fraction of that): every token takes the same experts with
# weights of its own, and no choice rests on a rounding.  The 32-bit engine runs the routers that choose token by token.
STEADY = ("odd",)
STEADY_GAP, STEADY_SHARE = 1.5, 0.2


def variant(name: str, dtype: str) -> str:
    """The name of the model folder that a test of `name` in `dtype` uses."""
    return name + "/steady" if dtype == "bfloat16" and name in STEADY else name


def make_model_dir(folder: str, name: str) -> str:
    import os
    import torch
    from safetensors.torch import load_file, save_file
    from hymt2sharp_b200.config import RutetarConfig
    from hymt2sharp_b200.weights import write_random_model
    name, _, steady = name.partition("/")
    spec = CONFIGS[name]
    write_random_model(folder, RutetarConfig.from_dict(spec["config"]), spec["seed"], spec["sigma"])
    # routers with a wide spread of outputs: a choice between two experts that rests on the last bits would make the
    # comparison of two precisions a comparison of two different sums
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(spec["seed"])
    for k in sorted(tensors):
        if steady and k.endswith(".mlp.router"):
            tensors[k] = (tensors[k].float() * STEADY_SHARE).to(tensors[k].dtype)
        elif steady and k.endswith(".mlp.router.b"):
            n = tensors[k].numel()
            tensors[k] = (torch.randperm(n, generator=gen).float() * STEADY_GAP).to(tensors[k].dtype)
        elif k.endswith(".mlp.router") or k.endswith(".mlp.router.b"):
            tensors[k] = (tensors[k].float() * ROUTER_SPREAD).to(tensors[k].dtype)
    save_file(tensors, path)
    return folder
