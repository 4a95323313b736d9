"""Small Zatasun configurations for the tests; they differ from one another in
every size, in their feed-forwards and in their constants."""
from __future__ import annotations

import torch

from tiny_fiferax import make_folder as _make_folder


def _mixer(heads, kv_heads, dim, vdim, rot_dims, base, scaling, scale, left_scale, width, blocks, conv, right_scale):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale},
            "left_scale": left_scale, "right": {"width": width, "blocks": blocks, "conv": conv},
            "right_scale": right_scale}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _layer(mixer, mlp=None):
    return {"type": "parallel", "mixer": mixer, "mlp": mlp}


# odd sizes that no tensor-core kernel takes; no grouping of heads; rotary on half a head without stretching;
# one block of gates and a convolution of one tap (no history); scales that are 1; two of five experts with
# a shared one; a layer without a feed-forward; every expert chosen (top = experts) without a shared one
ZA = {
    "architecture": "Zatasun", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
    "layers": [
        _layer(_mixer(4, 4, 12, 20, 6, 100.0, None, 0.4, 1.0, 44, 1, 1, 1.0), _dense(100)),
        _layer(_mixer(2, 1, 20, 20, 20, 3000.0, (8.0, 1.0, 3.0, 64), 0.25, 0.6, 30, 3, 4, 1.3),
               _moe(5, 2, 36, 1.0, (28, 0.7))),
        _layer(_mixer(3, 1, 8, 4, 8, 50.0, (2.0, 0.5, 2.0, 16), 0.3, 0.8, 24, 2, 2, 0.9)),
        _layer(_mixer(2, 2, 16, 12, 4, 10.0, None, 0.35, 1.2, 36, 4, 3, 0.4), _moe(3, 3, 20, 0.5)),
    ],
}

# sizes the bfloat16 tensor-core kernels take: head size 64 with three query heads a kv head, values of 96 (padded
# to 128), head size 128; frequencies stretched so that all three regimes occur; one expert of eight
ZB = {
    "architecture": "Zatasun", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.25,
    "layers": [
        _layer(_mixer(6, 2, 64, 64, 64, 10000.0, (4.0, 1.0, 4.0, 256), 0.125, 0.9, 256, 2, 4, 0.7), _dense(256)),
        _layer(_mixer(2, 2, 64, 96, 32, 500.0, None, 0.2, 1.1, 128, 8, 2, 0.5), _moe(8, 1, 64, 2.0, (128, 1.0))),
        _layer(_mixer(2, 1, 128, 128, 128, 30000.0, (16.0, 2.0, 8.0, 128), 0.09, 0.75, 192, 3, 3, 0.85),
               _moe(4, 3, 96, 1.5)),
    ],
}

# nothing divides by four: a width of 50, key sizes of 10 and 6, no rotation at all in one attention; the right
# mixer switched off in one layer and the left one in another (a scale of 0); seven of seven and one of two experts
ZC = {
    "architecture": "Zatasun", "vocab": 97, "width": 50, "norm": {"eps": 1e-4}, "logit_scale": 2.0,
    "layers": [
        _layer(_mixer(3, 1, 10, 6, 0, 10.0, None, 0.5, 1.0, 30, 5, 2, 0.0), _moe(7, 7, 9, 0.8, (11, 3.0))),
        _layer(_mixer(1, 1, 6, 14, 6, 77.0, (3.0, 1.0, 2.0, 10), 0.3, 0.0, 26, 13, 5, 1.0), _dense(22)),
        _layer(_mixer(5, 5, 6, 10, 2, 20.0, None, 0.7, 0.5, 18, 1, 3, 2.0), _moe(2, 1, 13, 4.0)),
    ],
}

CONFIGS = {"A": ZA, "B": ZB, "C": ZC}


def spread(name: str, t):
    """Random tensors as the tests want them: decays from fast to very slow (lam from -7 to 1), taps of the
    convolution that differ, sinks of the size of the scores."""
    if name.endswith(".lam"):
        return torch.linspace(-7.0, 1.0, t.numel()).reshape(t.shape)[torch.randperm(t.numel(), generator=torch.Generator().manual_seed(1))]
    if name.endswith(".conv"):
        return (t - 1.0) * 6.0 + 0.4
    if name.endswith(".sink"):
        return t * 10.0 + 1.0
    return t


def make_folder(cfg_dict, seed=0, store_dtype="bfloat16", root=None, edit=None):
    """A random model folder; ``edit(name, tensor)`` may change tensors on their way out (after :func:`spread`)."""
    def both(name, t):
        t = spread(name, t)
        return edit(name, t) if edit is not None else t
    return _make_folder(cfg_dict, seed=seed, store_dtype=store_dtype, root=root, edit=both)
