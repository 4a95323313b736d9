"""Small Tarorax configurations for the tests; they differ from one another in every size, in the
order of their layers, in their feed-forwards and in their constants."""
from __future__ import annotations

from tiny_fiferax import make_folder  # noqa: F401  (the writer of random model folders)


def _gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _att(heads, kv_heads, dim, vdim, scale, diff, conv=None, softcap=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if conv is not None:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# odd sizes that no tensor-core kernel takes; three streams; an attention layer first; no grouping of heads in one
# attention and three query heads a kv head in the other; a temperature that steps every 7 positions; a layer
# without a feed-forward; two of six experts out of two of three groups; key and value sizes that differ
TA = {
    "architecture": "Tarorax", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [
        _layer("attention", _att(2, 2, 12, 20, 0.3, 0.4, conv=3, softcap=4.0, q_temp=(0.7, 7)), _dense(100)),
        _layer("gla", _gla(3, 8, 20, 4.0, 5), _moe(6, 2, 36, 1.5, (3, 2))),
        _layer("gla", _gla(2, 24, 10, 9.0, 3)),
        _layer("attention", _att(3, 1, 10, 6, 0.25, 0.8, conv=2, softcap=30.0, q_temp=(0.2, 16)), _moe(4, 1, 20, 1.0, (2, 1))),
    ],
}

# sizes the bfloat16 tensor-core kernels take: maps and values of 64, of 128, and values twice the maps' size
# (padded); key channels of 64 and 128 in the linear attention; four streams; eight experts of which four
TB = {
    "architecture": "Tarorax", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "streams": 4,
    "layers": [
        _layer("gla", _gla(2, 64, 64, 12.0, 16), _dense(256)),
        _layer("attention", _att(4, 2, 64, 64, 0.125, 0.55, conv=4, softcap=40.0, q_temp=(0.4, 48)), _moe(8, 4, 64, 1.75, (4, 3))),
        _layer("gla", _gla(1, 128, 128, 2.0, 8), _moe(8, 2, 96, 2.5, (2, 2))),
        _layer("attention", _att(2, 1, 128, 128, 0.09, 0.3, conv=4, softcap=20.0, q_temp=(1.0, 32)), _dense(192)),
        _layer("attention", _att(2, 2, 32, 64, 0.2, 0.5, conv=2, q_temp=(0.5, 3))),
    ],
}

# nothing divides by four; no "streams" at all (one stream, no connection weights: the plain pre-norm layer); an
# attention without convolution, cap or temperature; every expert chosen (top = experts, no groups); one expert
# of two; a decay exponent of 1 (tau = 1)
TC = {
    "architecture": "Tarorax", "vocab": 97, "width": 50, "norm": {"eps": 1e-4},
    "layers": [
        _layer("gla", _gla(3, 10, 6, 1.0, 2), _moe(3, 3, 22, 1.0)),
        _layer("attention", _att(3, 1, 10, 14, 0.3, 0.1), _dense(36)),
        _layer("attention", _att(2, 2, 6, 10, 0.4, 0.9, conv=5, softcap=2.0), _moe(2, 1, 18, 3.0)),
        _layer("gla", _gla(1, 14, 22, 30.0, 1)),
    ],
}

# one stream that still has its connection weights; every size odd
TD = {
    "architecture": "Tarorax", "vocab": 31, "width": 51, "norm": {"eps": 1e-5}, "streams": 1,
    "layers": [
        _layer("attention", _att(1, 1, 7, 9, 0.5, 0.5, conv=1, q_temp=(0.3, 1)), _dense(17)),
        _layer("gla", _gla(3, 5, 3, 8.0, 1), _moe(5, 5, 9, 0.5, (5, 5))),
    ],
}

CONFIGS = {"A": TA, "B": TB, "C": TC, "D": TD}
