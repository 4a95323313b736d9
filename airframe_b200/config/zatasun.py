"""Zatasun: a decoder-only model whose every layer runs two mixers side by side
on the same input, summed with a scale each (``layers[i].type`` = ``parallel``):

left    causal softmax attention with grouped heads: q and k RMS-normed over
        their whole projection (all heads at once, weights of that size), then
        rotated (pairs i, i + dims/2 on the first ``rot.dims`` elements of a head,
        frequencies optionally stretched by wavelength), a score scale from the
        configuration, values of a size of their own, and a learned sink per head
        in the softmax's denominator;
right   a real-gated linear recurrence behind a short causal convolution, its
        gates from block-diagonal matrices.

A layer is x += norm1(mixer(x)); x += norm2(ff(x)): the sublayers read the stream
itself and the only norms stand on their outputs.  The feed-forward is dense
(SiLU-gated), a mixture of experts (sigmoid router, the weight on the expert's
input, a clamped activation, optionally a shared expert with a gate), or absent.
The embedding's rows are normed before they become the stream, and the logits are
the normed stream times the embedding table times ``logit_scale``.

config.json gives every size and every constant that differs between models.
Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1|norm2``, ``l<i>.mix.left.*``,
``l<i>.mix.right.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry)

LAYER_TYPES = ("parallel",)
MLP_KINDS = ("dense", "moe")

# Positions enter the rotary angles as 32-bit floats, which hold integers exactly up to here.
MAX_POSITIONS = 1 << 24

# The recurrence's decay is exp(-DECAY_RATE * r * softplus(lam)); the design fixes the factor.
DECAY_RATE = 8.0


@dataclass
class ZatasunConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: list = field(default_factory=list)      # the entries of config.json's "layers", checked

    architecture = "Zatasun"

    # ------------------------------------------------------------------ reading

    @staticmethod
    def _check_mixer(i: int, m: dict) -> None:
        where = f"config.json: layers[{i}].mixer"
        r = KeyReader(m, where)
        r.number("left_scale")
        r.number("right_scale")
        left = KeyReader(m.get("left"), where + ".left")
        heads, groups = left.integer("heads", minimum=1), left.integer("kv_heads", minimum=1)
        dim = left.integer("dim", minimum=1)
        left.integer("vdim", minimum=1)
        if heads % groups:
            raise ConfigError(f"{where}.left: {heads} heads are not a multiple of {groups} kv_heads")
        left.number("scale")
        rot = KeyReader(left.data.get("rot"), where + ".left.rot")
        dims = rot.integer("dims", minimum=0)
        rot.number("base", positive=True)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{where}.left.rot: dims {dims} must be even and at most dim {dim}")
        if rot.data.get("scaling") is not None:
            sc = KeyReader(rot.data["scaling"], where + ".left.rot.scaling")
            sc.number("factor", positive=True)
            sc.number("original", positive=True)
            if not sc.number("high", positive=True) > sc.number("low", positive=True):
                raise ConfigError(f"{where}.left.rot.scaling: 'high' must exceed 'low'")
        right = KeyReader(m.get("right"), where + ".right")
        width, blocks = right.integer("width", minimum=1), right.integer("blocks", minimum=1)
        right.integer("conv", minimum=1)
        if width % blocks:
            raise ConfigError(f"{where}.right: width {width} does not come in {blocks} equal blocks")

    @staticmethod
    def _check_mlp(i: int, mlp: dict) -> None:
        where = f"config.json: layers[{i}].mlp"
        mr = KeyReader(mlp, where)
        kind = mr.string("kind")
        if kind not in MLP_KINDS:
            raise ConfigError(f"{where}.kind '{kind}' is unknown (known: {list(MLP_KINDS)})")
        if kind == "dense":
            mr.integer("ff", minimum=1)
            return
        ex = KeyReader(mlp.get("expert"), where + ".expert")
        ex.integer("ff", minimum=1)
        ex.number("limit", positive=True)
        ro = KeyReader(mlp.get("router"), where + ".router")
        n, top = ro.integer("experts", minimum=1), ro.integer("top", minimum=1)
        if top > n:
            raise ConfigError(f"{where}.router: top {top} of {n} experts")
        if mlp.get("shared") is not None:
            sh = KeyReader(mlp["shared"], where + ".shared")
            sh.integer("ff", minimum=1)
            sh.number("limit", positive=True)

    @classmethod
    def from_dict(cls, data: dict) -> "ZatasunConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        checked = []
        for i, layer in enumerate(layers):
            lr = KeyReader(layer, f"config.json: layers[{i}]")
            kind = lr.string("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type '{kind}' is unknown (known: {list(LAYER_TYPES)})")
            if not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"config.json: layers[{i}].mixer must be an object")
            cls._check_mixer(i, layer["mixer"])
            mlp = layer.get("mlp")
            if mlp is not None:
                cls._check_mlp(i, mlp)
            checked.append(copy.deepcopy({"type": kind, "mixer": layer["mixer"], "mlp": mlp}))
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=KeyReader(data.get("norm"), "config.json: norm").number("eps", positive=True),
                   logit_scale=r.number("logit_scale"), layers=checked)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "layers": copy.deepcopy(self.layers),
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width}

    # ------------------------------------------------------------------ the model

    def _mixer(self, p: str, m: dict) -> PartSpec:
        h, eps = self.width, self.norm_eps
        left, right = m["left"], m["right"]
        lp, rp = p + "left.", p + "right."
        rot = {"theta": float(left["rot"]["base"]), "rotary_dim": left["rot"]["dims"], "pairing": "half",
               "precise_angles": True}
        if left["rot"].get("scaling") is not None:
            sc = left["rot"]["scaling"]
            rot["scaling"] = {"kind": "wavelength", "factor": float(sc["factor"]), "low": float(sc["low"]),
                              "high": float(sc["high"]), "original": float(sc["original"])}
        attention = PartSpec("attention", {
            "hidden_size": h, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "value_dim": left["vdim"], "scale": float(left["scale"]), "softcap": 0.0, "window": None,
            "position": PartSpec("rope", rot),
            "q_weight": lp + "q", "k_weight": lp + "k", "v_weight": lp + "v", "o_weight": lp + "o", "wide_output": True,
            "qk_norm": {"whole": True, "q_weight": lp + "q.norm", "k_weight": lp + "k.norm", "eps": eps},
            "sink_weight": lp + "sink"})
        names = {"y": rp + "y", "y_bias": rp + "y.b", "x": rp + "x", "x_bias": rp + "x.b", "conv": rp + "conv",
                 "conv_bias": rp + "conv.b", "a": rp + "ra", "a_bias": rp + "ra.b", "i": rp + "ri", "i_bias": rp + "ri.b",
                 "lam": rp + "lam", "o": rp + "o"}
        recurrence = PartSpec("rglru", {"hidden_size": h, "width": right["width"], "blocks": right["blocks"],
                                        "taps": right["conv"], "decay_rate": DECAY_RATE, "weights": names})
        return PartSpec("parallel", {"branches": [{"mixer": attention, "scale": float(m["left_scale"])},
                                                  {"mixer": recurrence, "scale": float(m["right_scale"])}]})

    def _feed_forward(self, p: str, mlp) -> PartSpec:
        h = self.width
        if mlp is None:
            return PartSpec("none")
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": mlp["ff"], "activation": "silu",
                                          "wide_output": True, "gate_weight": p + "gate", "up_weight": p + "up",
                                          "down_weight": p + "down"})
        params = {"hidden_size": h, "intermediate_size": mlp["expert"]["ff"], "limit": float(mlp["expert"]["limit"]),
                  "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                  "router_weight": p + "router", "expert_weights": p + "e{e}.{role}"}
        if mlp.get("shared") is not None:
            sp = p + "shared."
            params["shared"] = {"intermediate_size": mlp["shared"]["ff"], "limit": float(mlp["shared"]["limit"]),
                                "gate_weight": sp + "gate", "up_weight": sp + "up", "down_weight": sp + "down",
                                "mix_weight": sp + "sg"}
        return PartSpec("routed_experts", params)

    def model_spec(self) -> ModelSpec:
        h = self.width

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"weight": name, "size": h, "eps": self.norm_eps, "weight_offset": 0.0})

        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            norms = {"post_mixer": norm(p + "norm1")}
            if layer["mlp"] is not None:
                norms["post_feed_forward"] = norm(p + "norm2")
            layers.append(LayerSpec(prefix=p, block=PartSpec("postnorm"), mixer=self._mixer(p + "mix.", layer["mixer"]),
                                    feed_forward=self._feed_forward(p + "mlp.", layer["mlp"]), norms=norms))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=h, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": h,
                                                   "scale": 1.0, "norm": norm("embed.norm")}),
            layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": h, "softcap": 0.0, "tied_to": "embed",
                                      "scale": self.logit_scale}),
            stop_token_ids=[])
        spec.validate()
        return spec
