"""Tarorax: a decoder-only model whose residual stream is kept in several copies
(``streams``; hyper-connections: every sublayer reads one weighted sum of the copies
and rewrites all of them) and whose layers mix tokens in one of two ways
(``layers[i].type``):

gla         gated linear attention: a matrix state per head that decays by a factor
            per key channel and token, alpha = sigmoid(W_a2 W_a1 h + b)^(1 / tau);
            the heads' outputs RMS-normed with a shared weight, times silu(W_g h);
attention   differential attention: two score maps per head over the same values,
            o = a_1 - lambda a_2, RMS-normed, times (1 - diff); biased projections, a
            short causal convolution on q, k and v, a query temperature that grows
            with the logarithm of the position, capped scores, no rotation, grouped
            heads, an output gate sigmoid(W_g h).

A layer is pre-norm with norms that act as (1 + w), a per-channel layer scale on
every sublayer's result, and a feed-forward that is dense (tanh-GELU gated), absent,
or a mixture of experts: sigmoid router in 32 bits, a correction added for the
choice only, the choice restricted to the best groups of experts, the chosen scores
divided by their sum and scaled, experts W_down gelu(W_up h) with the exact GELU.
The logits are the normed sum of the streams times the embedding table.

config.json gives every size and every constant that differs between models.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``, ``l<i>.hc1|hc2.in|mix|out``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Optional

from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry)

LAYER_TYPES = ("gla", "attention")
MLP_KINDS = ("dense", "moe")

# Positions enter the query temperature as integers and the state mixers have no bound of their own; a
# 32-bit float holds positions exactly up to here.
MAX_POSITIONS = 1 << 24


@dataclass
class TaroraxConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    streams: Optional[int] = None                   # None: config.json has no "streams" (one stream, no connection weights)
    layers: list = field(default_factory=list)      # the entries of config.json's "layers", checked

    architecture = "Tarorax"

    # ------------------------------------------------------------------ reading

    @staticmethod
    def _check_mixer(i: int, kind: str, m: dict) -> None:
        where = f"config.json: layers[{i}].mixer"
        r = KeyReader(m, where)
        r.integer("heads", minimum=1)
        r.integer("dim", minimum=1)
        r.integer("vdim", minimum=1)
        if kind == "gla":
            r.number("tau", positive=True)
            return
        heads, groups = r.integer("heads"), r.integer("kv_heads", minimum=1)
        if heads % groups:
            raise ConfigError(f"{where}: {heads} heads are not a multiple of {groups} kv_heads")
        r.number("scale")
        r.number("diff")
        r.integer("conv", default=1, minimum=1)
        r.optional_number("softcap", default=None)
        if m.get("q_temp") is not None:
            qt = KeyReader(m["q_temp"], where + ".q_temp")
            qt.number("coef")
            qt.integer("every", minimum=1)

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
        KeyReader(mlp.get("expert"), where + ".expert").integer("ff", minimum=1)
        ro = KeyReader(mlp.get("router"), where + ".router")
        n, top = ro.integer("experts", minimum=1), ro.integer("top", minimum=1)
        ro.number("scale", default=1.0)
        if top > n:
            raise ConfigError(f"{where}.router: top {top} of {n} experts")
        if ro.data.get("groups") is not None:
            gr = KeyReader(ro.data["groups"], where + ".router.groups")
            count, keep = gr.integer("count", minimum=1), gr.integer("keep", minimum=1)
            if n % count or keep > count or keep * (n // count) < top:
                raise ConfigError(f"{where}.router.groups: {n} experts in {count} groups of which {keep} are kept "
                                  f"cannot give {top} choices")

    @classmethod
    def from_dict(cls, data: dict) -> "TaroraxConfig":
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
            cls._check_mixer(i, kind, layer["mixer"])
            mlp = layer.get("mlp")
            if mlp is not None:
                cls._check_mlp(i, mlp)
            checked.append(copy.deepcopy({"type": kind, "mixer": layer["mixer"], "mlp": mlp}))
        streams = r.integer("streams", minimum=1) if data.get("streams") is not None else None
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   norm_eps=KeyReader(data.get("norm"), "config.json: norm").number("eps", positive=True),
                   streams=streams, layers=checked)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    # ------------------------------------------------------------------ the model

    def _mixer(self, p: str, kind: str, m: dict) -> PartSpec:
        h, eps = self.width, self.norm_eps
        if kind == "gla":
            names = {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "a1": p + "a1", "a2": p + "a2",
                     "a2_bias": p + "a2.b", "norm": p + "norm", "o": p + "o"}
            params = {"hidden_size": h, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                      "tau": float(m["tau"]), "eps": eps, "weights": names}
            if m.get("rank") is not None:
                params["decay_rank"] = int(m["rank"])
            return PartSpec("gated_linear_attention", params)
        names = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_bias": p + "q.b", "k_bias": p + "k.b",
                 "v_bias": p + "v.b", "o_bias": p + "o.b", "g": p + "g", "lq1": p + "lq1", "lk1": p + "lk1",
                 "lq2": p + "lq2", "lk2": p + "lk2"}
        params = {"hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                  "value_dim": m["vdim"], "scale": float(m["scale"]), "diff": float(m["diff"]), "eps": eps,
                  "softcap": float(m["softcap"]) if m.get("softcap") else 0.0, "window": None, "weights": names}
        if m.get("conv") is not None:
            names.update({"q_conv": p + "q.conv", "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
            params["taps"] = int(m["conv"])
        if m.get("q_temp") is not None:
            params["q_temp"] = {"coef": float(m["q_temp"]["coef"]), "every": int(m["q_temp"]["every"])}
        return PartSpec("diff_attention", params)

    def _feed_forward(self, p: str, mlp) -> PartSpec:
        h = self.width
        if mlp is None:
            return PartSpec("none")
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": mlp["ff"], "activation": "gelu_tanh",
                                          "wide_output": True, "gate_weight": p + "gate", "up_weight": p + "up",
                                          "down_weight": p + "down"})
        ro = mlp["router"]
        router = {"correction_weight": p + "correction", "normalise": True, "scale": float(ro.get("scale", 1.0))}
        if ro.get("groups") is not None:
            router["groups"] = {"count": int(ro["groups"]["count"]), "keep": int(ro["groups"]["keep"])}
        return PartSpec("routed_experts", {
            "hidden_size": h, "intermediate_size": mlp["expert"]["ff"], "num_experts": ro["experts"], "top": ro["top"],
            "expert": "gelu_erf", "router_weight": p + "router", "expert_weights": p + "e{e}.{role}", "router": router})

    def model_spec(self) -> ModelSpec:
        h = self.width
        streams = self.streams or 1

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"weight": name, "size": h, "eps": self.norm_eps, "weight_offset": 1.0})

        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            norms = {"pre_mixer": norm(p + "norm1")}
            block = {"streams": streams, "hidden_size": h, "scales": [p + "ls1", p + "ls2" if layer["mlp"] is not None else None]}
            if self.streams is not None:
                block["connections"] = [{"in": f"{p}hc{q}.in", "mix": f"{p}hc{q}.mix", "out": f"{p}hc{q}.out"} for q in (1, 2)]
            if layer["mlp"] is not None:
                norms["pre_feed_forward"] = norm(p + "norm2")
            layers.append(LayerSpec(prefix=p, block=PartSpec("hyper", block),
                                    mixer=self._mixer(p + "mix.", layer["type"], layer["mixer"]),
                                    feed_forward=self._feed_forward(p + "mlp.", layer["mlp"]), norms=norms))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=h, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": h,
                                                   "scale": 1.0}),
            layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": h, "softcap": 0.0, "tied_to": "embed"}),
            stop_token_ids=[], streams=streams)
        spec.validate()
        return spec
