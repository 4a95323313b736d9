"""Named configurations for the random-weights mode: the two tiny test
models, the layer sizes of the released Gemma-2 models, a small Fiferax, a small Banitar, a small Zatasun and a small Tarorax, as
config.json dictionaries.  Nothing here is read by the model code: a configuration always
reaches it through ``config_from_dict``."""
from __future__ import annotations

_COMMON = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True, "rms_norm_eps": 1e-6,
}

PRESETS = {
    "tinyA": dict(_COMMON, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                  head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0, sliding_window=8,
                  query_pre_attn_scalar=16, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                  max_position_embeddings=64, torch_dtype="float32"),
    "tinyB": dict(_COMMON, num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1,
                  head_dim=32, intermediate_size=320, vocab_size=384, rope_theta=100000.0, sliding_window=16,
                  query_pre_attn_scalar=24, attn_logit_softcapping=20.0, final_logit_softcapping=15.0,
                  max_position_embeddings=128, torch_dtype="float32"),
    "2b": dict(_COMMON, num_hidden_layers=26, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4,
               head_dim=256, intermediate_size=9216, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
               query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
               max_position_embeddings=8192, torch_dtype="bfloat16"),
    "9b": dict(_COMMON, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
               head_dim=256, intermediate_size=14336, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
               query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
               max_position_embeddings=8192, torch_dtype="bfloat16"),
    "27b": dict(_COMMON, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, intermediate_size=36864, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
                query_pre_attn_scalar=144, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                max_position_embeddings=8192, torch_dtype="bfloat16"),
}


def _fiferax_small() -> dict:
    """Fiferax with four layers, one of each kind and a second delta rule (sizes of no released model)."""
    delta = {"heads": 8, "dim": 64, "rank": 32}
    par = {"left": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "mask": {"size": 256},
                    "rot": {"base": 10000.0, "dims": 32}, "scale": 0.125}, "left_scale": 1.0,
           "right": {"heads": 8, "dim": 32, "vdim": 64, "decay": [1.0 - 2.0 ** -(3 + h) for h in range(8)]},
           "right_scale": 1.0}
    layers = [{"type": "general_delta", "mixer": delta, "mlp": None},
              {"type": "parallel", "mixer": par, "mlp": {"kind": "dense", "ff": 1536}},
              {"type": "general_delta", "mixer": delta, "mlp": None},
              {"type": "mingru", "mixer": {"width": 768}, "mlp": {"kind": "dense", "ff": 1536}}]
    return {"architecture": "Fiferax", "vocab": 8192, "width": 512, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": layers}


PRESETS["fiferax-small"] = _fiferax_small()


def _banitar_small() -> dict:
    """Banitar with four layers, the two in the middle run twice (sizes of no released model)."""
    attn = {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "mask": {"size": 256}, "scale": 0.125,
            "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 512, "fast": 32.0, "slow": 1.0}}}
    latent = {"heads": 8, "dim": 32, "rot_dim": 32, "vdim": 64, "kv_rank": 96, "mask": {"size": 192}, "scale": 0.125,
              "rot": {"base": 10000.0, "dims": 32}}
    layers = [{"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": 1536}},
              {"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": 1536}},
              {"type": "attention", "mixer": attn, "mlp": None},
              {"type": "latent_attention", "mixer": latent, "mlp": {"kind": "dense", "ff": 1536}}]
    return {"architecture": "Banitar", "vocab": 8192, "width": 512, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": layers, "loop": {"start": 1, "stop": 3, "times": 2}}


PRESETS["banitar-small"] = _banitar_small()


def _zatasun_small() -> dict:
    """Zatasun with four layers, dense and routed feed-forwards in turn (sizes of no released model)."""
    mixer = {"left": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125,
                      "rot": {"base": 10000.0, "dims": 64,
                              "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 1024}}},
             "left_scale": 1.0, "right": {"width": 512, "blocks": 4, "conv": 4}, "right_scale": 1.0}
    moe = {"kind": "moe", "expert": {"ff": 256, "limit": 7.0}, "router": {"experts": 8, "top": 2},
           "shared": {"ff": 512, "limit": 7.0}}
    layers = [{"type": "parallel", "mixer": mixer, "mlp": {"kind": "dense", "ff": 1536} if i % 2 == 0 else moe}
              for i in range(4)]
    return {"architecture": "Zatasun", "vocab": 8192, "width": 512, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": layers}


PRESETS["zatasun-small"] = _zatasun_small()


def _tarorax_small() -> dict:
    """Tarorax with four layers over four streams, the third of them differential attention; dense and routed
    feed-forwards in turn (sizes of no released model)."""
    gla = {"heads": 8, "dim": 64, "vdim": 64, "tau": 8.0, "rank": 32}
    att = {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 128, "conv": 4, "diff": 0.5, "scale": 0.125, "softcap": 30.0,
           "q_temp": {"coef": 0.3, "every": 128}}
    moe = {"kind": "moe", "expert": {"ff": 256}, "router": {"experts": 8, "top": 2, "scale": 2.5,
                                                            "groups": {"count": 4, "keep": 2}}}
    layers = [{"type": "attention" if i == 2 else "gla", "mixer": att if i == 2 else gla,
               "mlp": {"kind": "dense", "ff": 1536} if i % 2 == 0 else moe} for i in range(4)]
    return {"architecture": "Tarorax", "vocab": 8192, "width": 512, "norm": {"eps": 1e-6}, "streams": 4, "layers": layers}


PRESETS["tarorax-small"] = _tarorax_small()


def preset(name: str) -> dict:
    """The config.json dictionary of a named configuration (a copy)."""
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}' (known: {', '.join(sorted(PRESETS))})")
    return dict(PRESETS[name])
