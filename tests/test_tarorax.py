"""Tarorax through the engine against the plain implementation (``plain_tarorax``): every way of
cutting the same requests into steps, in 32-bit and bfloat16, on configurations that differ in every
size, in the order of their layers, in their feed-forwards and in their constants."""
import copy
import io
import json
import math

import pytest
import torch

import plain_tarorax as plain
import replay
from tiny_tarorax import CONFIGS, TA, TB, TC, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

F64 = torch.float64


# ---------------------------------------------------------------- configuration (no GPU)

def test_config_round_trip_and_registry():
    from airframe_b200.config import TaroraxConfig, config_from_dict
    cfg = config_from_dict(TA)
    assert isinstance(cfg, TaroraxConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    spec = cfg.model_spec()
    assert spec.streams == 3
    assert [(layer.block.kind, layer.mixer.kind, layer.feed_forward.kind) for layer in spec.layers] == \
        [("hyper", "diff_attention", "gated_mlp"), ("hyper", "gated_linear_attention", "routed_experts"),
         ("hyper", "gated_linear_attention", "none"), ("hyper", "diff_attention", "routed_experts")]
    att = spec.layers[0].mixer.params
    assert (att["num_heads"], att["num_kv_heads"], att["head_dim"], att["value_dim"]) == (2, 2, 12, 20)
    assert (att["scale"], att["diff"], att["softcap"], att["taps"], att["q_temp"]) == (0.3, 0.4, 4.0, 3, {"coef": 0.7, "every": 7})
    assert att["weights"]["q_conv"] == "l0.mix.q.conv" and att["weights"]["o_bias"] == "l0.mix.o.b"
    gla = spec.layers[1].mixer.params
    assert (gla["num_heads"], gla["head_dim"], gla["value_dim"], gla["tau"], gla["decay_rank"]) == (3, 8, 20, 4.0, 5)
    ff = spec.layers[1].feed_forward.params
    assert (ff["num_experts"], ff["top"], ff["expert"]) == (6, 2, "gelu_erf")
    assert ff["router"] == {"correction_weight": "l1.mlp.correction", "normalise": True, "scale": 1.5,
                            "groups": {"count": 3, "keep": 2}}
    assert spec.layers[2].norms.keys() == {"pre_mixer"} and spec.layers[0].norms.keys() == {"pre_mixer", "pre_feed_forward"}
    assert spec.layers[0].norms["pre_mixer"].params["weight_offset"] == 1.0
    assert spec.layers[0].block.params["connections"][1]["mix"] == "l0.hc2.mix"
    assert spec.head.params["tied_to"] == "embed"
    # no "streams": one stream and no connection weights; an attention without convolution, cap or temperature
    plain_spec = config_from_dict(TC).model_spec()
    assert plain_spec.streams == 1 and "connections" not in plain_spec.layers[0].block.params
    bare = plain_spec.layers[1].mixer.params
    assert "taps" not in bare and "q_temp" not in bare and bare["softcap"] == 0.0 and "q_conv" not in bare["weights"]
    assert "groups" not in plain_spec.layers[0].feed_forward.params["router"]


def test_config_refuses_what_it_does_not_know():
    from airframe_b200.config import ConfigError, config_from_dict

    def broken(edit):
        d = copy.deepcopy(TA)
        edit(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)

    broken(lambda d: d["layers"][0].update(type="parallel"))
    broken(lambda d: d["layers"][3]["mixer"].update(heads=3, kv_heads=2))
    broken(lambda d: d["layers"][0]["mixer"].pop("diff"))
    broken(lambda d: d["layers"][0]["mixer"].pop("scale"))
    broken(lambda d: d["layers"][0]["mixer"].update(conv=0))
    broken(lambda d: d["layers"][0]["mixer"]["q_temp"].update(every=0))
    broken(lambda d: d["layers"][1]["mixer"].pop("tau"))
    broken(lambda d: d["layers"][1]["mixer"].update(tau=0.0))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="sparse"))
    broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=7))
    broken(lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(count=4))
    broken(lambda d: d["layers"][1]["mlp"]["router"]["groups"].update(keep=4))
    broken(lambda d: d["layers"][3]["mlp"]["router"].update(top=3))       # the one kept group holds two experts
    broken(lambda d: d["layers"][1]["mlp"]["expert"].pop("ff"))
    broken(lambda d: d.pop("norm"))
    broken(lambda d: d.update(streams=0))
    broken(lambda d: d.update(layers=[]))
    from airframe_b200.engine.model import declared_weights
    with pytest.raises(ConfigError):          # more streams than the kernels keep in registers: refused when the model is put together
        declared_weights(config_from_dict(dict(copy.deepcopy(TA), streams=17)).model_spec())


def test_declared_tensors():
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    decls = {d.name: tuple(d.shape) for d in declared_weights(config_from_dict(TA).model_spec())}
    assert decls["embed"] == (211, 72) and decls["final.norm"] == (72,) and "head" not in decls
    assert decls["l0.mix.q"] == (48, 72) and decls["l0.mix.k"] == (48, 72) and decls["l0.mix.v"] == (40, 72)
    assert decls["l3.mix.q"] == (60, 72) and decls["l3.mix.k"] == (20, 72) and decls["l3.mix.v"] == (6, 72)
    assert decls["l0.mix.q.b"] == (48,) and decls["l0.mix.v.b"] == (40,) and decls["l0.mix.o.b"] == (72,)
    assert decls["l0.mix.q.conv"] == (48, 3) and decls["l3.mix.v.conv"] == (6, 2) and decls["l0.mix.lk2"] == (12,)
    assert decls["l0.mix.g"] == (40, 72) and decls["l0.mix.o"] == (72, 40)
    assert decls["l1.mix.q"] == (24, 72) and decls["l1.mix.v"] == (60, 72) and decls["l1.mix.g"] == (60, 72)
    assert decls["l1.mix.a1"] == (5, 72) and decls["l1.mix.a2"] == (24, 5) and decls["l1.mix.a2.b"] == (24,)
    assert decls["l1.mix.norm"] == (20,) and decls["l1.mix.o"] == (72, 60)
    assert decls["l0.mlp.gate"] == (100, 72) and decls["l0.mlp.down"] == (72, 100)
    assert decls["l1.mlp.router"] == (6, 72) and decls["l1.mlp.correction"] == (6,)
    assert decls["l1.mlp.e5.up"] == (36, 72) and decls["l1.mlp.e0.down"] == (72, 36) and "l1.mlp.e0.gate" not in decls
    assert decls["l0.hc1.in"] == (3,) and decls["l0.hc2.mix"] == (3, 3) and decls["l2.hc1.out"] == (3,)
    assert decls["l0.ls1"] == (72,) and decls["l0.ls2"] == (72,) and decls["l2.ls1"] == (72,)
    assert "l2.norm2" not in decls and "l2.ls2" not in decls and "l2.hc2.in" not in decls and "l1.mlp.e6.up" not in decls
    none = {d.name for d in declared_weights(config_from_dict(TC).model_spec())}
    assert not any(".hc" in n or ".conv" in n for n in none if n.startswith("l1.")) and "l2.mix.q.conv" in none


# ---------------------------------------------------------------- the plain implementation on cases known by hand

def test_plain_streams():
    X = [torch.tensor([[1.0, 2.0]], dtype=F64), torch.tensor([[10.0, 20.0]], dtype=F64)]
    assert plain.streams_read(X, torch.tensor([0.5, 0.25], dtype=F64)).tolist() == [[3.0, 6.0]]
    mix = torch.tensor([[1.0, 2.0], [0.0, 3.0]], dtype=F64)          # [from, to]
    y = torch.tensor([[100.0, 200.0]], dtype=F64)
    new = plain.streams_write(X, y, mix, torch.tensor([1.0, -1.0], dtype=F64))
    assert new[0].tolist() == [[101.0, 202.0]]                        # 1 * x0 + 0 * x1 + y
    assert new[1].tolist() == [[2.0 + 30.0 - 100.0, 4.0 + 60.0 - 200.0]]     # 2 * x0 + 3 * x1 - y, from the OLD x0


def test_plain_decay_and_scan():
    h = torch.tensor([[1.0, 0.0]], dtype=F64)
    w1 = torch.tensor([[2.0, 0.0]], dtype=F64)
    w2 = torch.tensor([[1.0], [-1.0]], dtype=F64)
    a = plain.channel_decay(h, w1, w2, torch.tensor([0.0, 2.0], dtype=F64), 4.0)
    assert abs(float(a[0, 0]) - (1 / (1 + math.exp(-2.0))) ** 0.25) < 1e-15 and abs(float(a[0, 1]) - 0.5 ** 0.25) < 1e-15
    q = torch.tensor([[1.0, 1.0], [1.0, 1.0]], dtype=F64)
    k = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=F64)
    v = torch.tensor([[1.0], [10.0]], dtype=F64)
    alpha = torch.tensor([[0.0, 0.0], [0.5, 0.25]], dtype=F64)
    o = plain.decayed_outer_product_scan(q, k, v, alpha)
    # the decay acts on the rows of the key channels: S_1 = diag(.5, .25) [[1], [2]] + [[30], [40]]
    assert o[:, 0].tolist() == [3.0, 0.5 + 0.5 + 70.0]


def test_plain_convolution_temperature_and_difference():
    u = torch.tensor([[1.0], [10.0], [100.0]], dtype=F64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)
    assert plain.short_convolution(u, w)[:, 0].tolist() == [1.0, 12.0, 123.0]      # the last tap is the token's own
    t = plain.query_temperature(8, 0.5, 4)
    assert t[:3].tolist() == [1.0, 1.0, 1.0] and abs(float(t[3]) - (1 + 0.5 * math.log(2.0))) < 1e-15      # p = 3: floor(4 / 4) = 1
    assert abs(float(t[7]) - (1 + 0.5 * math.log(3.0))) < 1e-15
    W = {"p.lq1": torch.tensor([1.0, 1.0], dtype=F64), "p.lk1": torch.tensor([0.5, 0.5], dtype=F64),
         "p.lq2": torch.tensor([0.0, 2.0], dtype=F64), "p.lk2": torch.tensor([9.0, 0.0], dtype=F64)}
    assert abs(plain.difference_factor(W, "p.", 0.25) - (math.e - 1.0 + 0.25)) < 1e-15
    p = plain.capped_causal_softmax(torch.tensor([[0.0], [100.0]], dtype=F64), torch.tensor([[1.0], [1.0]], dtype=F64), 1.0, 2.0)
    assert p[0].tolist() == [1.0, 0.0] and abs(float(p[1, 0]) - 0.5) < 1e-15          # equal capped scores


def test_plain_router():
    # four experts in two groups; the correction moves the choice, not the weights; the groups' scores are sums of two
    W = {"m.router": torch.tensor([[0.0], [2.0], [1.0], [1.0]], dtype=F64),
         "m.correction": torch.tensor([3.0, 0.0, 0.0, 0.0], dtype=F64)}
    h = torch.tensor([[1.0]], dtype=F64)
    s = [0.5, 1 / (1 + math.exp(-2.0)), 1 / (1 + math.exp(-1.0)), 1 / (1 + math.exp(-1.0))]
    ids, w, margin = plain.route(h, W, "m.", {"experts": 4, "top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}})
    assert ids.tolist() == [[0, 1]]                                   # group 0 wins with 3.5 + 0.88 against 2 * 0.73
    assert abs(float(w[0, 0]) - 2.0 * s[0] / (s[0] + s[1])) < 1e-15 and abs(float(w.sum()) - 2.0) < 1e-12
    ids, w, _ = plain.route(h, W, "m.", {"experts": 4, "top": 2, "scale": 1.0})
    assert ids.tolist() == [[0, 1]]
    W["m.correction"] = torch.tensor([-3.0, -3.0, 0.0, 0.0], dtype=F64)          # negative choice scores in the losing group
    ids, w, _ = plain.route(h, W, "m.", {"experts": 4, "top": 1, "scale": 1.0, "groups": {"count": 2, "keep": 1}})
    assert ids.tolist() == [[2]] and abs(float(w[0, 0]) - 1.0) < 1e-12          # equal scores: the lower index


# ---------------------------------------------------------------- the engine

gpu = pytest.mark.gpu


@pytest.fixture(params=["float32", "bfloat16"])
def dtype(request):
    return request.param


_CASES = {}


def rms_rel(got, ref) -> float:
    d = got.double().cpu() - ref.double()
    return float(d.pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt())


CLOSE_CALL = 0.01      # a router's margin (in scores) below which bfloat16 may choose another expert or group
AFTERMATH = 24         # positions after such a token that still feel its other choice (the states, the keys)


class Ref:
    """Reference logits; per position whether every router chose by a clear margin there and at the positions
    before; and ``noise``: how far the plain logits move (root mean square against that of the logits) when nothing
    but every sublayer's input is rounded to bfloat16 - the least that any bfloat16 computation of them must show."""
    def __init__(self, logits, sure, noise=0.0):
        self.logits, self.sure, self.noise = logits, sure, noise

    def __getitem__(self, k):
        return Ref(self.logits[k], self.sure[k], self.noise)


def agrees(got, ref, dtype, what=None, rms=3e-2, worst=0.15):
    """32-bit: the largest difference against the largest reference logit, at every position.  bfloat16: the root
    mean square of the differences against that of the logits, and a looser bound on the largest one, over the
    positions whose routers, and those of the positions before, chose by a clear margin; the bounds are ``rms`` and
    ``worst``, or three times what rounding the sublayers' inputs alone does to the plain logits where that is more
    (the difference of two maps that nearly cancel, and a router between near-equal scores, multiply what rounding does)."""
    sure = None
    if isinstance(ref, Ref):
        rms, worst = max(rms, 3.0 * ref.noise), max(worst, 12.0 * ref.noise)
        ref, sure = ref.logits, ref.sure
    if dtype == "float32":
        assert rel_err(got, ref) < VS_PLAIN[dtype], what
        return
    if sure is not None:
        if not bool(sure.any()):
            return
        got, ref = got.cpu()[sure], ref[sure]
    assert rms_rel(got, ref) < rms, what
    assert rel_err(got, ref) < worst, what


def case(name, tmp_path_factory, edit=None, key=None, cfg_edit=None):
    key = key or name
    if key not in _CASES:
        cfg_dict = copy.deepcopy(CONFIGS[name])
        if cfg_edit is not None:
            cfg_edit(cfg_dict)
        folder = make_folder(cfg_dict, seed=41 + len(_CASES), root=tmp_path_factory.mktemp("tx" + key), edit=edit)
        cfg, w = plain.read_model_folder(folder)
        _CASES[key] = {"folder": folder, "cfg": cfg, "w": w, "ref": {}}
    return _CASES[key]


def reference(c, ids):
    k = tuple(ids)
    if k not in c["ref"]:
        clear = plain.routing_margins(c["cfg"], c["w"], ids) > CLOSE_CALL
        # (a wrong choice stays in a state for good; its weight fades: the positions right behind are left out)
        sure = torch.tensor([bool(clear[max(0, i - AFTERMATH): i + 1].all()) for i in range(len(ids))])
        exact = plain.logits(c["cfg"], c["w"], ids)
        rounded = plain.forward(c["cfg"], c["w"], ids, round_h=lambda z: z.to(torch.bfloat16).to(F64))
        at = sure if bool(sure.any()) else slice(None)
        c["ref"][k] = Ref(exact, sure, rms_rel(rounded[at], exact[at]))
    return c["ref"][k]


def load(c, dtype, max_tokens=64 * 24, **kw):
    from airframe_b200.engine import GpuRuntime
    return GpuRuntime.load(c["folder"], dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    """A prompt in one step; the same tokens with the last 40 one by one (the captured decode step); a prompt
    of one token followed by single tokens only (the convolution's history and the states begin at zero); a
    prompt shorter than the convolution's taps."""
    c = case(name, tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 150, 5)
    ref = reference(c, ids)
    whole = replay.run_whole(rt, ids)
    agrees(whole, ref, dtype)
    tail = replay.run_tail(rt, ids, 40)
    agrees(tail, ref, dtype)
    if dtype == "float32":
        assert rel_err(tail, whole) < SPLITS[dtype] * 4
    agrees(replay.run_tail(rt, ids[:70], 69), ref[:70], dtype)
    agrees(replay.run_whole(rt, ids[:1]), ref[:1], dtype)
    agrees(replay.run_tail(rt, ids[:9], 7), ref[:9], dtype)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_and_slots_used_again(name, dtype, tmp_path_factory):
    """Requests of unequal lengths (one of a single token) in batches, then decoded together, the shorter ones
    leaving; twice, so that slots, their states, histories and pages are used again by other requests."""
    c = case(name, tmp_path_factory)
    rt = load(c, dtype)
    V = c["cfg"]["vocab"]
    reqs = [replay.random_ids(V, n, 100 + n) for n in (90, 1, 37, 160, 66, 12)]
    refs = [reference(c, r) for r in reqs]
    prompt_lens = [70, 1, 5, 150, 64, 2]
    seen = []
    for rnd in range(2):
        out, slots = replay.run_batches(rt, reqs, 4, prompt_lens)
        seen.append(slots)
        for i, r in enumerate(refs):
            agrees(out[i], r, dtype, (rnd, i))
    assert seen[0] == seen[1]
    alone = replay.run_tail(rt, reqs[3], 10)
    if dtype == "float32":
        assert rel_err(alone, out[3]) < SPLITS[dtype] * 4
    else:
        agrees(alone, refs[3], dtype)


@gpu
def test_long_decoding_over_pages(dtype, tmp_path_factory):
    """Three tokens of prompt, then 290 single tokens: cache pages begin at 64, 128, 192 and 256, states and
    histories are carried 290 times, every key stays visible, and the temperature steps several times."""
    c = case("B", tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 293, 9)
    tail = replay.run_tail(rt, ids, 290)
    # (the same tokens as one prompt stand as far from the plain logits, and the two ways of cutting near one another)
    agrees(tail, reference(c, ids), dtype)
    whole = replay.run_whole(rt, ids)
    agrees(whole, reference(c, ids), dtype)
    if dtype == "float32":
        assert rms_rel(tail, whole.double()) < 1e-5
    else:           # (two roundings of the same logits stand a root of two further apart than either from the truth)
        r = reference(c, ids)
        agrees(tail, Ref(whole.double(), r.sure, 1.5 * r.noise), dtype, rms=5e-2, worst=0.3)


@gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_prompts_whose_scan_is_cut_into_chunks(name, dtype, tmp_path_factory):
    """Prompts long enough that the linear attention's scan runs as chunks side by side (five and a half chunks; a
    last chunk of one token): alone, with their last tokens one by one, and two of them beside a short request in
    one step, against the plain implementation."""
    c = case(name, tmp_path_factory)
    rt = load(c, dtype, max_tokens=64 * 40)
    V = c["cfg"]["vocab"]
    reqs = [replay.random_ids(V, n, 500 + n) for n in (700, 513, 5)]
    refs = [reference(c, r) for r in reqs]
    agrees(replay.run_whole(rt, reqs[0]), refs[0], dtype)
    agrees(replay.run_tail(rt, reqs[0], 30), refs[0], dtype)
    out, _ = replay.run_batches(rt, reqs, 3, [690, 513, 3])
    for i, r in enumerate(refs):
        agrees(out[i], r, dtype, i)


def _loud_first_token(name, t):
    """The embedding of token 0 made large: what the first position leaves in keys, values and states is then seen
    from far away through the norms."""
    if name == "embed":
        t = t.clone()
        t[0] *= 6.0
    return t


@gpu
@pytest.mark.parametrize("name", ["B", "C"])
def test_far_tokens_show(name, dtype, tmp_path_factory):
    """The first token reaches the last logits 259 positions on, over four cache pages and through 259 decays."""
    c = case(name, tmp_path_factory, key=name + "-far", edit=_loud_first_token)
    cfg, w = c["cfg"], c["w"]
    ids = [0] + replay.random_ids(cfg["vocab"] - 1, 259, 33)
    ids = [ids[0]] + [i + 1 for i in ids[1:]]
    ref = reference(c, ids)
    other = [1] + ids[1:]
    assert rel_err(plain.logits(cfg, w, other)[-8:], ref.logits[-8:]) > 10 * VS_PLAIN["float32"]
    rt = load(c, dtype)
    agrees(replay.run_tail(rt, ids, 8)[-8:], ref[-8:], dtype)
    agrees(replay.run_whole(rt, ids)[-8:], ref[-8:], dtype)
    agrees(replay.run_tail(rt, ids, 200)[-8:], ref[-8:], dtype)


@gpu
def test_what_a_mechanism_left_out_would_do(dtype, tmp_path_factory):
    """Leaving out the second map, the convolution's earlier taps, the temperature, the correction of the router,
    the layer scale, the mixing of the streams or an output bias moves the plain logits far beyond the tolerance
    that the engine keeps."""
    c = case("A", tmp_path_factory)
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 60, 8)
    ref = reference(c, ids)

    def moved(w2=None, cfg2=None):
        return rms_rel(plain.logits(cfg2 or cfg, w2 or w, ids), ref.logits)

    no_taps = {k: (torch.cat([torch.zeros_like(v[:, :-1]), v[:, -1:]], 1) if k.endswith(".conv") else v) for k, v in w.items()}
    assert moved(no_taps) > 0.04
    assert moved({k: (torch.zeros_like(v) if k.endswith(".correction") else v) for k, v in w.items()}) > 0.02
    assert moved({k: (torch.ones_like(v) if ".ls" in k else v) for k, v in w.items()}) > 0.04
    assert moved({k: (torch.eye(v.shape[0], dtype=F64) if k.endswith(".mix") and ".hc" in k else v) for k, v in w.items()}) > 0.04
    assert moved({k: (torch.zeros_like(v) if k.endswith(".o.b") else v) for k, v in w.items()}) > 0.02
    assert moved({k: (torch.full_like(v, -30.0) if k.endswith("lq2") else v) for k, v in w.items()}) > 0.02
    cold = copy.deepcopy(cfg)
    for layer in cold["layers"]:
        layer["mixer"].pop("q_temp", None)
    assert moved(cfg2=cold) > 0.02
    rt = load(c, dtype)
    agrees(replay.run_whole(rt, ids), ref, dtype)
    agrees(replay.run_tail(rt, ids, 45), ref, dtype)


@gpu
def test_layers_agree_one_by_one(tmp_path_factory):
    """The sum of the streams after every layer, 32-bit, against the plain implementation's."""
    from airframe_b200.engine import StepEntry

    class Keep:
        def __init__(self):
            self.x = []

        def after(self, run, layer, x, batch):
            if run >= 0:
                self.x.append(x.detach().cpu().double())

    for name in ("A", "B", "C", "D"):
        c = case(name, tmp_path_factory)
        rt = load(c, "float32")
        ids = replay.random_ids(c["cfg"]["vocab"], 75, 2)
        per_layer = []
        plain.forward(c["cfg"], c["w"], ids, layers_out=per_layer)
        s = rt.engine.take_slot()
        keep = Keep()
        rt.engine.step([StepEntry(s, ids, [0])], probe=keep)
        rt.engine.free_slot(s)
        assert len(keep.x) == len(per_layer)
        for i, (got, ref) in enumerate(zip(keep.x, per_layer)):
            assert rel_err(got, ref) < 2e-5, (name, i)


@gpu
def test_greedy_generation_through_the_runtime(tmp_path_factory):
    from airframe_b200.sampling import SamplingParams
    c = case("A", tmp_path_factory)
    rt = load(c, "float32")
    V = c["cfg"]["vocab"]
    prompts = [replay.random_ids(V, n, 60 + n) for n in (9, 1, 30)]
    params = SamplingParams(max_tokens=12, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    got = rt.generate(prompts, params)
    want = [plain.generate_greedy(c["cfg"], c["w"], p, 12) for p in prompts]
    assert got == want
    assert rt.generate(prompts[2], params) == want[2]
    rt16 = load(c, "bfloat16")
    out = rt16.generate(prompts, params)
    assert [len(o) for o in out] == [12, 12, 12]


@gpu
def test_trace_replay_of_a_tarorax_folder(tmp_path, tmp_path_factory):
    from airframe_b200.cli.trace_run import main
    c = case("C", tmp_path_factory)
    V = c["cfg"]["vocab"]
    a, b = replay.random_ids(V, 20, 1), replay.random_ids(V, 7, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:18], "want": [0, 17]},
                                     {"id": "b", "tokens": b[:6], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[18]], "want": [0]},
                                     {"id": "b", "tokens": [b[6]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[19]], "want": []}], "end": ["a"]}]
    out = io.StringIO()
    code = main(["--model", str(c["folder"]), "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"), stdout=out)
    assert code == 0 and out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
    import numpy as np
    ra, rb = reference(c, a).logits, reference(c, b).logits
    s0 = torch.from_numpy(np.fromfile(tmp_path / "0.f32", dtype="<f4")).view(2, V)
    s1 = torch.from_numpy(np.fromfile(tmp_path / "1.f32", dtype="<f4")).view(2, V)
    assert rel_err(s0, ra[[0, 17]]) < VS_PLAIN["float32"]
    assert rel_err(s1, torch.stack([ra[18], rb[6]])) < VS_PLAIN["float32"]
    assert not (tmp_path / "2.f32").exists()


@gpu
def test_long_prompt_at_layer_sizes_beyond_the_plain_implementation(tmp_path_factory):
    """The named small configuration (tensor-core products and attention, routed experts on the tensor cores) on a
    prompt of 2,500 tokens, then 70 single tokens: too long for the plain implementation, so the engine is held
    against itself: the 32-bit logits must not depend on where the prompt ends and the single tokens begin, and
    bfloat16 must agree with 32-bit within its rounding."""
    from airframe_b200.config.presets import preset
    folder = make_folder(preset("tarorax-small"), seed=4, root=tmp_path_factory.mktemp("txsmall"))
    from airframe_b200.engine import GpuRuntime, StepEntry
    ids = replay.random_ids(8192, 2570, 17)
    want = [0, 1, 255, 256, 257, 1023, 2047, 2499]

    def run(dtype, cut):
        rt = GpuRuntime.load(folder, dtype=dtype, max_tokens=64 * 48, max_context=4096)
        s = rt.engine.take_slot()
        out = [rt.step([StepEntry(s, ids[:cut], [w for w in want if w < cut])]).cpu()]
        for t in ids[cut:]:
            out.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        rt.engine.free_slot(s)
        return torch.cat(out)

    a = run("float32", 2500)
    assert torch.isfinite(a).all()
    b = run("float32", 2540)
    assert rel_err(b[-30:], a[-30:]) < 1e-4
    c = run("bfloat16", 2500)
    assert rms_rel(c, a) < 6e-2
