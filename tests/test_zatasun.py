"""Zatasun through the engine against the plain implementation (``plain_zatasun``): every way of
cutting the same requests into steps, in 32-bit and bfloat16, on configurations that differ in every
size, in their feed-forwards and in their constants."""
import copy
import io
import json
import math

import pytest
import torch

import plain_zatasun as plain
import replay
from tiny_zatasun import CONFIGS, ZA, ZB, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

F64 = torch.float64


# ---------------------------------------------------------------- configuration (no GPU)

def test_config_round_trip_and_registry():
    from airframe_b200.config import ZatasunConfig, config_from_dict
    cfg = config_from_dict(ZA)
    assert isinstance(cfg, ZatasunConfig)
    again = config_from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    spec = cfg.model_spec()
    assert [(layer.block.kind, layer.mixer.kind, layer.feed_forward.kind) for layer in spec.layers] == \
        [("postnorm", "parallel", "gated_mlp"), ("postnorm", "parallel", "routed_experts"),
         ("postnorm", "parallel", "none"), ("postnorm", "parallel", "routed_experts")]
    left, right = (b["mixer"] for b in spec.layers[1].mixer.params["branches"])
    assert [b["scale"] for b in spec.layers[1].mixer.params["branches"]] == [0.6, 1.3]
    assert left.kind == "attention" and left.params["value_dim"] == 20 and left.params["qk_norm"]["whole"] is True
    assert left.params["sink_weight"] == "l1.mix.left.sink" and left.params["scale"] == 0.25
    rot = left.params["position"].params
    assert rot["pairing"] == "half" and rot["rotary_dim"] == 20 and rot["scaling"]["kind"] == "wavelength"
    assert rot["scaling"]["original"] == 64.0 and "scaling" not in spec.layers[0].mixer.params["branches"][0]["mixer"].params["position"].params
    assert right.kind == "rglru" and (right.params["width"], right.params["blocks"], right.params["taps"]) == (30, 3, 4)
    ff = spec.layers[1].feed_forward.params
    assert (ff["num_experts"], ff["top"], ff["limit"], ff["shared"]["limit"]) == (5, 2, 1.0, 0.7)
    assert "shared" not in spec.layers[3].feed_forward.params
    assert spec.layers[2].norms.keys() == {"post_mixer"} and spec.layers[0].norms.keys() == {"post_mixer", "post_feed_forward"}
    assert spec.embedding.params["norm"].params["weight"] == "embed.norm"
    assert spec.head.params["tied_to"] == "embed" and spec.head.params["scale"] == 1.0
    assert config_from_dict(ZB).model_spec().head.params["scale"] == 0.25


def test_config_refuses_what_it_does_not_know():
    from airframe_b200.config import ConfigError, config_from_dict

    def broken(edit):
        d = copy.deepcopy(ZA)
        edit(d)
        with pytest.raises(ConfigError):
            config_from_dict(d)

    broken(lambda d: d["layers"][0].update(type="attention"))
    broken(lambda d: d["layers"][1]["mixer"]["left"].update(heads=3, kv_heads=2))
    broken(lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=22))
    broken(lambda d: d["layers"][1]["mixer"]["left"]["rot"]["scaling"].pop("low"))
    broken(lambda d: d["layers"][1]["mixer"]["left"]["rot"]["scaling"].update(high=1.0))
    broken(lambda d: d["layers"][1]["mixer"]["right"].update(blocks=4))
    broken(lambda d: d["layers"][1]["mixer"]["right"].update(conv=0))
    broken(lambda d: d["layers"][1]["mixer"].pop("left_scale"))
    broken(lambda d: d["layers"][0]["mlp"].update(kind="sparse"))
    broken(lambda d: d["layers"][1]["mlp"]["router"].update(top=6))
    broken(lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"))
    broken(lambda d: d["layers"][1]["mlp"]["shared"].pop("ff"))
    broken(lambda d: d.pop("norm"))
    broken(lambda d: d.pop("logit_scale"))
    broken(lambda d: d.update(layers=[]))


def test_declared_tensors():
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    decls = {d.name: tuple(d.shape) for d in declared_weights(config_from_dict(ZA).model_spec())}
    assert decls["embed"] == (211, 72) and decls["embed.norm"] == (72,) and decls["final.norm"] == (72,)
    assert "head" not in decls
    assert decls["l1.mix.left.q"] == (40, 72) and decls["l1.mix.left.k"] == (20, 72) and decls["l1.mix.left.v"] == (20, 72)
    assert decls["l1.mix.left.q.norm"] == (40,) and decls["l1.mix.left.k.norm"] == (20,)
    assert decls["l0.mix.left.q.norm"] == (48,) and decls["l0.mix.left.o"] == (72, 80) and decls["l0.mix.left.sink"] == (4,)
    assert decls["l1.mix.right.y"] == (30, 72) and decls["l1.mix.right.x.b"] == (30,) and decls["l1.mix.right.conv"] == (30, 4)
    assert decls["l1.mix.right.conv.b"] == (30,) and decls["l1.mix.right.ra"] == (3, 10, 10) and decls["l1.mix.right.ri.b"] == (3, 10)
    assert decls["l1.mix.right.lam"] == (30,) and decls["l1.mix.right.o"] == (72, 30)
    assert decls["l0.mlp.gate"] == (100, 72) and decls["l0.mlp.down"] == (72, 100) and decls["l0.norm2"] == (72,)
    assert decls["l1.mlp.router"] == (5, 72) and decls["l1.mlp.e4.up"] == (36, 72) and decls["l1.mlp.e0.down"] == (72, 36)
    assert decls["l1.mlp.shared.gate"] == (28, 72) and decls["l1.mlp.shared.sg"] == (1, 72)
    assert "l2.norm2" not in decls and "l2.mlp.gate" not in decls and "l3.mlp.shared.sg" not in decls and "l1.mlp.e5.up" not in decls


# ---------------------------------------------------------------- the plain implementation on cases known by hand

def test_plain_frequencies_and_rotation():
    # base 100, 8 dims: f = 1, 100^-1/4, 100^-1/2, 100^-3/4; wavelengths 6.28, 19.9, 62.8, 198.7.  Trained for
    # 100 positions with high 4 and low 1: shorter than 25 stays, longer than 100 is divided, 62.8 is mixed
    f = plain.stretched_frequencies(100.0, 8)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=F64))
    g = plain.stretched_frequencies(100.0, 8, {"factor": 5.0, "low": 1.0, "high": 4.0, "original": 100})
    assert g[0] == f[0] and g[1] == f[1] and abs(float(g[3]) - float(f[3]) / 5.0) < 1e-15
    s = (100 / (2 * math.pi / 0.1) - 1.0) / 3.0
    assert abs(float(g[2]) - ((1 - s) * 0.1 / 5.0 + s * 0.1)) < 1e-15 and 0 < s < 1
    x = torch.randn(3, 2, 10, dtype=F64)
    y = plain.rotate_half(x, torch.tensor([0, 1, 2]), f)
    one = torch.tensor(1.0, dtype=F64)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
    assert torch.allclose(y[1, 0, 0], x[1, 0, 0] * torch.cos(one) - x[1, 0, 4] * torch.sin(one))
    assert torch.allclose(y[1, 0, 4], x[1, 0, 4] * torch.cos(one) + x[1, 0, 0] * torch.sin(one))
    assert torch.allclose(y[2, 1, 6], x[2, 1, 6] * torch.cos(0.2 * one) + x[2, 1, 2] * torch.sin(0.2 * one))
    assert torch.equal(plain.rotate_half(x, torch.tensor([0, 1, 2]), plain.stretched_frequencies(10.0, 0)), x)


def test_plain_sink_attention_and_norms():
    q = torch.zeros(2, 2, 3, dtype=F64)
    k = torch.zeros(2, 1, 3, dtype=F64)
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=F64)
    sink = torch.tensor([0.0, math.log(2.0)], dtype=F64)
    o = plain.sink_attention(q, k, v, 0.7, sink)
    # scores are 0: the sink counts once as exp(sink), has no value, and is not scaled
    assert torch.allclose(o[0, 0], torch.tensor([0.5, 0.0], dtype=F64)) and torch.allclose(o[1, 0], torch.tensor([1 / 3, 1 / 3], dtype=F64))
    assert torch.allclose(o[0, 1], torch.tensor([1 / 3, 0.0], dtype=F64)) and torch.allclose(o[1, 1], torch.tensor([0.25, 0.25], dtype=F64))
    x = torch.tensor([3.0, 4.0], dtype=F64)
    assert torch.allclose(plain.rms(x, 0.5), x / math.sqrt(13.0))
    assert torch.allclose(plain.rms(x, 0.0, torch.tensor([2.0, 0.5], dtype=F64)), torch.tensor([6.0, 2.0], dtype=F64) / math.sqrt(12.5))
    assert abs(float(plain.gelu_tanh(torch.tensor(1.0, dtype=F64))) - 0.8411919906082768) < 1e-12


def test_plain_convolution_and_recurrence():
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=F64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)
    out = plain.causal_conv(x, w, torch.tensor([0.5], dtype=F64))
    assert out[:, 0].tolist() == [1.5, 12.5, 123.5]          # the last tap is the current token's; zeros before the start
    u = torch.tensor([[2.0], [3.0]], dtype=F64)
    r = torch.tensor([[0.5], [0.25]], dtype=F64)
    i = torch.tensor([[0.5], [1.0]], dtype=F64)
    lam = torch.tensor([0.0], dtype=F64)
    S = plain.gated_linear_recurrence(u, r, i, lam)
    a0, a1 = math.exp(-8 * 0.5 * math.log(2.0)), math.exp(-8 * 0.25 * math.log(2.0))
    s0 = math.sqrt(1 - a0 * a0) * 0.5 * 2.0                    # the first token has no special case
    assert abs(float(S[0]) - s0) < 1e-15 and abs(float(S[1]) - (a1 * s0 + math.sqrt(1 - a1 * a1) * 3.0)) < 1e-15
    assert abs(a0 - 1 / 16) < 1e-15


def test_plain_experts():
    W = {"e.gate": torch.tensor([[1.0, 0.0]], dtype=F64), "e.up": torch.tensor([[0.0, 1.0]], dtype=F64),
         "e.down": torch.tensor([[1.0], [2.0]], dtype=F64)}
    h = torch.tensor([[5.0, -9.0], [0.5, 0.25]], dtype=F64)
    y = plain.clamped_expert(h, W, "e.", 2.0)
    g0 = 2.0 * (1 / (1 + math.exp(-1.702 * 2.0))) * (-2.0 + 1.0)          # gate cut from above, up from both sides
    g1 = 0.5 * (1 / (1 + math.exp(-1.702 * 0.5))) * 1.25
    assert torch.allclose(y, torch.tensor([[g0, 2 * g0], [g1, 2 * g1]], dtype=F64))
    # two experts, one chosen: the score multiplies the input (which a clamp then cuts), not the output
    W = {"m.router": torch.tensor([[1.0, 0.0], [-1.0, 0.0]], dtype=F64)}
    for e in (0, 1):
        W[f"m.e{e}.gate"] = torch.tensor([[float(e + 1), 0.0]], dtype=F64)
        W[f"m.e{e}.up"] = torch.zeros(1, 2, dtype=F64)
        W[f"m.e{e}.down"] = torch.tensor([[1.0], [0.0]], dtype=F64)
    mlp = {"router": {"experts": 2, "top": 1}, "expert": {"limit": 100.0}}
    h = torch.tensor([[1.0, 0.0], [-1.0, 0.0]], dtype=F64)
    out = plain.routed_ff(h, W, "m.", mlp)
    s = 1 / (1 + math.exp(-1.0))
    assert abs(float(out[0, 0]) - s * (1 / (1 + math.exp(-1.702 * s)))) < 1e-15       # expert 0 on s * h
    assert abs(float(out[1, 0]) - (-2 * s) * (1 / (1 + math.exp(1.702 * 2 * s)))) < 1e-15    # expert 1 on s * h
    # a shared expert is added, times its own sigmoid gate
    W.update({"m.shared.gate": torch.tensor([[1.0, 0.0]], dtype=F64), "m.shared.up": torch.zeros(1, 2, dtype=F64),
              "m.shared.down": torch.tensor([[0.0], [1.0]], dtype=F64), "m.shared.sg": torch.tensor([[0.0, 0.0]], dtype=F64)})
    both = plain.routed_ff(h, W, "m.", dict(mlp, shared={"limit": 0.25}))
    assert torch.allclose(both[:, 0], out[:, 0])
    assert abs(float(both[0, 1]) - 0.5 * 0.25 * (1 / (1 + math.exp(-1.702 * 0.25)))) < 1e-15


# ---------------------------------------------------------------- the engine

gpu = pytest.mark.gpu


@pytest.fixture(params=["float32", "bfloat16"])
def dtype(request):
    return request.param


_CASES = {}


def rms_rel(got, ref) -> float:
    d = got.double().cpu() - ref.double()
    return float(d.pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt())


CLOSE_CALL = 0.006     # a router's margin (in scores) below which bfloat16 may choose another expert
AFTERMATH = 10         # positions after such a token that still feel its other choice (convolution, state, keys)


class Ref:
    """Reference logits with, per position, whether every router chose by a clear margin there and at the
    ``AFTERMATH`` positions before."""
    def __init__(self, logits, sure):
        self.logits, self.sure = logits, sure

    def __getitem__(self, k):
        return Ref(self.logits[k], self.sure[k])


def agrees(got, ref, dtype, what=None, rms=3e-2, worst=0.15):
    """32-bit: the largest difference against the largest reference logit, at every position.  bfloat16: the root
    mean square of the differences against that of the logits, and a looser bound on the largest one, over the
    positions whose routers, and those of the few positions before, chose by a clear margin (elsewhere bfloat16
    may rightly choose the runner-up)."""
    sure = None
    if isinstance(ref, Ref):
        ref, sure = ref.logits, ref.sure
    if dtype == "float32":
        assert rel_err(got, ref) < VS_PLAIN[dtype], what
        return
    if sure is not None:
        assert len(sure) < 100 or float(sure.double().mean()) > 0.2, what
        if not bool(sure.any()):
            return
        got, ref = got.cpu()[sure], ref[sure]
    assert rms_rel(got, ref) < rms, what
    assert rel_err(got, ref) < worst, what


def case(name, tmp_path_factory, edit=None, key=None, cfg_edit=None):
    """Folder, plain configuration and weights of a configuration (made once a session)."""
    key = key or name
    if key not in _CASES:
        cfg_dict = copy.deepcopy(CONFIGS[name])
        if cfg_edit is not None:
            cfg_edit(cfg_dict)
        folder = make_folder(cfg_dict, seed=23 + len(_CASES), root=tmp_path_factory.mktemp("zt" + key), edit=edit)
        cfg, w = plain.read_model_folder(folder)
        _CASES[key] = {"folder": folder, "cfg": cfg, "w": w, "ref": {}}
    return _CASES[key]


def reference(c, ids):
    k = tuple(ids)
    if k not in c["ref"]:
        clear = plain.routing_margins(c["cfg"], c["w"], ids) > CLOSE_CALL
        sure = torch.tensor([bool(clear[max(0, i - AFTERMATH): i + 1].all()) for i in range(len(ids))])
        c["ref"][k] = Ref(plain.logits(c["cfg"], c["w"], ids), sure)
    return c["ref"][k]


def load(c, dtype, max_tokens=64 * 24, **kw):
    from airframe_b200.engine import GpuRuntime
    return GpuRuntime.load(c["folder"], dtype=dtype, max_tokens=max_tokens, **kw)


@gpu
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_and_token_by_token(name, dtype, tmp_path_factory):
    """A prompt in one step; the same tokens with the last 40 one by one (the captured decode step);
    and a prompt of one token followed by single tokens only (the first tokens of a sequence, decoded:
    the convolution's history and the recurrence's state begin at zero)."""
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
    short = ids[:70]
    agrees(replay.run_tail(rt, short, 69), ref[:70], dtype)
    agrees(replay.run_whole(rt, ids[:1]), ref[:1], dtype)
    agrees(replay.run_tail(rt, ids[:9], 7), ref[:9], dtype)          # a prompt of two tokens, shorter than the taps


@gpu
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_and_slots_used_again(name, dtype, tmp_path_factory):
    """Requests of unequal lengths (one of a single token) in batches, then decoded together, the shorter
    ones leaving; twice, so that slots, their states and their pages are used again by other requests."""
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
    assert seen[0] == seen[1]                      # the same slots served other requests in between
    alone = replay.run_tail(rt, reqs[3], 10)
    if dtype == "float32":
        assert rel_err(alone, out[3]) < SPLITS[dtype] * 4        # each alone gives what it gave in company
    else:
        agrees(alone, refs[3], dtype)


@gpu
def test_long_decoding_over_pages(dtype, tmp_path_factory):
    """Three tokens of prompt, then 290 single tokens: cache pages begin at 64, 128, 192 and 256, the state is
    carried 290 times, and every key stays visible."""
    c = case("B", tmp_path_factory)
    rt = load(c, dtype)
    ids = replay.random_ids(c["cfg"]["vocab"], 293, 9)
    agrees(replay.run_tail(rt, ids, 290), reference(c, ids), dtype)


def _only(side):
    def edit(cfg):
        for layer in cfg["layers"]:
            layer["mixer"]["left_scale" if side == "right" else "right_scale"] = 0.0
    return edit


@gpu
@pytest.mark.parametrize("side", ["left", "right"])
def test_far_tokens_show(side, dtype, tmp_path_factory):
    """With one of the two mixers switched off, the first token reaches the last logits 259 positions on through
    the other alone: through attention's keys (over four cache pages), or through the slow channels of the
    recurrence."""
    c = case("B", tmp_path_factory, key="B-" + side, cfg_edit=_only(side))
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 260, 33)
    ref = reference(c, ids)
    first = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    assert rel_err(plain.logits(cfg, w, first)[-8:], ref.logits[-8:]) > 10 * VS_PLAIN["float32"]
    rt = load(c, dtype)
    agrees(replay.run_tail(rt, ids, 8)[-8:], ref[-8:], dtype)
    agrees(replay.run_whole(rt, ids)[-8:], ref[-8:], dtype)
    agrees(replay.run_tail(rt, ids, 200)[-8:], ref[-8:], dtype)


@gpu
def test_what_a_mechanism_left_out_would_do(dtype, tmp_path_factory):
    """Leaving out the sink, the norm over the whole projection (for one per head), the stretching of the
    frequencies, the convolution's earlier taps, the weight on an expert's input (for its output) or the
    embedding's norm moves the plain logits far beyond the tolerance that the engine keeps."""
    c = case("A", tmp_path_factory)
    cfg, w = c["cfg"], c["w"]
    ids = replay.random_ids(cfg["vocab"], 60, 8)
    ref = reference(c, ids)
    no_sink = {k: (torch.full_like(v, -1e30) if k.endswith(".sink") else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, no_sink, ids), ref.logits) > 0.04
    no_taps = {k: (torch.cat([torch.zeros_like(v[:, :-1]), v[:, -1:]], 1) if k.endswith(".conv") else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, no_taps, ids), ref.logits) > 0.04
    no_stretch = copy.deepcopy(cfg)
    for layer in no_stretch["layers"]:
        layer["mixer"]["left"]["rot"].pop("scaling", None)
    assert rms_rel(plain.logits(no_stretch, w, ids), ref.logits) > 0.04
    flat = {k: (torch.ones_like(v) if k == "embed.norm" else v) for k, v in w.items()}
    assert rms_rel(plain.logits(cfg, flat, ids), ref.logits) > 0.04
    top_all = copy.deepcopy(cfg)
    top_all["layers"][1]["mlp"]["router"]["top"] = 3
    assert rms_rel(plain.logits(top_all, w, ids), ref.logits) > 0.04
    rt = load(c, dtype)
    agrees(replay.run_whole(rt, ids), ref, dtype)
    agrees(replay.run_tail(rt, ids, 45), ref, dtype)


@gpu
def test_layers_agree_one_by_one(tmp_path_factory):
    """The residual stream after every layer, 32-bit, against the plain implementation's."""
    from airframe_b200.engine import StepEntry

    class Keep:
        def __init__(self):
            self.x = []

        def after(self, run, layer, x, batch):
            if run >= 0:
                self.x.append(x.detach().cpu().double())

    for name in ("A", "B", "C"):
        c = case(name, tmp_path_factory)
        rt = load(c, "float32")
        ids = replay.random_ids(c["cfg"]["vocab"], 75, 2)
        per_layer = []
        plain.hidden_states(c["cfg"], c["w"], ids, per_layer)
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
def test_trace_replay_of_a_zatasun_folder(tmp_path, tmp_path_factory):
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
    """The named small configuration (tensor-core products, two of eight experts and a shared one) on a prompt of
    2,500 tokens, then 70 single tokens: too long for the plain implementation, so the engine is held against
    itself: the 32-bit logits must not depend on where the prompt ends and the single tokens begin, and bfloat16
    must agree with 32-bit within its rounding."""
    from airframe_b200.config.presets import preset
    folder = make_folder(preset("zatasun-small"), seed=4, root=tmp_path_factory.mktemp("ztsmall"))
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
    # the last 30 tokens were single tokens in both runs; tokens 2500..2539 single in one, of the prompt in the other
    assert rel_err(b[-30:], a[-30:]) < 1e-4
    c = run("bfloat16", 2500)
    assert rms_rel(c, a) < 4e-2
