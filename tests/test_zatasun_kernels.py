"""The kernels behind Zatasun's mechanisms, each alone against the plain implementation's functions
(``plain_zatasun``, float64): the convolution with its history in the state, the block-diagonal gates, the
scan of the recurrence (prompts, single tokens, portions down to two tokens, slots used again), the router
with its choice, the experts' products over sorted rows, the norm over a whole projection with the rotation
behind it, and the residual step that norms a weighted sum."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_zatasun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def K():
    from airframe_b200 import kernels
    return kernels


def close(got, ref, tol):
    ref = ref.double().cpu()
    err = float((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
    assert err < tol, err


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def batch_of(lens, slots, before=None):
    """What the kernels read of a step: sequences packed one after the other, ``before`` tokens seen already."""
    before = before or [0] * len(lens)
    starts, seq, pos = [0], [], []
    for b, n in enumerate(lens):
        starts.append(starts[-1] + n)
        seq += [b] * n
        pos += list(range(before[b], before[b] + n))
    return SimpleNamespace(seq_starts=i32(starts), slots=i32(slots), n_seqs=len(lens), n_tokens=starts[-1],
                           seq_of_token=i32(seq), positions=i32(pos), len_after=i32([a + n for a, n in zip(before, lens)]))


# ---------------------------------------------------------------- the recurrence

def plain_recurrent_rows(px, py, w, cut=None):
    """u, S and S * gelu(y) of one sequence from its projection rows, by the plain functions."""
    u = plain.causal_conv(px + w["bx"], w["cw"], w["cb"])
    T, width = u.shape
    blocks = w["wa"].shape[0]
    ub = u.view(T, blocks, width // blocks)
    r = plain.sigmoid(torch.einsum("boi,tbi->tbo", w["wa"], ub) + w["ba"].view(blocks, -1)).reshape(T, width)
    i = plain.sigmoid(torch.einsum("boi,tbi->tbo", w["wi"], ub) + w["bi"].view(blocks, -1)).reshape(T, width)
    S = plain.gated_linear_recurrence(u, r, i, w["lam"])
    return u, S, S * plain.gelu_tanh(py + w["by"])


def run_recurrent_step(K, w, proj, batch, state, out_dtype, gate_dtype):
    """One step as the mixer runs it: convolution, gates, scan."""
    width, T = w["lam"].numel(), proj.shape[0]
    dev = lambda t, dt=torch.float32: t.to(dt).to(DEV).contiguous()
    rate = dev(8.0 * plain.softplus(w["lam"]))
    u = torch.empty(T, width, device=DEV)
    K.conv_rows(u, proj, width, dev(w["bx"]), dev(w["cw"].t()), dev(w["cb"]), state, batch)
    decay, inp = torch.empty_like(u), torch.empty_like(u)
    K.gate_rows(decay, inp, u, dev(w["wa"], gate_dtype), dev(w["wi"], gate_dtype), dev(w["ba"]), dev(w["bi"]), rate)
    y = torch.empty(T, width, dtype=out_dtype, device=DEV)
    K.decay_scan(y, decay, inp, proj, 0, width, dev(w["by"]), dev(w["bx"]), state, batch)
    return u, y


def recurrent_weights(width, blocks, taps, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    bw = width // blocks
    return {"bx": r(width), "by": r(width), "cw": r(width, taps), "cb": r(width), "wa": r(blocks, bw, bw) / math.sqrt(bw),
            "wi": r(blocks, bw, bw) / math.sqrt(bw), "ba": r(width), "bi": r(width),
            "lam": torch.linspace(-7.0, 1.5, width, dtype=F64)}      # decays from a = 0.99 a token down to nothing


@pytest.mark.parametrize("width,blocks,taps", [(44, 1, 1), (30, 3, 4), (256, 2, 4), (26, 13, 5), (128, 8, 2), (300, 4, 3), (640, 2, 3), (48, 2, 9), (64, 4, 8)])
def test_convolution_gates_and_scan(K, width, blocks, taps):
    w = recurrent_weights(width, blocks, taps, width)
    lens, slots = [61, 1, 6, 2], [4, 0, 2, 5]       # (70 rows: the convolution's window kernel, sequences that begin inside a thread's four tokens)
    g = torch.Generator().manual_seed(7)
    seqs = [torch.randn(n + 9, 2 * width, generator=g, dtype=F64) for n in lens]     # [y | x] rows, 9 more to decode
    want = [plain_recurrent_rows(s[:, width:], s[:, :width], w) for s in seqs]
    for out_dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        state = torch.full((6, taps, width), 7.0, device=DEV)
        state[slots] = 0.0                                   # (a slot begins at zero; the others' rows must not be read)
        proj = torch.cat([s[:n] for s, n in zip(seqs, lens)]).float().to(DEV)
        u, y = run_recurrent_step(K, w, proj, batch_of(lens, slots), state, out_dtype, torch.float32)
        at = 0
        for (ru, rS, ry), n, slot in zip(want, lens, slots):
            close(u[at:at + n], ru[:n], 2e-6)
            close(y[at:at + n], ry[:n], tol)
            close(state[slot, 0], rS[n - 1], 3e-6)
            at += n
        assert float(state[1].min()) == 7.0 and float(state[3].max()) == 7.0
        # nine single tokens each, all four together: the history of the convolution and the state come from the slots
        for t in range(9):
            proj = torch.stack([s[n + t] for s, n in zip(seqs, lens)]).float().to(DEV)
            u, y = run_recurrent_step(K, w, proj, batch_of([1] * 4, slots, [n + t for n in lens]), state, out_dtype,
                                      torch.float32)
            for b, ((ru, rS, ry), n, slot) in enumerate(zip(want, lens, slots)):
                close(u[b], ru[n + t], 2e-6)
                close(y[b], ry[n + t], tol)
                close(state[slot, 0], rS[n + t], 4e-6)


@pytest.mark.parametrize("width,blocks,taps", [(30, 3, 4), (128, 8, 2), (44, 1, 1), (60, 2, 6)])
def test_portions_and_a_slot_used_again(K, width, blocks, taps):
    """A sequence fed in portions of 2, 7, 1, 3, 19 and 70 tokens gives what it gives whole; then another sequence in
    the same slot, once its rows are zero again, knows nothing of the first."""
    w = recurrent_weights(width, blocks, taps, 3 * width)
    g = torch.Generator().manual_seed(11)
    for round_, n_total in enumerate((102, 102)):
        rows = torch.randn(n_total, 2 * width, generator=g, dtype=F64)
        ru, rS, ry = plain_recurrent_rows(rows[:, width:], rows[:, :width], w)
        if round_ == 0:
            state = torch.zeros(3, taps, width, device=DEV)
        else:
            state[1] = 0.0
        at = 0
        for n in (2, 7, 1, 3, 19, 70):       # (the last portion: many rows that begin in the slot's history)
            u, y = run_recurrent_step(K, w, rows[at:at + n].float().to(DEV), batch_of([n], [1], [at]), state,
                                      torch.float32, torch.float32)
            close(u, ru[at:at + n], 2e-6)
            close(y, ry[at:at + n], 4e-6)
            at += n
        close(state[1, 0], rS[-1], 4e-6)
        if taps > 1:       # the rows behind the state hold the last inputs of the convolution, the oldest first
            close(state[1, 1:], (rows[-(taps - 1):, width:] + w["bx"]), 2e-6)


def test_gates_in_bfloat16_and_slow_channels(K):
    """Gate matrices in bfloat16 (sums in 32 bits); a channel whose decay is 1 - 3e-7 a token keeps its state over 400
    tokens as the 64-bit recurrence does (1 - a is what the scan is given, so that a's distance from 1 survives)."""
    width, blocks, taps = 64, 4, 3
    w = recurrent_weights(width, blocks, taps, 5)
    w["lam"] = torch.linspace(-18.0, -10.0, width, dtype=F64)
    w["wa"], w["wi"] = w["wa"].bfloat16().double(), w["wi"].bfloat16().double()
    rows = torch.randn(400, 2 * width, generator=torch.Generator().manual_seed(2), dtype=F64)
    ru, rS, ry = plain_recurrent_rows(rows[:, width:], rows[:, :width], w)
    state = torch.zeros(1, taps, width, device=DEV)
    _, y = run_recurrent_step(K, w, rows[:300].float().to(DEV), batch_of([300], [0]), state, torch.float32, torch.bfloat16)
    close(y, ry[:300], 2e-5)
    for t in range(300, 400):
        _, y = run_recurrent_step(K, w, rows[t:t + 1].float().to(DEV), batch_of([1], [0], [t]), state, torch.float32,
                                  torch.bfloat16)
    close(y[0], ry[399], 2e-5)
    close(state[0, 0], rS[399], 2e-5)
    assert float(rS[399].abs().max()) > 1e-3        # (the slow channels have gathered something to keep)


# ---------------------------------------------------------------- routed experts

def expert_weights(E, H, F, seed, shared=None):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).bfloat16().double()
    W = {"m.router": r(E, H) * 4.0}
    for e in range(E):
        W.update({f"m.e{e}.gate": r(F, H) * 2.0, f"m.e{e}.up": r(F, H) * 2.0, f"m.e{e}.down": r(H, F)})
    if shared:
        W.update({"m.shared.gate": r(shared, H) * 2.0, "m.shared.up": r(shared, H) * 2.0, "m.shared.down": r(H, shared),
                  "m.shared.sg": r(1, H) * 4.0})
    return W


@pytest.mark.parametrize("E,top,H,F,T,limit", [(5, 2, 72, 36, 50, 1.0), (8, 1, 128, 64, 300, 2.0), (3, 3, 50, 13, 7, 0.5),
                                                (2, 1, 40, 24, 1, 4.0), (12, 4, 64, 96, 130, 1.5), (1, 1, 24, 8, 33, 0.7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_plan_and_expert_products(K, E, top, H, F, T, limit, dtype):
    W = expert_weights(E, H, F, E * 100 + T, shared=20)
    h = torch.randn(T, H, generator=torch.Generator().manual_seed(T)).bfloat16().double()
    mlp = {"router": {"experts": E, "top": top}, "expert": {"limit": limit}}
    want = plain.routed_ff(h, W, "m.", mlp)
    x = h.to(dtype).to(DEV)
    router = torch.cat([W["m.router"], W["m.shared.sg"]]).float().to(DEV)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    mix = torch.empty(T, device=DEV)
    K.expert_route(ids, wts, mix, x, router, E)
    s = plain.sigmoid(h @ W["m.router"].T)
    order = torch.tensor([sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top] for t in range(T)])
    assert torch.equal(ids.cpu().long(), order)
    close(wts, s.gather(1, order), 2e-6)
    close(mix, plain.sigmoid(h @ W["m.shared.sg"].T)[:, 0], 2e-6)
    perm = torch.empty(T * top, dtype=torch.int32, device=DEV)
    plan = torch.empty(1 + 3 * K.expert_max_tiles(T * top, E), dtype=torch.int32, device=DEV)
    K.expert_plan(perm, plan, ids, E)
    p = perm.cpu().long()
    assert sorted(p.tolist()) == list(range(T * top))
    by_expert = ids.cpu().long().reshape(-1)[p]
    assert torch.equal(by_expert, by_expert.sort().values)               # the sorted rows go expert by expert
    tiles = plan.cpu()[1: 1 + 3 * int(plan[0])].view(-1, 3)
    covered = []
    for e, first, rows in tiles.tolist():
        assert 0 < rows <= K.EXPERT_TILE and set(by_expert[first: first + rows].tolist()) == {e}
        covered += list(range(first, first + rows))
    assert covered == list(range(T * top))
    stack = lambda role: torch.stack([W[f"m.e{e}.{role}"] for e in range(E)]).to(dtype).to(DEV).contiguous()
    mid = torch.empty(T * top, F, dtype=dtype, device=DEV)
    K.expert_rows(mid, x, stack("gate"), stack("up"), perm=perm, plan=plan, pair_weight=wts, n_tokens=T, top=top, limit=limit)
    out = torch.empty(top, T, H, device=DEV)
    K.expert_rows(out, mid, stack("down"), perm=perm, plan=plan, n_tokens=T, top=top)
    close(out.sum(0), want, 2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("E,top,H", [(5, 2, 72), (7, 3, 50), (40, 4, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_chooses_alike_for_a_prompt_and_for_single_tokens(K, E, top, H, dtype):
    """The router over a prompt of 1,030 tokens (several tokens a block) against the plain scores, and bit for bit
    against the same tokens routed a few at a time (the form a decode step takes)."""
    T = 1030
    g = torch.Generator().manual_seed(E)
    h = torch.randn(T, H, generator=g).bfloat16().double()
    router = torch.randn(E + 1, H, generator=g, dtype=F64) / math.sqrt(H)
    x, r = h.to(dtype).to(DEV), router.float().to(DEV)
    ids, wts, mix = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV), torch.empty(T, device=DEV)
    K.expert_route(ids, wts, mix, x, r, E)
    s = plain.sigmoid(h @ router[:E].float().double().T)
    best = s.sort(dim=1, descending=True).values[:, :top]
    close(wts, best, 2e-6)
    close(mix, plain.sigmoid(h @ router[E:].float().double().T)[:, 0], 2e-6)
    for first in (0, 512, 1027):
        n = min(3, T - first)
        ids1, wts1, mix1 = torch.empty(n, top, dtype=torch.int32, device=DEV), torch.empty(n, top, device=DEV), torch.empty(n, device=DEV)
        K.expert_route(ids1, wts1, mix1, x[first:first + n].contiguous(), r, E)
        assert torch.equal(ids1, ids[first:first + n]) and torch.equal(wts1, wts[first:first + n])
        assert torch.equal(mix1, mix[first:first + n])


# ---------------------------------------------------------------- the norm over a whole projection, and the rotation

@pytest.mark.parametrize("nq,nkv,hd,dv,rot,scaling", [(4, 4, 12, 20, 6, None), (2, 1, 20, 20, 20, (8.0, 1.0, 3.0, 64)),
                                                      (6, 2, 64, 64, 64, (4.0, 1.0, 4.0, 256)), (3, 1, 10, 6, 0, None),
                                                      (2, 2, 64, 96, 32, None)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_norm_and_rotation(K, nq, nkv, hd, dv, rot, scaling, dtype):
    from airframe_b200.parts.base import BuildContext, build_part
    from airframe_b200.config.base import PartSpec
    T, eps = 9, 1e-5
    g = torch.Generator().manual_seed(nq * 10 + hd)
    proj = torch.randn(T, (nq + nkv) * hd + nkv * dv, generator=g, dtype=F64) * 3
    wq, wk = torch.randn(nq * hd, generator=g, dtype=F64), torch.randn(nkv * hd, generator=g, dtype=F64)
    positions = [0, 1, 2, 3, 700, 701, 5000, 70000, 1 << 20]
    sc = dict(zip(("factor", "low", "high", "original"), scaling)) if scaling else None
    freqs = plain.stretched_frequencies(3000.0, rot, sc)
    pos = torch.tensor(positions)
    q = plain.rotate_half(plain.rms(proj[:, : nq * hd], eps, wq).view(T, nq, hd), pos, freqs)
    k = plain.rotate_half(plain.rms(proj[:, nq * hd: (nq + nkv) * hd], eps, wk).view(T, nkv, hd), pos, freqs)
    params = {"theta": 3000.0, "rotary_dim": rot, "pairing": "half", "precise_angles": True}
    if sc:
        params["scaling"] = dict(sc, kind="wavelength")
    rope = build_part("position", PartSpec("rope", params), BuildContext(dtype, torch.device(DEV)))
    rope.load({})
    if rot:
        close(rope.inv_freq, freqs, 1e-6)
    batch = SimpleNamespace(positions=i32(positions), seq_of_token=i32(list(range(T))), slots=i32(list(range(T))),
                            len_after=i32([p + 1 for p in positions]), aux={})
    qkv = torch.empty(T, (nq + nkv) * hd + nkv * dv, dtype=dtype, device=DEV)
    K.qk_norm_rope_store(qkv, proj.float().to(DEV), batch, nq, nkv, hd, rope.inv_freq, rot, "half",
                         q_weight=wq.float().to(DEV), k_weight=wk.float().to(DEV), eps=eps, dv=dv, whole_norm=True,
                         table=rope.precise_table(batch))
    tol = 3e-6 if dtype == torch.float32 else 6e-3
    close(qkv[:, : nq * hd], q.reshape(T, -1), tol)
    close(qkv[:, nq * hd: (nq + nkv) * hd], k.reshape(T, -1), tol)
    close(qkv[:, (nq + nkv) * hd:], proj[:, (nq + nkv) * hd:], tol)


# ---------------------------------------------------------------- x += norm(a weighted sum)

@pytest.mark.parametrize("H", [50, 72, 256, 1032, 4104])
def test_residual_step_norms_a_weighted_sum(K, H):
    T = 300 if H == 1032 else 21        # (many rows of some width: two groups of four values a thread)
    g = torch.Generator().manual_seed(H)
    x = torch.randn(T, H, generator=g)
    a, b, parts = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g).bfloat16(), torch.randn(3, T, H, generator=g)
    w, w2 = torch.randn(H, generator=g), torch.randn(H, generator=g)
    for terms, total in (([(a, 0.6), (b, 1.3)], 0.6 * a.double() + 1.3 * b.double()),
                         ([(parts, 1.0), (a, 1.0)], parts.double().sum(0) + a.double()),
                         ([(a, 0.0), (b, 2.0)], 2.0 * b.double()),
                         ([(a, 1.0), (b, 1.0), (parts[0], 0.5)], a.double() + b.double() + 0.5 * parts[0].double())):
        dev_terms = [(t.to(DEV), s) for t, s in terms]
        want = x.double() + plain.rms(total, 1e-5, w.double())
        for out_dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 6e-3)):
            x1 = x.clone().to(DEV)
            y = torch.empty(T, H, dtype=out_dtype, device=DEV)
            K.add_normed_terms(x1, dev_terms, w.to(DEV), 1e-5, y=y, w_next=w2.to(DEV), eps_next=1e-6)
            close(x1, want, 2e-6)
            close(y, plain.rms(want, 1e-6, w2.double()), tol)
            x2 = x.clone().to(DEV)
            K.add_normed_terms(x2, dev_terms, w.to(DEV), 1e-5, y=y)
            close(y, want, tol)
            assert torch.equal(x1, x2)


@pytest.mark.parametrize("E,top,H,F,T,limit,tiles", [(5, 2, 72, 40, 50, 1.0, (16, 32)), (8, 1, 128, 64, 300, 2.0, (16, 64, 256)),
                                                      (3, 3, 56, 16, 7, 0.5, (16,)), (2, 1, 40, 24, 1, 4.0, (16,)),
                                                      (12, 4, 64, 96, 130, 1.5, (32, 128)), (1, 1, 24, 8, 33, 0.7, (32,)),
                                                      (4, 2, 320, 200, 700, 1.2, (128, 256)), (16, 2, 256, 136, 8, 3.0, (16,))])
def test_expert_products_on_the_tensor_cores(K, E, top, H, F, T, limit, tiles):
    """The grouped products over sorted rows: row tiles of every size (an expert's rows in several tiles, tiles
    that begin in the middle of a box, the last rows of the last expert), feature tiles that end inside a
    tile of 128 and reach into the next expert's matrix, K that is no multiple of 64; and one expert without a
    plan (the shared expert's form, scaled per token)."""
    W = expert_weights(E, H, F, E * 100 + T, shared=24)
    h = torch.randn(T, H, generator=torch.Generator().manual_seed(T)).bfloat16().double()
    mlp = {"router": {"experts": E, "top": top}, "expert": {"limit": limit}}
    want = plain.routed_ff(h, W, "m.", mlp)
    x = h.bfloat16().to(DEV)
    router = torch.cat([W["m.router"], W["m.shared.sg"]]).float().to(DEV)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    mix = torch.empty(T, device=DEV)
    K.expert_route(ids, wts, mix, x, router, E)
    stack = lambda role: torch.stack([W[f"m.e{e}.{role}"] for e in range(E)]).bfloat16().to(DEV).contiguous()
    wg, wu, wd = stack("gate"), stack("up"), stack("down")
    assert K.expert_rows_tc_supported(x, wg)
    for tile in tiles + (K.expert_tc_tile(T * top, E),):
        perm = torch.empty(T * top, dtype=torch.int32, device=DEV)
        plan = torch.full((1 + 3 * K.expert_max_tiles(T * top, E, tile),), -1, dtype=torch.int32, device=DEV)
        K.expert_plan(perm, plan, ids, E, tile)
        entries = plan.cpu()[1: 1 + 3 * int(plan[0])].view(-1, 3)
        assert int(entries[:, 2].max()) <= tile and int(entries[:, 2].sum()) == T * top
        rows = torch.empty(T * top, H, dtype=torch.bfloat16, device=DEV)
        K.expert_gather(rows, x, perm, top)
        assert torch.equal(rows, x[(perm.long() // top)])
        mid = torch.full((T * top, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.expert_rows_tc(mid, rows, wg, wu, perm=perm, plan=plan, pair_weight=wts, n_tokens=T, top=top, limit=limit, tile=tile)
        out = torch.full((top, T, H), float("nan"), device=DEV)
        K.expert_rows_tc(out, mid, wd, perm=perm, plan=plan, n_tokens=T, top=top, tile=tile)
        close(out.sum(0), want, 2e-2)
        # the same rows on the CUDA cores: the two paths differ by the activation's rounding alone
        mid2 = torch.empty_like(mid)
        plan32 = torch.empty(1 + 3 * K.expert_max_tiles(T * top, E), dtype=torch.int32, device=DEV)
        perm2 = torch.empty_like(perm)
        K.expert_plan(perm2, plan32, ids, E)
        K.expert_rows(mid2, x, wg, wu, perm=perm2, plan=plan32, pair_weight=wts, n_tokens=T, top=top, limit=limit)
        close(mid[perm.long().argsort()], mid2[perm2.long().argsort()], 2e-2)      # (pair by pair: an expert's pairs come in any order)
    K.check_device_errors(DEV)
    # one expert, the rows as they are, a scale per token behind the activation
    sg, su, sd = (W[f"m.shared.{r}"].bfloat16().to(DEV).unsqueeze(0).contiguous() for r in ("gate", "up", "down"))
    smid = torch.empty(T, 24, dtype=torch.bfloat16, device=DEV)
    K.expert_rows_tc(smid, x, sg, su, scale_out=mix, n_tokens=T, top=1, limit=0.9)
    sout = torch.empty(1, T, H, device=DEV)
    K.expert_rows_tc(sout, smid, sd, n_tokens=T, top=1)
    close(sout[0], plain.sigmoid(h @ W["m.shared.sg"].T) * plain.clamped_expert(h, W, "m.shared.", 0.9), 2e-2)
    K.check_device_errors(DEV)


@pytest.mark.parametrize("width,blocks,T", [(128, 8, 70), (256, 2, 300), (144, 3, 64), (1024, 4, 700), (320, 1, 129)])
def test_gates_on_the_tensor_cores(K, width, blocks, T):
    """The block-diagonal products of the gates as a grouped tensor-core product (blocks of 16 to 320 channels:
    K below, at and beyond a K step of 64, output tiles that end inside 128; rows in one to three tiles), against the
    plain functions on the bfloat16 rounding of u that the products read."""
    w = recurrent_weights(width, blocks, 2, width + T)
    w["wa"], w["wi"] = w["wa"].bfloat16().double(), w["wi"].bfloat16().double()
    u = torch.randn(T, width, generator=torch.Generator().manual_seed(T), dtype=F64).float()
    u16 = u.bfloat16()
    bw = width // blocks
    ub = u16.double().view(T, blocks, bw)
    r = plain.sigmoid(torch.einsum("boi,tbi->tbo", w["wa"], ub) + w["ba"].view(blocks, -1)).reshape(T, width)
    i = plain.sigmoid(torch.einsum("boi,tbi->tbo", w["wi"], ub) + w["bi"].view(blocks, -1)).reshape(T, width)
    a = torch.exp(-8.0 * r * plain.softplus(w["lam"]))
    dev = lambda t, dt=torch.float32: t.to(dt).to(DEV).contiguous()
    decay, inp = torch.empty(T, width, device=DEV), torch.empty(T, width, device=DEV)
    K.gate_rows_tc(decay, inp, dev(u), dev(u16, torch.bfloat16), dev(w["wa"], torch.bfloat16), dev(w["wi"], torch.bfloat16),
                   dev(w["ba"]), dev(w["bi"]), dev(8.0 * plain.softplus(w["lam"])))
    close(decay, 1.0 - a, 1e-5)
    close(inp, torch.sqrt(1.0 - a * a) * i * u.double(), 1e-5)
    K.check_device_errors(DEV)
