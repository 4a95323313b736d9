"""The kernels behind Tarorax's mechanisms, each alone against the plain implementation's functions
(``plain_tarorax``, float64): the streams' read and rewrite, the decay per key channel and the scan that uses it
(prompts, single tokens, slots used again), the gated norm of the heads, the convolution with its history and the
packing of the two maps as heads of their own (cache rows included), the attention kernels over that packing with
one key made to stand out at chosen distances, the join of the two maps, the router with correction and groups,
and the experts of one matrix and the exact GELU on the CUDA cores and on the tensor cores."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_tarorax as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64
PAGE = 64


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
    after = [a + n for a, n in zip(before, lens)]
    return SimpleNamespace(seq_starts=i32(starts), slots=i32(slots), n_seqs=len(lens), n_tokens=starts[-1],
                           seq_of_token=i32(seq), positions=i32(pos), len_after=i32(after), is_prefill=not any(before),
                           max_len=max(lens), seq_lens=list(lens), max_len_after=max(after), aux={})


def batch_of_aux(lens, slots, some_device_tensor):
    b = batch_of(lens, slots)
    b.tokens = some_device_tensor
    return b


# ---------------------------------------------------------------- the streams

@pytest.mark.parametrize("S,W,T", [(1, 50, 3), (3, 72, 9), (4, 128, 40), (8, 36, 5), (2, 2052, 2), (11, 64, 600), (16, 130, 4)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_streams_read_and_rewrite(K, S, W, T, out_dtype):
    g = torch.Generator().manual_seed(S * 1000 + W)
    x = torch.randn(T, S, W, generator=g)
    w_in, w_out = torch.randn(S, generator=g), torch.randn(S, generator=g)
    mix = torch.randn(S, S, generator=g)
    nw, nw2 = torch.randn(W, generator=g) * 0.3, torch.randn(W, generator=g) * 0.3
    ls = torch.randn(W, generator=g)
    in2 = torch.randn(S, generator=g)
    eps = 1e-5
    tol = 1e-5 if out_dtype == torch.float32 else 6e-3
    X = [x[:, s].double() for s in range(S)]
    xd = x.reshape(T, S * W).to(DEV).contiguous()
    y = torch.empty(T, W, dtype=out_dtype, device=DEV)
    K.hc_read(y, xd, w_in.to(DEV), nw.to(DEV), eps, 1.0, S)
    close(y, plain.zero_centred_norm(plain.streams_read(X, w_in.double()), nw.double(), eps), tol)
    # the result as a 16-bit tensor, as 32-bit partial sums, and as two terms with scales
    a16 = torch.randn(T, W, generator=g).to(torch.bfloat16)
    parts = torch.randn(3, T, W, generator=g)
    b32 = torch.randn(T, W, generator=g)
    for terms, total in (([(a16.to(DEV), 1.0)], a16.double()), ([(parts.to(DEV), 1.0)], parts.double().sum(0)),
                         ([(b32.to(DEV), 0.5), (parts.to(DEV), -2.0)], 0.5 * b32.double() - 2.0 * parts.double().sum(0))):
        for scaled in (True, False):
            for nxt in (True, False):
                xs = xd.clone()
                y2 = torch.empty(T, W, dtype=out_dtype, device=DEV) if nxt else None
                K.hc_write(xs, terms, mix.to(DEV).contiguous(), w_out.to(DEV), S, scale=ls.to(DEV) if scaled else None, y=y2,
                           in_next=in2.to(DEV) if nxt else None, w_next=nw2.to(DEV) if nxt else None, eps=eps, offset=1.0)
                new = plain.streams_write(X, total * (ls.double() if scaled else 1.0), mix.double(), w_out.double())
                close(xs.view(T, S, W), torch.stack(new, 1), 1e-5)
                if nxt:
                    close(y2, plain.zero_centred_norm(plain.streams_read(new, in2.double()), nw2.double(), eps), tol)
    e = torch.randn(T, W, generator=g).to(DEV)
    xs = torch.empty(T, S * W, device=DEV)
    K.stream_copy(xs, e, S)
    assert all(torch.equal(xs.view(T, S, W)[:, s], e) for s in range(S))
    total = torch.empty(T, W, device=DEV)
    K.stream_sum(total, xd, S)
    close(total, x.double().sum(1), 1e-6)


# ---------------------------------------------------------------- gated linear attention

@pytest.mark.parametrize("n,rank,T,tau", [(24, 5, 1, 4.0), (128, 12, 17, 10.0), (130, 1, 40, 1.0), (300, 33, 3, 2.5), (256, 128, 50, 6.0)])
def test_decay_per_key_channel(K, n, rank, T, tau):
    g = torch.Generator().manual_seed(n)
    proj = torch.randn(T, 7 + rank + 3, generator=g) * 3
    w2 = torch.randn(n, rank, generator=g)
    b = torch.randn(n, generator=g) * 4          # (sigmoids near 0 and near 1 among them)
    alpha = torch.empty(T, n, device=DEV)
    K.channel_decay(alpha, proj.to(DEV), 7, w2.t().contiguous().to(DEV), b.to(DEV), tau)
    z = proj[:, 7:7 + rank].double() @ w2.double().T + b.double()
    close(alpha, torch.exp(torch.log(plain.sigmoid(z)) / tau), 1e-5)
    # a token's decays do not depend on how many tokens the step holds (the kernel for few tokens adds in the same order)
    for t0, cnt in ((0, 1), (T - 1, 1), (0, min(T, 16)), (max(0, T - 5), min(T, 5))):
        part = torch.empty(cnt, n, device=DEV)
        K.channel_decay(part, proj[t0:t0 + cnt].contiguous().to(DEV), 7, w2.t().contiguous().to(DEV), b.to(DEV), tau)
        assert torch.equal(part, alpha[t0:t0 + cnt])
    # far down the sigmoid's tail the logarithm is taken without the sigmoid underflowing
    deep = torch.full((1, 7 + rank + 3), 0.0)
    K.channel_decay(alpha[:1], deep.to(DEV), 7, w2.t().contiguous().to(DEV), torch.full((n,), -200.0, device=DEV), 100.0)
    close(alpha[:1], torch.full((1, n), math.exp(-2.0), dtype=F64), 1e-5)


@pytest.mark.parametrize("heads,dk,dv", [(2, 8, 8), (3, 24, 40), (1, 32, 32), (2, 64, 16), (1, 128, 128), (2, 6, 10), (1, 5, 3)])
def test_scan_with_a_decay_per_channel(K, heads, dk, dv):
    """Two sequences in one step against the plain recurrence; then the longer one again in steps of unequal sizes
    down to single tokens (the state is carried), in a slot that another sequence used before; a padding row
    (slot -1) changes nothing and leaves zeros."""
    lens = [37, 5]
    T = sum(lens)
    g = torch.Generator().manual_seed(dk * 131 + dv)
    q, k, v = (torch.randn(T, heads * n, generator=g) for n in (dk, dk, dv))
    alpha = torch.rand(T, heads * dk, generator=g) * 0.6 + 0.4
    alpha[3] = 1.0                                # nothing forgotten at one token, everything at another
    alpha[20] = 0.0

    def ref_of(s):
        return torch.cat([plain.decayed_outer_product_scan(q[s, h * dk:(h + 1) * dk].double(), k[s, h * dk:(h + 1) * dk].double(),
                                                           v[s, h * dv:(h + 1) * dv].double(), alpha[s, h * dk:(h + 1) * dk].double())
                          for h in range(heads)], dim=1)

    ref = [ref_of(slice(0, 37)), ref_of(slice(37, 42))]
    state = torch.zeros(4, heads, dv, dk, device=DEV)
    dev = [t.to(DEV) for t in (q, k, v, alpha)]
    out = torch.full((T, heads * dv), 7.0, device=DEV)
    K.state_scan("channel", out, dev[0], dev[1], dev[2], state, batch_of(lens, [2, 0]), heads, dk, dv, w=dev[3])
    close(out[:37], ref[0], 2e-5)
    close(out[37:], ref[1], 2e-5)
    assert float(state[1].abs().sum()) == 0 and float(state[3].abs().sum()) == 0
    state[0].zero_()
    got, at = [], 0
    for n in (19, 13, 2, 1, 1, 1):
        rows = [t[at:at + n].contiguous() for t in dev]
        pad = [torch.cat([t, torch.ones(1, t.shape[1], device=DEV)]) for t in rows]
        o = torch.full((n + 1, heads * dv), 7.0, device=DEV)
        before = state.clone()
        K.state_scan("channel", o, pad[0], pad[1], pad[2], state, batch_of([n, 1], [0, -1]), heads, dk, dv, w=pad[3])
        assert float(o[n].abs().sum()) == 0 and torch.equal(before[1:], state[1:])
        got.append(o[:n])
        at += n
    close(torch.cat(got), ref[0], 2e-5)


@pytest.mark.parametrize("heads,dk,dv,lens,chunk", [(2, 8, 8, [300, 1, 130], 128), (3, 24, 40, [257], 64), (1, 64, 100, [64, 65, 200], 64),
                                                    (2, 128, 128, [520], 128), (1, 5, 3, [33, 70], 32), (2, 70, 33, [129, 2], 128)])
def test_chunks_scanned_side_by_side_and_joined(K, heads, dk, dv, lens, chunk):
    """Sequences cut into chunks (a last chunk of one token, of a whole chunk, sequences shorter than a chunk), from
    states that earlier steps left: outputs and new states against the token-by-token kernel and the plain
    recurrence; a channel that forgets everything at once inside a chunk, and one that forgets nothing."""
    T = sum(lens)
    g = torch.Generator().manual_seed(dk * 7 + dv + T)
    q, k, v = (torch.randn(T, heads * n, generator=g) for n in (dk, dk, dv))
    alpha = torch.rand(T, heads * dk, generator=g) * 0.5 + 0.5
    alpha[:, 0] = 1.0
    alpha[T // 2, 1 % (heads * dk)] = 0.0
    alpha[:, -1] = 0.05                      # (its cumulated decay leaves the range of 32-bit floats within a chunk)
    slots = list(range(1, len(lens) + 1))
    start = torch.randn(len(lens) + 2, heads, dv, dk, generator=g)
    dev = [t.to(DEV) for t in (q, k, v, alpha)]
    b = batch_of(lens, slots)
    b.tokens = dev[0]
    want_state = start.clone().to(DEV)
    want = torch.empty(T, heads * dv, device=DEV)
    K.state_scan("channel", want, dev[0], dev[1], dev[2], want_state, b, heads, dk, dv, w=dev[3])
    got_state = start.clone().to(DEV)
    got = torch.full((T, heads * dv), 7.0, device=DEV)
    K.state_scan_chunked(got, dev[0], dev[1], dev[2], dev[3], got_state, b, heads, dk, dv, chunk=chunk)
    close(got, want, 2e-5)
    close(got_state, want_state, 2e-5)
    assert torch.equal(got_state[0], start[0].to(DEV)) and torch.equal(got_state[-1], start[-1].to(DEV))
    # and against the plain recurrence from a zero state
    zero = torch.zeros_like(got_state)
    K.state_scan_chunked(got, dev[0], dev[1], dev[2], dev[3], zero, batch_of_aux(lens, slots, dev[0]), heads, dk, dv, chunk=chunk)
    at = 0
    for n in lens:
        s = slice(at, at + n)
        ref = torch.cat([plain.decayed_outer_product_scan(q[s, h * dk:(h + 1) * dk].double(), k[s, h * dk:(h + 1) * dk].double(),
                                                          v[s, h * dv:(h + 1) * dv].double(), alpha[s, h * dk:(h + 1) * dk].double())
                         for h in range(heads)], dim=1)
        close(got[s], ref, 3e-5)
        at += n


@pytest.mark.parametrize("heads,dv", [(3, 20), (2, 64), (1, 7)])
def test_heads_normed_with_a_shared_weight_and_a_silu_gate(K, heads, dv):
    T, n = 11, heads * dv
    g = torch.Generator().manual_seed(n)
    o, gate, w = torch.randn(T, n, generator=g) * 5, torch.randn(T, n + 3, generator=g) * 2, torch.randn(dv, generator=g)
    y = torch.empty(T, n, device=DEV)
    gd = gate.to(DEV)
    K.gated_group_norm(y, o.to(DEV), w.repeat(heads).to(DEV), gd[:, 3:], dv, 1e-3, gate_act="silu", in_scale=0.3)
    ref = plain.rms((0.3 * o.double()).view(T, heads, dv), 1e-3) * w.double()
    close(y, ref.reshape(T, n) * plain.silu(gate[:, 3:].double()), 1e-5)


# ---------------------------------------------------------------- differential attention

def _unpack(qkv, H, G, d, dv, pk, pv):
    """The packed rows back in the projection's layout: q [T, H, 2, d], k [T, G, 2, d], v per map [T, G, 2, dv]."""
    T, rep = qkv.shape[0], H // G
    q = qkv[:, : 2 * H * pk].view(T, G, 2, rep, pk)[..., :d].permute(0, 1, 3, 2, 4).reshape(T, H, 2, d)
    k = qkv[:, 2 * H * pk: (2 * H + 2 * G) * pk].view(T, G, 2, pk)[..., :d]
    v = qkv[:, (2 * H + 2 * G) * pk:].view(T, G, 2, pv)[..., :dv]
    return q, k, v


@pytest.mark.parametrize("H,G,d,dv,pk,pv,taps", [(2, 2, 12, 20, 12, 20, 3), (3, 1, 10, 6, 10, 6, 2), (4, 2, 64, 64, 64, 64, 4),
                                                 (2, 1, 40, 80, 128, 128, 4), (1, 1, 7, 9, 8, 10, 1), (2, 2, 6, 10, 6, 10, 11)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolution_history_and_packing(K, H, G, d, dv, pk, pv, taps, dtype):
    """Two sequences as prompts, then in steps of 2, 1, 1 and 5 tokens from the history; against the plain
    convolution of the whole sequences.  The padding behind a head is zero; a slot is used again from zeros."""
    C = H * 2 * d + G * 2 * d + G * dv
    lens = [9, 2]
    more = [2, 1, 1, 5]
    g = torch.Generator().manual_seed(C + taps)
    full = [torch.randn(n + sum(more), C + 5, generator=g) for n in lens]
    bias = torch.randn(C, generator=g)
    cw = torch.randn(C, taps, generator=g)
    coef, every = 0.7, 3
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    refs = []
    for f in full:
        u = plain.short_convolution(f[:, :C].double() + bias.double(), cw.double())
        temp = plain.query_temperature(f.shape[0], coef, every)
        cq = H * 2 * d
        refs.append((u[:, :cq].view(-1, H, 2, d) * temp[:, None, None, None], u[:, cq:cq + G * 2 * d].view(-1, G, 2, d),
                     u[:, cq + G * 2 * d:].view(-1, G, dv)))
    hist = torch.zeros(5, max(taps - 1, 1), C, device=DEV)
    hist[1] = 9.0            # (a slot that nobody holds: it must stay as it is)
    width = (2 * H + 2 * G) * pk + 2 * G * pv
    done = [0, 0]
    for step in [lens] + [[m, m] for m in more]:
        rows = torch.cat([f[a:a + n] for f, a, n in zip(full, done, step)]).to(DEV)
        b = batch_of(step, [3, 0], before=list(done))
        qkv = torch.full((rows.shape[0], width), 7.0, dtype=dtype, device=DEV)
        K.conv_pack(qkv, rows, b, H, G, d, dv, pk, pv, bias=bias.to(DEV), taps_w=cw.t().contiguous().to(DEV),
                    history=hist if taps > 1 else None, temp_coef=coef, temp_every=every)
        q, k, v = _unpack(qkv.float().cpu(), H, G, d, dv, pk, pv)
        at = 0
        for i, n in enumerate(step):
            s = slice(done[i], done[i] + n)
            close(q[at:at + n], refs[i][0][s], tol)
            close(k[at:at + n], refs[i][1][s], tol)
            close(v[at:at + n, :, 0], refs[i][2][s], tol)
            assert torch.equal(v[at:at + n, :, 0], v[at:at + n, :, 1])          # a group's values once per map
            at += n
            done[i] += n
        if pk > d:
            assert float(qkv[:, : (2 * H + 2 * G) * pk].reshape(-1, pk)[:, d:].abs().sum()) == 0
        if pv > dv:
            assert float(qkv[:, (2 * H + 2 * G) * pk:].reshape(-1, pv)[:, dv:].abs().sum()) == 0
    assert float((hist[1] - 9.0).abs().sum()) == 0
    if taps > 1:      # the history holds the last taps - 1 inputs (bias in), oldest first
        want = (full[0][:, :C] + bias)[done[0] - (taps - 1): done[0]]
        close(hist[3], want, 1e-6)


@pytest.mark.parametrize("d,dv,pk,pv,n,dtype", [(12, 20, 12, 20, 70, torch.float32), (64, 64, 64, 64, 200, torch.bfloat16),
                                                (40, 80, 128, 128, 130, torch.bfloat16), (32, 32, 32, 32, 129, torch.float32)])
def test_attention_over_the_packed_maps_with_a_key_that_stands_out(K, d, dv, pk, pv, n, dtype):
    """Packed by ``conv_pack`` (cache pages included, in a scrambled page table), the two maps go through the
    library's attention kernels: a prompt of n tokens, then single tokens over the cache.  In map 1 the key at one
    position is made to score far above the rest for every later query, in map 2 another position's: the maps'
    outputs are then those positions' values, whichever page they lie in (position 0, a page's last row, the first
    row of the next page, and far back)."""
    H, G = 4, 2
    C = H * 2 * d + G * 2 * d + G * dv
    cq, ck = H * 2 * d, G * 2 * d
    extra = 3
    for far1, far2 in ((0, PAGE), (PAGE - 1, 1), (PAGE, n - 2)):
        g = torch.Generator().manual_seed(n + far1)
        rows = torch.randn(n + extra, C, generator=g) * 0.1
        q = rows[:, :cq].view(-1, H, 2, d)
        k = rows[:, cq:cq + ck].view(-1, G, 2, d)
        q[..., 0] = 6.0                            # every query asks for channel 0; the chosen keys answer loudest
        k[..., 0] = 0.0
        k[far1, :, 0, 0] = 8.0
        k[far2, :, 1, 0] = 8.0
        v = rows[:, cq + ck:].view(-1, G, dv)
        kv = SimpleNamespace(k=torch.zeros(8, 2 * G, PAGE, pk, dtype=dtype, device=DEV),
                             v=torch.zeros(8, 2 * G, PAGE, pv, dtype=dtype, device=DEV),
                             page_table=i32([[5, 2, 7, 0, -1, -1], [1, 3, 4, 6, -1, -1]]), ring_rows=0)
        width = (2 * H + 2 * G) * pk + 2 * G * pv
        outs = []
        fed = 0
        for step in [n] + [1] * extra:
            b = batch_of([step], [1], before=[fed])
            qkv = torch.empty(step, width, dtype=dtype, device=DEV)
            K.conv_pack(qkv, rows[fed:fed + step].to(DEV), b, H, G, d, dv, pk, pv, kv=kv)
            ctx = torch.empty(step, 2 * H * pv, dtype=dtype, device=DEV)
            qq = qkv[:, : 2 * H * pk]
            if fed == 0:
                K.attn_prefill(ctx, qq, qkv[:, 2 * H * pk: (2 * H + 2 * G) * pk], qkv[:, (2 * H + 2 * G) * pk:], b, 2 * H, 2 * G,
                               pk, 1.0, 0.0, 0, dv=pv)
            else:
                K.attn_decode(ctx, qq, kv, b, 2 * H, 2 * G, pk, 1.0, 0.0, 0, dv=pv)
            outs.append(ctx.float().cpu())
            fed += step
        ctx = torch.cat(outs).view(-1, G, 2, H // G, pv)[..., :dv]          # [token, group, map, head of the group, value]
        tol = 2e-3 if dtype == torch.float32 else 2e-2
        for t in list(range(max(far1, far2), n + extra))[:: max(1, n // 9)] + [n, n + extra - 1]:
            for grp in range(G):
                for j in range(H // G):
                    assert float((ctx[t, grp, 0, j] - v[far1, grp]).abs().max()) < tol, (t, "map 1")
                    assert float((ctx[t, grp, 1, j] - v[far2, grp]).abs().max()) < tol, (t, "map 2")
        # before a loud key exists, a map is an ordinary average: the query right before far2 does not see it
        if far2 > far1 + 1:
            t = far2 - 1
            assert float((ctx[t, 0, 1, 0] - v[far2, 0]).abs().max()) > 10 * tol


@pytest.mark.parametrize("H,G,dv,pv,ones", [(2, 2, 20, 20, 1), (3, 1, 6, 6, 0), (4, 2, 64, 64, 1), (2, 1, 80, 128, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_join_of_the_two_maps(K, H, G, dv, pv, ones, dtype):
    T, rep = 7, H // G
    g = torch.Generator().manual_seed(H * dv)
    ctx = torch.randn(T, G, 2, rep, pv, generator=g).to(dtype)
    gate = torch.randn(T, H * dv + 2, generator=g) * 2
    lam, eps, post = 0.73, 1e-5, 0.4
    width = -(-(H * dv + ones) // 8) * 8
    y = torch.full((T, width), 7.0, dtype=dtype, device=DEV)
    K.diff_join(y, ctx.reshape(T, -1).to(DEV), gate.to(DEV)[:, 2:], H, G, dv, pv, lam, eps, post, ones=ones)
    a = ctx.double()[..., :dv]
    o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, H, dv)
    ref = (plain.rms(o, eps) * post).reshape(T, H * dv) * plain.sigmoid(gate[:, 2:].double())
    close(y[:, : H * dv], ref, 1e-5 if dtype == torch.float32 else 6e-3)
    tail = y[:, H * dv:].float().cpu()
    assert torch.equal(tail[:, :ones], torch.ones(T, ones)) and float(tail[:, ones:].abs().sum()) == 0


# ---------------------------------------------------------------- the router and the experts

@pytest.mark.parametrize("E,top,groups,keep,T,H", [(6, 2, 3, 2, 9, 72), (8, 4, 4, 3, 300, 128), (4, 1, 2, 1, 5, 50), (5, 5, 5, 5, 3, 51),
                                                    (3, 3, 1, 1, 4, 50), (64, 6, 8, 3, 33, 96), (8, 2, 8, 2, 7, 40)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router_with_correction_and_groups(K, E, top, groups, keep, T, H, dtype):
    g = torch.Generator().manual_seed(E * 7 + top)
    h = torch.randn(T, H, generator=g).to(dtype)
    W = {"m.router": torch.randn(E, H, generator=g).double() * 0.3, "m.correction": torch.randn(E, generator=g).double() * 0.7}
    r = {"experts": E, "top": top, "scale": 2.5}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    ids_ref, w_ref, margin = plain.route(h.double(), W, "m.", r)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    K.expert_route(ids, wts, None, h.to(DEV), W["m.router"].float().to(DEV), E, correction=W["m.correction"].float().to(DEV),
                   groups=groups, keep=keep, normalise=True, out_scale=2.5)
    sure = margin > 1e-4
    assert bool(sure.any())
    assert torch.equal(ids.cpu()[sure].long(), ids_ref[sure])
    close(wts.cpu()[sure], w_ref[sure], 1e-5)
    assert bool((wts.cpu()[sure].sum(-1) - 2.5).abs().max() < 1e-4)


@pytest.mark.parametrize("E,top,H,F,T", [(5, 2, 72, 36, 9), (3, 3, 50, 22, 40), (8, 4, 128, 64, 300), (2, 1, 51, 9, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_of_one_matrix_and_the_exact_gelu(K, E, top, H, F, T, dtype):
    """Router, plan and the two products on the CUDA cores against W_down gelu(W_up h) weighed behind the
    activation; where the sizes allow, the same on the tensor cores."""
    g = torch.Generator().manual_seed(E * 100 + T)
    h = torch.randn(T, H, generator=g).to(dtype)
    up = (torch.randn(E, F, H, generator=g) * 0.3).to(dtype)
    down = (torch.randn(E, H, F, generator=g) * 0.3).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g) + 0.1
    ref = torch.zeros(T, H, dtype=F64)
    for t in range(T):
        for j in range(top):
            e = int(ids[t, j])
            ref[t] += float(wts[t, j]) * (down[e].double() @ plain.gelu_erf(up[e].double() @ h[t].double()))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    hd, upd, downd, idd, wd = h.to(DEV), up.to(DEV), down.to(DEV), ids.to(DEV), wts.to(DEV)
    for fast in (False, True):
        if fast and not (K.expert_rows_tc_supported(hd, upd) and F % 8 == 0):
            continue
        tile = K.expert_tc_tile(T * top, E) if fast else K.EXPERT_TILE
        perm = torch.empty(T * top, dtype=torch.int32, device=DEV)
        plan = torch.empty(1 + 3 * K.expert_max_tiles(T * top, E, tile), dtype=torch.int32, device=DEV)
        K.expert_plan(perm, plan, idd, E, tile)
        mid = torch.empty(T * top, F, dtype=dtype, device=DEV)
        out = torch.empty(top, T, H, dtype=torch.float32, device=DEV)
        if fast:
            rows = torch.empty(T * top, H, dtype=dtype, device=DEV)
            K.expert_gather(rows, hd, perm, top)
            K.expert_rows_tc(mid, rows, upd, perm=perm, plan=plan, pair_weight=wd, n_tokens=T, top=top, tile=tile, act="gelu_erf")
            K.expert_rows_tc(out, mid, downd, perm=perm, plan=plan, n_tokens=T, top=top, tile=tile)
        else:
            K.expert_rows(mid, hd, upd, perm=perm, plan=plan, pair_weight=wd, n_tokens=T, top=top, act="gelu_erf")
            K.expert_rows(out, mid, downd, perm=perm, plan=plan, n_tokens=T, top=top)
        K.check_device_errors(torch.device(DEV))
        close(out.sum(0), ref, tol)
