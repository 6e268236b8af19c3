"""Zuvulorn on the GPU against the plain implementation (tests/plain/zuvulorn_plain.py): each kernel alone, each
mixer alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with
pages and state slots that are used again, keys far back and at page borders with and without the sink's share,
the first tokens of a sequence, long decoding, and greedy generation through the engine's scheduler."""

import math
import types

import pytest
import torch

from zuvulorn_helpers import (CONFIGS, ZP, to_bf16_and_back, attn, compare, delta, draw_weights, every_expert, experts, layer, model, model_folder,
                              rglru, write_folder)
from helpers import random_tokens, run_trace, trace_budget, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def step_ctx(qlens, slots):
    seg_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=DEV)
    tok_seg = torch.cat([torch.full((n,), s) for s, n in enumerate(qlens)]).to(torch.int32).to(DEV)
    return types.SimpleNamespace(seg_start=seg_start, tok_seg=tok_seg, S=len(qlens), max_q_len=max(qlens),
                                 state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV),
                                 alloc=lambda shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))


def cut(total, sizes):
    out, at, k = [], 0, 0
    while at < total:
        n = min(sizes[k % len(sizes)], total - at)
        out.append((at, n))
        at, k = at + n, k + 1
    return out


# ---------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("s, T, W", [(2, 9, 64), (3, 5, 72), (1, 4, 33), (8, 3, 256), (4, 70, 1030)])
@pytest.mark.parametrize("rms", [False, True])
def test_the_copies_of_the_stream_are_updated_read_and_normed_in_one_launch(s, T, W, rms):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(s * 100 + T)
    x = torch.randn(s, T, W, generator=g) + 0.5
    d = torch.randn(2, T, W, generator=g)
    mix, ow, iw = torch.randn(s, s, generator=g), torch.randn(s, generator=g), torch.randn(s, generator=g)
    w = torch.randn(W, generator=g) * 0.2 + 1
    new = torch.einsum("ij,itd->jtd", mix, x) + ow[:, None, None] * d.sum(0)[None]
    u = torch.einsum("j,jtd->td", iw, new)
    ref = ZP.rms(u, 1e-5) * w if rms else ZP.layer_norm(u, w, 1e-5)
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 3e-2)):
        xd = x.to(DEV)
        h = torch.empty(T, W, dtype=dtype, device=DEV)
        ops.hyper_norm(xd, s, xd, d.to(DEV), mix.to(DEV), ow.to(DEV), iw.to(DEV), w.to(DEV), 1e-5, h, None, rms)
        assert float((xd.cpu() - new).abs().max()) <= 1e-5 * max(1.0, float(new.abs().max()))
        assert float((h.float().cpu() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))
    # some rows only: the copies stay as they are, the update is seen by the norm all the same
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    xd = x.to(DEV)
    h = torch.empty(2, W, device=DEV)
    ops.hyper_norm(xd, s, None, d.to(DEV), mix.to(DEV), ow.to(DEV), iw.to(DEV), w.to(DEV), 1e-5, h, rows, rms)
    assert torch.equal(xd.cpu(), x)
    assert float((h.cpu() - ref[[T - 1, 0]]).abs().max()) <= 2e-5 * max(1.0, float(ref.abs().max()))
    # the first sublayer of a model: one set of rows read as equal copies, nothing left open; no weights: plain sums
    x0 = x[0].contiguous().to(DEV)
    out = torch.empty(s, T, W, device=DEV)
    h = torch.empty(T, W, device=DEV)
    ops.hyper_norm(x0, s, out, None, None, None, iw.to(DEV), w.to(DEV), 1e-5, h, None, rms)
    u0 = x[0] * iw.sum()
    ref0 = ZP.rms(u0, 1e-5) * w if rms else ZP.layer_norm(u0, w, 1e-5)
    assert torch.equal(out.cpu(), x[0][None].repeat(s, 1, 1))
    assert float((h.cpu() - ref0).abs().max()) <= 2e-5 * max(1.0, float(ref0.abs().max()))
    xd = x.to(DEV)
    ops.hyper_norm(xd, s, xd, d[0].contiguous().to(DEV), None, None, None, w.to(DEV), 1e-5, h, None, rms)
    u1 = (x + d[0][None]).sum(0)
    ref1 = ZP.rms(u1, 1e-5) * w if rms else ZP.layer_norm(u1, w, 1e-5)
    assert float((xd.cpu() - (x + d[0][None])).abs().max()) <= 1e-6
    assert float((h.cpu() - ref1).abs().max()) <= 2e-5 * max(1.0, float(ref1.abs().max()))


@pytest.mark.parametrize("C, K", [(40, 4), (33, 3), (8, 1), (256, 2), (5, 7)])
def test_short_convolution_with_its_tail_in_portions_and_token_by_token(C, K):
    """Portions shorter than the convolution's reach, so that the tail is partly moved up and partly refilled; then
    token by token with the kernel moving the tail itself, two requests side by side, one a step behind."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(C + K)
    n = 29
    x = torch.randn(n, C + 3, generator=g)
    taps, bias = torch.randn(C, K, generator=g) * 0.6, torch.randn(C, generator=g)
    ref = ZP.causal_conv(x[:, 2:2 + C].contiguous(), taps, bias)
    xd = x.to(DEV)[:, 2:2 + C]
    tail = torch.zeros(3, max(K - 1, 0), C, device=DEV)
    got = torch.empty(n, C)
    for a, m in cut(n, (1, 2, 1, 1, 7, 3, 2)):
        ctx = step_ctx([m], [1])
        out = torch.empty(m, C, device=DEV)
        ops.causal_conv(xd[a:a + m], taps.to(DEV), bias.to(DEV), tail, ctx, out)
        ops.state_tail(xd[a:a + m], tail, ctx)
        got[a:a + m] = out.cpu()
    assert float((got - ref).abs().max()) <= 1e-5
    if K > 1:
        assert float((tail[1].cpu() - x[n - (K - 1):, 2:2 + C]).abs().max()) == 0.0
        assert float(tail[0].abs().max()) == 0.0 and float(tail[2].abs().max()) == 0.0
    tail.zero_()
    for a in range(n + 1):
        rows = [r for r in (a, a - 1) if 0 <= r < n]
        ctx = step_ctx([1] * len(rows), [2 if r == a else 0 for r in rows])
        out = torch.empty(len(rows), C, device=DEV)
        ops.causal_conv(xd[rows], taps.to(DEV), None, tail, ctx, out, move_tail=True)
        for j, r in enumerate(rows):
            assert float((out[j].cpu() - (ref[r] - bias)).abs().max()) <= 1e-5, (a, r)


@pytest.mark.parametrize("blocks, bs", [(5, 8), (3, 64), (1, 8), (4, 1), (2, 33), (1, 300)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_block_gates_and_the_recurrence_in_pieces(blocks, bs, wdt):
    """The gates per block of channels, the coefficients from them, and the recurrence: two requests cut into
    portions down to one token, their states in slots 2 and 0, a neighbour's slot untouched."""
    from prism_b200 import ops
    C = blocks * bs
    g = torch.Generator().manual_seed(C)
    lens = [70, 23]
    wr = (torch.randn(blocks, bs, bs, generator=g) / bs ** 0.5).to(wdt)
    wi = (torch.randn(blocks, bs, bs, generator=g) / bs ** 0.5).to(wdt)
    br, bi, lam = (torch.randn(blocks, bs, generator=g) * 0.5).to(wdt), (torch.randn(blocks, bs, generator=g) * 0.5).to(wdt), \
        (torch.randn(C, generator=g) - 2.0).to(wdt)
    data = []
    for n in lens:
        u, y = torch.randn(n, C, generator=g), torch.randn(n, C, generator=g)
        ub = u.view(n, blocks, bs)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wr.float()) + br.float()).reshape(n, C)
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wi.float()) + bi.float()).reshape(n, C)
        a = torch.exp(-8.0 * r * ZP.softplus(lam.float()))
        b = torch.sqrt(1 - a * a) * i * u
        S, out = torch.zeros(C), torch.empty(n, C)
        for t in range(n):
            S = a[t] * S + b[t]
            out[t] = S * ZP.gelu_tanh(y[t])
        data.append((u, y, a, b, out))
    state = torch.zeros(4, C, device=DEV)
    state[1] = 9.0
    cuts = [cut(lens[0], (30, 1, 1, 17, 2)), cut(lens[1], (5, 2, 1, 9))]
    got = [torch.empty(n, C) for n in lens]
    for step in range(max(len(c) for c in cuts)):
        act = [(r, cuts[r][step]) for r in range(2) if step < len(cuts[r])]
        u = torch.cat([data[r][0][a:a + n] for r, (a, n) in act]).to(DEV)
        y = torch.cat([data[r][1][a:a + n] for r, (a, n) in act]).to(DEV)
        T = u.shape[0]
        ag = torch.empty(2, T, C, device=DEV)
        ops.block_gates(u, wr.to(DEV), wi.to(DEV), br.to(DEV), bi.to(DEV), lam.to(DEV), 8.0, ag[0], ag[1])
        ra = torch.cat([data[r][2][a:a + n] for r, (a, n) in act])
        rb = torch.cat([data[r][3][a:a + n] for r, (a, n) in act])
        assert float((ag[0].cpu() - ra).abs().max()) <= 2e-5 and float((ag[1].cpu() - rb).abs().max()) <= 5e-5
        ctx = step_ctx([n for _, (_, n) in act], [(2, 0)[r] for r, _ in act])
        o = torch.empty(T, C, device=DEV)
        ops.rglru_scan(ag[0], ag[1], y, state, ctx, o, gelu=True)
        at = 0
        for r, (a, n) in act:
            got[r][a:a + n] = o[at:at + n].cpu()
            at += n
    for r in range(2):
        assert float((got[r] - data[r][4]).abs().max()) <= 1e-4 * max(1.0, float(data[r][4].abs().max())), r
    assert float((state[1] - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("C", [5, 64, 200])
def test_long_stretches_of_the_recurrence_run_in_chunks(C):
    """Requests of unequal length in one step, some longer than the size from which the scan runs in chunks (ends at
    a chunk's last token, one past it, one short of it), from states that are not zero, into slots in any order;
    then one more token each from the states left."""
    from prism_b200 import ops
    qlens = [300, 1, 128, 129, 127, 64, 513]
    slots = [3, 0, 6, 1, 5, 2, 4]
    g = torch.Generator().manual_seed(C)
    T = sum(qlens)
    a = torch.rand(T, C, generator=g) * 0.5 + 0.5
    a[10:200] = 1.0 - 1e-4 * torch.rand(190, C, generator=g)          # a long memory across several chunks
    b = torch.randn(T, C, generator=g)
    y = torch.randn(T, C, generator=g)
    st0 = torch.randn(7, C, generator=g)
    want = torch.zeros(T, C, dtype=torch.float64)
    last = torch.zeros(7, C, dtype=torch.float64)
    at = 0
    for n, sl in zip(qlens, slots):
        S = st0[sl].double()
        for t in range(at, at + n):
            S = a[t].double() * S + b[t].double()
            want[t] = S * y[t].double()
        last[sl] = S
        at += n
    ctx = step_ctx(qlens, slots)
    assert ctx.max_q_len >= ops.RGLRU_CHUNKED_FROM
    state = st0.clone().to(DEV)
    out = torch.empty(T, C, device=DEV)
    ops.rglru_scan(a.to(DEV), b.to(DEV), y.to(DEV), state, ctx, out, gelu=False)
    scale = float(want.abs().max())
    assert float((out.cpu().double() - want).abs().max()) <= 2e-5 * scale
    assert float((state.cpu().double() - last).abs().max()) <= 2e-5 * float(last.abs().max())
    # the chunks' form against the token-by-token kernel on the same step
    state2 = st0.clone().to(DEV)
    out2 = torch.empty(T, C, device=DEV)
    ctx.max_q_len = 1
    ops.rglru_scan(a.to(DEV), b.to(DEV), y.to(DEV), state2, ctx, out2, gelu=False)
    assert float((out2 - out).abs().max()) <= 2e-5 * scale


@pytest.mark.parametrize("G, rep, dk, dv", [(2, 2, 12, 20), (1, 1, 1, 1), (1, 3, 7, 5), (3, 1, 64, 32), (1, 2, 128, 128), (1, 1, 300, 16)])
def test_delta_rule_with_a_decay_per_key_channel_in_pieces(G, rep, dk, dv):
    """Decay, error against the decayed state, write, then the read-out that sees the write; two requests of unequal
    length cut into portions down to one token, the plain loop runs each whole."""
    from prism_b200 import ops
    H = G * rep
    g = torch.Generator().manual_seed(dk * 100 + dv)
    lens = [110, 37]
    data = []
    for n in lens:
        q = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1) * dk ** -0.5
        k = torch.nn.functional.normalize(torch.randn(n, G, dk, generator=g), dim=-1)
        v = torch.randn(n, H, dv, generator=g)
        beta, dec = torch.rand(n, H, generator=g), torch.rand(n, H, dk, generator=g) * 0.7 + 0.3
        ref = torch.empty(n, H, dv)
        for h in range(H):
            S = torch.zeros(dk, dv)
            for t in range(n):
                S = dec[t, h][:, None] * S
                u = beta[t, h] * (v[t, h] - S.T @ k[t, h // rep])
                S = S + torch.outer(k[t, h // rep], u)
                ref[t, h] = S.T @ q[t, h // rep]
        data.append((torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1), beta, dec.reshape(n, -1), ref))
    state = torch.zeros(4, H, dv, dk, device=DEV)
    state[1] = 9.0
    cuts = [cut(lens[0], (40, 1, 1, 17, 2, 64)), cut(lens[1], (5, 2, 1, 30))]
    got = [torch.empty(n, H, dv) for n in lens]
    for step in range(max(len(c) for c in cuts)):
        act = [(r, cuts[r][step]) for r in range(2) if step < len(cuts[r])]
        x = torch.cat([data[r][0][a:a + n] for r, (a, n) in act]).to(DEV)
        beta = torch.cat([data[r][1][a:a + n] for r, (a, n) in act]).to(DEV).contiguous()
        ww = torch.cat([data[r][2][a:a + n] for r, (a, n) in act]).to(DEV).contiguous()
        ctx = step_ctx([n for _, (_, n) in act], [(2, 0)[r] for r, _ in act])
        o = torch.empty(x.shape[0], H, dv, device=DEV)
        ops.recurrent_scan(ops.SCAN_CHANNEL, x[:, :G * dk], x[:, G * dk:2 * G * dk], x[:, 2 * G * dk:], state, ctx, H, rep, dk, dv, o,
                           bg=beta, ww=ww)
        at = 0
        for r, (a, n) in act:
            got[r][a:a + n] = o[at:at + n].cpu()
            at += n
    for r in range(2):
        assert float((got[r] - data[r][3]).abs().max()) <= 2e-5 * max(1.0, float(data[r][3].abs().max())), r
    assert float((state[1] - 9.0).abs().max()) == 0.0


@pytest.mark.parametrize("T, R, H, per", [(1, 16, 4, 16), (9, 5, 3, 20), (70, 64, 2, 150), (8, 1, 1, 1), (3, 100, 5, 26)])
def test_second_halves_of_the_low_rank_products_with_their_epilogues(T, R, H, per):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T * R)
    N = H * per
    low = torch.randn(T, R + 3, generator=g)
    w2, w0, rate = torch.randn(N, R, generator=g) / R ** 0.5, torch.randn(N, generator=g), torch.randn(H, generator=g) * 0.5
    z = low[:, 3:] @ w2.T
    out = torch.empty(T, N, device=DEV)
    ops.lowrank_decay(low.to(DEV)[:, 3:], w2.t().contiguous().to(DEV), w0.to(DEV), out, inner_tanh=False,
                      epilogue=ops.LR_SOFTPLUS, rate_log=rate.to(DEV), per=per)
    ref = torch.exp(-torch.exp(rate).repeat_interleave(per)[None] * ZP.softplus(z + w0))
    assert float((out.cpu() - ref).abs().max()) <= 3e-6
    ops.lowrank_decay(low.to(DEV)[:, 3:], w2.t().contiguous().to(DEV), None, out, inner_tanh=False, epilogue=ops.LR_SIGMOID)
    assert float((out.cpu() - torch.sigmoid(z)).abs().max()) <= 3e-6


@pytest.mark.parametrize("G, H, dk, dv, K", [(1, 2, 8, 16, 4), (2, 4, 6, 5, 3), (1, 1, 1, 1, 1), (1, 3, 3, 2, 6)])
def test_convolutions_of_q_k_v_unit_vectors_and_beta(G, H, dk, dv, K):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(K + dk)
    C = 2 * G * dk + H * dv
    n = 19
    proj = torch.randn(n, C + H + 3, generator=g)
    taps = torch.randn(C, K, generator=g) * 0.6
    y = ZP.silu(ZP.causal_conv(proj[:, :C].contiguous(), taps))
    q = ZP.unit(y[:, :G * dk].view(n, G, dk)) * dk ** -0.5
    k = ZP.unit(y[:, G * dk:2 * G * dk].view(n, G, dk))
    ref = torch.cat([q.reshape(n, -1), k.reshape(n, -1), y[:, 2 * G * dk:]], 1)
    tail = torch.zeros(2, max(K - 1, 0), C, device=DEV)
    got, got_b = torch.empty(n, C), torch.empty(n, H)
    pd = proj.to(DEV)
    for a, m in cut(n, (1, 2, 1, 5, 3)):
        ctx = step_ctx([m], [1])
        qkv, beta = torch.empty(m, C, device=DEV), torch.empty(m, H, device=DEV)
        single = m == 1
        ops.conv_unit_gates(pd[a:a + m], C, 0, taps.to(DEV), tail, None, None, ctx, G, H, dk, dv, 1e-6, qkv, beta, move_tail=single)
        if not single:
            ops.state_tail(pd[a:a + m], tail, ctx)
        got[a:a + m], got_b[a:a + m] = qkv.cpu(), beta.cpu()
    assert float((got - ref).abs().max()) <= 1e-5
    assert float((got_b - torch.sigmoid(proj[:, C:C + H])).abs().max()) <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_times_a_ready_gate(dtype):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(4)
    o, gate, w = torch.randn(6, 3, 14, generator=g), torch.rand(6, 50, generator=g), torch.randn(14, generator=g) * 0.2 + 1
    out = torch.empty(6, 42, dtype=dtype, device=DEV)
    ops.headnorm_gate(o.to(DEV), gate.to(DEV)[:, 8:], w.to(DEV), 1e-5, 1.0, out, gate_act="none")
    ref = (ZP.rms(o, 1e-5) * w).reshape(6, 42) * gate[:, 8:]
    assert float((out.float().cpu() - ref).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, float(ref.abs().max()))


def paged_case(segs, nkv, dk, dv, page_size, dtype, seed):
    """``segs``: (cached, new) per request.  Keys and values of every position in pages handed out in a scrambled
    order; returns the step's descriptor arrays, the planes, and the dense keys/values per request."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [(-(-(c + n) // page_size)) for c, n in segs]
    total = sum(pages_per)
    order = torch.randperm(total + 3, generator=g).tolist()
    bt = torch.full((len(segs), max(pages_per)), total + 3, dtype=torch.int32)
    kc = torch.randn(total + 4, page_size, nkv, dk, generator=g)
    vc = torch.randn(total + 4, page_size, nkv, dv, generator=g)
    dense, o = [], 0
    for s, (c, n) in enumerate(segs):
        ids = order[o:o + pages_per[s]]
        o += pages_per[s]
        bt[s, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        dense.append((kc[ids].reshape(-1, nkv, dk)[:c + n], vc[ids].reshape(-1, nkv, dv)[:c + n]))
    pos = torch.cat([torch.arange(c, c + n) for c, n in segs]).to(torch.int32)
    tok_seg = torch.cat([torch.full((n,), s) for s, (c, n) in enumerate(segs)]).to(torch.int32)
    seg_start = torch.tensor([0] + list(torch.tensor([n for _, n in segs]).cumsum(0)), dtype=torch.int32)
    ctx = types.SimpleNamespace(
        positions=pos.to(DEV), tok_seg=tok_seg.to(DEV), seg_start=seg_start.to(DEV),
        cached_len=torch.tensor([c for c, _ in segs], dtype=torch.int32, device=DEV), S=len(segs),
        max_q_len=max(n for _, n in segs), max_kv_len=max(c + n for c, n in segs),
        decode_only=all(n == 1 for _, n in segs), err=torch.zeros(1, dtype=torch.int32, device=DEV))
    return ctx, kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), bt.to(DEV), total + 4, dense


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, dk, dv, rot", [(6, 2, 16, 24, 8), (3, 3, 10, 14, 6), (1, 1, 8, 8, 0), (4, 1, 64, 32, 64), (2, 1, 6, 6, 6)])
def test_norm_over_the_whole_projection_rotation_in_halves_and_store(dtype, nh, nkv, dk, dv, rot):
    """q and k are divided by the root mean square of ALL their heads' entries together, weighted entry by entry,
    then entry i of a head's first ``rot`` turns with entry i + rot/2; k and v land in their pages.  Also the
    layer without keys of its own: q alone."""
    from prism_b200 import ops
    from prism_b200.parts.positions import ScaledRotaryEmbedding
    segs = [(0, 3), (9000, 6), (63, 2)]
    ctx, kc, vc, bt, npages, _ = paged_case(segs, nkv, dk, dv, 64, dtype, 2)
    T = 11
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(T, nh * dk + nkv * dk + nkv * dv + 5, generator=g) * 2.0
    proj[:, :dk] *= 4.0                                   # one head much larger than the others: a per-head norm would differ
    wq, wk = torch.randn(nh * dk, generator=g) * 0.3 + 1, torch.randn(nkv * dk, generator=g) * 0.3 + 1
    scaling = dict(factor=4.0, low=1.0, high=4.0, original=64)
    freq = ScaledRotaryEmbedding(rot, 300.0, scaling, interleaved=False).frequencies() if rot else None
    pd = proj.to(DEV)
    a, b, c = nh * dk, nh * dk + nkv * dk, nh * dk + nkv * dk + nkv * dv
    q_out = torch.empty(T, nh, dk, dtype=dtype, device=DEV)
    ops.qk_norm_rope_store(pd[:, :a], pd[:, a:b], pd[:, b:c], wq.to(DEV), wk.to(DEV), 1e-5, None if freq is None else freq.to(DEV),
                           rot, q_out, kc, vc, bt, ctx.positions, ctx.tok_seg, npages, 1 << 20, ctx.err, whole=True, halves=True)
    assert int(ctx.err.item()) == 0
    pos = ctx.positions.cpu().long()
    f = ZP.band_frequencies(300.0, rot, scaling, torch.float32)
    q_ref = ZP.rotate_halves((ZP.rms(proj[:, :a], 1e-5) * wq).view(T, nh, dk), pos, f)
    k_ref = ZP.rotate_halves((ZP.rms(proj[:, a:b], 1e-5) * wk).view(T, nkv, dk), pos, f)
    tol = 2e-3 if dtype == torch.float32 else 4e-2          # float32 sin/cos of angles up to 9,005 radians
    assert float((q_out.float().cpu() - q_ref).abs().max()) <= tol
    seg_of = ctx.tok_seg.cpu().tolist()
    for t in range(T):
        p = int(pos[t])
        page = int(bt[seg_of[t], p // 64])
        assert float((kc[page, p % 64].float().cpu() - k_ref[t]).abs().max()) <= tol
        assert float((vc[page, p % 64].float().cpu() - proj[t, b:c].view(nkv, dv)).abs().max()) <= (1e-6 if dtype == torch.float32 else 4e-2)
    before = kc.clone()
    q2 = torch.empty_like(q_out)
    ops.qk_norm_rope_store(pd[:, :a], None, None, wq.to(DEV), None, 1e-5, None if freq is None else freq.to(DEV), rot, q2, None, None,
                           bt, ctx.positions, ctx.tok_seg, npages, 1 << 20, ctx.err, whole=True, halves=True, nkv=nkv)
    assert torch.equal(q2, q_out) and torch.equal(before, kc)


def plain_sink_attention(q, dense, segs, nh, nkv, scale, sink):
    outs, t = [], 0
    for (c, n), (k, v) in zip(segs, dense):
        vis = torch.ones(c + n, c + n, dtype=torch.bool).tril()[c:]
        o = torch.empty(n, nh, v.shape[-1])
        for h in range(nh):
            g = h // (nh // nkv)
            s = ((q[t:t + n, h] @ k[:, g].T) * scale).masked_fill(~vis, -math.inf)
            o[:, h] = ZP.sink_softmax(s) @ v[:, g] if sink else torch.softmax(s, -1) @ v[:, g]
        outs.append(o.reshape(n, -1))
        t += n
    return torch.cat(outs)


def run_attention(kernel, segs, shape, page_size, seed, scale, sink=True, boost=None):
    from prism_b200 import ops
    nh, nkv, dk, dv = shape
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    ctx, kc, vc, bt, npages, dense = paged_case(segs, nkv, dk, dv, page_size, dtype, seed)
    T = int(ctx.positions.shape[0])
    q = torch.randn(T, nh, dk, generator=torch.Generator().manual_seed(seed + 1))
    if boost is not None:
        boost(q, kc, vc, bt, dense)
    dense = [(k.to(dtype).float(), v.to(dtype).float()) for k, v in dense]
    qd = q.to(dtype).to(DEV)
    out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
    sk = torch.zeros(nh, device=DEV) if sink else None
    if kernel.startswith("generic"):
        ops.attention_masked_generic(qd, out, kc, vc, bt, ctx.positions, ctx.tok_seg, npages, ops.KeyMask.causal(), scale, sk, ctx.err)
    else:
        few = kernel.startswith("tc_decode")
        ns = int(kernel.split(":")[1]) if ":" in kernel else 1
        ops.attention_masked_bf16(qd, out, kc, vc, bt, ctx.seg_start, ctx.cached_len, ctx.S, ctx.max_q_len, npages,
                                  ops.KeyMask.causal(), scale, sk, few, ctx.err, nsplit=ns)
    assert int(ctx.err.item()) == 0
    return out.float().cpu(), plain_sink_attention(qd.float().cpu(), dense, segs, nh, nkv, scale, sink)


KERNELS = ["generic_f32", "generic_bf16", "tc_portions", "tc_decode", "tc_decode:3"]


def tc_takes(kernel, shape):
    from prism_b200 import ops
    nh, nkv, dk, dv = shape
    return not kernel.startswith("tc") or (ops.lib().prism_attention_masked_supported(dk, dv, nh, nkv) and dv % 8 == 0)


@pytest.mark.parametrize("shape", [(6, 2, 16, 24), (3, 1, 32, 32), (6, 6, 64, 16), (2, 1, 7, 5), (16, 4, 128, 128), (1, 1, 8, 8)],
                         ids=lambda s: "h%d_g%d_k%d_v%d" % s)
@pytest.mark.parametrize("kernel", KERNELS)
def test_causal_attention_with_one_added_to_the_denominator(shape, kernel):
    """Requests of unequal length in scrambled pages: first tokens, page borders, portions behind a long cache.
    The small scale keeps the sum of the exponentials of the order of one, so that leaving the sink out (or
    counting it twice) moves every row."""
    if not tc_takes(kernel, shape):
        pytest.skip("the tensor-core kernel leaves this shape to the generic one")
    if kernel.startswith("tc_decode"):
        segs = [(0, 1), (1, 1), (12, 1), (63, 1), (64, 1), (130, 1), (257, 1)]
    else:
        segs = [(0, 1), (0, 37), (5, 2), (60, 9), (100, 80), (199, 1), (3, 130)]
    dk = shape[2]
    got, ref = run_attention(kernel, segs, shape, 16 if dk < 64 else 64, 5, 0.5 * dk ** -0.5)
    tol = 2e-5 if kernel == "generic_f32" else 2e-2
    assert float((got - ref).abs().max()) <= tol
    _, no_sink = run_attention(kernel, segs, shape, 16 if dk < 64 else 64, 5, 0.5 * dk ** -0.5, sink=False)
    assert float((got - no_sink).abs().max()) > 20 * tol          # the test would see a softmax without the sink


@pytest.mark.parametrize("kernel", KERNELS)
def test_the_sink_takes_its_share_and_a_far_key_is_found(kernel):
    """One key of a long context gets a score far above all others and a value of its own: the output is that
    value wherever the key lies - the first token, far back among hundreds, either side of a page border, the
    query's own position.  With every score far below zero the sink takes everything and the output vanishes;
    with one score of exactly zero beside such scores the key and the sink share evenly."""
    nh, nkv, dk, dv = 4, 2, 32, 32
    ctx_len = 700
    decode = kernel.startswith("tc_decode")
    tol = 2e-5 if kernel == "generic_f32" else 3e-2
    for qpos in (ctx_len - 1, ctx_len - 40):
        for key in (0, 1, 63, 64, 65, 127, 128, 300, 639, 640, qpos - 1, qpos):
            segs = [(qpos, 1)] if decode else [(qpos - 5, 9)]
            row = 0 if decode else 5

            def boost(q, kc, vc, bt, dense, key=key, level=30.0):
                k, v = dense[0]
                k[key] = 0.0
                k[key, :, 0] = level
                v[key] = 7.0
                q[row, :, 0] = 30.0
                page, at = int(bt[0, key // 64]), key % 64
                kc[page, at] = k[key].to(kc.dtype)
                vc[page, at] = v[key].to(vc.dtype)
            got, ref = run_attention(kernel, segs, (nh, nkv, dk, dv), 64, 9, dk ** -0.5, boost=boost)
            assert float((got[row].view(nh, dv) - 7.0).abs().max()) < 0.05, (qpos, key)
            assert float((got - ref).abs().max()) <= tol, (qpos, key)
    # all keys far below the sink; then one of them level with it
    for level, want in ((None, 0.0), (0.0, 3.5)):
        segs = [(299, 1)] if decode else [(290, 10)]
        row = 0 if decode else 9

        def boost(q, kc, vc, bt, dense, level=level):
            k, v = dense[0]
            q[row] = 0.0
            q[row, :, 0] = 8.0
            k[:, :, 0] = -40.0
            if level is not None:
                k[77, :, 0] = level
                v[77] = 7.0
            for key in range(k.shape[0]):
                page, at = int(bt[0, key // 64]), key % 64
                kc[page, at] = k[key].to(kc.dtype)
                vc[page, at] = v[key].to(vc.dtype)
        got, ref = run_attention(kernel, segs, (nh, nkv, dk, dv), 64, 10, dk ** -0.5, boost=boost)
        assert float((got[row] - want).abs().max()) < 1e-3 + tol, level
        assert float((got - ref).abs().max()) <= tol


def plain_experts(x, logits, gu, dn, top, F):
    s = torch.sigmoid(logits)
    out = torch.zeros(top, x.shape[0], x.shape[1])
    chosen = torch.topk(s, top, dim=-1).indices
    for t in range(x.shape[0]):
        for j, e in enumerate(chosen[t].tolist()):
            a = s[t, e] * x[t]
            out[j, t] = (ZP.silu(a @ gu[e, :F].T) * (a @ gu[e, F:].T)) @ dn[e].T
    return out.sum(0)


@pytest.mark.parametrize("T, W, F, E, top", [(1, 72, 24, 6, 2), (37, 64, 40, 3, 1), (130, 128, 96, 8, 3), (5, 33, 7, 5, 5), (9, 16, 8, 1, 1),
                                             (300, 64, 32, 64, 2), (2, 256, 64, 16, 1), (700, 256, 200, 5, 2), (20, 136, 328, 4, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_take_their_tokens_scaled_by_the_score(T, W, F, E, top, dtype):
    """Scores spread by a large router, so that the choice does not hang on rounding; every choice of a token is a
    plane of the result, which the caller adds up."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(dtype)
    logits = torch.randn(T, E + 2, generator=g) * 2.0
    gu = (torch.randn(E, 2 * F, W, generator=g) / W ** 0.5).to(dtype)
    dn = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(dtype)
    ctx = step_ctx([T], [0])
    y = ops.moe_feed_forward(ctx, x.to(DEV), logits.to(DEV)[:, 1:E + 1], gu.to(DEV), dn.to(DEV), top)
    assert y.shape == (top, T, W) and y.dtype == torch.float32
    ref = plain_experts(x.float(), logits[:, 1:E + 1], gu.float(), dn.float(), top, F)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert float((y.sum(0).cpu() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))
    # the other conventions of the same kernels: softmax scores renormalized over the chosen, on the expert's output
    y2 = ops.moe_feed_forward(ctx, x.to(DEV), logits.to(DEV)[:, 1:E + 1], gu.to(DEV), dn.to(DEV), top, softmax=True, renorm=True,
                              scale_input=False)
    p = torch.softmax(logits[:, 1:E + 1], -1)
    ch = torch.topk(p, top, dim=-1)
    ref2 = torch.zeros(T, W)
    for t in range(T):
        for wgt, e in zip((ch.values[t] / ch.values[t].sum()).tolist(), ch.indices[t].tolist()):
            a = x[t].float()
            ref2[t] += wgt * ((ZP.silu(a @ gu[e, :F].float().T) * (a @ gu[e, F:].float().T)).to(dtype).float() @ dn[e].float().T)
    assert float((y2.sum(0).cpu() - ref2).abs().max()) <= tol * max(1.0, float(ref2.abs().max()))


@pytest.mark.parametrize("T, W, F, E, top", [(3, 64, 24, 4, 2), (33, 192, 136, 6, 3), (64, 128, 128, 2, 2), (65, 128, 72, 9, 1),
                                             (500, 320, 264, 7, 2)])
def test_experts_on_tensor_cores_against_cuda_cores(T, W, F, E, top):
    """bf16: tiles of one expert each on the tensor cores against the CUDA-core kernels on the same choice; experts
    without a token, stretches that end inside a tile, feature counts that are no multiple of the tile."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T * 7 + E)
    x = torch.randn(T, W, generator=g).to(torch.bfloat16).to(DEV)
    logits = (torch.randn(T, E, generator=g) * 2.0).to(DEV)
    if E > 2:
        logits[:, 1] = -30.0                     # nobody chooses expert 1
    gu = (torch.randn(E, 2 * F, W, generator=g) / W ** 0.5).to(torch.bfloat16).to(DEV)
    dn = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(torch.bfloat16).to(DEV)
    ctx = step_ctx([T], [0])
    assert ops.lib().prism_moe_tcgen05_supported(W, F)
    for kw in (dict(), dict(softmax=True, renorm=True, scale_input=False, act="gelu_tanh")):
        ops.moe_tensor_cores = False
        try:
            ref = ops.moe_feed_forward(ctx, x, logits, gu, dn, top, **kw).clone()
        finally:
            ops.moe_tensor_cores = True
        got = ops.moe_feed_forward(ctx, x, logits, gu, dn, top, **kw)
        ops.check_tc_errors()
        assert float((got - ref).abs().max()) <= 2e-2 * max(1.0, float(ref.abs().max()))


# ---------------------------------------------------------------------------------------------------------
# the model through the engine's step function
# ---------------------------------------------------------------------------------------------------------

LIMIT = {"float32": 3e-5, "bfloat16": 4e-2}
ILL = {"float32": 0.0, "bfloat16": 0.05}        # see zuvulorn_helpers.judge
LENGTHS = {"A": [1, 9, 40, 71, 130], "B": [2, 65, 128, 200, 333], "C": [1, 5, 33], "D": [3, 26, 61], "E": [1, 20, 70], "F": [3, 70, 150, 257]}


def runner_for(folder, dtype, max_tokens, page_size, max_live=4):
    from prism_b200.engine.replay import build_runner
    return build_runner(folder, dtype, max_tokens, page_size, max_live)[3]


def sequences(name):
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name[0]])}


def served(name, dtype):
    """The configuration a dtype is tested on: in bfloat16 the variant in which every expert is chosen
    (``zuvulorn_helpers.every_expert``)."""
    return name + "x" if dtype == "bfloat16" else name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "small_portions", "mixed"])
def test_cutting(name, dtype, mode):
    """Whole prompts, a decoded tail, portions (one schedule of twos and threes only), and mixed batches of up
    to four live requests in a pool that holds no more than the schedule needs, so that pages and state slots
    come back and are used again."""
    name = served(name, dtype)
    seqs = sequences(name)
    steps = {"whole": trace_whole, "tail": lambda s: trace_tail(s, 48), "portions": trace_portions,
             "small_portions": lambda s: trace_portions(s, (2, 3, 2, 2, 5, 2)),
             "mixed": lambda s: trace_mixed(s, seed=3)}[mode](seqs)
    ps = CONFIGS[name][2]
    runner = runner_for(model_folder(name), dtype, trace_budget(steps, max(ps, 64)), ps)
    got = run_trace(runner, steps)
    assert len(got) == sum(len(s) for s in seqs.values())
    compare(name, seqs, got, LIMIT[dtype], ILL[dtype], dtype)
    assert runner.cache.pages_in_use() == 0 and len(runner.cache.requests) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_stream_after_every_layer(dtype):
    """The sum of the copies after each layer, whole prompt, against the plain model's: a fault shows in the layer
    that has it."""
    from prism_b200.engine.batch import Segment
    from prism_b200.parts.base import StreamUpdate
    for name in (served("A", dtype), served("D", dtype)):
        raw, seed, ps = CONFIGS[name]
        seq = random_tokens(raw["vocab"], 45, 7)
        wd = {k: v.double() for k, v in draw_weights(raw, seed).items()}
        _, after = ZP.forward(raw, wd, seq, return_layers=True)
        rounded = ZP.forward(raw, wd, seq, return_layers=True, rnd=to_bf16_and_back)[1] if dtype == "bfloat16" else after
        runner = runner_for(model_folder(name), dtype, 64, ps)
        kept = []

        def watch(block):
            inner = block.forward

            def forward(ctx, residual, delta, cache):
                x, d = inner(ctx, residual, delta, cache)          # the copies, and the update the block left open
                open_ = d.delta if isinstance(d, StreamUpdate) else d
                y = open_.float() if open_.dim() == 2 else open_.float().sum(0)
                xs = x if x.dim() == 3 else x[None]
                if isinstance(d, StreamUpdate) and d.mix is not None:
                    n = xs.shape[0]
                    new = torch.einsum("ij,itw->jtw", d.mix.float().view(n, n), xs) + d.out.float()[:, None, None] * y[None]
                else:
                    new = xs + y[None]
                kept.append(new.sum(0).cpu())
                return x, d
            block.forward = forward
        for block in runner.model.layers:
            watch(block)
        runner.begin_request("a")
        runner.step([Segment("a", seq, [44])])
        runner.check_errors()
        assert len(kept) == len(raw["layers"])
        for i, x in enumerate(kept):
            scale = float(after[i].pow(2).mean().sqrt())
            err = float((x - after[i]).pow(2).mean().sqrt()) / scale
            own = float((rounded[i] - after[i]).pow(2).mean().sqrt()) / scale          # what rounding alone does here
            assert err <= (2e-5 if dtype == "float32" else max(1e-2, 3 * own)), (name, i, err, own)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_pages(dtype):
    name = served("B", dtype)
    seq = random_tokens(CONFIGS[name][0]["vocab"], 420, 9)
    runner = runner_for(model_folder(name), dtype, 448, 64)
    got = run_trace(runner, trace_tail({"a": seq}, 300))
    compare(name, {"a": seq}, got, LIMIT[dtype], ILL[dtype], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests_against_each_alone(dtype):
    seqs = sequences("A")
    ps = CONFIGS["A"][2]
    alone = run_trace(runner_for(model_folder("A"), dtype, 4096, ps), trace_portions(seqs, (5, 2, 9)))
    together = run_trace(runner_for(model_folder("A"), dtype, 4096, ps, max_live=5), trace_mixed(seqs, seed=11, max_live=5))
    tol = 2e-5 if dtype == "float32" else 8e-2
    for key, row in alone.items():
        assert float((row - together[key]).abs().max()) <= tol * max(1.0, float(row.abs().max())), key


def test_a_state_slot_that_is_used_again_starts_from_zero():
    """One slot only: the second request gets the slot the first one left, and must not inherit its states or the
    convolutions' tails."""
    seqs = {"a": random_tokens(90, 40, 1), "b": random_tokens(90, 25, 2), "c": random_tokens(90, 2, 3)}
    runner = runner_for(model_folder("E"), "float32", 64, 16, max_live=1)
    got = run_trace(runner, trace_portions(seqs, (7, 1, 3)))
    compare("E", seqs, got, LIMIT["float32"])


ONE_LAYER = {
    "attention": [layer("attention", attn(4, 2, 16, 8, scale=0.4, rot_dims=8, base=300.0, scaling=(2.0, 1.0, 2.0, 32)), None)],
    "attention_on_anothers_keys": [layer("attention", attn(3, 1, 32, 32, scale=0.2), None),
                                   layer("attention", attn(3, 1, 32, 32, scale=0.3, kv_from=0), None)],
    "channel_delta": [layer("channel_delta", delta(4, 2, 24, 12, 5, 6, 3), None)],
    "rglru": [layer("rglru", rglru(56, 7, 3), None)],
    "experts": [layer("rglru", rglru(8, 1, 2), experts(20, 5, 2))],
    "odd_sizes": [layer("attention", attn(2, 1, 7, 5, rot_dims=4), experts(9, 3, 2)), layer("channel_delta", delta(3, 3, 5, 3, 2, 2, 5), None),
                  layer("rglru", rglru(27, 3, 5), experts(5, 2, 1))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mixer_alone(which, dtype):
    odd = which == "odd_sizes"
    raw = model(51 if odd else 97, 37 if odd else 48, ONE_LAYER[which], streams=3 if odd else 2)
    if dtype == "bfloat16":
        raw = every_expert(raw)
    w = draw_weights(raw, 21)
    folder = write_folder(raw, w)
    seq = random_tokens(raw["vocab"], 75, 4)
    ref = ZP.forward(raw, {k: v.float() for k, v in w.items()}, seq)
    runner = runner_for(folder, dtype, 128, 16)
    got = run_trace(runner, trace_portions({"a": seq}, (20, 1, 1, 30, 2, 1)))
    scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    errs = sorted(float((got[("a", p)] - ref[p] - (got[("a", p)] - ref[p]).mean()).pow(2).mean().sqrt()) / scale for p in range(75))
    assert errs[-1] <= LIMIT[dtype] * (8 if ILL[dtype] else 1) and errs[int(len(errs) * (1 - ILL[dtype])) - 1] <= LIMIT[dtype], errs[-4:]


def test_a_token_far_back_decides_through_attention_alone():
    """A model of one attention layer whose first token differs between two prompts that are otherwise equal and
    several hundred tokens long: the logits at the end differ, in a whole prompt and when the end is decoded
    token by token, and each agrees with the plain model."""
    raw = model(60, 64, [layer("attention", attn(4, 2, 16, 16, scale=0.02, rot_dims=16, base=10000.0), None)], streams=2)
    w = draw_weights(raw, 5)
    folder = write_folder(raw, w)
    base = random_tokens(60, 390, 6)
    seqs = {"a": [3] + base, "b": [4] + base}
    wf = {k: v.double() for k, v in w.items()}
    refs = {k: ZP.forward(raw, wf, s) for k, s in seqs.items()}
    tol = 2e-5 * float(refs["a"].abs().max())
    assert float((refs["a"][-1] - refs["b"][-1]).abs().max()) > 50 * tol
    for steps in (trace_whole(seqs), trace_tail(seqs, 70)):
        got = run_trace(runner_for(folder, "float32", 1024, 64), steps)
        for rid in seqs:
            for pos in (0, 1, 63, 64, 320, 389, 390):
                assert float((got[(rid, pos)] - refs[rid][pos]).abs().max()) <= tol, (rid, pos)


def test_greedy_generation_through_the_scheduler():
    """Engine.generate (scheduler, batching, sampling, CUDA graphs for the decode steps) picks the plain
    model's greedy tokens; more prompts than request slots, so that state slots are used again."""
    from prism_b200.config.engine_config import EngineConfig, SchedulerConfig
    from prism_b200.engine.llm import Engine
    from prism_b200.sampling.sampler import SamplingParams
    raw, seed, ps = CONFIGS["A"]
    w = {k: v.float() for k, v in draw_weights(raw, seed).items()}
    prompts = [random_tokens(raw["vocab"], n, 40 + n) for n in (3, 17, 30, 8, 1, 12)]
    n_new = 24
    folder = model_folder("A")
    for graphs in (False, True):
        eng = Engine(folder, EngineConfig(kv_page_size=ps, num_pages=40, max_seq_len=128, use_cuda_graph=graphs,
                                          graph_batch_sizes=(1, 2, 4, 8),
                                          scheduler=SchedulerConfig(max_batch_tokens=48, max_num_seqs=4, prefill_chunk=16)),
                     dtype="float32")
        assert eng.runner.use_cuda_graph == graphs
        res = eng.generate(prompts, SamplingParams(max_new_tokens=n_new, ignore_eos=True))
        for p, r in zip(prompts, res):
            seq = list(p)
            for tok in r.token_ids:
                logits = ZP.forward(raw, w, seq)[-1]
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) > 1e-3:          # a near tie may fall either way
                    assert tok == int(logits.argmax()), (graphs, len(p), len(seq))
                seq.append(tok)
            assert len(r.token_ids) == n_new
        assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_serves_the_design(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Zuvulorn folder: the model class is found by config.json, the ranks of
    the low-rank products by the model file, the pool holds what --max-tokens says and there are four state slots."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = served("B", dtype)
    raw = CONFIGS[name][0]
    folder = model_folder(name)
    vocab = raw["vocab"]
    seqs = {f"q{i}": random_tokens(vocab, n, 500 + i) for i, n in enumerate([70, 33, 90, 12, 64, 5])}
    steps = trace_mixed(seqs, seed=17)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(trace_budget(steps, 64))],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, fed = {}, {}
    for s in steps:
        n_want = sum(len(e["want"]) for e in s["entries"])
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in s["entries"]:
            for w in e["want"]:
                got[(e["id"], fed.get(e["id"], 0) + w)] = torch.from_numpy(data[r].copy())
                r += 1
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
    assert len(got) == sum(len(s) for s in seqs.values())
    compare(name, seqs, got, LIMIT[dtype], ILL[dtype], dtype)
