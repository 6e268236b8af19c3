"""Tagelorn on the GPU against the plain implementation (tests/plain/tagelorn_plain.py): each kernel alone, each
mixer alone, whole prompts against token-by-token decoding, portions down to two tokens, mixed batches with pages
and state slots that are used again, keys far back, at page borders and just inside and outside the window, the
first tokens of a sequence, long decoding, and greedy generation through the engine's scheduler."""

import math
import types

import pytest
import torch

from tagelorn_helpers import (CONFIGS, LENGTHS, TP, attn, compare, delta, dense, draw_weights, every_expert, layer, model, model_folder,
                              moe, to_bf16_and_back, write_folder)
from helpers import random_tokens, run_trace, trace_budget, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LIMIT = {"float32": 2e-5, "bfloat16": 2e-2}
ILL = {"float32": 0.0, "bfloat16": 0.05}


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

@pytest.mark.parametrize("W", [32, 33, 336])
def test_embedding_rows_scaled_with_sine_and_cosine_of_the_position(W):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(W)
    table = torch.randn(50, W, generator=g)
    ids = torch.randint(0, 50, (9,), generator=g)
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 4095, 12345, 7], dtype=torch.int32)
    i = torch.arange((W + 1) // 2, dtype=torch.float64)
    freq = (10000.0 ** (-2.0 * i / W)).float().to(DEV)
    out = torch.empty(9, W, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(ids.to(torch.int32).to(DEV), table.to(DEV), out, err, 2.0, pos.to(DEV), freq)
    ref = table.double()[ids] * 2.0
    for r, p in enumerate(pos.tolist()):
        ref[r] += TP.sinusoid(p + 1, W, torch.float64)[p]
    assert int(err.item()) == 0
    assert float((out.cpu().double() - ref).abs().max()) <= 2e-3          # the angle itself is a float32 product
    assert float((out.cpu().double() - ref)[:5].abs().max()) <= 1e-5


@pytest.mark.parametrize("C, K", [(5, 1), (40, 2), (33, 4), (352, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_input_convolution_beside_the_skip_path_in_portions_and_token_by_token(C, K, dtype):
    """Two requests in slots 2 and 0 (slot 1 is a neighbour's and must stay), cut into portions shorter and longer than
    the tail and into single tokens, against the plain convolution over the whole sequence.  Steps of sixteen tokens and
    more with the taps also given as float32 ``[K, C]`` take the kernel that works in tiles of tokens (a tile may hold the
    end of one request and the start of the other)."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(C + K)
    lens = (70, 33)
    xs = [torch.randn(n, C, generator=g) for n in lens]
    taps = torch.randn(C, K, generator=g) * 0.5
    refs = [TP.input_conv(x.double(), taps.double()) for x in xs]
    for sizes in ((1,), (2, 7, 1, 3), (30,), (21, 2, 40)):
        tail = torch.zeros(3, max(K - 1, 0), C, device=DEV)
        tail[1] = 7.0
        got = [torch.empty(n, C) for n in lens]
        for k, parts in enumerate(zip(*[cut(n, sizes) + [None] * 80 for n in lens])):
            live = [(s, p) for s, p in enumerate(parts) if p is not None]
            if not live:
                break
            ctx = step_ctx([p[1] for _, p in live], [(2, 0)[s] for s, _ in live])
            x = torch.cat([xs[s][a:a + n] for s, (a, n) in live]).to(DEV)
            out = torch.empty(x.shape[0], C, dtype=dtype, device=DEV)
            single = all(p[1] == 1 for _, p in live)
            ops.causal_conv(x, taps.to(DEV), None, tail, ctx, out, move_tail=single, add_input=True,
                            taps_t=taps.t().contiguous().to(DEV) if k % 2 == 0 else None)
            if not single and K > 1:
                ops.state_tail(x, tail, ctx)
            o = 0
            for s, (a, n) in live:
                got[s][a:a + n] = out[o:o + n].float().cpu()
                o += n
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for s in range(2):
            assert float((got[s].double() - refs[s]).abs().max()) <= tol * max(1.0, float(refs[s].abs().max())), (sizes, s)
        if K > 1:
            assert float((tail[1] - 7.0).abs().max()) == 0.0


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
    dense_kv, o = [], 0
    for s, (c, n) in enumerate(segs):
        ids = order[o:o + pages_per[s]]
        o += pages_per[s]
        bt[s, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        dense_kv.append((kc[ids].reshape(-1, nkv, dk)[:c + n], vc[ids].reshape(-1, nkv, dv)[:c + n], ids))
    pos = torch.cat([torch.arange(c, c + n) for c, n in segs]).to(torch.int32)
    tok_seg = torch.cat([torch.full((n,), s) for s, (c, n) in enumerate(segs)]).to(torch.int32)
    seg_start = torch.tensor([0] + list(torch.tensor([n for _, n in segs]).cumsum(0)), dtype=torch.int32)
    ctx = types.SimpleNamespace(
        positions=pos.to(DEV), tok_seg=tok_seg.to(DEV), seg_start=seg_start.to(DEV),
        cached_len=torch.tensor([c for c, _ in segs], dtype=torch.int32, device=DEV), S=len(segs),
        max_q_len=max(n for _, n in segs), max_kv_len=max(c + n for c, n in segs),
        decode_only=all(n == 1 for _, n in segs), err=torch.zeros(1, dtype=torch.int32, device=DEV))
    return ctx, kc, vc, bt.to(DEV), total + 4, dense_kv


def plain_biased_attention(q, dense_kv, segs, nh, nkv, scale, size, keep, rel, far, sink):
    """Softmax over the visible keys and the sink, scores ``q.k * scale + rel[bucket(distance)]``, float64."""
    outs, t = [], 0
    rows = rel.shape[0]
    for (c, n), (k, v, _) in zip(segs, dense_kv):
        o = torch.zeros(n, nh, v.shape[-1], dtype=torch.float64)
        for i in range(n):
            p = c + i
            js = [j for j in range(p + 1) if TP.visible(p, j, size, keep)]
            b = torch.tensor([TP.distance_bucket(p - j, rows, far) for j in js])
            for h in range(nh):
                g = h // (nh // nkv)
                s = (k[js, g].double() @ q[t + i, h].double()) * scale + rel[b, h].double()
                m = max(float(s.max()), float(sink[h]))
                e = torch.exp(s - m)
                o[i, h] = (e / (e.sum() + math.exp(float(sink[h]) - m))) @ v[js, g].double()
        outs.append(o.reshape(n, -1))
        t += n
    return torch.cat(outs)


def run_attention(kernel, segs, shape, page_size, seed, scale, size, keep, rows, far, boost=None):
    from prism_b200 import ops
    from prism_b200.parts.attention import distance_bucket
    nh, nkv, dk, dv = shape
    dtype = torch.float32 if kernel == "generic_f32" else torch.bfloat16
    ctx, kc, vc, bt, npages, dense_kv = paged_case(segs, nkv, dk, dv, page_size, dtype, seed)
    g = torch.Generator().manual_seed(seed + 1)
    T = int(ctx.positions.shape[0])
    q = torch.randn(T, nh, dk, generator=g)
    rel, sink = torch.randn(rows, nh, generator=g) * 1.5, torch.randn(nh, generator=g)
    if boost is not None:
        boost(q, kc, vc, dense_kv)
    kc, vc = kc.to(dtype), vc.to(dtype)
    dense_kv = [(kc[ids].reshape(-1, nkv, dk)[:c + n].float(), vc[ids].reshape(-1, nkv, dv)[:c + n].float(), ids)
                for (c, n), (_, _, ids) in zip(segs, dense_kv)]
    qd = q.to(dtype).to(DEV)
    out = torch.empty(T, nh * dv, dtype=dtype, device=DEV)
    idx = torch.tensor([distance_bucket(n, rows, far) for n in range(far + 1)])
    table = rel[idx].t().contiguous().to(DEV)
    mask = ops.KeyMask.window(size, keep)
    if kernel.startswith("generic"):
        ops.attention_masked_generic(qd, out, kc.to(DEV), vc.to(DEV), bt, ctx.positions, ctx.tok_seg, npages, mask, scale, sink.to(DEV),
                                     ctx.err, table)
    else:
        few = kernel.startswith("tc_decode")
        ns = int(kernel.split(":")[1]) if ":" in kernel else 1
        ops.attention_masked_bf16(qd, out, kc.to(DEV), vc.to(DEV), bt, ctx.seg_start, ctx.cached_len, ctx.S, ctx.max_q_len, npages,
                                  mask, scale, sink.to(DEV), few, ctx.err, nsplit=ns, dist_bias=table)
    assert int(ctx.err.item()) == 0
    return out.float().cpu(), plain_biased_attention(qd.float().cpu(), dense_kv, segs, nh, nkv, scale, size, keep, rel, far, sink).float()


KERNELS = ["generic_f32", "generic_bf16", "tc_portions", "tc_decode", "tc_decode:3"]
PORTIONS = [(0, 3), (200, 40), (63, 2), (0, 130)]
DECODING = [(0, 1), (63, 1), (64, 1), (300, 1), (129, 1)]


def tc_takes(kernel, shape):
    from prism_b200 import ops
    nh, nkv, dk, dv = shape
    return not kernel.startswith("tc") or (ops.lib().prism_attention_masked_supported(dk, dv, nh, nkv) and dv % 8 == 0)


@pytest.mark.parametrize("mask", [(80, 5, 24, 200), (9, 2, 10, 30), (40, 0, 6, 11), (33, 70, 16, 64), (1, 1, 1, 1), (500, 0, 2, 3)],
                         ids=lambda m: "w%d_k%d_r%d_f%d" % m)
@pytest.mark.parametrize("shape", [(5, 1, 64, 64), (6, 2, 16, 24), (4, 4, 10, 6), (8, 2, 32, 64), (1, 1, 8, 8)],
                         ids=lambda s: "h%d_g%d_k%d_v%d" % s)
@pytest.mark.parametrize("kernel", KERNELS)
def test_attention_under_a_window_with_kept_positions_a_bias_by_distance_and_a_sink(mask, shape, kernel):
    if not tc_takes(kernel, shape):
        pytest.skip("the tensor-core kernel does not take this shape")
    size, keep, rows, far = mask
    segs = DECODING if kernel.startswith("tc_decode") else PORTIONS
    got, ref = run_attention(kernel, segs, shape, 64, 5, 0.3, size, keep, rows, far)
    tol = 2e-5 if kernel == "generic_f32" else 2e-2
    assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("kernel", KERNELS)
@pytest.mark.parametrize("where", ["kept_far", "first_not_kept", "last_inside", "first_outside", "page_border", "own"])
def test_one_key_that_stands_out(kernel, where):
    """A request of 400 positions behind a window of 80 that keeps 5: one key's score is raised far above the rest, and
    its value is a row of hundreds.  Where the key is visible the output is that row, where it is not, nothing of it
    arrives: a window or a kept run that is one token off shows in every head."""
    size, keep = 80, 5
    qpos = 399
    key = {"kept_far": 4, "first_not_kept": 5, "last_inside": qpos - size + 1, "first_outside": qpos - size, "page_border": 383,
           "own": qpos}[where]
    seen = where not in ("first_not_kept", "first_outside")
    segs = [(qpos, 1)] if kernel.startswith("tc_decode") else [(380, 20)]

    def boost(q, kc, vc, dense_kv):
        _, _, ids = dense_kv[0]
        page, slot = ids[key // 64], key % 64
        kc[page, slot] = q[-1, 0][None, :] * 4.0
        vc[page, slot] = 300.0
        q[-1] = q[-1, 0][None, :]
    got, ref = run_attention(kernel, segs, (4, 2, 32, 16), 64, 9, 0.5, size, keep, 24, 200, boost)
    tol = 2e-5 if kernel == "generic_f32" else 2e-2
    assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))
    last = ref[-1]
    assert (float(last.abs().min()) > 200.0) == seen and (float(last.abs().max()) < 30.0) == (not seen)


@pytest.mark.parametrize("H, d", [(1, 1), (3, 7), (2, 20), (4, 32), (2, 64), (2, 128), (1, 300)])
def test_generalized_delta_rule_in_pieces(H, d):
    """Two requests in slots 2 and 0, cut into portions and single tokens, against the plain recurrence over the whole
    sequence in float64; the neighbour's slot stays as it was."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(H * 1000 + d)
    lens = (37, 12)
    A = H * d
    rows = [torch.randn(n, 3 * A, generator=g) for n in lens]                    # r | k | v
    decay = [torch.rand(n, A, generator=g) * 0.4 + 0.6 for n in lens]
    ex = []
    for s, n in enumerate(lens):
        k = rows[s][:, A:2 * A].view(n, H, d)
        e = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        ex.append(torch.cat([e.reshape(n, A), (torch.rand(n, H, d, generator=g) * e).reshape(n, A)], 1))
    refs = []
    for s, n in enumerate(lens):
        r, k, v = (rows[s][:, i * A:(i + 1) * A].double().view(n, H, d) for i in range(3))
        w, e, c = decay[s].double().view(n, H, d), ex[s][:, :A].double().view(n, H, d), ex[s][:, A:].double().view(n, H, d)
        S = torch.zeros(H, d, d, dtype=torch.float64)
        o = torch.zeros(n, H, d, dtype=torch.float64)
        for t in range(n):
            for h in range(H):
                S[h] = w[t, h][:, None] * S[h] - c[t, h][:, None] * (e[t, h] @ S[h])[None, :] + k[t, h][:, None] * v[t, h][None, :]
                o[t, h] = S[h].T @ r[t, h]
        refs.append(o)
    for sizes in ((1,), (2, 9, 1, 17), (50,)):
        state = torch.zeros(3, H, d, d, device=DEV)
        state[1] = 3.0
        got = [torch.empty(n, H, d) for n in lens]
        for parts in zip(*[cut(n, sizes) + [None] * 60 for n in lens]):
            live = [(s, p) for s, p in enumerate(parts) if p is not None]
            if not live:
                break
            ctx = step_ctx([p[1] for _, p in live], [(2, 0)[s] for s, _ in live])
            x = torch.cat([rows[s][a:a + n] for s, (a, n) in live]).to(DEV)
            ww = torch.cat([decay[s][a:a + n] for s, (a, n) in live]).to(DEV)
            ee = torch.cat([ex[s][a:a + n] for s, (a, n) in live]).contiguous().to(DEV)
            out = torch.empty(x.shape[0], H, d, device=DEV)
            ops.recurrent_scan(ops.SCAN_GENERAL, x[:, :A], x[:, A:2 * A], x[:, 2 * A:], state, ctx, H, 1, d, d, out, ww=ww, ex=ee)
            o = 0
            for s, (a, n) in live:
                got[s][a:a + n] = out[o:o + n].cpu()
                o += n
        for s in range(2):
            assert float((got[s].double() - refs[s]).abs().max()) <= 2e-5 * max(1.0, float(refs[s].abs().max())), (sizes, s)
        assert float((state[1] - 3.0).abs().max()) == 0.0


@pytest.mark.parametrize("T, H, d, R", [(1, 1, 1, 1), (5, 3, 7, 5), (40, 2, 64, 16), (17, 4, 32, 3)])
def test_unit_key_removal_and_the_decay_between_a_bound_and_one(T, H, d, R):
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T + d)
    A = H * d
    proj = torch.randn(T, 2 * A + R + 3, generator=g)
    ab, w2, w0 = torch.randn(A, generator=g), torch.randn(A, R, generator=g), torch.randn(A, generator=g)
    pd = proj.to(DEV)
    ex = torch.empty(T, 2 * A, device=DEV)
    ops.unit_removal(pd[:, :A], pd[:, A:2 * A], ab.to(DEV), 1e-6, H, d, ex)
    k = proj[:, :A].double().view(T, H, d)
    e = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    c = torch.sigmoid(proj[:, A:2 * A].double() + ab.double()).view(T, H, d) * e
    assert float((ex.cpu().double() - torch.cat([e.reshape(T, A), c.reshape(T, A)], 1)).abs().max()) <= 1e-5
    ww = torch.empty(T, A, device=DEV)
    rate = math.exp(-0.5)
    ops.lowrank_decay(pd[:, 2 * A:2 * A + R], w2.t().contiguous().to(DEV), w0.to(DEV), ww, epilogue=ops.LR_EXPSIG, rate=rate)
    ref = torch.exp(-rate * torch.sigmoid(torch.tanh(proj[:, 2 * A:2 * A + R].double()) @ w2.double().T + w0.double()))
    assert float((ww.cpu().double() - ref).abs().max()) <= 1e-5
    assert float(ww.min()) > math.exp(-rate) - 1e-6 and float(ww.max()) < 1.0


def plain_routed(x, z, corr, up, down, top, groups, keep, scale):
    out = torch.zeros(x.shape[0], down.shape[1], dtype=x.dtype)
    for t in range(x.shape[0]):
        chosen, weights = TP.route(z[t], corr, top, groups, keep, scale)
        for e, w in zip(chosen, weights):
            out[t] += w * (TP.relu2(x[t] @ up[e].T) @ down[e].T)
    return out


@pytest.mark.parametrize("T, W, F, E, top, groups, keep", [(1, 32, 16, 1, 1, 1, 1), (7, 72, 24, 6, 3, 3, 2), (40, 48, 32, 4, 1, 2, 1),
                                                         (130, 128, 64, 8, 4, 4, 3), (9, 37, 11, 12, 4, 4, 2), (33, 64, 40, 64, 6, 8, 3),
                                                         (5, 40, 8, 8, 8, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_without_a_gate_chosen_by_groups_with_a_correction(T, W, F, E, top, groups, keep, dtype):
    """The choice by corrected scores among the kept groups (corrections large enough to change it, some scores
    negative with them), weights from the scores without the correction over their sum, times a constant; experts
    ``down(relu(up x)^2)``.  In bfloat16 the logits are given, so rounding has no choice to make."""
    from prism_b200 import ops
    g = torch.Generator().manual_seed(T * 7 + E)
    x = torch.randn(T, W, generator=g)
    z = torch.randn(T, E, generator=g) * 2.0
    corr = torch.randn(E, generator=g) * (1.0 / E) - 0.3 / E
    up, down = torch.randn(E, F, W, generator=g) / math.sqrt(W), torch.randn(E, W, F, generator=g) / math.sqrt(F)
    if dtype == torch.bfloat16:
        x, up, down = (to_bf16_and_back(t) for t in (x, up, down))
    ref = plain_routed(x.double(), z.double(), corr.double(), up.double(), down.double(), top, groups, keep, 2.5)
    ctx = types.SimpleNamespace(alloc=lambda shape, dt: torch.empty(shape, dtype=dt, device=DEV))
    choice = ops.MoeChoice(corr.to(DEV), groups, keep, 2.5, 1e-20)
    for cores in ((False, True) if dtype == torch.bfloat16 else (False,)):
        ops.moe_tensor_cores = cores
        try:
            y = ops.moe_feed_forward(ctx, x.to(dtype).to(DEV), z.to(DEV), up.to(dtype).to(DEV), down.to(dtype).to(DEV), top, True, True,
                                     False, "relu2", False, choice)
        finally:
            ops.moe_tensor_cores = True
        got = y.sum(0).cpu().double()
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), cores
    ops.check_tc_errors()


def test_small_kernels_of_the_design():
    from prism_b200 import ops
    g = torch.Generator().manual_seed(3)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        gu = torch.randn(6, 2 * 35, generator=g).to(dtype)
        out = torch.empty(6, 35, dtype=dtype, device=DEV)
        ops.glu(gu.to(DEV), out, "gelu_tanh")
        ref = TP.gelu_tanh(gu[:, :35].double()) * gu[:, 35:].double()
        assert float((out.cpu().double() - ref).abs().max()) <= tol * 4
        z, table = torch.randn(5, 7, generator=g), torch.randn(20, 30, generator=g).to(dtype)
        ids = torch.tensor([3, 0, 19, 7, 7], dtype=torch.int32)
        o2 = torch.empty(5, 7, dtype=dtype, device=DEV)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.gather_gate(z.to(DEV), ids.to(DEV), table.to(DEV), 14, o2, "gelu_tanh", err)
        ref = TP.gelu_tanh(z.double()) * table.double()[ids.long()][:, 14:21]
        assert float((o2.cpu().double() - ref).abs().max()) <= tol * 4 and int(err.item()) == 0
        res, d = torch.randn(4, 50, generator=g), torch.randn(3, 4, 50, generator=g)
        rd, copy = res.to(DEV), torch.empty(4, 50, dtype=dtype, device=DEV)
        ops.add_rows(rd, d.to(DEV), copy)
        assert float((rd.cpu() - (res + d.sum(0))).abs().max()) <= 1e-5
        assert float((copy.float().cpu() - (res + d.sum(0))).abs().max()) <= tol * 4
    lg = torch.randn(3, 100, generator=g) * 30
    ld = lg.to(DEV)
    ops.softcap(ld, 15.0)
    assert float((ld.cpu() - 15.0 * torch.tanh(lg / 15.0)).abs().max()) <= 1e-5


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------

def runner_for(folder, dtype, max_tokens, page_size, max_live=4):
    from prism_b200.engine.replay import build_runner
    return build_runner(folder, dtype, max_tokens, page_size, max_live)[3]


def sequences(name):
    vocab = CONFIGS[name][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, 300 + i) for i, n in enumerate(LENGTHS[name[0]])}


def served(name, dtype):
    """The configuration a dtype is tested on: in bfloat16 the variant in which every expert is chosen
    (``tagelorn_helpers.every_expert``)."""
    return name + "x" if dtype == "bfloat16" else name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "small_portions", "mixed"])
def test_cutting(name, dtype, mode):
    """Whole prompts, a decoded tail, portions (one schedule of twos and threes only), and mixed batches of up to four
    live requests in a pool that holds no more than the schedule needs, so that pages and state slots come back and
    are used again."""
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
    """The residual rows after each layer, whole prompt, against the plain model's: a fault shows in the layer that has it."""
    from prism_b200.engine.batch import Segment
    for name in (served("A", dtype), served("B", dtype)):
        raw, seed, ps = CONFIGS[name]
        seq = random_tokens(raw["vocab"], 45, 7)
        wd = {k: v.double() for k, v in draw_weights(raw, seed).items()}
        after, rounded = [], []
        TP.forward(raw, wd, seq, streams=after)
        if dtype == "bfloat16":
            TP.forward(raw, wd, seq, rnd=to_bf16_and_back, streams=rounded)
        else:
            rounded = after
        runner = runner_for(model_folder(name), dtype, 64, ps)
        kept = []

        def watch(block):
            inner = block.forward

            def forward(ctx, residual, delta, cache):
                x, d = inner(ctx, residual, delta, cache)
                kept.append((x + (d.float() if d.dim() == 2 else d.float().sum(0))).cpu())
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
def test_long_decoding_across_pages_and_past_the_window(dtype):
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
    runner = runner_for(model_folder("D"), "float32", 64, 16, max_live=1)
    got = run_trace(runner, trace_portions(seqs, (7, 1, 3)))
    compare("D", seqs, got, LIMIT["float32"])


ONE_LAYER = {
    "attention": [layer("attention", attn(4, 2, 16, 8, scale=0.4, size=11, keep_first=3, bias_rows=8, bias_max=25), None)],
    "attention_without_kept_positions": [layer("attention", attn(3, 1, 32, 32, scale=0.2, size=30, bias_rows=4, bias_max=9), None)],
    "general_delta": [layer("general_delta", delta(4, 24, 6), None)],
    "dense": [layer("general_delta", delta(1, 4, 1), dense(40))],
    "experts": [layer("general_delta", delta(1, 4, 1), moe(20, 6, 2, count=3, keep=2, scale=1.5, shared=12))],
    "experts_without_shared": [layer("general_delta", delta(1, 4, 1), moe(20, 5, 2))],
    "odd_sizes": [layer("attention", attn(2, 1, 7, 5, size=6, keep_first=1, bias_rows=4, bias_max=7), moe(9, 3, 2)),
                  layer("general_delta", delta(3, 5, 2), dense(13))],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(ONE_LAYER))
def test_each_mixer_alone(which, dtype):
    odd = which == "odd_sizes"
    raw = model(51 if odd else 97, 37 if odd else 48, ONE_LAYER[which], taps=2 if odd else 4, side=3 if odd else None,
                softcap=None if odd else 12.0)
    if dtype == "bfloat16":
        raw = every_expert(raw)
    w = draw_weights(raw, 21)
    folder = write_folder(raw, w)
    seq = random_tokens(raw["vocab"], 75, 4)
    ref = TP.forward(raw, {k: v.double() for k, v in w.items()}, seq).float()
    runner = runner_for(folder, dtype, 128, 16)
    got = run_trace(runner, trace_portions({"a": seq}, (20, 1, 1, 30, 2, 1)))
    scale = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
    errs = sorted(float((got[("a", p)] - ref[p] - (got[("a", p)] - ref[p]).mean()).pow(2).mean().sqrt()) / scale for p in range(75))
    assert errs[-1] <= LIMIT[dtype] * (8 if ILL[dtype] else 1) and errs[int(len(errs) * (1 - ILL[dtype])) - 1] <= LIMIT[dtype], errs[-4:]


def test_a_kept_token_far_back_decides_through_attention_alone():
    """A model of one attention layer whose first token differs between two prompts that are otherwise equal and several
    hundred tokens long; the window is far shorter, but the first positions are kept: the logits at the end differ, in a
    whole prompt and when the end is decoded token by token, and each agrees with the plain model.  With the second
    token (not kept) different instead, the ends agree."""
    raw = model(60, 64, [layer("attention", attn(4, 2, 16, 16, scale=0.3, size=50, keep_first=1, bias_rows=8, bias_max=100), None)],
                taps=1)
    w = draw_weights(raw, 5)
    folder = write_folder(raw, w)
    base = random_tokens(60, 390, 6)
    seqs = {"a": [3] + base, "b": [4] + base, "c": [3, 9] + base[1:]}
    wf = {k: v.double() for k, v in w.items()}
    refs = {k: TP.forward(raw, wf, s).float() for k, s in seqs.items()}
    tol = 2e-5 * float(refs["a"].abs().max())
    assert float((refs["a"][-1] - refs["b"][-1]).abs().max()) > 50 * tol
    assert float((refs["a"][-1] - refs["c"][-1]).abs().max()) == 0.0
    for steps in (trace_whole(seqs), trace_tail(seqs, 70)):
        got = run_trace(runner_for(folder, "float32", 1536, 64), steps)
        for rid in seqs:
            for pos in (0, 1, 49, 50, 51, 63, 64, 320, 389, 390):
                assert float((got[(rid, pos)] - refs[rid][pos]).abs().max()) <= tol, (rid, pos)


def test_greedy_generation_through_the_scheduler():
    """Engine.generate (scheduler, batching, sampling, CUDA graphs for the decode steps) picks the plain model's greedy
    tokens; more prompts than request slots, so that state slots are used again."""
    from prism_b200.config.engine_config import EngineConfig, SchedulerConfig
    from prism_b200.engine.llm import Engine
    from prism_b200.sampling.sampler import SamplingParams
    raw, seed, ps = CONFIGS["A"]
    w = {k: v.double() for k, v in draw_weights(raw, seed).items()}
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
                logits = TP.forward(raw, w, seq)[-1]
                top = torch.topk(logits, 2).values
                if float(top[0] - top[1]) > 1e-3:          # a near tie may fall either way
                    assert tok == int(logits.argmax()), (graphs, len(p), len(seq))
                seq.append(tok)
            assert len(r.token_ids) == n_new
        assert eng.cache.pages_in_use() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_replay_program_serves_the_design(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Tagelorn folder: the model class is found by config.json, the distance
    table's rows and the decay's rank by the model file, the pool holds what --max-tokens says and there are four slots."""
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
