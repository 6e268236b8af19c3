"""Prefill and decode throughput of the Dolezen, the Pofazen, the Zuvulorn or the Tagelorn design at layer sizes that resemble real models
(random weights, bf16), beside the Qwen2 architecture at equal width, depth and parameter count (Tagelorn also beside
Zuvulorn, the closest of the other designs: attention with a sink, a delta rule with a decay per key channel, experts), and the
design's own kernels beside the like kernels on the same problem with their fractions of the measured peaks.

    python bench.py --design dolezen|pofazen|zuvulorn|tagelorn [--sizes 2k,4k] [--steps K] [--warmup W]
    python benchmarks/design_bench.py [--design pofazen] [--sizes 2k] [--kernels-only] [--once KERNEL]

One JSON line.  Timing: CUDA events after W >= 3 warm-up runs; every timed step reads all weights (more than
the 126 MB L2) and the kernel timings flush L2 between launches.
"""

import argparse
import json
import os
import sys
import time
import types

import torch

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
sys.path.insert(0, ROOT)

DEV = "cuda:0"
PAGE = 64
# width, feed-forward, heads / kv heads / key size / value size of the chunked layers, and of the latent layers
# heads / plain size / rotated size / value size / query rank / latent rank; mask sizes
SIZES = {
    "2k": dict(width=2048, ff=8192, heads=16, kv_heads=4, dim=128, vdim=128, lat_heads=16, lat_dim=128, rot=64,
               lat_vdim=128, q_rank=768, kv_rank=192, chunk=1024, window=512, layers=8, vocab=32768),
    "4k": dict(width=4096, ff=14336, heads=32, kv_heads=8, dim=128, vdim=128, lat_heads=32, lat_dim=128, rot=64,
               lat_vdim=128, q_rank=1536, kv_rank=192, chunk=1024, window=512, layers=8, vocab=32768),
}


def dolezen_config(s):
    att = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], mask=dict(size=s["chunk"]),
               scale=s["dim"] ** -0.5)
    lat = dict(heads=s["lat_heads"], dim=s["lat_dim"], rot_dim=s["rot"], vdim=s["lat_vdim"], q_rank=s["q_rank"],
               kv_rank=s["kv_rank"], mask=dict(size=s["window"]), rot=dict(base=10000.0, dims=s["rot"]),
               scale=(s["lat_dim"] + s["rot"]) ** -0.5)
    mlp = dict(kind="dense", ff=s["ff"])
    layers = []
    for i in range(s["layers"]):          # own keys, shared keys, latent, own keys, ...
        k = i % 4
        if k == 2:
            layers.append(dict(type="latent_attention", mixer=dict(lat), mlp=mlp))
        elif k == 1:
            layers.append(dict(type="attention", mixer=dict(att, kv_from=i - 1), mlp=mlp))
        else:
            layers.append(dict(type="attention", mixer=dict(att), mlp=mlp))
    return dict(architecture="Dolezen", vocab=s["vocab"], width=s["width"], norm=dict(eps=1e-6),
                embedding=dict(scale=1.0), layers=layers, max_positions=8192)


def pofazen_config(s):
    """Layers: parallel (windowed attention that keeps the first tokens + gated delta rule), wkv, wkv, parallel, ...;
    every layer with a gated feed-forward of Qwen2's size."""
    left = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
                mask=dict(size=s["window"], keep_first=4),
                rot=dict(base=10000.0, dims=s["dim"] // 2, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    right = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], conv=4)
    par = dict(left=left, right=right, left_scale=1.0, right_scale=1.0)
    wkv = dict(heads=s["width"] // 64, dim=64, decay_rank=64)
    mlp = dict(kind="dense", ff=s["ff"] * 2 // 3 // 256 * 256)
    layers = [dict(type="parallel", mixer=par, mlp=mlp) if i % 4 in (0, 3) else dict(type="wkv", mixer=wkv, mlp=mlp)
              for i in range(s["layers"])]
    return dict(architecture="Pofazen", vocab=s["vocab"], width=s["width"], norm=dict(eps=1e-6), postln_alpha=2.0,
                layers=layers, max_positions=8192)


MOE_EXPERTS, MOE_TOP = 8, 2


def zuvulorn_config(s):
    """Layers: attention with keys of its own, attention on the keys of the layer before, delta rule with a decay
    per key channel, real-gated linear recurrence, ...; every layer under hyper-connections with two copies of the
    stream and a mixture of 8 experts (2 per token) whose weights together are Qwen2's feed-forward."""
    att = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
               rot=dict(base=500000.0, dims=s["dim"], scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    cd = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], conv=4, decay_rank=64, gate_rank=64)
    rg = dict(width=s["width"], blocks=s["width"] // 128, conv=4)
    mlp = dict(kind="moe", expert=dict(ff=moe_ff(s)), router=dict(experts=MOE_EXPERTS, top=MOE_TOP))
    layers = []
    for i in range(s["layers"]):
        k = i % 4
        if k == 0:
            layers.append(dict(type="attention", mixer=dict(att), mlp=mlp))
        elif k == 1:
            layers.append(dict(type="attention", mixer=dict(att, kv_from=i - 1), mlp=mlp))
        elif k == 2:
            layers.append(dict(type="channel_delta", mixer=cd, mlp=mlp))
        else:
            layers.append(dict(type="rglru", mixer=rg, mlp=mlp))
    return dict(architecture="Zuvulorn", vocab=s["vocab"], width=s["width"], norm=dict(eps=1e-6), streams=2, layers=layers,
                max_positions=8192)


def moe_ff(s):
    return s["ff"] * 2 // 3 // 256 * 256 // MOE_EXPERTS // 32 * 32


def qwen2_config(s):
    # the same width, depth and head shape; a gated feed-forward has three matrices where the dense one has two
    return dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", num_hidden_layers=s["layers"],
                hidden_size=s["width"], num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"],
                head_dim=s["dim"], intermediate_size=s["ff"] * 2 // 3 // 256 * 256, vocab_size=s["vocab"],
                rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=8192,
                use_sliding_window=False)


def timeit(fn, reps=10, flush=True, warmup=3):
    junk = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        if flush:
            junk.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps       # ms


def engine_numbers(raw, prompt_len, batch, steps, warmup):
    """Prefill tokens/s (one prompt of ``prompt_len`` tokens a step) and decode tokens/s (``batch`` requests
    behind ``prompt_len`` tokens each, CUDA graphs) through the engine's step function."""
    from prism_b200 import Engine, EngineConfig, SchedulerConfig, ops
    from prism_b200.engine.batch import Segment
    ctx_len = prompt_len + steps + warmup + 8
    pages = (ctx_len + PAGE - 1) // PAGE
    ec = EngineConfig(kv_page_size=PAGE, num_pages=(batch + 1) * pages + 8, max_seq_len=pages * PAGE, use_cuda_graph=True,
                      graph_batch_sizes=(batch,),
                      scheduler=SchedulerConfig(max_batch_tokens=prompt_len, max_num_seqs=batch + 1, prefill_chunk=prompt_len))
    eng = Engine(None, ec, dtype="bfloat16", config=raw, random_seed=0)
    runner = eng.runner
    g = torch.Generator().manual_seed(1)
    V = eng.model.spec.vocab_size
    prompt = lambda: torch.randint(0, V, (prompt_len,), generator=g).tolist()
    n = [0]

    def prefill_once():
        rid = f"p{n[0]}"
        n[0] += 1
        runner.begin_request(rid)
        runner.step([Segment(rid, prompt(), [prompt_len - 1])])
        runner.end_request(rid)
    l0 = ops.launch_count
    pre_ms = timeit(prefill_once, reps=max(3, min(steps, 8)), flush=False, warmup=max(3, warmup))
    ids = [f"d{i}" for i in range(batch)]
    for rid in ids:
        runner.begin_request(rid)
        runner.step([Segment(rid, prompt(), [])])
    out = torch.empty(batch, dtype=torch.int32, device=DEV)

    def decode_once():
        logits = runner.step([Segment(rid, [1], [0]) for rid in ids])
        ops.sample(logits, None, None, out)
    for _ in range(max(3, warmup)):
        decode_once()
    torch.cuda.synchronize()
    g0 = runner.graph_kernel_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        decode_once()
    e1.record()
    torch.cuda.synchronize()
    dec_ms = e0.elapsed_time(e1) / steps
    runner.check_errors()
    res = dict(prefill_tokens_per_s=round(prompt_len / pre_ms * 1e3), prefill_ms=round(pre_ms, 3),
               decode_tokens_per_s=round(batch / dec_ms * 1e3), decode_ms_per_step=round(dec_ms, 4),
               weights_gb=round(eng.pool.total_gb, 3), launches_per_decode_step=(runner.graph_kernel_launches - g0) // steps,
               launches=ops.launch_count - l0 + runner.graph_kernel_launches - g0)
    del eng, runner
    torch.cuda.empty_cache()
    return res


def paged(batch, ctx, q_len, nkv, dk, dv, values_in_keys=False):
    pages_per = (ctx + q_len + PAGE - 1) // PAGE
    n_pages = batch * pages_per + 1
    kc = torch.randn(n_pages, PAGE, nkv, dk, device=DEV, dtype=torch.bfloat16)
    vc = kc[..., :dv] if values_in_keys else torch.randn(n_pages, PAGE, nkv, dv, device=DEV, dtype=torch.bfloat16)
    bt = torch.arange(batch * pages_per, dtype=torch.int32, device=DEV).view(batch, pages_per)
    i32 = lambda x: x.to(torch.int32).to(DEV)
    ctx_ns = types.SimpleNamespace(
        positions=i32(torch.cat([torch.arange(ctx, ctx + q_len) for _ in range(batch)])),
        tok_seg=i32(torch.arange(batch).repeat_interleave(q_len)), seg_start=i32(torch.arange(batch + 1) * q_len),
        cached_len=torch.full((batch,), ctx, dtype=torch.int32, device=DEV), S=batch, max_q_len=q_len,
        max_kv_len=ctx + q_len,
        decode_only=q_len == 1, err=torch.zeros(1, dtype=torch.int32, device=DEV))
    return ctx_ns, kc, vc, bt, n_pages


def visible_pairs(T0, n, mask):
    return sum(p - mask.first_key(p) + 1 for p in range(T0, T0 + n))


def kernel_numbers(s, pk, once=None):
    """The attention kernels alone: Dolezen's chunked and latent layers against Qwen2's causal layer of the same
    head shape, prefill of 2,048 tokens and a decode step of 8 and 64 requests behind 2,047 tokens."""
    from prism_b200 import ops
    out = {}
    T = 2048
    cases = [("chunked_sink", s["heads"], s["kv_heads"], s["dim"], s["vdim"], False, ops.KeyMask.chunk(s["chunk"]), True),
             ("latent", s["lat_heads"], 1, s["kv_rank"] + s["rot"], s["kv_rank"], True, ops.KeyMask.window(s["window"]), False)]
    for name, nh, nkv, dk, dv, vin, mask, sink in cases:
        sk = torch.randn(nh, device=DEV) if sink else None
        for label, batch, cached, q_len in (("prefill_2048", 1, 0, T), ("decode_b8", 8, T - 1, 1), ("decode_b64", 64, T - 1, 1)):
            if once and once != f"{name}_{label}":
                continue
            c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, dk, dv, vin)
            q = torch.randn(batch * q_len, nh, dk, device=DEV, dtype=torch.bfloat16)
            o = torch.empty(batch * q_len, nh * dv, device=DEV, dtype=torch.bfloat16)
            fn = lambda: ops.masked_attention(c, q, o, kc, vc, bt, npages, mask, dk ** -0.5, sk)
            if once:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                return {}
            ms = timeit(fn)
            pairs = batch * visible_pairs(cached, q_len, mask)
            flops = 2 * pairs * nh * (dk + dv)
            keys = batch * min(cached + q_len, mask.size or cached + q_len) if q_len == 1 else batch * (cached + q_len)
            nbytes = 2 * (keys * nkv * (dk + (0 if vin else dv)) + 2 * batch * q_len * nh * (dk + dv) // 2)
            out[f"{name}_{label}"] = dict(us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 1),
                                          frac_bf16_peak_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4),
                                          gbs=round(nbytes / ms / 1e6, 1),
                                          frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    # the closest model's kernels on its causal layer of the same head shape
    nh, nkv, hd = s["heads"], s["kv_heads"], s["dim"]
    for label, batch, cached, q_len in (("prefill_2048", 1, 0, T), ("decode_b8", 8, T - 1, 1), ("decode_b64", 64, T - 1, 1)):
        if once:
            continue
        c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, hd, hd)
        q = torch.randn(batch * q_len, nh, hd, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(batch * q_len, nh * hd, device=DEV, dtype=torch.bfloat16)
        causal = ops.KeyMask.causal()
        if q_len == 1:
            ns = ops.decode_splits(batch, nkv, cached + 1, None)
            po = torch.empty(batch, nh, ns, hd, device=DEV)
            pml = torch.empty(batch, nh, ns, 2, device=DEV)
            fn = lambda: ops.attention_decode_bf16(q, o, kc, vc, bt, c.positions, c.tok_seg, npages, None, hd ** -0.5, ns,
                                                   po, pml, c.err)
            variants = [("qwen2_causal", fn)]
        else:
            variants = [("qwen2_causal_tcgen05", lambda: ops.attention_prefill_tc(q, o, kc, vc, bt, c.seg_start, c.cached_len, q_len,
                                                                                  npages, None, hd ** -0.5, c.err)),
                        ("qwen2_causal_mma_sync", lambda: ops.attention_prefill_bf16(q, o, kc, vc, bt, c.seg_start, c.cached_len,
                                                                                     q_len, npages, None, hd ** -0.5, c.err))]
        for vname, fn in variants:
            ms = timeit(fn)
            pairs = batch * visible_pairs(cached, q_len, causal)
            flops = 4 * pairs * nh * hd
            nbytes = 2 * (batch * (cached + q_len) * nkv * 2 * hd + 2 * batch * q_len * nh * hd)
            out[f"{vname}_{label}"] = dict(us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 1),
                                           frac_bf16_peak_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4),
                                           gbs=round(nbytes / ms / 1e6, 1),
                                           frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
    return out


def _rates(ms, flops, nbytes, pk):
    return dict(us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 2),
                frac_bf16_peak_of_measured=round(flops / ms / 1e9 / pk["bf16_tflops"], 4), gbs=round(nbytes / ms / 1e6, 1),
                frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))


def pofazen_kernel_numbers(s, pk, once=None):
    """The design's kernels alone: attention under a window that keeps the first tokens against Qwen2's
    kernels under the same window (same head shape), and the two recurrent scans (prefill of 2,048 tokens: float32
    FMA work, one token after another; decode: the float32 state read and written once a step)."""
    from prism_b200 import ops
    out = {}
    T = 2048
    nh, nkv, dk, dv, win = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"]
    mask = ops.KeyMask.window(win, 4)
    shapes = (("prefill_2048", 1, 0, T), ("decode_b8", 8, T - 1, 1), ("decode_b64", 64, T - 1, 1))
    for label, batch, cached, q_len in shapes:
        name = f"window_keep_{label}"
        if once and once != name:
            continue
        c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, dk, dv)
        q = torch.randn(batch * q_len, nh, dk, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(batch * q_len, nh * dv, device=DEV, dtype=torch.bfloat16)
        fn = lambda: ops.masked_attention(c, q, o, kc, vc, bt, npages, mask, dk ** -0.5, None)
        if once:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            return {}
        ms = timeit(fn)
        pairs = batch * sum(min(p + 1, win) + min(4, max(0, p + 1 - win)) for p in range(cached, cached + q_len))
        keys = batch * (min(cached + q_len, win + 4) if q_len == 1 else cached + q_len)
        out[name] = _rates(ms, 2 * pairs * nh * (dk + dv), 2 * (keys * nkv * (dk + dv) + batch * q_len * nh * (dk + dv)), pk)
    for label, batch, cached, q_len in shapes:          # the closest model's kernels under the same window, no kept tokens
        if once:
            break
        c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, dk, dk)
        q = torch.randn(batch * q_len, nh, dk, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(batch * q_len, nh * dk, device=DEV, dtype=torch.bfloat16)
        if q_len == 1:
            ns = ops.decode_splits(batch, nkv, cached + 1, win)
            po = torch.empty(batch, nh, ns, dk, device=DEV)
            pml = torch.empty(batch, nh, ns, 2, device=DEV)
            variants = [("qwen2_window", lambda: ops.attention_decode_bf16(q, o, kc, vc, bt, c.positions, c.tok_seg, npages, win,
                                                                           dk ** -0.5, ns, po, pml, c.err))]
        else:
            variants = [("qwen2_window_tcgen05", lambda: ops.attention_prefill_tc(q, o, kc, vc, bt, c.seg_start, c.cached_len, q_len,
                                                                                  npages, win, dk ** -0.5, c.err)),
                        ("qwen2_window_mma_sync", lambda: ops.attention_prefill_bf16(q, o, kc, vc, bt, c.seg_start, c.cached_len,
                                                                                     q_len, npages, win, dk ** -0.5, c.err))]
        for vname, fn in variants:
            ms = timeit(fn)
            pairs = batch * sum(min(p + 1, win) for p in range(cached, cached + q_len))
            keys = batch * (min(cached + q_len, win) if q_len == 1 else cached + q_len)
            out[f"{vname}_{label}"] = _rates(ms, 4 * pairs * nh * dk, 2 * (keys * nkv * 2 * dk + 2 * batch * q_len * nh * dk), pk)
    # the recurrent scans
    wh, wd = s["width"] // 64, 64
    for sname, mode, H, rep, kd, vd in (("delta_scan", ops.SCAN_DELTA, nh, nh // nkv, dk, dv), ("bonus_scan", ops.SCAN_BONUS, wh, 1, wd, wd)):
        for label, batch, cached, q_len in shapes:
            name = f"{sname}_{label}"
            if once and once != name:
                continue
            Tt = batch * q_len
            G = H // rep
            c = types.SimpleNamespace(seg_start=(torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV),
                                      state_slots=torch.arange(batch, dtype=torch.int32, device=DEV), S=batch)
            state = torch.zeros(batch + 1, H, vd, kd, device=DEV)
            o = torch.empty(Tt, H, vd, device=DEV)
            if mode == ops.SCAN_DELTA:
                x = torch.nn.functional.normalize(torch.randn(Tt, 2 * G + H, kd, device=DEV), dim=-1).view(Tt, -1)
                bg = torch.rand(Tt, 2 * H, device=DEV) * 0.5 + 0.5
                fn = lambda: ops.recurrent_scan(mode, x[:, :G * kd], x[:, G * kd:2 * G * kd], x[:, 2 * G * kd:], state, c, H, rep, kd,
                                                vd, o, bg=bg)
            else:
                x = torch.randn(Tt, 3 * H * kd, device=DEV) * 0.1
                ww = torch.randn(Tt, H * kd, device=DEV)
                w0, u = torch.zeros(H * kd, device=DEV), torch.randn(H * kd, device=DEV) * 0.1
                ready = q_len > 1                   # as the mixer does: a step of many tokens forms the decay beforehand
                if ready:
                    ops.decay_from_exponent(ww, w0)
                fn = lambda: ops.recurrent_scan(mode, x[:, :H * kd], x[:, H * kd:2 * H * kd], x[:, 2 * H * kd:], state, c, H, 1, kd,
                                                vd, o, ww=ww, w0=w0, u=u, decay_ready=ready)
            if once:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                return {}
            ms = timeit(fn)
            flops = 6 * Tt * H * kd * vd                    # three multiply-adds per state entry and token
            nbytes = 4 * (2 * batch * H * kd * vd + Tt * H * (2 * kd + 2 * vd))
            out[name] = dict(us=round(ms * 1e3, 1), fp32_tflops=round(flops / ms / 1e9, 2), gbs=round(nbytes / ms / 1e6, 1),
                             frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4),
                             us_per_token=round(ms * 1e3 / q_len, 3))
    return out


def zuvulorn_kernel_numbers(s, pk, once=None):
    """The design's kernels alone, each beside the like kernel of the closest model on the same problem: causal
    attention with one added to the denominator beside Qwen2's causal kernels; the delta rule with a decay per
    key channel beside the delta rule with one decay per head; the real-gated recurrence with its gates; the
    experts' grouped products beside Qwen2's dense feed-forward of the same total weight; the norm that also
    updates and reads the copies of the stream beside the plain add + norm."""
    from prism_b200 import ops
    out = {}
    T = 2048
    nh, nkv, dk, dv, W = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["width"]
    shapes = (("prefill_2048", 1, 0, T), ("decode_b8", 8, T - 1, 1), ("decode_b64", 64, T - 1, 1))
    causal = ops.KeyMask.causal()

    def run(name, fn, flops, nbytes, fp32=False):
        if once:
            if once == name:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
            return
        ms = timeit(fn)
        if fp32:
            out[name] = dict(us=round(ms * 1e3, 1), fp32_tflops=round(flops / ms / 1e9, 2), gbs=round(nbytes / ms / 1e6, 1),
                             frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
        else:
            out[name] = _rates(ms, flops, nbytes, pk)

    sink = torch.zeros(nh, device=DEV)
    for label, batch, cached, q_len in shapes:
        c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, dk, dv)
        q = torch.randn(batch * q_len, nh, dk, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(batch * q_len, nh * dv, device=DEV, dtype=torch.bfloat16)
        pairs = batch * visible_pairs(cached, q_len, causal)
        flops = 2 * pairs * nh * (dk + dv)
        nbytes = 2 * (batch * (cached + q_len) * nkv * (dk + dv) + batch * q_len * nh * (dk + dv))
        run(f"sink_causal_{label}", lambda: ops.masked_attention(c, q, o, kc, vc, bt, npages, causal, dk ** -0.5, sink), flops, nbytes)
        if q_len == 1:
            ns = ops.decode_splits(batch, nkv, cached + 1, None)
            po = torch.empty(batch, nh, ns, dk, device=DEV)
            pml = torch.empty(batch, nh, ns, 2, device=DEV)
            run(f"qwen2_causal_{label}", lambda: ops.attention_decode_bf16(q, o, kc, vc, bt, c.positions, c.tok_seg, npages, None,
                                                                           dk ** -0.5, ns, po, pml, c.err), flops, nbytes)
        else:
            run(f"qwen2_causal_tcgen05_{label}", lambda: ops.attention_prefill_tc(q, o, kc, vc, bt, c.seg_start, c.cached_len, q_len,
                                                                                  npages, None, dk ** -0.5, c.err), flops, nbytes)
            run(f"qwen2_causal_mma_sync_{label}", lambda: ops.attention_prefill_bf16(q, o, kc, vc, bt, c.seg_start, c.cached_len,
                                                                                     q_len, npages, None, dk ** -0.5, c.err), flops, nbytes)
    # the matrix-state scans: a decay per key channel (this design) beside one per head (the like kernel)
    H, rep, G = nh, nh // nkv, nkv
    for label, batch, cached, q_len in shapes:
        Tt = batch * q_len
        c = types.SimpleNamespace(seg_start=(torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV),
                                  state_slots=torch.arange(batch, dtype=torch.int32, device=DEV), S=batch, max_q_len=q_len)
        state = torch.zeros(batch + 1, H, dv, dk, device=DEV)
        o = torch.empty(Tt, H, dv, device=DEV)
        x = torch.nn.functional.normalize(torch.randn(Tt, 2 * G + H, dk, device=DEV), dim=-1).view(Tt, -1)
        beta = torch.rand(Tt, H, device=DEV)
        bg = torch.rand(Tt, 2 * H, device=DEV) * 0.5 + 0.5
        ww = torch.rand(Tt, H * dk, device=DEV) * 0.5 + 0.5
        flops = 6 * Tt * H * dk * dv
        nbytes = 4 * (2 * batch * H * dk * dv + Tt * H * (2 * dk + 2 * dv))
        run(f"channel_scan_{label}", lambda: ops.recurrent_scan(ops.SCAN_CHANNEL, x[:, :G * dk], x[:, G * dk:2 * G * dk], x[:, 2 * G * dk:],
                                                                state, c, H, rep, dk, dv, o, bg=beta, ww=ww), flops, nbytes, fp32=True)
        run(f"delta_scan_{label}", lambda: ops.recurrent_scan(ops.SCAN_DELTA, x[:, :G * dk], x[:, G * dk:2 * G * dk], x[:, 2 * G * dk:],
                                                              state, c, H, rep, dk, dv, o, bg=bg), flops, nbytes, fp32=True)
    # the real-gated recurrence: gates (two block-diagonal products, float32) and the scan per channel
    actx = types.SimpleNamespace(alloc=lambda shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
    C, nb = W, W // 128
    bs = C // nb
    wr, wi = (torch.randn(nb, bs, bs, device=DEV, dtype=torch.bfloat16) / bs ** 0.5 for _ in range(2))
    br, bi, lam = (torch.zeros(nb, bs, device=DEV, dtype=torch.bfloat16) for _ in range(2)) , None, torch.zeros(C, device=DEV, dtype=torch.bfloat16)
    br, bi = br
    for label, batch, cached, q_len in shapes:
        Tt = batch * q_len
        c = types.SimpleNamespace(seg_start=(torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV),
                                  state_slots=torch.arange(batch, dtype=torch.int32, device=DEV), S=batch, max_q_len=q_len,
                                  alloc=actx.alloc)
        u, y = torch.randn(Tt, C, device=DEV), torch.randn(Tt, C, device=DEV)
        ag = torch.empty(2, Tt, C, device=DEV)
        st = torch.zeros(batch + 1, C, device=DEV)
        o = torch.empty(Tt, C, device=DEV, dtype=torch.bfloat16)
        run(f"block_gates_{label}", lambda: ops.block_gates(u, wr, wi, br, bi, lam, 8.0, ag[0], ag[1]), 4 * Tt * C * bs,
            4 * 3 * Tt * C + 2 * 2 * nb * bs * bs, fp32=True)
        run(f"rglru_scan_{label}", lambda: ops.rglru_scan(ag[0], ag[1], y, st, c, o), 3 * Tt * C, 4 * 3 * Tt * C + 2 * Tt * C + 8 * batch * C,
            fp32=True)
    # the experts beside the dense feed-forward of the same total weight
    E, top, F = MOE_EXPERTS, MOE_TOP, moe_ff(s)
    Fd = s["ff"] * 2 // 3 // 256 * 256
    gu = torch.randn(E, 2 * F, W, device=DEV, dtype=torch.bfloat16) / W ** 0.5
    dn = torch.randn(E, W, F, device=DEV, dtype=torch.bfloat16) / F ** 0.5
    gud = torch.randn(2 * Fd, W, device=DEV, dtype=torch.bfloat16) / W ** 0.5
    dnd = torch.randn(W, Fd, device=DEV, dtype=torch.bfloat16) / Fd ** 0.5
    actx = types.SimpleNamespace(alloc=lambda shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
    for label, Tt in (("prefill_2048", T), ("decode_b8", 8), ("decode_b64", 64)):
        xx = torch.randn(Tt, W, device=DEV, dtype=torch.bfloat16)
        logits = torch.randn(Tt, E, device=DEV)
        used = min(E, Tt * top)
        run(f"experts_{label}", lambda: ops.moe_feed_forward(actx, xx, logits, gu, dn, top), 6 * Tt * top * F * W,
            2 * (3 * used * F * W + Tt * W * (1 + 2 * top)))
        run(f"qwen2_feed_forward_{label}", lambda: ops.feed_forward_swiglu(actx, xx, gud, dnd), 6 * Tt * Fd * W,
            2 * (3 * Fd * W + 3 * Tt * W))
    # the norm that carries out the stream update and the read-in, beside add + norm on one stream
    wn = torch.ones(W, device=DEV)
    for label, Tt in (("prefill_2048", T), ("decode_b64", 64)):
        xs = torch.randn(2, Tt, W, device=DEV)
        d = torch.randn(Tt, W, device=DEV)
        mix, ow, iw = torch.eye(2, device=DEV), torch.ones(2, device=DEV), torch.ones(2, device=DEV)
        h = torch.empty(Tt, W, device=DEV, dtype=torch.bfloat16)
        run(f"hyper_norm_{label}", lambda: ops.hyper_norm(xs, 2, xs, d, mix, ow, iw, wn, 1e-6, h), 0, 4 * Tt * W * 5 + 2 * Tt * W, fp32=True)
        x1 = torch.randn(Tt, W, device=DEV)
        run(f"qwen2_add_norm_{label}", lambda: ops.add_rmsnorm(x1, d, wn, 1e-6, h), 0, 4 * Tt * W * 3 + 2 * Tt * W, fp32=True)
    return out


TAGELORN_BIAS_ROWS, TAGELORN_BIAS_FAR, TAGELORN_SIDE = 32, 2048, 64


def tagelorn_ff(s):
    """Inner width of a Tagelorn expert (two matrices each): eight routed experts and the shared one together weigh what
    Qwen2's gated feed-forward of three matrices does."""
    return s["ff"] * 2 // 3 // 256 * 256 * 3 // 2 // (MOE_EXPERTS + 1) // 32 * 32


def tagelorn_config(s):
    """Layers: windowed attention (keeps the first four positions, bias by distance, sink), generalized delta rule, ...;
    every layer behind an input convolution of four taps and followed by a token input; the first layer's feed-forward
    dense, the others 8 experts in 4 groups (2 groups kept, 2 experts a token) and a shared one."""
    att = dict(heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], vdim=s["vdim"], scale=s["dim"] ** -0.5,
               mask=dict(size=s["window"], keep_first=4), bias_max=TAGELORN_BIAS_FAR, bias_rows=TAGELORN_BIAS_ROWS)
    gd = dict(heads=s["heads"], dim=s["dim"], decay_rank=64)
    F = tagelorn_ff(s)
    routed = dict(kind="moe", expert=dict(ff=F), shared=dict(ff=F),
                  router=dict(experts=MOE_EXPERTS, top=MOE_TOP, scale=2.5, groups=dict(count=4, keep=2)))
    layers = []
    for i in range(s["layers"]):
        mlp = dict(kind="dense", ff=s["ff"] * 2 // 3 // 256 * 256) if i == 0 else routed
        layers.append(dict(type="attention" if i % 2 == 0 else "general_delta", mixer=dict(att if i % 2 == 0 else gd), mlp=mlp))
    return dict(architecture="Tagelorn", vocab=s["vocab"], width=s["width"], norm=dict(eps=1e-6), canon=dict(taps=4),
                embedding=dict(scale=1.0), token_side=dict(dim=TAGELORN_SIDE), logit_softcap=30.0, layers=layers,
                max_positions=8192)


def tagelorn_kernel_numbers(s, pk, once=None):
    """The design's kernels alone, each beside the like kernel of the closest model on the same problem: attention
    under a window with kept positions, a sink and the bias by distance beside the same kernel without the bias (and
    Qwen2's kernels under the window); the generalized delta rule beside the delta rule with a decay per key channel;
    the experts without a gate, routed by groups, beside gated experts of the same total weight; the input
    convolution beside the skip path, the sinusoid embedding, and the token input's small kernels by their bytes."""
    from prism_b200 import ops
    from prism_b200.parts.attention import distance_bucket
    out = {}
    T = 2048
    nh, nkv, dk, dv, W, win = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["width"], s["window"]
    shapes = (("prefill_2048", 1, 0, T), ("decode_b8", 8, T - 1, 1), ("decode_b64", 64, T - 1, 1))
    mask = ops.KeyMask.window(win, 4)

    def run(name, fn, flops, nbytes, fp32=False):
        if once:
            if once == name:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
            return
        ms = timeit(fn)
        if fp32:
            out[name] = dict(us=round(ms * 1e3, 1), fp32_tflops=round(flops / ms / 1e9, 2), gbs=round(nbytes / ms / 1e6, 1),
                             frac_hbm_of_measured=round(nbytes / ms / 1e6 / pk["hbm_gbs"], 4))
        else:
            out[name] = _rates(ms, flops, nbytes, pk)

    sink = torch.randn(nh, device=DEV)
    rel = torch.randn(TAGELORN_BIAS_ROWS, nh)
    idx = torch.tensor([distance_bucket(n, TAGELORN_BIAS_ROWS, TAGELORN_BIAS_FAR) for n in range(TAGELORN_BIAS_FAR + 1)])
    table = rel[idx].t().contiguous().to(DEV)
    for label, batch, cached, q_len in shapes:
        c, kc, vc, bt, npages = paged(batch, cached, q_len, nkv, dk, dv)
        q = torch.randn(batch * q_len, nh, dk, device=DEV, dtype=torch.bfloat16)
        o = torch.empty(batch * q_len, nh * dv, device=DEV, dtype=torch.bfloat16)
        pairs = batch * sum(min(p + 1, win) + min(4, max(0, p + 1 - win)) for p in range(cached, cached + q_len))
        keys = batch * (min(cached + q_len, win + 4) if q_len == 1 else cached + q_len)
        flops, nbytes = 2 * pairs * nh * (dk + dv), 2 * (keys * nkv * (dk + dv) + batch * q_len * nh * (dk + dv))
        run(f"biased_window_{label}", lambda: ops.masked_attention(c, q, o, kc, vc, bt, npages, mask, dk ** -0.5, sink, table), flops, nbytes)
        run(f"like_window_sink_{label}", lambda: ops.masked_attention(c, q, o, kc, vc, bt, npages, mask, dk ** -0.5, sink), flops, nbytes)
        if q_len == 1:
            ns = ops.decode_splits(batch, nkv, cached + 1, win)
            po = torch.empty(batch, nh, ns, dk, device=DEV)
            pml = torch.empty(batch, nh, ns, 2, device=DEV)
            run(f"qwen2_window_{label}", lambda: ops.attention_decode_bf16(q, o, kc, vc, bt, c.positions, c.tok_seg, npages, win,
                                                                           dk ** -0.5, ns, po, pml, c.err), flops, nbytes)
        else:
            run(f"qwen2_window_tcgen05_{label}", lambda: ops.attention_prefill_tc(q, o, kc, vc, bt, c.seg_start, c.cached_len, q_len,
                                                                                  npages, win, dk ** -0.5, c.err), flops, nbytes)
            run(f"qwen2_window_mma_sync_{label}", lambda: ops.attention_prefill_bf16(q, o, kc, vc, bt, c.seg_start, c.cached_len,
                                                                                     q_len, npages, win, dk ** -0.5, c.err), flops, nbytes)
    # the matrix-state scans: decay and removal per key channel (this design) beside a decay per key channel (the like kernel)
    H = nh
    for label, batch, cached, q_len in shapes:
        Tt = batch * q_len
        c = types.SimpleNamespace(seg_start=(torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV),
                                  state_slots=torch.arange(batch, dtype=torch.int32, device=DEV), S=batch, max_q_len=q_len)
        state = torch.zeros(batch + 1, H, dv, dk, device=DEV)
        o = torch.empty(Tt, H, dv, device=DEV)
        x = torch.nn.functional.normalize(torch.randn(Tt, 3 * H, dk, device=DEV), dim=-1).view(Tt, -1)
        ww = torch.rand(Tt, H * dk, device=DEV) * 0.4 + 0.6
        ex = torch.cat([x[:, H * dk:2 * H * dk], x[:, H * dk:2 * H * dk] * 0.5], 1).contiguous()
        beta = torch.rand(Tt, H, device=DEV)
        flops = 6 * Tt * H * dk * dv
        run(f"general_scan_{label}", lambda: ops.recurrent_scan(ops.SCAN_GENERAL, x[:, :H * dk], x[:, H * dk:2 * H * dk], x[:, 2 * H * dk:],
                                                                state, c, H, 1, dk, dv, o, ww=ww, ex=ex), flops,
            4 * (2 * batch * H * dk * dv + Tt * H * (5 * dk + 2 * dv)), fp32=True)
        run(f"like_channel_scan_{label}", lambda: ops.recurrent_scan(ops.SCAN_CHANNEL, x[:, :H * dk], x[:, H * dk:2 * H * dk], x[:, 2 * H * dk:],
                                                                     state, c, H, 1, dk, dv, o, bg=beta, ww=ww), flops,
            4 * (2 * batch * H * dk * dv + Tt * H * (3 * dk + 2 * dv)), fp32=True)
    # experts without a gate, routed by groups, beside gated experts of the same total weight (the like kernels) and the dense layer
    E, top, F, Fz = MOE_EXPERTS, MOE_TOP, tagelorn_ff(s) * (MOE_EXPERTS + 1) // MOE_EXPERTS // 32 * 32, moe_ff(s)
    Fd = s["ff"] * 2 // 3 // 256 * 256
    up = torch.randn(E, F, W, device=DEV, dtype=torch.bfloat16) / W ** 0.5
    dn = torch.randn(E, W, F, device=DEV, dtype=torch.bfloat16) / F ** 0.5
    guz = torch.randn(E, 2 * Fz, W, device=DEV, dtype=torch.bfloat16) / W ** 0.5
    dnz = torch.randn(E, W, Fz, device=DEV, dtype=torch.bfloat16) / Fz ** 0.5
    gud = torch.randn(2 * Fd, W, device=DEV, dtype=torch.bfloat16) / W ** 0.5
    dnd = torch.randn(W, Fd, device=DEV, dtype=torch.bfloat16) / Fd ** 0.5
    actx = types.SimpleNamespace(alloc=lambda shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
    choice = ops.MoeChoice(torch.randn(E, device=DEV) * 0.05, 4, 2, 2.5, 1e-20)
    for label, Tt in (("prefill_2048", T), ("decode_b8", 8), ("decode_b64", 64)):
        xx = torch.randn(Tt, W, device=DEV, dtype=torch.bfloat16)
        logits = torch.randn(Tt, E, device=DEV)
        used = min(E, Tt * top)
        run(f"grouped_experts_{label}", lambda: ops.moe_feed_forward(actx, xx, logits, up, dn, top, True, True, False, "relu2", False, choice),
            4 * Tt * top * F * W, 2 * (2 * used * F * W + Tt * W * (1 + 2 * top)))
        run(f"like_gated_experts_{label}", lambda: ops.moe_feed_forward(actx, xx, logits, guz, dnz, top), 6 * Tt * top * Fz * W,
            2 * (3 * used * Fz * W + Tt * W * (1 + 2 * top)))
        run(f"gelu_feed_forward_{label}", lambda: ops.feed_forward_glu(actx, xx, gud, dnd, "gelu_tanh"), 6 * Tt * Fd * W,
            2 * (3 * Fd * W + 3 * Tt * W))
        run(f"qwen2_feed_forward_{label}", lambda: ops.feed_forward_swiglu(actx, xx, gud, dnd), 6 * Tt * Fd * W,
            2 * (3 * Fd * W + 3 * Tt * W))
    # the input convolution beside the skip path (float32 normed rows in, compute dtype out), beside add + norm on the same rows
    taps = torch.randn(W, 4, device=DEV, dtype=torch.bfloat16)
    wn = torch.ones(W, device=DEV)
    for label, batch, q_len in (("prefill_2048", 1, T), ("decode_b64", 64, 1)):
        Tt = batch * q_len
        c = types.SimpleNamespace(seg_start=(torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV),
                                  tok_seg=torch.arange(batch, dtype=torch.int32).repeat_interleave(q_len).to(DEV),
                                  state_slots=torch.arange(batch, dtype=torch.int32, device=DEV), S=batch, max_q_len=q_len)
        h32 = torch.randn(Tt, W, device=DEV)
        tail = torch.zeros(batch + 1, 3, W, device=DEV)
        h = torch.empty(Tt, W, device=DEV, dtype=torch.bfloat16)
        taps_t = taps.float().t().contiguous()
        run(f"input_conv_{label}", lambda: ops.causal_conv(h32, taps, None, tail, c, h, move_tail=q_len == 1, add_input=True, taps_t=taps_t), 0,
            4 * Tt * W + 2 * Tt * W + (8 * 3 * batch * W if q_len == 1 else 0), fp32=True)
        d = torch.randn(Tt, W, device=DEV)
        x1 = torch.randn(Tt, W, device=DEV)
        run(f"qwen2_add_norm_{label}", lambda: ops.add_rmsnorm(x1, d, wn, 1e-6, h), 0, 4 * Tt * W * 3 + 2 * Tt * W, fp32=True)
    return out


DESIGNS = {"dolezen": (dolezen_config, kernel_numbers), "pofazen": (pofazen_config, pofazen_kernel_numbers),
           "zuvulorn": (zuvulorn_config, zuvulorn_kernel_numbers), "tagelorn": (tagelorn_config, tagelorn_kernel_numbers)}
# designs measured beside another design as well as beside Qwen2: the closest of the models that ran before
BESIDE = {"tagelorn": ("zuvulorn", zuvulorn_config)}


def run(sizes, steps, warmup, prompt_len=2048, batch=8, kernels_only=False, once=None, peaks=None, design="dolezen"):
    pk = peaks or dict(hbm_gbs=6650.0, bf16_tflops=1590.0)
    make_config, design_kernels = DESIGNS[design]
    result = dict(metric=f"prefill and decode tokens/s, {design.capitalize()} beside Qwen2 at equal size", unit="tokens/s", n_gpus=1,
                  steps=steps, warmup=warmup, dtype="bf16", data="synthetic (random weights, random token ids)",
                  peaks=pk, sizes={})
    launches = 0
    for name in sizes:
        s = SIZES[name]
        entry = dict(shape=s)
        if not kernels_only and not once:
            models = [(design, make_config(s)), ("qwen2", qwen2_config(s))]
            if design in BESIDE:
                models.append((BESIDE[design][0], BESIDE[design][1](s)))
            for label, raw in models:
                entry[label] = engine_numbers(raw, prompt_len, batch, steps, warmup)
                launches += entry[label].pop("launches")
            if design in BESIDE:
                other = BESIDE[design][0]
                entry[f"{design}_over_{other}"] = dict(
                    prefill=round(entry[design]["prefill_tokens_per_s"] / entry[other]["prefill_tokens_per_s"], 3),
                    decode=round(entry[design]["decode_tokens_per_s"] / entry[other]["decode_tokens_per_s"], 3))
            entry[f"{design}_over_qwen2"] = dict(
                prefill=round(entry[design]["prefill_tokens_per_s"] / entry["qwen2"]["prefill_tokens_per_s"], 3),
                decode=round(entry[design]["decode_tokens_per_s"] / entry["qwen2"]["decode_tokens_per_s"], 3))
        entry["kernels"] = design_kernels(s, pk, once)
        result["sizes"][name] = entry
    result["gpu_launches"] = launches
    result["config"] = dict(prompt_len=prompt_len, decode_batch=batch, page_size=PAGE, l2="inputs larger than L2 (weights); "
                            "kernel timings flush L2 between launches")
    return result


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--design", default="dolezen", choices=sorted(DESIGNS))
    ap.add_argument("--sizes", default="2k,4k")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernels-only", action="store_true")
    ap.add_argument("--once", default=None, help="launch one kernel case a few times without timing (for a profiler)")
    a = ap.parse_args(argv)
    print(json.dumps(run(a.sizes.split(","), a.steps, max(3, a.warmup), kernels_only=a.kernels_only, once=a.once,
                         design=a.design)))


if __name__ == "__main__":
    main()
