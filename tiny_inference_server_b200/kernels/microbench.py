"""Runs single kernels at the shapes of a model, for timing and for profiler captures.

    python -m tiny_inference_server_b200.kernels.microbench attention --batch 8 --context 4096
    python -m tiny_inference_server_b200.kernels.microbench attention-prefill --tokens 2048
    python -m tiny_inference_server_b200.kernels.microbench rowwise --tokens 2048
    python -m tiny_inference_server_b200.kernels.microbench gemm --rows 8        (weight-streaming kernel)
    python -m tiny_inference_server_b200.kernels.microbench gemm --rows 4096     (tcgen05 kernel, above 64 rows)
    python -m tiny_inference_server_b200.kernels.microbench prefill --tokens 2048 --layers 4
    python -m tiny_inference_server_b200.kernels.microbench sampling --rows 8 --vocab 49152
    python -m tiny_inference_server_b200.kernels.microbench seqmix --window 1024   (windowed attention, short
        convolution, delta rule and gating, each beside the like kernel of the rotary GQA model)
    python -m tiny_inference_server_b200.kernels.microbench latent-linear-routed   (attention over compressed keys
        and values, recurrences with a decay per head, routed experts, each beside the like kernel of an earlier model)
    python -m tiny_inference_server_b200.kernels.microbench differential-latent-forget   (two score maps a head,
        windowed attention over compressed rows with head gates, the recurrence whose forget gate writes, a norm behind a
        sublayer, each beside the like kernel of an earlier model)
    python -m tiny_inference_server_b200.kernels.microbench all

``--reps N --no-timing`` launches the kernel N times and exits (a profiler attaches to that);
without it the kernels are timed with CUDA events, replayed from a CUDA graph that holds 40
launches over buffers larger than L2 (so a time includes the gap between dependent kernels,
as inside a decode step).  Default sizes are the upstream 0.9B model's: width 1536, 12 query
and 3 kv heads of 128, SwiGLU 4096.
"""
from __future__ import annotations

import argparse
import sys
import tempfile

import torch

from . import ops


def _graph_time(fn, n=40):
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n * 1e3


class _Step:
    """The little of a StepContext that the attention operation reads."""

    decode_only = True

    def __init__(self, tiles, max_position):
        self._tiles = tiles
        self.max_position = max_position
        self.min_position = max_position

    def plan(self, planner):
        return self._tiles


def attention(args):
    from .attention_plan import infer_tiles
    dev = "cuda"
    H, KVH, hd, page, ctx, B = args.heads, args.kv_heads, args.head_dim, args.page_size, args.context, args.batch
    pages_per = (ctx + page - 1) // page
    num_pages = B * pages_per
    n_planes = max(2, min(12, (400 << 20) // max(1, B * ctx * 2 * KVH * hd * 2)))
    planes = [torch.randn(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(n_planes)]
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(B, pages_per).contiguous()
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    qkv = torch.randn(B, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty(B, H * hd, device=dev, dtype=torch.bfloat16)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, slots, H // KVH), ctx - 1)
    rotary = None
    if args.rotary:          # as in a decode step: the kernel rotates q and k and writes the cache itself
        rotary = (torch.ones(ctx, hd // 2, device=dev), torch.zeros(ctx, hd // 2, device=dev))

    def run(i):
        ops.paged_attention(qkv, out, planes[i % n_planes], table, positions, slots, H, KVH, hd, page, None, fault, step,
                            rotary=rotary)

    kv_bytes = B * ctx * 2 * KVH * hd * 2
    if args.no_timing:
        for i in range(args.reps):
            run(i)
        torch.cuda.synchronize()
        print(f"attention batch {B} context {ctx}: {args.reps} launches, fault {int(fault[0])}")
        return
    t = _graph_time(run)
    print(f"attention decode  batch {B:3d} context {ctx}: {t:8.2f} us  {kv_bytes / t / 1e3:8.1f} GB/s of keys and values")


def attention_prefill(args):
    """Attention of one portion of ``--tokens`` rows at positions start..start+tokens-1 of a prompt
    (``--start 0``: a prompt over its own keys)."""
    from .attention_plan import infer_tiles
    dev = "cuda"
    H, KVH, hd, page, n = args.heads, args.kv_heads, args.head_dim, args.page_size, args.tokens
    num_pages = (args.start + n + page - 1) // page
    planes = [torch.randn(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(4)]
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(1, num_pages).contiguous()
    positions = torch.arange(args.start, args.start + n, dtype=torch.int32, device=dev)
    slots = torch.zeros(n, dtype=torch.int32, device=dev)
    qkv = torch.randn(n, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n, H * hd, device=dev, dtype=torch.bfloat16)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, slots, H // KVH), args.start + n - 1)
    step.min_position = args.start

    def run(i):
        ops.paged_attention(qkv, out, planes[i % 4], table, positions, slots, H, KVH, hd, page, None, fault, step)

    flops = 4 * H * hd * (n * (n + 1) / 2 + n * args.start)
    if args.no_timing:
        for i in range(args.reps):
            run(i)
        torch.cuda.synchronize()
        print(f"attention prefill {n} rows: {args.reps} launches, fault {int(fault[0])}")
        return
    ops.TC_ATTENTION_MIN_TILES = 1            # time both kernels whatever the choice would be
    for tc in (True, False):
        ops.TC_ATTENTION = tc
        t = _graph_time(run, 10)
        print(f"attention prefill {n:5d} rows, {'tcgen05 ' if tc else 'mma.sync'}: {t:8.2f} us  {flops / t / 1e6:7.1f} TFLOP/s  "
              f"fault {int(fault[0])}")
    ops.TC_ATTENTION = True


def rowwise(args):
    """The memory-bound kernels between the products, at ``--tokens`` rows of the model's widths."""
    dev = "cuda"
    n, d, F, H, KVH, hd, page = args.tokens, args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    bufs = 6                                                   # rotate buffers so that not everything stays in L2
    res = [torch.randn(n, d, device=dev) for _ in range(bufs)]
    delta = [torch.randn(n, d, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    normed = torch.empty(n, d, device=dev, dtype=torch.bfloat16)
    scale = torch.ones(d, device=dev)
    t = _graph_time(lambda i: ops.add_rmsnorm(res[i % bufs], delta[i % bufs], scale, 1e-6, normed), 12)
    mb = n * d * (4 + 2 + 4 + 2) / 1e6
    print(f"add_rmsnorm    {n} x {d}: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")
    gu = [torch.randn(n, 2 * F, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    hid = torch.empty(n, F, device=dev, dtype=torch.bfloat16)
    t = _graph_time(lambda i: ops.swiglu(gu[i % bufs], hid, 32), 12)
    mb = n * F * 6 / 1e6
    print(f"swiglu         {n} x {F}: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")
    qkv = [torch.randn(n, (H + 2 * KVH) * hd, device=dev, dtype=torch.bfloat16) for _ in range(bufs)]
    num_pages = (n + page - 1) // page
    plane = torch.zeros(num_pages, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16)
    table = torch.arange(num_pages, dtype=torch.int32, device=dev).reshape(1, num_pages).contiguous()
    positions = torch.arange(n, dtype=torch.int32, device=dev)
    slots = torch.zeros(n, dtype=torch.int32, device=dev)
    cos = torch.ones(n, hd // 2, device=dev)
    sin = torch.zeros(n, hd // 2, device=dev)
    fault = torch.zeros(4, dtype=torch.int32, device=dev)
    t = _graph_time(lambda i: ops.rope_kv_write(qkv[i % bufs], positions, slots, cos, sin, plane, table, H, KVH, hd, page,
                                                fault), 12)
    mb = n * ((H + 2 * KVH) * hd * 2 + (H + 2 * KVH) * hd * 2) / 1e6
    print(f"rope_kv_write  {n} rows: {t:7.2f} us  {mb / t * 1e3:7.1f} GB/s")


class _PortionStep:
    """A step that holds one portion of a prompt (or ``decode``: one row per request), with whatever a planner
    makes of its device arrays."""

    def __init__(self, positions, row_slot, decode=False):
        self.positions, self.row_slot, self.decode_only = positions, row_slot, decode
        self.max_position = int(positions.max())
        self.min_position = int(positions.min())
        self._plans = {}

    def plan(self, planner):
        if planner.key not in self._plans:
            self._plans[planner.key] = planner.infer(self.positions, self.row_slot)
        return self._plans[planner.key]


def seqmix(args, hbm_gbs=None, tflops=None):
    """The kernels of the mixers that are not rotary attention, each beside the kernel of the rotary GQA model
    that does the like work at equal sizes (``None``: that model has none).  Returns {name: {us, rate, unit,
    like_us, like_rate}}; ``rate`` is GB/s of the bytes the kernel must move, or TFLOP/s for the prompt attention."""
    from .attention_plan import infer_tiles
    dev = "cuda"
    d, F, H, G, hd, page = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    n, B, ctx, W = args.tokens, args.batch, args.context, args.window
    bf = dict(device=dev, dtype=torch.bfloat16)
    i32 = dict(device=dev, dtype=torch.int32)
    fault = torch.zeros(4, **i32)
    out = {}

    def put(name, us, work, unit, like_us=None, like_work=None):
        e = {"us": round(us, 2), "rate": round(work / us / 1e3, 1) if unit == "GB/s" else round(work / us / 1e6, 1), "unit": unit}
        if like_us is not None:
            lw = work if like_work is None else like_work
            e["like_us"] = round(like_us, 2)
            e["like_rate"] = round(lw / like_us / 1e3, 1) if unit == "GB/s" else round(lw / like_us / 1e6, 1)
        out[name] = e
        like = f"   like kernel {e['like_us']:9.2f} us {e['like_rate']:9.1f} {unit}" if like_us is not None else ""
        print(f"{name:34s} {e['us']:9.2f} us {e['rate']:9.1f} {unit}{like}")

    # ---- attention over a prompt portion: n rows of one request from position 0, window W
    num_pages = (n + page - 1) // page
    planes = [torch.randn(num_pages, 2, G, page, hd, **bf) for _ in range(2)]
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    pos = torch.arange(n, **i32)
    slot = torch.zeros(n, **i32)
    q = torch.randn(n, (H + 2 * G) * hd, **bf)
    gate = torch.randn(n, H * hd, **bf)
    o = torch.empty(n, H * hd, **bf)
    r1 = torch.rand(H, device=dev) + 0.2
    r2 = torch.rand(H, device=dev) + 0.1
    step = _PortionStep(pos, slot)
    pairs = sum(min(p + 1, W) for p in range(n))
    flops = 4.0 * H * hd * pairs
    t_new = _graph_time(lambda i: ops.window_attention(q, gate, o, planes[i % 2][:, 0], planes[i % 2][:, 1], table, pos, slot, H,
                                                       page, W, hd ** -0.5, r1, r2, fault, step), 10)
    gstep = _Step(infer_tiles(pos, slot, H // G), n - 1)
    gstep.decode_only = False
    gstep.min_position = 0
    t_like = _graph_time(lambda i: ops.paged_attention(q, o, planes[i % 2], table, pos, slot, H, G, hd, page, W, fault, gstep), 10)
    put(f"attention, {n} rows, window {W}", t_new, flops, "TFLOP/s", t_like)
    # ---- attention of B decode rows at position ctx - 1
    pages_per = (ctx + page - 1) // page
    n_planes = max(2, min(12, (300 << 20) // max(1, B * ctx * 2 * G * hd * 2)))
    planes = [torch.randn(B * pages_per, 2, G, page, hd, **bf) for _ in range(n_planes)]
    table = torch.arange(B * pages_per, **i32).reshape(B, pages_per).contiguous()
    pos = torch.full((B,), ctx - 1, **i32)
    slot = torch.arange(B, **i32)
    qd, gd, od = q[:B].contiguous(), gate[:B].contiguous(), torch.empty(B, H * hd, **bf)
    dstep = _PortionStep(pos, slot, decode=True)
    kv_bytes = B * min(W, ctx) * 2 * G * hd * 2
    t_new = _graph_time(lambda i: ops.window_attention(qd, gd, od, planes[i % n_planes][:, 0], planes[i % n_planes][:, 1], table,
                                                       pos, slot, H, page, W, hd ** -0.5, r1, r2, fault, dstep))
    gstep = _Step(infer_tiles(pos, slot, H // G), ctx - 1)
    t_like = _graph_time(lambda i: ops.paged_attention(qd, od, planes[i % n_planes], table, pos, slot, H, G, hd, page, W, fault,
                                                       gstep))
    put(f"attention, {B} decode rows, window {W}", t_new, kv_bytes, "GB/s", t_like)
    del planes
    # ---- between the projections and the cache
    bufs = 4
    num_pages = (n + page - 1) // page
    plane = torch.zeros(num_pages, 2, G, page, hd, **bf)
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    pos = torch.arange(n, **i32)
    slot = torch.zeros(n, **i32)
    last = torch.full((n,), n - 1, **i32)
    nq, nk = H * hd, G * hd
    qkv = [torch.randn(n, nq + 2 * nk, **bf) for _ in range(bufs)]
    other = torch.randn(n, nk, **bf)
    wq, wk, lam = torch.ones(nq, device=dev), torch.ones(nk, device=dev), torch.full((1,), 0.3, device=dev)
    t_new = _graph_time(lambda i: ops.norm_mix_store(qkv[i % bufs], nq, nk, nk, wq, wk, 1e-6, other, lam, plane[:, 0], plane[:, 1],
                                                     table, pos, slot, page, fault), 12)
    cos, sin = torch.ones(n, hd // 2, device=dev), torch.zeros(n, hd // 2, device=dev)
    t_like = _graph_time(lambda i: ops.rope_kv_write(qkv[i % bufs], pos, slot, cos, sin, plane, table, H, G, hd, page, fault), 12)
    moved = n * (nq + 2 * nk) * 2 * 2
    put(f"norm, mix, cache write, {n} rows", t_new, moved + n * nk * 2, "GB/s", t_like, moved)
    # ---- short convolutions: the mixer's input (with the residual) and its projections
    state = torch.zeros(2, 3 * (nq + 2 * nk), device=dev)
    x = [torch.randn(n, d, **bf) for _ in range(bufs)]
    y = torch.empty(n, d, **bf)
    w4 = torch.randn(4, d, device=dev)
    t_new = _graph_time(lambda i: ops.causal_conv(x[i % bufs], w4, state, y, slot, last, residual=True), 12)
    res = [torch.randn(n, d, device=dev) for _ in range(bufs)]
    ones = torch.ones(d, device=dev)
    t_like = _graph_time(lambda i: ops.add_rmsnorm(res[i % bufs], x[i % bufs], ones, 1e-6, y, kind="mean_eps"), 12)
    put(f"input convolution, {n} x {d}", t_new, n * d * 4, "GB/s", t_like, n * d * 12)
    yc = torch.empty(n, nq + 2 * nk, **bf)
    wc = torch.randn(4, nq + 2 * nk, device=dev)
    t_new = _graph_time(lambda i: ops.causal_conv(qkv[i % bufs], wc, state, yc, slot, last, silu=True), 12)
    put(f"convolution of q, k, v, {n} rows", t_new, n * (nq + 2 * nk) * 4, "GB/s")
    # ---- gating of the feed-forward
    gu = [torch.randn(n, 2 * F, **bf) for _ in range(bufs)]
    hid = torch.empty(n, F + 8, **bf)
    bg, bu = torch.zeros(F, device=dev), torch.zeros(F, device=dev)
    t_new = _graph_time(lambda i: ops.glu_clamped(gu[i % bufs], bg, bu, 7.0, 1.702, 1.0, hid, F), 12)
    hid2 = torch.empty(n, F, **bf)
    t_like = _graph_time(lambda i: ops.swiglu(gu[i % bufs], hid2, 32), 12)
    put(f"gating, {n} x {F}", t_new, n * F * 6, "GB/s", t_like)
    # ---- the delta rule: a prompt portion, and B decode rows
    nv = H * hd
    rows = [torch.randn(n, 2 * nk + nv, **bf) for _ in range(2)]
    beta, a, gt = torch.randn(n, H, **bf), torch.randn(n, H * hd, **bf), torch.randn(n, nv, **bf)
    a_log, dtb, nw = torch.zeros(H, device=dev), torch.zeros(H * hd, device=dev), torch.ones(hd, device=dev)
    st = torch.zeros(max(B, 1), H * hd * hd, device=dev)
    od = torch.empty(n, nv, **bf)
    t_new = _graph_time(lambda i: ops.delta_rule(rows[i % 2], beta, a, gt, a_log, dtb, nw, 1e-6, 1e-6, hd ** -0.5, st, od, slot, last,
                                                 H, G, hd, hd, requests=1, segments=(torch.zeros(1, **i32), 1)), 4)
    put(f"delta rule, {n} rows of one request", t_new, 6.0 * n * H * hd * hd, "TFLOP/s")
    slot_b = torch.arange(B, **i32)
    t_new = _graph_time(lambda i: ops.delta_rule(rows[i % 2][:B], beta[:B], a[:B], gt[:B], a_log, dtb, nw, 1e-6, 1e-6, hd ** -0.5, st,
                                                 od[:B], slot_b, slot_b, H, G, hd, hd, requests=B, segments=(slot_b, B)), 12)
    put(f"delta rule, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s")
    return out



def latent_linear_routed(args):
    """The kernels of attention over compressed keys and values, of the recurrences with one decay per head (the delta
    rule, linear attention) and of routed experts, each beside the kernel of an earlier architecture of this engine
    that does the like work at equal sizes (``None``: there is none).  Sizes: ``heads`` heads; the recurrences with
    keys and values of ``head_dim``; attention with ``rank`` compressed elements and ``rot`` rotated ones a token;
    ``experts`` experts of ``ffn / (top + 1)`` hidden elements of which ``top`` run a token.  Returns {name: {us,
    rate, unit, like_us, like_rate}}."""
    dev = "cuda"
    d, F, H, G, hd, page = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    n, B, ctx = args.tokens, args.batch, args.context
    rank, rot, E, top = args.rank, args.rot, args.experts, args.top
    bf = dict(device=dev, dtype=torch.bfloat16)
    i32 = dict(device=dev, dtype=torch.int32)
    fault = torch.zeros(4, **i32)
    out = {}

    def put(name, us, work, unit, like_us=None, like_work=None):
        e = {"us": round(us, 2), "rate": round(work / us / 1e3, 1) if unit == "GB/s" else round(work / us / 1e6, 1), "unit": unit}
        if like_us is not None:
            lw = work if like_work is None else like_work
            e["like_us"] = round(like_us, 2)
            e["like_rate"] = round(lw / like_us / 1e3, 1) if unit == "GB/s" else round(lw / like_us / 1e6, 1)
        out[name] = e
        like = f"   like kernel {e['like_us']:9.2f} us {e['like_rate']:9.1f} {unit}" if like_us is not None else ""
        print(f"{name:44s} {e['us']:9.2f} us {e['rate']:9.1f} {unit}{like}")

    # ---- attention over a prompt portion of n rows from position 0: one kv head of rank + rot elements a key, whose first
    # rank elements are the value, H query heads, a sink; beside windowed attention with G kv heads of head_dim
    row = rank + rot
    num_pages = (n + page - 1) // page
    pages = [torch.randn(num_pages, 1, page, row, **bf) for _ in range(2)]
    like_planes = [torch.randn(num_pages, 2, G, page, hd, **bf) for _ in range(2)]
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    pos, slot = torch.arange(n, **i32), torch.zeros(n, **i32)
    last = torch.full((n,), n - 1, **i32)
    q = torch.randn(n, H * row, **bf)
    lat = torch.empty(n, H * rank, **bf)
    sink = torch.zeros(H, device=dev)
    step = _PortionStep(pos, slot)
    pairs = n * (n + 1) // 2
    t_new = _graph_time(lambda i: ops.window_attention(q, None, lat, pages[i % 2], pages[i % 2][..., :rank], table, pos, slot, H,
                                                       page, None, row ** -0.5, None, None, fault, step, sink=sink), 6)
    ql = torch.randn(n, H * hd, **bf)
    ol = torch.empty(n, H * hd, **bf)
    r1, r2 = torch.rand(H, device=dev) + 0.2, torch.rand(H, device=dev) + 0.1
    t_like = _graph_time(lambda i: ops.window_attention(ql, None, ol, like_planes[i % 2][:, 0], like_planes[i % 2][:, 1], table,
                                                        pos, slot, H, page, None, hd ** -0.5, r1, r2, fault, step), 6)
    put(f"latent attention, {n} rows", t_new, 2.0 * H * (row + rank) * pairs, "TFLOP/s", t_like, 4.0 * H * hd * pairs)
    # ---- B decode rows at position ctx - 1
    pages_per = (ctx + page - 1) // page
    n_bufs = max(2, min(12, (300 << 20) // max(1, B * ctx * row * 2)))
    pages = [torch.randn(B * pages_per, 1, page, row, **bf) for _ in range(n_bufs)]
    like_planes = [torch.randn(B * pages_per, 2, G, page, hd, **bf) for _ in range(2)]
    table = torch.arange(B * pages_per, **i32).reshape(B, pages_per).contiguous()
    pos_b, slot_b = torch.full((B,), ctx - 1, **i32), torch.arange(B, **i32)
    dstep = _PortionStep(pos_b, slot_b, decode=True)
    qd, ld = q[:B].contiguous(), lat[:B].contiguous()
    t_new = _graph_time(lambda i: ops.window_attention(qd, None, ld, pages[i % n_bufs], pages[i % n_bufs][..., :rank], table, pos_b,
                                                       slot_b, H, page, None, row ** -0.5, None, None, fault, dstep, sink=sink))
    qld, old = ql[:B].contiguous(), ol[:B].contiguous()
    t_like = _graph_time(lambda i: ops.window_attention(qld, None, old, like_planes[i % 2][:, 0], like_planes[i % 2][:, 1], table,
                                                        pos_b, slot_b, H, page, None, hd ** -0.5, r1, r2, fault, dstep))
    put(f"latent attention, {B} decode rows at {ctx}", t_new, B * ctx * row * 2, "GB/s", t_like, B * ctx * 2 * G * hd * 2)
    del pages, like_planes
    # ---- between the projections and the cache
    bufs = 4
    num_pages = (n + page - 1) // page
    kp = torch.zeros(num_pages, 1, page, row, **bf)
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    qdim = hd // 2 + rot
    proj = [torch.randn(n, H * qdim + row, **bf) for _ in range(bufs)]
    cw = torch.ones(rank, device=dev)
    cos, sin = torch.ones(n, rot // 2, device=dev), torch.zeros(n, rot // 2, device=dev)
    t_new = _graph_time(lambda i: ops.latent_prepare(proj[i % bufs], H * qdim, H, hd // 2, rot, rank, cw, 1e-6, cos, sin, q, kp, table,
                                                     pos, slot, page, fault), 12)
    plane = torch.zeros(num_pages, 2, G, page, hd, **bf)
    nq, nk = H * hd, G * hd
    qkv = [torch.randn(n, nq + 2 * nk, **bf) for _ in range(bufs)]
    wq, wk = torch.ones(nq, device=dev), torch.ones(nk, device=dev)
    t_like = _graph_time(lambda i: ops.norm_mix_store(qkv[i % bufs], nq, nk, nk, wq, wk, 1e-6, None, None, plane[:, 0], plane[:, 1],
                                                      table, pos, slot, page, fault), 12)
    put(f"rotation, norm, cache write, {n} rows", t_new, n * (2 * H * rot + 2 * row) * 2, "GB/s", t_like, n * (nq + 2 * nk) * 2 * 2)
    # ---- the recurrences: a prompt portion of one request, and B decode rows
    nv = H * hd
    rows = [torch.randn(n, 2 * nk + nv, **bf) for _ in range(2)]
    beta, a_h, a_c, gt = torch.randn(n, H, **bf), torch.randn(n, H, **bf), torch.randn(n, H * hd, **bf), torch.randn(n, nv, **bf)
    a_log, dt_h, dt_c, nw = torch.zeros(H, device=dev), torch.zeros(H, device=dev), torch.zeros(H * hd, device=dev), torch.ones(hd, device=dev)
    st = torch.zeros(max(B, 1), H * hd * hd, device=dev)
    od = torch.empty(n, nv, **bf)
    one = (torch.zeros(1, **i32), 1)
    t_new = _graph_time(lambda i: ops.delta_rule(rows[i % 2], beta, a_h, gt, a_log, dt_h, nw, 1e-6, 1e-6, hd ** -0.5, st, od, slot, last,
                                                 H, G, hd, hd, requests=1, segments=one, decay_per_head=True, gate_act="silu"), 4)
    t_like = _graph_time(lambda i: ops.delta_rule(rows[i % 2], beta, a_c, gt, a_log, dt_c, nw, 1e-6, 1e-6, hd ** -0.5, st, od, slot, last,
                                                  H, G, hd, hd, requests=1, segments=one), 4)
    put(f"delta rule, decay per head, {n} rows", t_new, 6.0 * n * H * hd * hd, "TFLOP/s", t_like)
    t_new = _graph_time(lambda i: ops.delta_rule(rows[i % 2][:B], beta[:B], a_h[:B], gt[:B], a_log, dt_h, nw, 1e-6, 1e-6, hd ** -0.5,
                                                 st, od[:B], slot_b, slot_b, H, G, hd, hd, requests=B, segments=(slot_b, B),
                                                 decay_per_head=True, gate_act="silu"), 12)
    t_like_d = _graph_time(lambda i: ops.delta_rule(rows[i % 2][:B], beta[:B], a_c[:B], gt[:B], a_log, dt_c, nw, 1e-6, 1e-6, hd ** -0.5,
                                                    st, od[:B], slot_b, slot_b, H, G, hd, hd, requests=B, segments=(slot_b, B)), 12)
    put(f"delta rule, decay per head, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s", t_like_d)
    lin = [torch.randn(n, 3 * nv, **bf) for _ in range(2)]
    decay, nwl = torch.full((H,), 0.97, device=dev), torch.ones(nv, device=dev)
    st.zero_()
    t_new = _graph_time(lambda i: ops.linear_attention(lin[i % 2], gt, decay, nwl, 1e-6, st, od, slot, last, H, hd, hd, requests=1,
                                                       segments=one), 4)
    put(f"linear attention, {n} rows", t_new, 4.0 * n * H * hd * hd, "TFLOP/s", t_like, 6.0 * n * H * hd * hd)
    t_new = _graph_time(lambda i: ops.linear_attention(lin[i % 2][:B], gt[:B], decay, nwl, 1e-6, st, od[:B], slot_b, slot_b, H, hd, hd,
                                                       requests=B, segments=(slot_b, B)), 12)
    put(f"linear attention, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s", t_like_d)
    # ---- routed experts: top experts of ffn / (top + 1) hidden elements a row, beside the dense gated unit of top times that
    Fe = max(32, F // (top + 1) // 32 * 32)
    w_gu = torch.randn(E, 2, Fe, d, **bf) * 0.02
    w_dn = torch.randn(E, d, Fe, **bf) * 0.02
    w_r = torch.randn(E, d, device=dev) * 0.1
    corr = torch.zeros(E, device=dev)
    w_sg = torch.randn(d, device=dev) * 0.02
    dense_gu = torch.randn(d, 2 * top * Fe, **bf) * 0.02
    dense_dn = torch.randn(top * Fe, d, **bf) * 0.02
    for label, m in ((f"{B} decode rows", B), (f"{n} rows", n)):
        xs = [torch.randn(m, d, **bf) for _ in range(bufs)]
        groups = 4 if E % 4 == 0 and top <= E // 2 else 0
        t_r = _graph_time(lambda i: ops.moe_route(xs[i % bufs], w_r, corr, w_sg, groups, 2 if groups else 0, top), 12)
        put(f"router, {label}", t_r, m * d * 2 + E * d * 4, "GB/s")
        chosen, weights, sgate = ops.moe_route(xs[0], w_r, corr, w_sg, groups, 2 if groups else 0, top)
        t_new = _graph_time(lambda i: ops.moe_experts(xs[i % bufs], chosen, weights, w_gu, w_dn, None, None), 12 if m <= 64 else 3)
        t_like = _graph_time(lambda i: ops.gemm(ops.gemm_swiglu(xs[i % bufs], dense_gu, top * Fe, 32), dense_dn), 12 if m <= 64 else 3)
        if m <= 64:
            used = min(E, m * top)
            put(f"experts, {label}", t_new, used * 3 * d * Fe * 2, "GB/s", t_like, top * 3 * d * Fe * 2)
        else:
            put(f"experts, {label}", t_new, 6.0 * m * top * d * Fe, "TFLOP/s", t_like)
    return out


def differential_latent_forget(args):
    """The kernels of differential attention (two score maps a head), of windowed attention over compressed keys and
    values with a gate per head, of the recurrence whose forget gate also writes, of a norm behind a sublayer and of an
    ungated activation, each beside the kernel of an earlier architecture of this engine that does the like work at
    equal sizes (``None``: there is none).  Sizes: ``heads`` query and ``kv_heads`` key/value heads; a score map with
    keys of ``head_dim / 2`` (a head's two maps together are ``head_dim`` wide) and values of ``head_dim``; ``rank``
    compressed elements a token, seen through a window of ``window`` keys; the recurrence with keys and values of
    ``head_dim``.  Returns {name: {us, rate, unit, like_us, like_rate}}."""
    dev = "cuda"
    d, F, H, G, hd, page = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    n, B, ctx, rank, W = args.tokens, args.batch, args.context, args.rank, args.window
    dim = hd // 2
    bf = dict(device=dev, dtype=torch.bfloat16)
    i32 = dict(device=dev, dtype=torch.int32)
    fault = torch.zeros(4, **i32)
    out = {}

    def put(name, us, work, unit, like_us=None, like_work=None):
        e = {"us": round(us, 2), "rate": round(work / us / 1e3, 1) if unit == "GB/s" else round(work / us / 1e6, 1), "unit": unit}
        if like_us is not None:
            lw = work if like_work is None else like_work
            e["like_us"] = round(like_us, 2)
            e["like_rate"] = round(lw / like_us / 1e3, 1) if unit == "GB/s" else round(lw / like_us / 1e6, 1)
        out[name] = e
        like = f"   like kernel {e['like_us']:9.2f} us {e['like_rate']:9.1f} {unit}" if like_us is not None else ""
        print(f"{name:52s} {e['us']:9.2f} us {e['rate']:9.1f} {unit}{like}")

    # ---- differential attention over a prompt portion of n rows from position 0: 2 H query heads as wide as a key row
    # (two maps of dim), G kv heads; beside attention of H heads with keys and values of head_dim over the same cache.
    # The work counted is the design's (two maps of dim against the keys, two sums of values), not the zeros the
    # query rows carry where the other map's part of a key lies.
    num_pages = (n + page - 1) // page
    planes = [torch.randn(num_pages, 2, G, page, hd, **bf) for _ in range(2)]
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    pos, slot = torch.arange(n, **i32), torch.zeros(n, **i32)
    last = torch.full((n,), n - 1, **i32)
    q2 = torch.randn(n, 2 * H * hd, **bf)
    maps = torch.empty(n, 2 * H * hd, **bf)
    ql, ol = torch.randn(n, H * hd, **bf), torch.empty(n, H * hd, **bf)
    step = _PortionStep(pos, slot)
    pairs = n * (n + 1) // 2
    t_new = _graph_time(lambda i: ops.window_attention(q2, None, maps, planes[i % 2][:, 0], planes[i % 2][:, 1], table, pos, slot,
                                                       2 * H, page, None, dim ** -0.5, None, None, fault, step), 6)
    t_like = _graph_time(lambda i: ops.window_attention(ql, None, ol, planes[i % 2][:, 0], planes[i % 2][:, 1], table, pos, slot,
                                                        H, page, None, hd ** -0.5, None, None, fault, step), 6)
    put(f"differential attention, {n} rows", t_new, 2.0 * 2 * H * (dim + hd) * pairs, "TFLOP/s", t_like, 4.0 * H * hd * pairs)
    pages_per = (ctx + page - 1) // page
    n_bufs = max(2, min(12, (300 << 20) // max(1, B * ctx * 2 * G * hd * 2)))
    planes = [torch.randn(B * pages_per, 2, G, page, hd, **bf) for _ in range(n_bufs)]
    dtable = torch.arange(B * pages_per, **i32).reshape(B, pages_per).contiguous()
    pos_b, slot_b = torch.full((B,), ctx - 1, **i32), torch.arange(B, **i32)
    dstep = _PortionStep(pos_b, slot_b, decode=True)
    q2d, mapsd, qld, old = q2[:B].contiguous(), maps[:B].contiguous(), ql[:B].contiguous(), ol[:B].contiguous()
    t_new = _graph_time(lambda i: ops.window_attention(q2d, None, mapsd, planes[i % n_bufs][:, 0], planes[i % n_bufs][:, 1], dtable,
                                                       pos_b, slot_b, 2 * H, page, None, dim ** -0.5, None, None, fault, dstep))
    t_like = _graph_time(lambda i: ops.window_attention(qld, None, old, planes[i % n_bufs][:, 0], planes[i % n_bufs][:, 1], dtable,
                                                        pos_b, slot_b, H, page, None, hd ** -0.5, None, None, fault, dstep))
    put(f"differential attention, {B} decode rows at {ctx}", t_new, B * ctx * 2 * G * hd * 2, "GB/s", t_like)
    del planes
    # ---- between the projections and the cache: bias, norm per head and map, temperature, cache write, padded queries
    bufs = 4
    plane = torch.zeros(num_pages, 2, G, page, hd, **bf)
    nq, nk = H * hd, G * hd
    qkv = [torch.randn(n, nq + 2 * nk, **bf) for _ in range(bufs)]
    bias, qw, kw = torch.zeros(nq + 2 * nk, device=dev), torch.ones(dim, device=dev), torch.ones(dim, device=dev)
    t_new = _graph_time(lambda i: ops.head_norm_store(qkv[i % bufs], H, G, 2, dim, hd, bias, qw, kw, 1e-6, 0.2, 128, q2, plane[:, 0],
                                                      plane[:, 1], table, pos, slot, page, fault), 12)
    wq, wk = torch.ones(nq, device=dev), torch.ones(nk, device=dev)
    t_like = _graph_time(lambda i: ops.norm_mix_store(qkv[i % bufs], nq, nk, nk, wq, wk, 1e-6, None, None, plane[:, 0], plane[:, 1],
                                                      table, pos, slot, page, fault), 12)
    put(f"bias, norms, temperature, cache write, {n} rows", t_new, n * ((nq + 2 * nk) + 2 * nq + 2 * nk) * 2, "GB/s", t_like,
        n * (nq + 2 * nk) * 2 * 2)
    mp = [torch.randn(n, 2 * H * hd, **bf) for _ in range(bufs)]
    t_new = _graph_time(lambda i: ops.diff_combine(mp[i % bufs], 0.8, 1e-6, 0.7, ol, H, hd, slot), 12)
    res = [torch.randn(n, d, device=dev) for _ in range(bufs)]
    delta = [torch.randn(n, d, **bf) for _ in range(bufs)]
    normed, scale = torch.empty(n, d, **bf), torch.ones(d, device=dev)
    t_plain = _graph_time(lambda i: ops.add_rmsnorm(res[i % bufs], delta[i % bufs], scale, 1e-6, normed), 12)
    put(f"two maps combined and normed, {n} rows", t_new, n * 3 * H * hd * 2, "GB/s", t_plain, n * d * 12)
    t_new = _graph_time(lambda i: ops.add_rmsnorm(res[i % bufs], delta[i % bufs], scale, 1e-6, normed, kind="mean_eps",
                                                  delta_norm=(scale, 1e-6, "mean_eps")), 12)
    put(f"normed update + sum + norm, {n} rows", t_new, n * d * 12, "GB/s", t_plain)
    up = [torch.randn(n, 2 * F, **bf) for _ in range(bufs)]
    hid = torch.empty(n, F, **bf)
    t_new = _graph_time(lambda i: ops.activation(up[i % bufs][:, :F], hid, "relu2"), 12)
    t_like = _graph_time(lambda i: ops.swiglu(up[i % bufs], hid, 32), 12)
    put(f"squared relu, {n} rows", t_new, n * F * 4, "GB/s", t_like, n * F * 6)
    # ---- windowed attention over compressed rows with a gate per head, beside the same cache without a window, with a
    # rotated slice and a sink (the design this one's latent attention grew from)
    rot = 64
    cpages = [torch.randn(num_pages, 1, page, rank, **bf) for _ in range(2)]
    rpages = [torch.randn(num_pages, 1, page, rank + rot, **bf) for _ in range(2)]
    qc, qr = torch.randn(n, H * rank, **bf), torch.randn(n, H * (rank + rot), **bf)
    lat, gates = torch.empty(n, H * rank, **bf), torch.randn(n, H, **bf)
    sink = torch.zeros(H, device=dev)
    seen = sum(min(p + 1, W) for p in range(n))
    t_new = _graph_time(lambda i: ops.window_attention(qc, gates, lat, cpages[i % 2], cpages[i % 2][..., :rank], table, pos, slot, H,
                                                       page, W, dim ** -0.5, None, None, fault, step, gate_per_head=True), 6)
    t_like = _graph_time(lambda i: ops.window_attention(qr, None, lat, rpages[i % 2], rpages[i % 2][..., :rank], table, pos, slot, H,
                                                        page, None, dim ** -0.5, None, None, fault, step, sink=sink), 6)
    put(f"latent attention, window {W}, head gates, {n} rows", t_new, 4.0 * H * rank * seen, "TFLOP/s", t_like,
        2.0 * H * (2 * rank + rot) * pairs)
    n_bufs = max(2, min(12, (300 << 20) // max(1, B * ctx * (rank + rot) * 2)))
    cpages = [torch.randn(B * pages_per, 1, page, rank, **bf) for _ in range(n_bufs)]
    rpages = [torch.randn(B * pages_per, 1, page, rank + rot, **bf) for _ in range(n_bufs)]
    qcd, qrd, latd, gd = qc[:B].contiguous(), qr[:B].contiguous(), lat[:B].contiguous(), gates[:B].contiguous()
    t_new = _graph_time(lambda i: ops.window_attention(qcd, gd, latd, cpages[i % n_bufs], cpages[i % n_bufs][..., :rank], dtable, pos_b,
                                                       slot_b, H, page, W, dim ** -0.5, None, None, fault, dstep, gate_per_head=True))
    t_like = _graph_time(lambda i: ops.window_attention(qrd, None, latd, rpages[i % n_bufs], rpages[i % n_bufs][..., :rank], dtable,
                                                        pos_b, slot_b, H, page, None, dim ** -0.5, None, None, fault, dstep, sink=sink))
    put(f"latent attention, window {W}, {B} decode rows at {ctx}", t_new, B * min(W, ctx) * rank * 2, "GB/s", t_like,
        B * ctx * (rank + rot) * 2)
    del cpages, rpages
    kp, kpr = torch.zeros(num_pages, 1, page, rank, **bf), torch.zeros(num_pages, 1, page, rank + rot, **bf)
    proj = [torch.randn(n, H * (dim + rot) + rank + rot, **bf) for _ in range(bufs)]
    cw = torch.ones(rank, device=dev)
    cos, sin = torch.ones(n, rot // 2, device=dev), torch.zeros(n, rot // 2, device=dev)
    t_new = _graph_time(lambda i: ops.latent_prepare(proj[i % bufs], H * dim, H, dim, 0, rank, cw, 1e-6, None, None, qc, kp, table,
                                                     pos, slot, page, fault), 12)
    t_like = _graph_time(lambda i: ops.latent_prepare(proj[i % bufs], H * (dim + rot), H, dim, rot, rank, cw, 1e-6, cos, sin, qr, kpr,
                                                      table, pos, slot, page, fault), 12)
    put(f"compressed vector normed into the cache, {n} rows", t_new, n * 2 * rank * 2, "GB/s", t_like,
        n * (2 * H * rot + 2 * (rank + rot)) * 2)
    # ---- the recurrence whose forget gate writes, beside linear attention with one decay per head
    nv = H * hd
    rows = [torch.randn(n, 3 * nv, **bf) for _ in range(2)]
    lower, fb, nw, nwl = torch.rand(nv, device=dev) * 0.9, torch.zeros(nv, device=dev), torch.ones(hd, device=dev), torch.ones(nv, device=dev)
    decay, gt = torch.full((H,), 0.97, device=dev), torch.randn(n, nv, **bf)
    st = torch.zeros(max(B, 1), H * hd * hd, device=dev)
    od = torch.empty(n, nv, **bf)
    one = (torch.zeros(1, **i32), 1)
    t_new = _graph_time(lambda i: ops.forget_gate_recurrence(rows[i % 2][:, :2 * nv], rows[i % 2][:, 2 * nv:], lower, fb, nw, 1e-6, st, od,
                                                             slot, last, H, hd, hd, requests=1, segments=one), 4)
    st.zero_()
    t_like = _graph_time(lambda i: ops.linear_attention(rows[i % 2], gt, decay, nwl, 1e-6, st, od, slot, last, H, hd, hd, requests=1,
                                                        segments=one), 4)
    put(f"forget-gate recurrence, {n} rows", t_new, 4.0 * n * H * hd * hd, "TFLOP/s", t_like)
    st.zero_()
    t_new = _graph_time(lambda i: ops.forget_gate_recurrence(rows[i % 2][:B, :2 * nv], rows[i % 2][:B, 2 * nv:], lower, fb, nw, 1e-6, st,
                                                             od[:B], slot_b, slot_b, H, hd, hd, requests=B, segments=(slot_b, B)), 12)
    st.zero_()
    t_like = _graph_time(lambda i: ops.linear_attention(rows[i % 2][:B], gt[:B], decay, nwl, 1e-6, st, od[:B], slot_b, slot_b, H, hd, hd,
                                                        requests=B, segments=(slot_b, B)), 12)
    put(f"forget-gate recurrence, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s", t_like)
    return out


def gated_space_tied(args):
    """The kernels of gated linear attention, of a selective state space (scan; skip, gate and norm in groups), of attention
    whose values are its keys (rotation and cache write; attention with a keyless softmax term), of the norm in groups with
    two updates and two outputs, of the embedding with a hashed second table and of routed experts without gates, each
    beside the kernel of an earlier architecture of this engine that does the like work at equal sizes.  Sizes: ``heads``
    heads with keys and values of ``head_dim`` for the recurrences and the attention (``kv_heads`` key heads), a state of
    ``head_dim`` per head for the state space.  Returns {name: {us, rate, unit, like_us, like_rate}}."""
    dev = "cuda"
    d, F, H, G, hd, page = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size
    n, B, ctx = args.tokens, args.batch, args.context
    E, top = args.experts, args.top
    bf = dict(device=dev, dtype=torch.bfloat16)
    i32 = dict(device=dev, dtype=torch.int32)
    fault = torch.zeros(4, **i32)
    out = {}

    def put(name, us, work, unit, like_us=None, like_work=None):
        e = {"us": round(us, 2), "rate": round(work / us / 1e3, 1) if unit == "GB/s" else round(work / us / 1e6, 1), "unit": unit}
        if like_us is not None:
            lw = work if like_work is None else like_work
            e["like_us"] = round(like_us, 2)
            e["like_rate"] = round(lw / like_us / 1e3, 1) if unit == "GB/s" else round(lw / like_us / 1e6, 1)
        out[name] = e
        like = f"   like kernel {e['like_us']:9.2f} us {e['like_rate']:9.1f} {unit}" if like_us is not None else ""
        print(f"{name:52s} {e['us']:9.2f} us {e['rate']:9.1f} {unit}{like}")

    pos, slot = torch.arange(n, **i32), torch.zeros(n, **i32)
    last = torch.full((n,), n - 1, **i32)
    slot_b = torch.arange(B, **i32)
    one = (torch.zeros(1, **i32), 1)
    nv = H * hd
    # ---- gated linear attention beside the recurrence whose forget gate writes (the same walk of a matrix state with a
    # gate per key channel; this one also reads keys) and, for decode rows, the same
    rows = [torch.randn(n, 4 * nv, **bf) for _ in range(2)]
    power, a_bias, nw = torch.full((H,), 1 / 8, device=dev), torch.full((nv,), 3.0, device=dev), torch.ones(hd, device=dev)
    lower, fb = torch.rand(nv, device=dev) * 0.9, torch.zeros(nv, device=dev)
    gate = torch.randn(n, nv, **bf)
    st = torch.zeros(max(B, 1), H * hd * hd, device=dev)
    od = torch.empty(n, nv, **bf)
    t_new = _graph_time(lambda i: ops.gated_linear_attention(rows[i % 2][:, :3 * nv], rows[i % 2][:, 3 * nv:], power, a_bias, gate, nw,
                                                             1e-6, hd ** -0.5, st, od, slot, last, H, hd, hd, requests=1, segments=one), 4)
    st.zero_()
    t_like = _graph_time(lambda i: ops.forget_gate_recurrence(rows[i % 2][:, :2 * nv], rows[i % 2][:, 2 * nv:3 * nv], lower, fb, nw, 1e-6,
                                                              st, od, slot, last, H, hd, hd, requests=1, segments=one), 4)
    put(f"gated linear attention, {n} rows", t_new, 4.0 * n * H * hd * hd, "TFLOP/s", t_like)
    st.zero_()
    t_new = _graph_time(lambda i: ops.gated_linear_attention(rows[i % 2][:B, :3 * nv], rows[i % 2][:B, 3 * nv:], power, a_bias, gate[:B],
                                                             nw, 1e-6, hd ** -0.5, st, od[:B], slot_b, slot_b, H, hd, hd, requests=B,
                                                             segments=(slot_b, B)), 12)
    st.zero_()
    t_like = _graph_time(lambda i: ops.forget_gate_recurrence(rows[i % 2][:B, :2 * nv], rows[i % 2][:B, 2 * nv:3 * nv], lower, fb, nw,
                                                              1e-6, st, od[:B], slot_b, slot_b, H, hd, hd, requests=B,
                                                              segments=(slot_b, B)), 12)
    put(f"gated linear attention, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s", t_like)
    # ---- the state space's scan (input and output matrices of G groups, a step size per head) beside the delta rule with
    # one decay per head (the same decay; it also corrects the state towards the value)
    gn = G * hd
    cbx = [torch.randn(n, 2 * gn + nv, **bf) for _ in range(2)]
    dt = torch.randn(n, H, **bf)
    a_log, dt_bias = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    beta = torch.randn(n, H, **bf)
    st.zero_()
    t_new = _graph_time(lambda i: ops.state_space_scan(cbx[i % 2], dt, a_log, dt_bias, st, slot, last, H, G, hd, hd, requests=1,
                                                       segments=one), 4)
    st.zero_()
    t_like = _graph_time(lambda i: ops.delta_rule(cbx[i % 2], beta, dt, gate, a_log, dt_bias, nw, 1e-6, 1e-6, hd ** -0.5, st, od, slot,
                                                  last, H, G, hd, hd, requests=1, segments=one, decay_per_head=True), 4)
    put(f"state space scan, {n} rows", t_new, 4.0 * n * H * hd * hd, "TFLOP/s", t_like, 6.0 * n * H * hd * hd)
    st.zero_()
    t_new = _graph_time(lambda i: ops.state_space_scan(cbx[i % 2][:B], dt[:B], a_log, dt_bias, st, slot_b, slot_b, H, G, hd, hd,
                                                       requests=B, segments=(slot_b, B)), 12)
    st.zero_()
    t_like = _graph_time(lambda i: ops.delta_rule(cbx[i % 2][:B], beta[:B], dt[:B], gate[:B], a_log, dt_bias, nw, 1e-6, 1e-6, hd ** -0.5,
                                                  st, od[:B], slot_b, slot_b, H, G, hd, hd, requests=B, segments=(slot_b, B),
                                                  decay_per_head=True), 12)
    put(f"state space scan, {B} decode rows", t_new, B * H * hd * hd * 8, "GB/s", t_like)
    bufs = 4
    raw = [torch.randn(n, nv, device=dev) for _ in range(bufs)]
    skip, nwl = torch.ones(H, device=dev), torch.ones(nv, device=dev)
    t_new = _graph_time(lambda i: ops.skip_gate_group_norm(raw[i % bufs], cbx[i % 2][:, 2 * gn:], skip, gate, nwl, 2, 1e-6, od, slot, H, hd), 12)
    mp = [torch.randn(n, 2 * nv, **bf) for _ in range(bufs)]
    t_like = _graph_time(lambda i: ops.diff_combine(mp[i % bufs], 0.8, 1e-6, 0.7, od, H, hd, slot), 12)
    put(f"skip, gate, norm in groups, {n} rows", t_new, n * nv * (4 + 2 * 3), "GB/s", t_like, n * 3 * nv * 2)
    # ---- attention with tied values: rotation and cache write beside the norm-and-store of windowed attention; attention
    # with the keyless term beside the same kernel without it
    num_pages = (n + page - 1) // page
    kp, vp = torch.zeros(num_pages, G, page, hd, **bf), torch.zeros(num_pages, G, page, hd, **bf)
    table = torch.arange(num_pages, **i32).reshape(1, num_pages).contiguous()
    nq, nk = H * hd, G * hd
    qk = [torch.randn(n, nq + 2 * nk, **bf) for _ in range(bufs)]
    rot = hd // 4
    cos, sin = torch.ones(n, rot // 2, device=dev), torch.zeros(n, rot // 2, device=dev)
    t_new = _graph_time(lambda i: ops.rotate_tie_store(qk[i % bufs], H, G, hd, rot, cos, sin, kp, vp, table, pos, slot, page, fault), 12)
    wq, wk = torch.ones(nq, device=dev), torch.ones(nk, device=dev)
    t_like = _graph_time(lambda i: ops.norm_mix_store(qk[i % bufs], nq, nk, nk, wq, wk, 1e-6, None, None, kp, vp, table, pos, slot, page,
                                                      fault), 12)
    put(f"rotation and tied cache write, {n} rows", t_new, n * (2 * H * rot + nk + 2 * nk) * 2, "GB/s", t_like, n * (nq + 2 * nk) * 2 * 2)
    step = _PortionStep(pos, slot)
    pairs = n * (n + 1) // 2
    kps = [torch.randn(num_pages, G, page, hd, **bf) for _ in range(2)]
    vps = [torch.randn(num_pages, G, page, hd, **bf) for _ in range(2)]
    q, o = torch.randn(n, nq, **bf), torch.empty(n, nq, **bf)
    sink = torch.zeros(H, device=dev)
    t_new = _graph_time(lambda i: ops.window_attention(q, None, o, kps[i % 2], vps[i % 2], table, pos, slot, H, page, None, hd ** -0.5,
                                                       None, None, fault, step, sink=sink), 6)
    t_like = _graph_time(lambda i: ops.window_attention(q, None, o, kps[i % 2], vps[i % 2], table, pos, slot, H, page, None, hd ** -0.5,
                                                        None, None, fault, step), 6)
    put(f"attention with a keyless term, {n} rows", t_new, 4.0 * H * hd * pairs, "TFLOP/s", t_like)
    pages_per = (ctx + page - 1) // page
    n_bufs = max(2, min(12, (300 << 20) // max(1, B * ctx * 2 * G * hd * 2)))
    kps = [torch.randn(B * pages_per, G, page, hd, **bf) for _ in range(n_bufs)]
    vps = [torch.randn(B * pages_per, G, page, hd, **bf) for _ in range(n_bufs)]
    dtable = torch.arange(B * pages_per, **i32).reshape(B, pages_per).contiguous()
    pos_b = torch.full((B,), ctx - 1, **i32)
    dstep = _PortionStep(pos_b, slot_b, decode=True)
    qd, odd = q[:B].contiguous(), o[:B].contiguous()
    t_new = _graph_time(lambda i: ops.window_attention(qd, None, odd, kps[i % n_bufs], vps[i % n_bufs], dtable, pos_b, slot_b, H, page,
                                                       None, hd ** -0.5, None, None, fault, dstep, sink=sink))
    t_like = _graph_time(lambda i: ops.window_attention(qd, None, odd, kps[i % n_bufs], vps[i % n_bufs], dtable, pos_b, slot_b, H, page,
                                                        None, hd ** -0.5, None, None, fault, dstep))
    put(f"attention with a keyless term, {B} decode rows at {ctx}", t_new, B * ctx * 2 * G * hd * 2, "GB/s", t_like)
    del kps, vps
    # ---- the norm in groups: two updates added, two outputs written, beside two launches of the plain fused norm
    res = [torch.randn(n, d, device=dev) for _ in range(bufs)]
    da, db = [torch.randn(n, d, **bf) for _ in range(bufs)], [torch.randn(n, d, **bf) for _ in range(bufs)]
    o1, o2, scale = torch.empty(n, d, **bf), torch.empty(n, d, **bf), torch.ones(d, device=dev)
    t_new = _graph_time(lambda i: ops.group_norm(res[i % bufs], da[i % bufs], db[i % bufs], 2, 1e-6, scale, o1, scale, o2), 12)

    def twice(i):
        ops.add_rmsnorm(res[i % bufs], da[i % bufs], scale, 1e-6, o1, kind="mean_eps")
        ops.add_rmsnorm(res[i % bufs], db[i % bufs], scale, 1e-6, o2, kind="mean_eps")
    t_like = _graph_time(twice, 12)
    put(f"two updates, norm in groups, two outputs, {n} rows", t_new, n * d * (8 + 4 + 4), "GB/s", t_like, n * d * (16 + 4 + 4))
    t_new = _graph_time(lambda i: ops.group_norm(res[i % bufs][:B], da[i % bufs][:B], db[i % bufs][:B], 2, 1e-6, scale, o1[:B], scale,
                                                 o2[:B]), 12)
    t_like = _graph_time(lambda i: (ops.add_rmsnorm(res[i % bufs][:B], da[i % bufs][:B], scale, 1e-6, o1[:B], kind="mean_eps"),
                                    ops.add_rmsnorm(res[i % bufs][:B], db[i % bufs][:B], scale, 1e-6, o2[:B], kind="mean_eps")), 12)
    put(f"two updates, norm in groups, two outputs, {B} rows", t_new, B * d * 16, "GB/s", t_like, B * d * 24)
    # ---- the embedding with the hashed pair table beside the plain gather
    vocab = 32768
    tab, prs = torch.randn(vocab, d, **bf), torch.randn(4100, d, **bf)
    toks = torch.randint(0, vocab, (n,), **i32)
    prev = torch.zeros(8, 1, **i32)
    t_new = _graph_time(lambda i: ops.embed_pairs(tab, prs, toks, pos, slot, last, prev, res[i % bufs], 2.0, 4099, 1009, 31), 12)
    t_like = _graph_time(lambda i: ops.embed_rows(tab, toks, res[i % bufs], 2.0), 12)
    put(f"embedding with a pair table, {n} rows", t_new, n * d * (2 + 2 + 4), "GB/s", t_like, n * d * (2 + 4))
    # ---- routed experts without gates (one matrix and an activation) beside the gated ones with as many weights
    fe = max(64, F // (top + 1) // 64 * 64)
    x = torch.randn(n, d, **bf)
    wr = torch.randn(E, d, device=dev)
    up1, up2 = torch.randn(E, fe * 3 // 2 // 64 * 64, d, **bf) * 0.02, torch.randn(E, 2, fe, d, **bf) * 0.02
    f1 = up1.shape[1]
    dn1, dn2 = torch.randn(E, d, f1, **bf) * 0.02, torch.randn(E, d, fe, **bf) * 0.02
    ch, wt, _ = ops.moe_route(x, wr, None, None, 0, 0, top, scores="softmax_chosen")
    t_new = _graph_time(lambda i: ops.moe_experts(x, ch, wt, up1, dn1, None, None, act="relu2"), 6)
    t_like = _graph_time(lambda i: ops.moe_experts(x, ch, wt, up2, dn2, None, None), 6)
    put(f"experts without gates, {n} rows", t_new, 2.0 * n * top * 2 * f1 * d, "TFLOP/s", t_like, 2.0 * n * top * 3 * fe * d)
    t_new = _graph_time(lambda i: ops.moe_experts(x[:B], ch[:B], wt[:B], up1, dn1, None, None, act="relu2"), 12)
    t_like = _graph_time(lambda i: ops.moe_experts(x[:B], ch[:B], wt[:B], up2, dn2, None, None), 12)
    put(f"experts without gates, {B} decode rows", t_new, B * top * 2 * f1 * d * 2, "GB/s", t_like, B * top * 3 * fe * d * 2)
    t_new = _graph_time(lambda i: ops.moe_route(x, wr, None, None, 0, 0, top, scores="softmax_chosen"), 12)
    t_like = _graph_time(lambda i: ops.moe_route(x, wr, None, None, 0, 0, top), 12)
    put(f"router, softmax over the chosen, {n} rows", t_new, n * d * 2, "GB/s", t_like)
    return out


def sampling(args):
    """The sampling kernel at ``--rows`` rows of ``--vocab`` logits, for the kinds of setting a row can have."""
    dev = "cuda"
    k, v = args.rows, args.vocab
    bufs = max(2, min(16, (300 << 20) // (k * v * 4)))
    logits = [torch.randn(k, v, device=dev) * 3 for _ in range(bufs)]
    slots = torch.arange(k, dtype=torch.int32, device=dev)
    seen = torch.zeros(k, (v + 31) // 32, dtype=torch.int32, device=dev)
    seeds = torch.arange(k, dtype=torch.int64, device=dev)
    counters = torch.zeros(k, dtype=torch.int64, device=dev)
    out = torch.empty(k, dtype=torch.int32, device=dev)
    for name, temp, top_k, top_p, pen in [("greedy", 0.0, 0, 0.0, 1.0), ("temperature", 1.0, 0, 0.0, 1.0),
                                          ("top-k 50", 1.0, 50, 0.0, 1.0), ("top-p 0.9", 1.0, 0, 0.9, 1.0),
                                          ("top-k 50, top-p 0.95, penalty 1.1", 0.8, 50, 0.95, 1.1)]:
        temps = torch.full((k,), temp, device=dev)
        top_ks = torch.full((k,), top_k, dtype=torch.int32, device=dev)
        top_ps = torch.full((k,), top_p, device=dev)
        pens = torch.full((k,), pen, device=dev)
        if args.no_timing:
            if pen == 1.0:
                continue                      # a profiler looks at the setting with everything in it
            for i in range(args.reps):
                ops.sample_rows(logits[i % bufs], temps, top_ks, top_ps, pens, slots, seen, seeds, counters, out, None)
            torch.cuda.synchronize()
            print(f"sampling {k} x {v} {name}: {args.reps} launches")
            return
        t = _graph_time(lambda i: ops.sample_rows(logits[i % bufs], temps, top_ks, top_ps, pens, slots, seen, seeds,
                                                  counters, out, None), 20)
        print(f"sampling {k} x {v}  {name:36s}: {t:7.2f} us")


def gemm(args):
    dev = "cuda"
    d, F, H, KVH, hd, n = args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.rows
    x = torch.randn(n, d, device=dev, dtype=torch.bfloat16)
    hm = torch.randn(n, F, device=dev, dtype=torch.bfloat16)
    shapes = (("qkv", d, (H + 2 * KVH) * hd, x, False), ("o", H * hd, d, x[:, : H * hd].contiguous(), False),
              ("gate_up+swiglu", d, 2 * F, x, True), ("down", F, d, hm, False))
    for name, K, N, inp, fused in shapes:
        if args.only and args.only != name:
            continue
        ws = [torch.randn(K, N, device=dev, dtype=torch.bfloat16) for _ in range(12)]

        def mine(i):
            if n > 64:
                ops.gemm_tc(inp, ws[i % 12], swiglu=fused)
            else:
                ops.gemm_skinny(inp, ws[i % 12], swiglu=fused)

        gu = torch.empty(n, N, device=dev, dtype=torch.bfloat16) if fused else None
        half = torch.empty(n, N // 2, device=dev, dtype=torch.bfloat16) if fused else None

        def lib(i):
            if fused:
                ops.swiglu(torch.mm(inp, ws[i % 12], out=gu), half, 32)
            else:
                torch.mm(inp, ws[i % 12])

        if args.no_timing:
            for i in range(args.reps):
                mine(i)
            torch.cuda.synchronize()
            print(f"gemm {name} rows {n}: {args.reps} launches")
            continue
        a, b = _graph_time(mine), _graph_time(lib)
        mb = K * N * 2 / 1e6
        extra = ""
        if n <= 64:
            # both weight-streaming kernels, whatever the dispatch would choose: the ring, the TMA boxes
            saved = (ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS)
            times = {}
            for label, sg in (("ring", False), ("boxes", True)):
                ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS = \
                    sg, 0, 1 << 30, 1 << 30, 64
                if not sg or ops._stream_fits(n, K, ops._ksplit(N, K)):
                    times[label] = _graph_time(mine)
            (ops.STREAM_GEMM, ops.STREAM_MIN_KC, ops.STREAM_MAX_KC, ops.STREAM_MAX_CTAS, ops.STREAM_MAX_ROWS) = saved
            times["tcgen05 swapped"] = _graph_time(lambda i: ops.gemm_swap(inp, ws[i % 12], swiglu=fused))
            extra = "   " + "  ".join(f"{k} {v:6.2f}" for k, v in times.items())
        print(f"gemm {name:15s} rows {n:4d} {mb:6.1f} MB: this kernel {a:7.2f} us ({mb / a * 1e3:7.1f} GB/s, "
              f"{2 * n * K * N / a / 1e6:6.1f} TFLOP/s)   library {b:7.2f} us{extra}")


def prefill(args):
    """One step of ``--tokens`` prompt tokens through ``--layers`` layers of the model."""
    from ..config import EngineConfig
    from ..engine import ModelRunner, StepEntry
    from ..registry import config_from_dict
    from ..weights import write_random_model
    cfg = config_from_dict(dict(architecture="gqa_mtp_transformer", vocab_size=49152, hidden_size=args.width,
                                num_layers=args.layers, num_heads=args.heads, num_kv_heads=args.kv_heads,
                                head_dim=args.head_dim, ffn_hidden=args.ffn, max_context=4096, num_mtp_heads=0))
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(tmp, cfg, seed=0)
        r = ModelRunner.from_folder(folder, EngineConfig(dtype="bfloat16", page_size=args.page_size,
                                                         num_pages=(args.tokens // args.page_size + 2) * 2,
                                                         max_batch=2, max_tokens_per_step=args.tokens))
    g = torch.Generator().manual_seed(0)
    for rep in range(max(3, args.reps)):
        ids = torch.randint(0, cfg.vocab_size, (args.tokens,), generator=g).tolist()
        s = r.add_request()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.step([StepEntry(s, ids, [args.tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        print(f"prefill {args.tokens} tokens, {args.layers} layers: {e0.elapsed_time(e1):.3f} ms", flush=True)
        r.release(s)


def timeline(args):
    """Where the time of a decode layer goes, from inside its kernels: the five launches of a layer (qkv, attention,
    o, gate/up, down — as the engine chains them, norms folded into the products) replayed from a graph of
    ``--layers`` layers, in a build of the kernels that stamps the global timer at named places (csrc/timeline.cuh;
    compiled for this command only).  Printed for a layer in the middle: per kernel and place the first, median
    and last CTA, in ns after the last CTA of the kernel before stored its result."""
    from . import build
    from .attention_plan import infer_tiles
    if "-DTIS_TIMELINE" not in build.NVCC_FLAGS:
        build.NVCC_FLAGS.append("-DTIS_TIMELINE")            # before the libraries are first asked for
    dev = "cuda"
    d, F, H, KVH, hd, page, ctx, B, L = (args.width, args.ffn, args.heads, args.kv_heads, args.head_dim, args.page_size,
                                         args.context, args.batch, args.layers)
    lib, alib = ops.library(), ops.attention_library(hd)
    slots = lib.tis_timeline_slots()
    pages_per = (ctx + page - 1) // page
    planes = [torch.randn(B * pages_per, 2, KVH, page, hd, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).reshape(B, pages_per).contiguous()
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    rows_slot = torch.arange(B, dtype=torch.int32, device=dev)
    step = _Step(infer_tiles(positions, rows_slot, H // KVH), ctx - 1)
    rotary = (torch.ones(ctx, hd // 2, device=dev), torch.zeros(ctx, hd // 2, device=dev))
    fault = torch.zeros(4, dtype=torch.int32, device=dev)

    def w(k, n):
        return [torch.randn(k, n, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(L)]
    w_qkv, w_o, w_gu, w_down = w(d, (H + 2 * KVH) * hd), w(H * hd, d), w(d, 2 * F), w(F, d)
    norm_w = torch.ones(d, device=dev)
    stream = torch.randn(B, d, device=dev)
    names = ("qkv", "attention", "o", "gate/up", "down")
    max_ctas = 1024
    stamps = torch.zeros(L * 5, max_ctas * slots, dtype=torch.int64, device=dev)
    attn_out = torch.empty(B, H * hd, device=dev, dtype=torch.bfloat16)

    def layer(l, x):
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 0]))
        qkv = ops.gemm(x, w_qkv[l])
        alib.tis_timeline_next(ops._p(stamps[l * 5 + 1]))
        ops.paged_attention(qkv, attn_out, planes[l], table, positions, rows_slot, H, KVH, hd, page, None, fault, step,
                            rotary=rotary)
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 2]))
        a = ops.gemm(attn_out, w_o[l], sink=ops.ResidualSink(stream, norm_w, 1e-6))
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 3]))
        h = ops.gemm_swiglu(a, w_gu[l], F, 32)
        lib.tis_timeline_next(ops._p(stamps[l * 5 + 4]))
        return ops.gemm(h, w_down[l], sink=ops.ResidualSink(stream, norm_w, 1e-6))

    def run():
        x = ops.ScaledRows(torch.randn(B, d, device=dev, dtype=torch.bfloat16),
                           torch.ones(B, (d + 63) // 64, device=dev), 1e-6)
        for l in range(L):
            x = layer(l, x)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        stamps.zero_()
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
    print(f"decode layer, {B} rows, context {ctx}: {e0.elapsed_time(e1) / L * 1e3:.2f} us a layer with the stamps "
          f"(fault words {fault.tolist()})")
    t = stamps.cpu().reshape(L * 5, max_ctas, slots)
    places = {
        "gemm": ("entry", "weights ordered", "dependency wait over", "first tile ready", "loop done", "cluster barrier passed",
                 "stored"),
        "attention": ("entry", "before the dependency wait", "dependency wait over", "first tile landed", "last tile landed",
                      "loop done", "partial results pushed", "partials of the cluster arrived", "stored"),
    }
    mid = L // 2
    prev = t[mid * 5 - 1]
    prev_end = int(prev[prev[:, 0] > 0].max())
    for k in range(5):
        rec = t[mid * 5 + k]
        rec = rec[rec[:, 0] > 0]
        kind = places["attention" if k == 1 else "gemm"]
        print(f"{names[k]} ({rec.shape[0]} CTAs): ns after the last CTA of the kernel before stored (first / median / last CTA)")
        for i, place in enumerate(kind):
            v = rec[:, i]
            v = v[v > 0] - prev_end
            if v.numel():
                print(f"  {place:32s} {int(v.min()):8d} {int(v.median()):8d} {int(v.max()):8d}")
        prev_end = int(rec[:, len(kind) - 1].max())


def main(argv=None):
    ap = argparse.ArgumentParser(prog="microbench", description=__doc__.split("\n\n")[0])
    ap.add_argument("what", choices=["attention", "attention-prefill", "rowwise", "gemm", "prefill", "sampling", "timeline",
                                     "seqmix", "latent-linear-routed", "differential-latent-forget", "gated-space-tied", "all"])
    ap.add_argument("--rank", type=int, default=128, help="latent-linear-routed: compressed elements a token")
    ap.add_argument("--rot", type=int, default=64, help="latent-linear-routed: rotated elements a token")
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top", type=int, default=3)
    ap.add_argument("--window", type=int, default=1024, help="seqmix: keys a row sees")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--start", type=int, default=0, help="attention-prefill: first position of the portion")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--only", default=None, help="gemm: one of qkv, o, gate_up+swiglu, down")
    ap.add_argument("--width", type=int, default=1536)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=3)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=49152)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--no-timing", action="store_true")
    ap.add_argument("--rotary", action="store_true", help="attention: rotary encoding and cache write inside the kernel")
    args = ap.parse_args(argv)
    if args.what == "timeline":
        if args.layers < 2:
            ap.error("timeline: at least two layers (the printed one has a layer before it)")
        return timeline(args) or 0
    ops.library()
    if args.what in ("attention", "all"):
        for b in ([args.batch] if args.what == "attention" else [1, 8, 64]):
            args.batch = b
            attention(args)
    if args.what in ("attention-prefill", "all"):
        attention_prefill(args)
    if args.what in ("rowwise", "all"):
        rowwise(args)
    if args.what in ("gemm", "all"):
        for n in ([args.rows] if args.what == "gemm" else [1, 8, 16]):
            args.rows = n
            gemm(args)
    if args.what in ("prefill", "all"):
        prefill(args)
    if args.what in ("sampling", "all"):
        sampling(args)
    if args.what in ("seqmix", "all"):
        seqmix(args)
    if args.what in ("latent-linear-routed", "all"):
        latent_linear_routed(args)
    if args.what in ("differential-latent-forget", "all"):
        differential_latent_forget(args)
    if args.what in ("gated-space-tied", "all"):
        gated_space_tied(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
