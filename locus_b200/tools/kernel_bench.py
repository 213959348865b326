"""Runs one kernel of the engine on synthetic inputs, for timing and for profiler captures.

    python -m locus_b200.tools.kernel_bench linear --m 2048 --n 6144 --k 2048 [--dual] [--accumulate] [--iters 20]
    python -m locus_b200.tools.kernel_bench attn_decode --batch 8 --ctx 4000 [--heads 16 --kv-heads 16 --head-dim 128]
    python -m locus_b200.tools.kernel_bench attn_chunk --tokens 2048 --ctx 0
    python -m locus_b200.tools.kernel_bench experts --tokens 2048 [--experts 60 --top-k 4 --k 2048 --n 1408] [--part up|down]
    python -m locus_b200.tools.kernel_bench recurrence --tokens 2048 --batch 1 [--heads 16 --head-dim 128 --v-dim 128]
                                                       [--per-group 1] [--ones] [--retention | --delta | --gla]
    python -m locus_b200.tools.kernel_bench head_prep --tokens 2048 --batch 1 [--window 4096]

Times with CUDA events after warm-up.  Weights rotate through enough copies that the L2
cannot hold them (``linear``); attention reads a cache larger than the L2 at the default
sizes.  Prints one line with microseconds per call, TFLOP/s and GB/s.  Under ``ncu`` use a
small ``--iters`` and ``-k regex:<kernel>``.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from .. import kernels as K


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time(fn, iters: int, graph: bool) -> float:
    """Microseconds per call.  ``graph``: replay the calls from a CUDA graph so that the
    host's launch cost does not hide a short kernel's time."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g), K.stream_scope():
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        a, b = _events()
        a.record()
        g.replay()
        b.record()
    else:
        a, b = _events()
        a.record()
        for _ in range(iters):
            fn()
        b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def bench_linear(args) -> None:
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    M, N, Kd = args.m, args.n, args.k
    wbytes = N * Kd * (2 if dt == torch.bfloat16 else 4) * (2 if args.dual else 1)
    copies = max(1, min(40, int(400e6 // wbytes)))
    ws = [(torch.randn(N, Kd, device=dev) * 0.02).to(dt) for _ in range(copies)]
    w2s = [(torch.randn(N, Kd, device=dev) * 0.02).to(dt) for _ in range(copies)] if args.dual else None
    x = torch.randn(M, Kd, device=dev).to(dt)
    out = torch.zeros(M, N, device=dev, dtype=torch.float32 if args.accumulate else dt)
    state = {"i": 0}

    def fn():
        i = state["i"] % copies
        state["i"] += 1
        K.linear(x, ws[i], out, w2=w2s[i] if args.dual else None, accumulate=args.accumulate)

    us = _time(fn, args.iters, args.graph)
    flops = 2.0 * M * N * Kd * (2 if args.dual else 1)
    print(f"linear M={M} N={N} K={Kd} dual={int(args.dual)} accumulate={int(args.accumulate)} {args.dtype}: "
          f"{us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s  weights {wbytes / us / 1e3:.1f} GB/s  "
          f"(tensor-core error word {K.tc_error() if dt == torch.bfloat16 else 0})")


def bench_experts(args) -> None:
    """The two grouped products of the routed experts as the sparse-MoE block runs them: SwiGLU of
    gate and up ([E, n, k] each) over the tokens laid out by expert, then down ([E, k, n]) with the
    routing weight of each row, into float32 rows.  Every token picks ``top_k`` distinct experts at
    random; the layers' weights rotate through copies so that the L2 cannot hold them."""
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    T, E, k, H, I = args.tokens, args.experts, args.top_k, args.k, args.n
    n_pairs = T * k
    g = torch.Generator(device="cpu").manual_seed(1)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32).reshape(-1).to(dev)
    wts = torch.rand(n_pairs, device=dev)
    el = 2 if dt == torch.bfloat16 else 4
    layer_bytes = 3 * E * I * H * el
    copies = max(1, min(8, int(3e9 // layer_bytes)))
    gate = [(torch.randn(E, I, H, device=dev) * 0.02).to(dt) for _ in range(copies)]
    up = [(torch.randn(E, I, H, device=dev) * 0.02).to(dt) for _ in range(copies)]
    down = [(torch.randn(E, H, I, device=dev) * 0.02).to(dt) for _ in range(copies)]
    h = torch.randn(T, H, device=dev).to(dt)
    tile = args.tile or (K.FEW_ROWS if T <= K.FEW_ROWS else K.expert_tile(n_pairs, E))
    streamed = tile <= (K.SKINNY_TILE_ROWS if dt == torch.bfloat16 else K.FEW_ROWS)
    if not streamed and dt != torch.bfloat16:
        tile = 64
    lay = K.ExpertLayout(n_pairs, E, 64, dev)
    K.moe_sort(ids, n_pairs, lay, tile)
    xs = torch.empty(n_pairs, H, device=dev, dtype=dt)
    K.gather_rows(h, lay.sorted_pair, k, xs, n_pairs)
    act = torch.empty(n_pairs, I, device=dev, dtype=dt)
    pair_out = torch.empty(n_pairs, H, device=dev, dtype=torch.float32)
    state = {"i": 0}

    def fn():
        i = state["i"] % copies
        state["i"] += 1
        if args.part in ("both", "up"):
            if streamed:
                K.linear(h, gate[i], act, w2=up[i], x_rows=lay.sorted_pair, x_row_div=k, layout=lay, n_rows=n_pairs)
            else:
                K.linear(xs, gate[i], act, w2=up[i], layout=lay, n_rows=n_pairs)
        if args.part in ("both", "down"):
            K.linear(act, down[i], pair_out, layout=lay, n_rows=n_pairs, row_scale=wts, scale_rows=lay.sorted_pair)

    us = _time(fn, args.iters, args.graph)
    share = {"both": 3, "up": 2, "down": 1}[args.part]
    used = int((torch.bincount(ids.long(), minlength=E) > 0).sum())
    flops = 2.0 * n_pairs * H * I * share
    wbytes = used * I * H * el * share
    print(f"experts T={T} E={E} top_k={k} hidden={H} inner={I} part={args.part} tile={tile} {args.dtype}: "
          f"{us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s  weights of the {used} experts used {wbytes / us / 1e3:.1f} GB/s  "
          f"(tensor-core error word {K.tc_error() if dt == torch.bfloat16 else 0})")


def _paged(args, B: int, ctx: int, new: int):
    dev = "cuda:0"
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    P, nh, nkv, hd = args.page_tokens, args.heads, args.kv_heads, args.head_dim
    per = -(-(ctx + new) // P)
    pool = torch.randn(B * per, 2, nkv, P, hd, device=dev).to(dt)
    table = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per).contiguous()
    q = torch.randn(B * new, nh * hd, device=dev).to(dt)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    meta = dict(seg_q0=i32([i * new for i in range(B)]), seg_qn=i32([new] * B), seg_ctx=i32([ctx] * B), block_table=table)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=args.window, scale=1 / math.sqrt(hd))
    if args.keep_first or args.sink:
        kw.update(keep_first=args.keep_first, sink=args.sink)
    return pool, q, torch.empty_like(q), meta, kw, i32


def bench_attn_decode(args) -> None:
    B, ctx = args.batch, args.ctx
    pool, q, out, meta, kw, i32 = _paged(args, B, ctx, 1)
    ms = ctx // K.DECODE_SPLIT + 1
    po = torch.empty(B * args.heads * ms * args.head_dim, device="cuda:0")
    pm = torch.empty(2 * B * args.heads * ms, device="cuda:0")
    items = i32(list(range(B)))
    cnt = torch.zeros(B * args.heads, dtype=torch.int32, device="cuda:0")

    def fn():
        K.attn_decode(q, pool, out, items=items, n_items=B, part_o=po, part_ml=pm, counters=cnt, max_splits=ms,
                      **meta, **kw)

    us = _time(fn, args.iters, args.graph)
    seen = ctx + 1 if not args.window else min(ctx + 1, args.window + args.keep_first)   # the keys a new token sees
    byts = B * seen * 2 * args.kv_heads * args.head_dim * pool.element_size()
    print(f"attn_decode batch={B} ctx={ctx} heads={args.heads}/{args.kv_heads} head_dim={args.head_dim} window={args.window} "
          f"keep_first={args.keep_first} sink={args.sink} {args.dtype}: "
          f"{us:.1f} us/call  cache read {byts / us / 1e3:.1f} GB/s")


def bench_attn_chunk(args) -> None:
    T, ctx = args.tokens, args.ctx
    pool, q, out, meta, kw, i32 = _paged(args, 1, ctx, T)
    mma = K.attn_chunk_mma_takes(q, args.head_dim) and not args.cuda_cores
    tile = K.MMA_QUERY_TILE if mma else 16
    items = torch.tensor([(0, o) for o in range(0, T, tile)], dtype=torch.int32, device="cuda:0")

    tc = mma and not args.mma_sync and K.attn_chunk_tc_takes(q, args.head_dim, args.page_tokens, T, ctx + T)

    extra = {}
    n_splits = 1
    if tc:
        n_splits = K.attn_chunk_tc_splits(items.shape[0], args.heads, ctx + T) if args.key_ranges < 0 else args.key_ranges
        if n_splits > 1:
            n_o, n_ml = T * args.heads * n_splits * args.head_dim, T * args.heads * n_splits * 2
            extra = dict(n_splits=n_splits, part_o=torch.empty(n_o, device="cuda:0"), part_ml=torch.empty(n_ml, device="cuda:0"))
    elif mma:
        n_splits = K.attn_chunk_mma_splits(items.shape[0], args.heads, ctx + T) if args.key_ranges < 0 else args.key_ranges
        if n_splits > 1:
            n_o, n_ml = K.attn_chunk_mma_scratch(args.head_dim)
            extra = dict(n_splits=n_splits, part_o=torch.empty(n_o, device="cuda:0"), part_ml=torch.empty(n_ml, device="cuda:0"))

    def fn():
        call = K.attn_chunk_tc if tc else (K.attn_chunk_mma if mma else K.attn_chunk)
        call(q, pool, out, items=items, n_items=items.shape[0], **meta, **kw, **extra)

    us = _time(fn, args.iters, args.graph)
    flops = 4.0 * args.heads * args.head_dim * (T * ctx + T * (T + 1) / 2)
    print(f"attn_chunk tokens={T} ctx={ctx} heads={args.heads}/{args.kv_heads} head_dim={args.head_dim} window={args.window} "
          f"keep_first={args.keep_first} sink={args.sink} "
          f"{f'tcgen05, {n_splits} key ranges' if tc else (f'mma.sync, {n_splits} key ranges' if mma else 'cuda cores')}: {us:.1f} us/call  {flops / us / 1e6:.1f} TFLOP/s (causal flops)")


def bench_recurrence(args) -> None:
    """The gated linear recurrence over ``--batch`` requests of ``--tokens`` new tokens each (1: the token-by-token
    kernel, as in a decode step; 16 and more: chunk by chunk), or with ``--retention`` the fixed-decay recurrence of the
    same sizes beside it.  Bytes: the states read and written and the operands read; FLOPs: what the chunked form does
    (a chunk's Q K^T and (Q K^T * D) V, Q S and the state's update) or, token by token, the update and S^T q."""
    dev = "cuda:0"
    B, n, H, d, dv, G = args.batch, args.tokens, args.heads, args.head_dim, args.v_dim, args.per_group
    dvx = dv + (1 if args.ones else 0)
    T = B * n
    g = torch.Generator().manual_seed(1)
    q0 = torch.arange(0, T, n, dtype=torch.int32, device=dev)
    qn = torch.full((B,), n, dtype=torch.int32, device=dev)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    if args.delta:
        return _bench_delta(args, B, n, H, d, dv, G, q0, qn, slots, g)
    if args.gla:
        return _bench_gla(args, B, n, H, d, dv, q0, qn, slots, g)
    if args.retention:
        rows = (torch.randn(T, 2 * H * d + 2 * H * dv, generator=g) * 0.3).to(dev)
        state = torch.zeros(B, H, d, dv, device=dev)
        decay = torch.full((H,), 0.99, device=dev)
        out = torch.zeros(T, H * dv, device=dev)

        def fn():
            K.retention_scan(rows, state, slots, q0, qn, B, decay, d ** -0.5, out, n_heads=H, dim=d, v_dim=dv,
                             short=n < K.RETENTION_CHUNK_FROM, long=n >= K.RETENTION_CHUNK_FROM, longest_new=n)
    else:
        Gn = H // G
        rows = (torch.randn(T, 2 * Gn * d + H * dv, generator=g) * 0.3).to(dev)
        keep = (torch.rand(T, H, generator=g) * 0.1 + 0.9).to(dev)
        take = torch.rand(T, H, generator=g).to(dev)
        state = torch.zeros(B, H * d * dvx, device=dev)
        out = torch.zeros(T, H * dvx, device=dev)

        def fn():
            K.gated_recurrence(rows, 0, rows, Gn * d, rows, 2 * Gn * d, keep, take, state, 0, slots, q0, qn, B, out,
                               n_heads=H, heads_per_group=G, dim=d, v_dim=dv, ones=args.ones,
                               short=n < K.RECURRENCE_CHUNK_FROM, long=n >= K.RECURRENCE_CHUNK_FROM, longest_new=n)
    us = _time(fn, args.iters, args.graph)
    by = 4.0 * (2 * B * H * d * dvx + rows.numel() + out.numel())
    fl = 2.0 * T * H * ((32 * d + 32 * dvx if n >= 16 else 0) + 2 * d * dvx)
    print(f"{'retention' if args.retention else 'gated recurrence'}: {B} x {n} tokens, {H} heads of {d} x {dvx}: {us:.1f} us/call, "
          f"{fl / us / 1e6:.2f} TFLOP/s (float32 FMA), {by / us / 1e3:.0f} GB/s")


def _bench_gla(args, B, n, H, d, dv, q0, qn, slots, g) -> None:
    """Gated linear attention at the same sizes: a decay per key channel near 1 (given as 1 - decay).  FLOPs: the decayed
    rank-one update and S^T q per token and head; bytes: the states read and written, the operands, the outputs."""
    dev, T = "cuda:0", B * n
    rows = (torch.randn(T, 2 * H * d + H * dv, generator=g) * 0.3).to(dev)
    lose = (torch.rand(T, H * d, generator=g) * 0.1).to(dev)
    state = torch.zeros(B, H * d * dv, device=dev)
    out = torch.zeros(T, H * dv, device=dev)

    def fn():
        K.gla_scan(rows, 0, rows, H * d, rows, 2 * H * d, lose, 0, state, 0, slots, q0, qn, B, out, n_heads=H, dim=d,
                   v_dim=dv, q_scale=d ** -0.5)
    us = _time(fn, args.iters, args.graph)
    by = 4.0 * (2 * B * H * d * dv + rows.numel() + lose.numel() + out.numel())
    fl = 2.0 * T * H * 2 * d * dv
    print(f"gated linear attention: {B} x {n} tokens, {H} heads of {d} x {dv}: {us:.1f} us/call, "
          f"{fl / us / 1e6:.2f} TFLOP/s (float32 FMA), {by / us / 1e3:.0f} GB/s")


def _bench_delta(args, B, n, H, d, dv, G, q0, qn, slots, g) -> None:
    """The gated delta rule at the same sizes: unit keys, steps in (0, 1), decays near 1.  FLOPs: S^T k, S^T q and the
    decayed rank-one update per token and head; bytes: the states read and written, the operands, the outputs."""
    dev, T, Gn = "cuda:0", B * n, H // G
    q = (torch.randn(T, Gn * d, generator=g) * d ** -0.5).to(dev)
    k = torch.nn.functional.normalize(torch.randn(T, Gn, d, generator=g), dim=-1).reshape(T, Gn * d).to(dev)
    v = (torch.randn(T, H * dv, generator=g) * 0.3).to(dev)
    beta = torch.rand(T, H, generator=g).to(dev)
    decay = (torch.rand(T, H, generator=g) * 0.1 + 0.9).to(dev)
    state = torch.zeros(B, H * d * dv, device=dev)
    out = torch.zeros(T, H * dv, device=dev)

    def fn():
        K.delta_rule(q, 0, k, 0, v, 0, beta, decay, state, 0, slots, q0, qn, B, out, n_heads=H, heads_per_group=G, dim=d,
                     v_dim=dv)
    us = _time(fn, args.iters, args.graph)
    by = 4.0 * (2 * B * H * d * dv + q.numel() + k.numel() + v.numel() + out.numel())
    fl = 2.0 * T * H * 3 * d * dv
    print(f"gated delta rule: {B} x {n} tokens, {H} heads of {d} x {dv}: {us:.1f} us/call, "
          f"{fl / us / 1e6:.2f} TFLOP/s (float32 FMA), {by / us / 1e3:.0f} GB/s")


def bench_head_prep(args) -> None:
    """What stands between a stacked projection and its attention or recurrence, on ``--batch`` requests of ``--tokens``
    new tokens: the short convolution from and into the slot, silu, unit norms and the gates (the delta rule's side), or
    with ``--window`` > 0 the convolution, the rotation, the head norms and the write into pages (the attention side).
    Bytes: the float32 rows read, the outputs written."""
    dev = "cuda:0"
    B, n, H, Hk, d, dv, taps = args.batch, args.tokens, args.heads, args.kv_heads, args.head_dim, args.v_dim, 4
    T = B * n
    g = torch.Generator().manual_seed(1)
    paged = args.window > 0
    heads, dims = ((H, Hk, Hk), (d, d, d)) if paged else ((Hk, Hk, H), (d, d, dv))
    widths = [h * x for h, x in zip(heads, dims)]
    C = sum(widths)
    gh = 0 if paged else H
    proj = (torch.randn(T, C + 2 * gh, generator=g) * 0.5).to(dev)
    conv = (torch.randn(C, taps, generator=g) * 0.5).to(dev).to(torch.bfloat16)
    state = torch.zeros(B, C * (taps - 1), device=dev)
    q0 = torch.arange(0, T, n, dtype=torch.int32, device=dev)
    qn = torch.full((B,), n, dtype=torch.int32, device=dev)
    slots = torch.arange(B, dtype=torch.int32, device=dev)
    pos = torch.arange(n, dtype=torch.int32).repeat(B).to(dev)
    odt = torch.bfloat16 if paged and args.dtype == "bfloat16" else torch.float32
    qo = torch.zeros(T, widths[0], dtype=odt, device=dev)
    offs = (0, widths[0], widths[0] + widths[1])
    if paged:
        P = args.page_tokens
        pool = torch.zeros(-(-T // P), 2, Hk, P, d, dtype=odt, device=dev)
        where = torch.arange(T, dtype=torch.int32, device=dev)
        inv = (1e4 ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)).to(dev)
        kw = dict(q_out=qo, pool=pool, slots=where, page_tokens=P, inv_freq=inv, rot=d, norm="rms", eps=1e-6)
    else:
        ko, vo = torch.zeros(T, widths[1], device=dev), torch.zeros(T, widths[2], device=dev)
        beta, decay = torch.zeros(T, H, device=dev), torch.zeros(T, H, device=dev)
        a_log, dtb = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        kw = dict(q_out=qo, k_out=ko, v_out=vo, act=True, norm="unit", eps=1e-6, q_scale=d ** -0.5,
                  gates=(beta, decay, C, C + H, a_log, dtb))

    def fn():
        K.head_prep(proj, offsets=offs, heads=heads, dims=dims, laid=dims, state_slots=slots, seg_q0=q0, seg_qn=qn, n_seg=B,
                    longest_new=n, positions=pos, conv=conv, state=state, conv_offset=0, **kw)
    us = _time(fn, args.iters, args.graph)
    by = 4.0 * proj.numel() + qo.numel() * qo.element_size() + (2 * T * Hk * d * qo.element_size() if paged else 4.0 * (widths[1] + widths[2] + 2 * H) * T)
    print(f"head_prep ({'attention side' if paged else 'delta side'}): {B} x {n} tokens, {C} channels, {taps} taps: "
          f"{us:.1f} us/call, {by / us / 1e3:.0f} GB/s")


def bench_sample(args) -> None:
    """The sampling kernel on --rows rows of --vocab random float32 logits: greedy, temperature 0.8 alone, with
    top-k 50, with top-p 0.9, with top-k 50 + top-p 0.9 + min-p 0.05.  --one-block keeps every row on the one-block
    kernel (up to 16 rows of 8,192 to 163,840 tokens otherwise go to the cluster kernel)."""
    dev = "cuda:0"
    R, V = args.rows, args.vocab
    K.sample_use_cluster(not args.one_block)
    logits = torch.randn(R, V, device=dev, generator=torch.Generator(dev).manual_seed(1)) * 3
    full = lambda v, dt: torch.full((R,), v, dtype=dt, device=dev)
    out = torch.zeros(R, dtype=torch.int32, device=dev)
    seeds, ctr = torch.arange(R, dtype=torch.int64, device=dev), torch.zeros(R, dtype=torch.int64, device=dev)
    for name, t, k, p, m in (("greedy", 0.0, 0, 1.0, 0.0), ("temperature", 0.8, 0, 1.0, 0.0), ("top-k 50", 0.8, 50, 1.0, 0.0),
                             ("top-p 0.9", 0.8, 0, 0.9, 0.0), ("top-k + top-p + min-p", 0.8, 50, 0.9, 0.05)):
        kw = dict(temperature=full(t, torch.float32), top_k=full(k, torch.int32), top_p=full(p, torch.float32),
                  min_p=full(m, torch.float32), seeds=seeds, counters=ctr, out=out)
        us = _time(lambda: K.sample(logits, **kw), args.iters, args.graph)
        print(f"sample rows={R} vocab={V} {'one block a row' if args.one_block else 'default'} {name}: {us:.1f} us/call")
    K.sample_use_cluster(True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench")
    ap.add_argument("kernel", choices=["linear", "attn_decode", "attn_chunk", "experts", "sample", "recurrence", "head_prep"])
    ap.add_argument("--rows", type=int, default=8, help="sample: rows of logits")
    ap.add_argument("--vocab", type=int, default=151936, help="sample: logits of a row")
    ap.add_argument("--one-block", action="store_true", help="sample: never the cluster kernel")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--graph", action="store_true", help="time a CUDA graph of the calls")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--dual", action="store_true", help="SwiGLU of two weight matrices")
    ap.add_argument("--accumulate", action="store_true", help="add into a float32 output")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4000)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--v-dim", type=int, default=128, help="recurrence: columns of a head's state")
    ap.add_argument("--per-group", type=int, default=1, help="recurrence: heads that share q and k")
    ap.add_argument("--ones", action="store_true", help="recurrence: one column more, whose v is 1")
    ap.add_argument("--retention", action="store_true", help="recurrence: the fixed-decay kernels instead")
    ap.add_argument("--delta", action="store_true", help="recurrence: the gated delta rule instead")
    ap.add_argument("--gla", action="store_true", help="recurrence: gated linear attention (a decay per key channel) instead")
    ap.add_argument("--page-tokens", type=int, default=64)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--keep-first", type=int, default=0, dest="keep_first",
                    help="attention: with --window, a request's first tokens stay in sight")
    ap.add_argument("--sink", action="store_true", help="attention: one more term of score 0 in the softmax's denominator")
    ap.add_argument("--experts", type=int, default=60)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--tile", type=int, default=0, help="experts: rows of a tile instead of the engine's choice")
    ap.add_argument("--part", default="both", choices=["both", "up", "down"], help="experts: which product")
    ap.add_argument("--skinny-rows", type=int, default=-1,
                    help="linear: most rows that go to the weight-streaming kernel instead of the engine's limit")
    ap.add_argument("--token-tile", type=int, default=0,
                    help="linear: token tile of the tcgen05 kernel instead of the engine's choice")
    ap.add_argument("--splits", type=int, default=0,
                    help="linear: with --token-tile, parts along K (0 = not split)")
    ap.add_argument("--cuda-cores", action="store_true", help="attn_chunk: the CUDA-core kernel")
    ap.add_argument("--key-ranges", type=int, default=-1,
                    help="attn_chunk, tensor-core kernels: ranges the keys are cut into (default: the engine's choice)")
    ap.add_argument("--mma-sync", action="store_true", help="attn_chunk: the mma.sync kernel where tcgen05 would run")
    args = ap.parse_args(argv)
    if args.skinny_rows >= 0:
        K.SKINNY_ROWS = args.skinny_rows
        K.FEW_ROWS = min(K.FEW_ROWS, args.skinny_rows)
    if args.token_tile:
        K.tc_plan = lambda m, n, k, dual: (args.token_tile, max(1, args.splits))
    if not torch.cuda.is_available():
        print("kernel_bench: no CUDA device", file=sys.stderr)
        return 1
    {"linear": bench_linear, "attn_decode": bench_attn_decode, "attn_chunk": bench_attn_chunk,
     "experts": bench_experts, "sample": bench_sample, "recurrence": bench_recurrence, "head_prep": bench_head_prep}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
