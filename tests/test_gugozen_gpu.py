"""The Gugozen design on the GPU against the plain implementation (float64), in float32 and in bfloat16: each mechanism
alone (one-layer models) and together, at sizes that are and are not multiples of 8; whole prompts, decoding token by
token, portions down to two tokens, mixed batches with pages and state slots that are used again; configurations drawn at
random on pages of 64; a far key among hundreds, in a prompt and while decoding; long decoding through CUDA graphs; heads
of 128 in long portions; the new kernels alone against their plain twins; greedy generation through the engine's entry
point and the command line; trace replay as a program.  Pages are filled with NaN when they are made and when they go
back."""
import json
import os
import subprocess
import sys

import pytest
import torch

import emulated_kernels as EK
from gugozen_cases import (CONFIGS, Case, attention, compare, compare_together, errors, gla, latent, make_runner, model, random_config, run_steps,
                           schedules, sharpen, with_mlp)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"

# max and mean |error| of the logits (their mean over the vocabulary taken off) relative to the largest |logit|
TOL = {torch.float32: (5e-5, 1e-5), torch.bfloat16: (3e-2, 5e-3)}
# how near a tie of router logits (relative to their spread) the engine may decide the other way
NEAR_TIE = {torch.float32: 2e-5, torch.bfloat16: 5e-2}
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
LENGTHS = {"mix": (1, 2, 37, 70, 45, 19, 130), "odd": (3, 90, 33, 16, 75), "wide": (150, 40, 260), "latent_only": (44, 3, 21),
           "attention_only": (50, 23), "gla_only": (70, 5), "moe_only": (40, 9)}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = Case(name, tmp_path_factory.mktemp("gugozen"), torch.bfloat16, requests=LENGTHS[name])
        return made[name]

    return get


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(LENGTHS))
def test_every_schedule_agrees_with_plain(name, dtype, cases):
    case = cases(name)
    runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=40, max_tokens=320)
    for sched_name, steps in schedules(case).items():
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched_name


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("seed", list(range(6)))
def test_drawn_configurations_on_pages_of_64(seed, dtype, tmp_path_factory):
    """Configurations drawn at random (layer order, head counts and sizes, rotated parts, latents and layers on other
    layers' latents, decays, experts, constants): portions of changing size and mixed batches of four live requests on
    pages of 64 whose pool only holds them when pages are used again."""
    import functools

    raw = random_config(300 + seed)
    # (sharp scores in five to seven post-norm layers amplify the rounding of bfloat16 activations: milder factors there)
    tweak = sharpen if dtype == torch.float32 else functools.partial(sharpen, strength=0.4)
    case = Case(f"drawn{seed}", tmp_path_factory.mktemp("drawn"), torch.bfloat16, raw=raw, requests=(230, 1, 150, 40, 97, 180),
                seed=seed, tweak=tweak)
    runner, cache = make_runner(case, dtype, DEV, page_tokens=64, n_pages=14, max_tokens=256, max_seq=512)
    sch = schedules(case)
    for name in ("mixed", "chunked"):
        got, routed = run_steps(runner, cache, case, sch[name])
        if dtype == torch.bfloat16:
            compare_together(case, got, routed, 0.1, 1.5e-2, one_in=10, cap=3.0)
        else:
            compare(case, got, routed, 2e-4, 4e-5, NEAR_TIE[dtype])   # (five to seven sharpened layers deep)
        assert cache.free_pages() == cache.total_pages()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("page_tokens", [8, 64])
def test_other_page_sizes_and_the_cuda_core_products(page_tokens, dtype, cases, monkeypatch):
    import locus_b200.kernels as K

    case = cases("mix")
    if page_tokens == 8:
        monkeypatch.setattr(K, "USE_TENSOR_CORES", False)   # bfloat16 on the CUDA-core products
    runner, cache = make_runner(case, dtype, DEV, page_tokens=page_tokens, n_pages=24 if page_tokens == 64 else 90,
                                max_tokens=320, max_seq=1024)
    sch = schedules(case)
    for steps in (sch["mixed"], sch["chunked"]):
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_heads_of_128_in_long_portions_on_pages_of_64(dtype, tmp_path_factory):
    """Heads of 128 with values of 96 and four query heads on every key/value head, portions of several hundred tokens
    (the attention kernels that long portions of that head size take, with the learned sink), a recurrence whose state
    has 128 rows, a latent layer on another one's rows, pages of 64."""
    raw = model(256, 301, [with_mlp(attention(8, 2, 128, 96, rot=64, base=5e5, scale=0.1), 8, 2, 96, 1.75, shared=(160, 2.5)),
                           with_mlp(gla(2, 128, 64, tau=12.0), 0),
                           with_mlp(latent(4, 64, 32, 48, 128, scale=0.11), 8, 1, 96, 1.75),
                           with_mlp(latent(4, 64, 32, 48, 128, kv_from=2, scale=0.11), 0)], alpha=3.0, bigram=(997, 131, 11))
    case = Case("big", tmp_path_factory.mktemp("big"), torch.bfloat16, raw=raw, requests=(700, 90))
    runner, cache = make_runner(case, dtype, DEV, page_tokens=64, n_pages=20, max_tokens=640, max_seq=1024)
    steps = [[("r0", 300), ("r1", 40)], [("r0", 399), ("r1", 1)], [("r0", 1), ("r1", 49)]]
    got, routed = run_steps(runner, cache, case, steps)
    if dtype == torch.bfloat16:
        compare_together(case, got, routed, *TOL[dtype])
    else:
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_through_graphs(dtype, cases, tmp_path):
    """Two requests decoded side by side for 200 tokens through CUDA graphs, past several pages: the replayed steps
    against the same steps launched kernel by kernel (whose agreement with the plain implementation the other tests
    hold), and the first and last rows against the plain implementation itself."""
    from locus_b200.engine.step import StepEntry

    case = Case("mix", tmp_path, torch.bfloat16, requests=(230, 215))
    rows = {}
    for graphs in (False, True):
        runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=40, max_tokens=64, use_graphs=graphs)
        seqs = {r: cache.open(r) for r in ("r0", "r1")}
        for r, n in (("r0", 30), ("r1", 15)):
            assert cache.ensure_capacity(seqs[r], n)
            runner.step([StepEntry(seqs[r], case.tokens[r][:n], [n - 1])])
        fed, got = {"r0": 30, "r1": 15}, []
        for _ in range(200):
            entries = []
            for r in ("r0", "r1"):
                assert cache.ensure_capacity(seqs[r], 1)
                entries.append(StepEntry(seqs[r], [case.tokens[r][fed[r]]], [0]))
                fed[r] += 1
            got.append(runner.step(entries).detach().cpu().double().clone())
        runner.check_device_errors()
        rows[graphs] = torch.stack(got)
        if graphs:
            assert runner.stats["graph_replays"] >= 190
    err, mean = errors(rows[True].reshape(400, -1), rows[False].reshape(400, -1))
    assert float(err.max()) <= TOL[dtype][0] and mean <= TOL[dtype][1], (float(err.max()), mean)
    first, _ = errors(rows[True][0, 0][None], case.ref("r0")[0][30][None])
    assert float(first.max()) <= TOL[dtype][0]


# ---------------------------------------------------------------------------
# the new kernels alone against their plain twins (float64)


def _cmp(a, b, tol):
    a, b = a.double().cpu(), b.double().cpu()
    assert bool(torch.isfinite(a).all())
    assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max())), float((a - b).abs().max())


@pytest.fixture
def precise(monkeypatch):
    monkeypatch.setattr(EK, "PRECISE", True)


@pytest.mark.parametrize("H,d,dv", [(2, 24, 16), (1, 7, 5), (3, 72, 40), (2, 128, 64), (1, 200, 12)])
def test_gla_scan_and_decay_against_twin(H, d, dv, precise):
    import locus_b200.kernels as K

    g = torch.Generator().manual_seed(H * 100 + d)
    qn = [1, 37, 2, 100]
    T = sum(qn)
    W = 2 * H * d + H * dv + 4   # (the parts need not start on 16-byte boundaries)
    proj = torch.randn(T, W, generator=g)
    off_q, off_k, off_v = 0, H * d, 2 * H * d + 3
    z = torch.randn(T, H * d, generator=g) * 3.0
    z[0, 0], z[1, 1] = 40.0, -40.0           # decays of 1 and of (nearly) 0
    state = torch.randn(5, H * d * dv + 7, generator=g)
    slots = torch.tensor([3, 0, 4, 1], dtype=torch.int32)
    q0 = torch.tensor([0, 1, 38, 40], dtype=torch.int32)   # (the segments' first rows)
    n = torch.tensor(qn, dtype=torch.int32)

    for tau in (1.0, 16.0):
        ref_z, ref_state, ref_out = z.clone().double(), state.clone().double(), torch.zeros(T, H * dv, dtype=torch.float64)
        EK.gla_decay(ref_z, 0, H * d, tau)
        EK.gla_scan(proj.double(), off_q, proj.double(), off_k, proj.double(), off_v, ref_z, 0, ref_state, 7, slots, q0, n, 4,
                    ref_out, n_heads=H, dim=d, v_dim=dv, q_scale=d ** -0.5)
        dz, ds, dp = z.to(DEV), state.to(DEV), proj.to(DEV)
        out = torch.zeros(T, H * dv, device=DEV)
        K.gla_decay(dz, 0, H * d, tau)
        _cmp(dz, ref_z, 2e-6)
        # cut in two launches: the first tokens of every segment, then the rest, through the state
        first = torch.tensor([min(x, 9) for x in qn], dtype=torch.int32)
        K.gla_scan(dp, off_q, dp, off_k, dp, off_v, dz, 0, ds, 7, slots.to(DEV), q0.to(DEV), first.to(DEV), 4, out,
                   n_heads=H, dim=d, v_dim=dv, q_scale=d ** -0.5)
        rest = n - first
        K.gla_scan(dp, off_q, dp, off_k, dp, off_v, dz, 0, ds, 7, slots.to(DEV), (q0 + first).to(DEV), rest.to(DEV), 4, out,
                   n_heads=H, dim=d, v_dim=dv, q_scale=d ** -0.5)
        # and whole, from the same start
        ds2, out2 = state.to(DEV), torch.zeros(T, H * dv, device=DEV)
        K.gla_scan(dp, off_q, dp, off_k, dp, off_v, dz, 0, ds2, 7, slots.to(DEV), q0.to(DEV), n.to(DEV), 4, out2,
                   n_heads=H, dim=d, v_dim=dv, q_scale=d ** -0.5)
        _cmp(out2, ref_out, 2e-5)
        _cmp(ds2, ref_state, 2e-5)
        _cmp(out, ref_out, 2e-5)
        _cmp(ds, ref_state, 2e-5)


def test_embed_pair_layernorm_post_and_span_norm_against_twins(precise):
    import locus_b200.kernels as K

    g = torch.Generator().manual_seed(3)
    H, V, B = 50, 300, 53
    for dt in (torch.float32, torch.bfloat16):
        table, pair = torch.randn(V, H, generator=g).to(dt), torch.randn(B + 1, H, generator=g).to(dt)
        qn = [1, 6, 9, 2]
        T = sum(qn)
        toks = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
        ctx = [5, 0, 7, 0]
        pos = torch.tensor([c + i for c, n in zip(ctx, qn) for i in range(n)], dtype=torch.int32)
        q0 = torch.tensor([0, 1, 7, 16], dtype=torch.int32)
        n = torch.tensor(qn, dtype=torch.int32)
        slots = torch.tensor([2, 0, 3, 1], dtype=torch.int32)
        last = torch.tensor([[11], [12], [299], [14]], dtype=torch.int32)
        ref, ref_last = torch.zeros(T, H, dtype=torch.float64), last.clone()
        kw = dict(n_seg=4, longest_new=9, mul_prev=1000003, mul_cur=65537)
        EK.embed_pair(toks, pos, table, pair, ref, seg_q0=q0, seg_qn=n, state_slots=slots, last=ref_last, **kw)
        out, dl = torch.zeros(T, H, device=DEV), last.to(DEV)
        K.embed_pair(toks.to(DEV), pos.to(DEV), table.to(DEV), pair.to(DEV), out, seg_q0=q0.to(DEV), seg_qn=n.to(DEV),
                     state_slots=slots.to(DEV), last=dl, **kw)
        _cmp(out, ref, 1e-6)
        assert dl.cpu().tolist() == ref_last.tolist()
        # the norm behind a sum, with the copy for the next sublayer
        x, y = torch.randn(T, H, generator=g) * 3, torch.randn(T + 2, H, generator=g)
        w, b = torch.randn(H, generator=g).to(dt), torch.randn(H, generator=g).to(dt)
        rx = x.clone().double()
        EK.layernorm_post(rx, y.double(), 2.5, w, b, 1e-5)
        dx, cast = x.to(DEV), torch.zeros(T, H, dtype=dt, device=DEV)
        K.layernorm_post(dx, y.to(DEV), 2.5, w.to(DEV), b.to(DEV), 1e-5, cast)
        _cmp(dx, rx, 2e-6)
        _cmp(cast, rx, 2e-6 if dt == torch.float32 else 8e-3)
        # norms over two spans of a wider row
        rows = torch.randn(T, 90, generator=g)
        w0, w1 = torch.randn(37, generator=g).to(dt), torch.randn(20, generator=g).to(dt)
        rr = rows.clone().double()
        EK.span_rmsnorm(rr, [(3, 37, w0), (50, 20, w1)], 1e-6)
        dr = rows.to(DEV)
        K.span_rmsnorm(dr, [(3, 37, w0.to(DEV)), (50, 20, w1.to(DEV))], 1e-6)
        _cmp(dr, rr, 2e-6)
        one = rows.to(DEV)
        K.span_rmsnorm(one, [(50, 20, w1.to(DEV))], 1e-6)
        _cmp(one[:, 50:70], rr[:, 50:70], 2e-6)
        assert torch.equal(one[:, :50].cpu(), rows[:, :50])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("M,tc", [(5, True), (14, True), (100, True), (300, True), (40, False)])
def test_the_clamped_gated_unit_on_every_product_kernel(M, tc, dtype, precise, monkeypatch):
    """The unit as an epilogue of the row-streaming, the weight-streaming, the tcgen05 and the CUDA-core kernel (which
    one runs follows the rows and the element type), with and without a scale on the input, plain and grouped."""
    import locus_b200.kernels as K

    if not tc:
        monkeypatch.setattr(K, "USE_TENSOR_CORES", False)
    g = torch.Generator().manual_seed(M)
    Kd, N, lim = 64, 48, 1.25
    x = (torch.randn(M, Kd, generator=g) * 1.5).to(dtype)
    w, w2 = torch.randn(N, Kd, generator=g).mul(0.3).to(dtype), torch.randn(N, Kd, generator=g).mul(0.3).to(dtype)
    scale, order = torch.rand(M, generator=g), torch.randperm(M, generator=g).to(torch.int32)
    tol = 3e-6 if dtype == torch.float32 else 1.2e-2
    for rs, sr in ((None, None), (scale, None), (scale, order)):
        ref = torch.zeros(M, N, dtype=torch.float64)
        EK.linear(x, w, ref, w2=w2, act="glu_clamp", act_limit=lim, row_scale=rs, scale_rows=sr)
        out = torch.zeros(M, N, dtype=dtype, device=DEV)
        K.linear(x.to(DEV), w.to(DEV), out, w2=w2.to(DEV), act="glu_clamp", act_limit=lim,
                 row_scale=None if rs is None else rs.to(DEV), scale_rows=None if sr is None else sr.to(DEV))
        _cmp(out, ref, tol)
    # grouped: three experts over rows laid out by expert
    E = 3
    we, we2 = torch.randn(E, N, Kd, generator=g).mul(0.3).to(dtype), torch.randn(E, N, Kd, generator=g).mul(0.3).to(dtype)
    ids = torch.randint(0, E, (M,), generator=g, dtype=torch.int32)
    for tile in ((8,) if M <= 8 else (16, 64) if dtype == torch.bfloat16 and tc else (64,)):
        lay_ref, lay = EK.ExpertLayout(M, E, tile, "cpu"), K.ExpertLayout(M, E, tile, DEV)
        EK.moe_sort(ids, M, lay_ref, tile)
        K.moe_sort(ids.to(DEV), M, lay, tile)
        ref = torch.zeros(M, N, dtype=torch.float64)
        EK.linear(x, we, ref, w2=we2, act="glu_clamp", act_limit=lim, row_scale=scale, scale_rows=lay_ref.sorted_pair,
                  x_rows=lay_ref.sorted_pair, layout=lay_ref, n_rows=M)
        out = torch.zeros(M, N, dtype=dtype, device=DEV)
        K.linear(x.to(DEV), we.to(DEV), out, w2=we2.to(DEV), act="glu_clamp", act_limit=lim, row_scale=scale.to(DEV),
                 scale_rows=lay.sorted_pair, x_rows=lay.sorted_pair, layout=lay, n_rows=M)
        _cmp(out, ref, tol)
    with pytest.raises(K.KernelError):
        K.linear(x.to(DEV), w.to(DEV), out, act="glu_clamp", act_limit=lim)


@pytest.mark.parametrize("nh,nkv,hd,dtype", [(6, 2, 128, torch.bfloat16), (8, 2, 64, torch.bfloat16), (2, 2, 128, torch.bfloat16),
                                             (3, 1, 96, torch.bfloat16), (4, 2, 64, torch.float32)],
                         ids=["6on2_128", "8on2_64", "2on2_128", "3on1_96", "f32_4on2_64"])
def test_every_attention_kernel_with_a_learned_sink(nh, nkv, hd, dtype):
    """A learned score per query head in the softmax's denominator, from far below the keys' scores to above them:
    the portion kernels (tcgen05 whole and with its keys cut into ranges, mma.sync, CUDA cores) and the decode kernels
    (streaming per head and per group of query heads in both variants, fixed ranges) against the twin in float64, a
    batch and requests alone; the sink is not multiplied by the scores' factor."""
    import locus_b200.kernels as K
    from test_mekizen_gpu import _close, _paged_attention_case

    P = 64
    sink = torch.linspace(-3.0, 2.5, nh)
    tol = 1.5e-2 if dtype == torch.bfloat16 else 2e-5
    # portions
    segs = [(0, 5), (33, 17), (100, 2), (64, 64), (190, 130), (600, 70)]
    pool, q, meta, T = _paged_attention_case(dtype, nh, nkv, hd, P, segs, 0, 0, seed=nh + hd)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=0, scale=0.11)
    items64 = torch.tensor([(s, o) for s, (c, n) in enumerate(segs) for o in range(0, n, K.MMA_QUERY_TILE)], dtype=torch.int32)
    items16 = torch.tensor([(s, o) for s, (c, n) in enumerate(segs) for o in range(0, n, 16)], dtype=torch.int32)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.PRECISE = True
    try:
        EK.attn_chunk(q, pool, ref, items=items16, n_items=len(items16), sink=sink, **meta, **kw)
        plain_ref = torch.zeros(T, nh * hd, dtype=torch.float64)
        EK.attn_chunk(q, pool, plain_ref, items=items16, n_items=len(items16), sink=True, **meta, **kw)
    finally:
        EK.PRECISE = False
    assert not _close(plain_ref, ref, 10 * tol)     # (a sink of score 0 in its place is far away)
    dev = {k: v.cuda() for k, v in meta.items()}
    dsink = sink.cuda()

    def fresh():
        return torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")

    if K.attn_chunk_tc_takes(q.cuda(), hd, P, T, 2048):
        out = fresh()
        K.attn_chunk_tc(q.cuda(), pool.cuda(), out, items=items64.cuda(), n_items=len(items64), sink=dsink, **dev, **kw)
        assert K.attn_tc_error() == 0 and _close(out, ref, tol), "attn_chunk_tc"
        for n_splits in (2, 7):
            part_o = torch.full((T * nh * n_splits * hd,), float("nan"), device="cuda")
            part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device="cuda")
            out = fresh()
            K.attn_chunk_tc(q.cuda(), pool.cuda(), out, items=items64.cuda(), n_items=len(items64), n_splits=n_splits,
                            part_o=part_o, part_ml=part_ml, sink=dsink, **dev, **kw)
            assert K.attn_tc_error() == 0 and _close(out, ref, tol), f"attn_chunk_tc in {n_splits} key ranges"
    if K.attn_chunk_mma_takes(q.cuda(), hd):
        out = fresh()
        K.attn_chunk_mma(q.cuda(), pool.cuda(), out, items=items64.cuda(), n_items=len(items64), sink=dsink, **dev, **kw)
        assert _close(out, ref, tol), "attn_chunk_mma"
        n_o, n_ml = K.attn_chunk_mma_scratch(hd)
        part_o, part_ml = torch.full((n_o,), float("nan"), device="cuda"), torch.full((n_ml,), float("nan"), device="cuda")
        some = items64[-2:]     # (the last request's tiles, behind 600 keys, cut into ranges)
        out = fresh()
        K.attn_chunk_mma(q.cuda(), pool.cuda(), out, items=some.cuda(), n_items=len(some), n_splits=4, part_o=part_o,
                         part_ml=part_ml, sink=dsink, **dev, **kw)
        lo = int(meta["seg_q0"][-1])
        assert _close(out[lo:], ref[lo:], tol), "attn_chunk_mma in 4 key ranges"
    out = fresh()
    K.attn_chunk(q.cuda(), pool.cuda(), out, items=items16.cuda(), n_items=len(items16), sink=dsink, **dev, **kw)
    assert _close(out, ref, tol), "attn_chunk"
    # single tokens
    ctxs = [0, 1, 31, 32, 33, 63, 64, 100, 130, 200, 263, 333, 461, 700, 1023, 1100]
    segs = [(c, 1) for c in ctxs]
    pool, q, meta, T = _paged_attention_case(dtype, nh, nkv, hd, P, segs, 0, 0, seed=nh + hd + 1)
    items = torch.arange(len(segs), dtype=torch.int32)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.PRECISE = True
    try:
        EK.attn_chunk(q, pool, ref, items=torch.stack([items, torch.zeros_like(items)], 1), n_items=len(items), sink=sink, **meta, **kw)
    finally:
        EK.PRECISE = False
    dev = {k: v.cuda() for k, v in meta.items()}
    max_splits = (max(ctxs) // K.DECODE_SPLIT) + 1
    units = K.decode_units(len(segs), nh, hd, dtype, max_splits, "cuda", page_tokens=P, n_kv_heads=nkv)
    part_o = torch.full((units * hd,), float("nan"), device="cuda")
    part_ml = torch.full((units * 2,), float("nan"), device="cuda")
    counters = torch.zeros(len(segs) * nh, dtype=torch.int32, device="cuda")
    use_gqa, ran_gqa = K.USE_GQA_DECODE, False
    try:
        for gqa, deep in [(g, d) for g in (True, False) for d in (None, True, False)]:
            if gqa and not K.attn_decode_gqa_takes(dtype, nh, nkv, hd, P, len(segs)):
                continue
            ran_gqa = ran_gqa or gqa
            K.USE_GQA_DECODE = gqa
            K.attn_decode_variant(deep)
            K.attn_decode_gqa_variant(deep)
            what = f"{'grouped' if gqa else 'per head'}, variant {deep}"
            out = fresh()
            K.attn_decode(q.cuda(), pool.cuda(), out, items=items.cuda(), n_items=len(items), part_o=part_o, part_ml=part_ml,
                          counters=counters, max_splits=max_splits, sink=dsink, **dev, **kw)
            assert K.attn_error() == 0 and K.attn_gqa_error() == 0
            assert _close(out, ref, tol), what
            assert int(counters.abs().sum()) == 0
            for lo, hi in ((5, 6), (len(segs) - 1, len(segs)), (len(segs) - 16, len(segs))):
                one = fresh()
                K.attn_decode(q.cuda(), pool.cuda(), one, items=items[lo:hi].cuda(), n_items=hi - lo, part_o=part_o,
                              part_ml=part_ml, counters=counters, max_splits=max_splits, sink=dsink, **dev, **kw)
                assert _close(one[lo:hi], ref[lo:hi], tol), f"{what}, requests {lo} to {hi} alone"
    finally:
        K.USE_GQA_DECODE = use_gqa
        K.attn_decode_variant(None)
        K.attn_decode_gqa_variant(None)
    if dtype == torch.bfloat16 and nh != nkv and hd in (64, 128):
        assert ran_gqa, "the grouped decode kernel did not take this shape"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_among_hundreds_in_a_prompt_and_in_decoding(dtype, tmp_path_factory):
    """One early token whose embedding is scaled up draws the attention of every later query (softmax and latent
    layers) and sits in every later state (the recurrence); the plain implementation without that token's scaling differs
    by far more than the tolerance at the probes, which lie hundreds of tokens and several pages later, once inside a
    prompt's portion and once decoded one by one."""
    def tweak(name, w):
        sharpen(name, w)
        w["embed"][7] = w["embed"][7] * 5.0

    raw = model(64, 60, [with_mlp(attention(4, 2, 16, 16, rot=8), 0), with_mlp(latent(2, 16, 8, 16, 24), 0),
                         with_mlp(gla(2, 16, 16, tau=64.0), 0)], bigram=(53, 31, 5))
    case = Case("far", tmp_path_factory.mktemp("far"), torch.bfloat16, raw=raw, requests=(420,), tweak=tweak)
    case.tokens["r0"] = [7 if i == 3 else (t if t != 7 else 8) for i, t in enumerate(case.tokens["r0"])]
    runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=40, max_tokens=448)
    for steps in ([[("r0", 420)]], [[("r0", 400)]] + [[("r0", 1)]] * 20, [[("r0", 333)], [("r0", 2)], [("r0", 85)]]):
        got, routed = run_steps(runner, cache, case, steps)
        compare(case, got, routed, *TOL[dtype], NEAR_TIE[dtype])
    # the probe is worth its name: without the marker the last rows are far away
    import plain_gugozen as plain
    other = list(case.tokens["r0"])
    other[3] = 9
    moved, _ = errors(plain.forward(case.cfg, case.weights, other)[0][400:], case.ref("r0")[0][400:])
    assert float(moved.median()) > 20 * TOL[torch.float32][0]


def test_generation_through_the_engine_and_the_command_line(cases):
    from locus_b200.engine.engine import Engine
    import plain_gugozen as plain

    case = cases("mix")
    prompts = [case.tokens["r2"], case.tokens["r5"]]
    eng = Engine.from_model_dir(case.dir, dtype="float32", ctx=512, page_tokens=16, max_batch_tokens=32, chunk=16, max_running=4)
    out = eng.generate(prompts, max_new_tokens=8)
    for p, o in zip(prompts, out):
        ref = plain.forward(case.cfg, case.weights, p + o)[0]
        for i, tok in enumerate(o):
            row = ref[len(p) + i - 1]
            assert float(row.max() - row[tok]) <= 1e-4 * float(ref.abs().max()), (i, tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), case.dir, ",".join(map(str, prompts[0])), "8",
                        "--dtype", "float32", "--page-tokens", "16", "--ctx", "512"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    said = [int(x) for x in r.stdout.replace(",", " ").split() if x.lstrip("-").isdigit()]
    assert said[-8:] == list(out[0]), (said[-8:], out[0])
    archs = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), "--archs"], capture_output=True, text=True)
    assert "Gugozen" in archs.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_program(dtype, cases, tmp_path):
    case = cases("mix")
    out = tmp_path / "out"
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": case.tokens["r2"][:20], "want": [0, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": case.tokens["r2"][20:22], "want": [1]},
                                     {"id": "b", "tokens": case.tokens["r5"], "want": [18]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": case.tokens["r2"][22:23], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", case.dir, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    import numpy as np
    ref2, ref5 = case.ref("r2")[0], case.ref("r5")[0]
    want = {0: ref2[[0, 19]], 1: torch.stack([ref2[21], ref5[18]]), 2: ref2[[22]]}
    tol = TOL[torch.float32 if dtype == "float32" else torch.bfloat16][0]
    for s, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(ref.shape[0], -1)).double()
        err, _ = errors(got, ref)
        assert float(err.max()) <= tol * 3, (s, float(err.max()))
