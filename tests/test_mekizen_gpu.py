"""The Mekizen design on the GPU against the plain implementation (float64), in float32 and in bfloat16: each
mechanism alone (one-layer models) and together, at sizes that are and are not multiples of 8; whole prompts, decoding
token by token, portions down to two tokens, mixed batches with pages and state slots that are used again; a key just
inside and just outside a window and the kept first tokens, in prompts and while decoding; long decoding through CUDA
graphs; other page sizes; heads of 128 in long portions; the new kernels alone against their plain twins; greedy
generation through the engine's entry point and the command line; trace replay as a program.  Pages are filled with
NaN when they are made and when they go back."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import emulated_kernels as EK
import plain_mekizen as plain
from mekizen_cases import (CONFIGS, Case, attention, compare, compare_together, make_runner, model, parallel, random_config,
                           run_steps, schedules, sharpen, tokens as draw, with_mlp)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"

# max and mean |error| of the logits (their mean over the vocabulary taken off) relative to the largest |logit|
TOL = {torch.float32: (5e-5, 1e-5), torch.bfloat16: (3e-2, 5e-3)}
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
# heads of 3 to 10 elements, a window of one token: in bfloat16 single rows amplify the activations' rounding
AMPLIFIES = {"odd"}
LENGTHS = {"mix": (1, 2, 37, 70, 45, 19, 130), "odd": (3, 90, 33, 16, 75), "wide": (150, 40, 260), "shared_kv": (44, 3, 21),
           "conv_attention_only": (70, 5), "delta_only": (70, 5), "attention_only": (50, 23)}


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = Case(name, tmp_path_factory.mktemp("mekizen"), torch.bfloat16, requests=LENGTHS[name])
        return made[name]

    return get


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(LENGTHS))
def test_every_schedule_agrees_with_plain(name, dtype, cases):
    case = cases(name)
    runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=40, max_tokens=320)
    for sched_name, steps in schedules(case).items():
        got = run_steps(runner, cache, case, steps)
        (compare_together if dtype == torch.bfloat16 and name in AMPLIFIES else compare)(case, got, *TOL[dtype])
        assert cache.free_pages() == cache.total_pages() and cache.state_slots.free == cache.state_slots.total, sched_name


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("seed", list(range(8)))
def test_drawn_configurations_on_pages_of_64(seed, dtype, tmp_path_factory):
    """Configurations drawn at random (layer order, head counts and sizes, rotated parts, windows, kept tokens, taps,
    layers on other layers' keys and values, constants): portions of changing size and mixed batches of four live
    requests on pages of 64 whose pool only holds them when pages are used again."""
    raw = random_config(200 + seed)
    case = Case(f"drawn{seed}", tmp_path_factory.mktemp("drawn"), torch.bfloat16, raw=raw, requests=(230, 1, 150, 40, 97, 180),
                seed=seed)
    full = any(l["type"] == "parallel" or "mask" not in l["mixer"] for l in raw["layers"])
    runner, cache = make_runner(case, dtype, DEV, page_tokens=64, n_pages=14 if full else 12, max_tokens=256, max_seq=512)
    sch = schedules(case)
    for name in ("mixed", "chunked"):
        got = run_steps(runner, cache, case, sch[name])
        (compare_together if dtype == torch.bfloat16 else compare)(case, got, *TOL[dtype])
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
        got = run_steps(runner, cache, case, steps)
        compare(case, got, *TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_heads_of_128_in_long_portions_on_pages_of_64(dtype, tmp_path_factory):
    """Heads of 128 with grouped queries on both sides, portions of several hundred tokens (the attention kernels that
    long portions of that head size take, with and without the window, the kept tokens and the sink), a delta rule
    whose state has 128 rows, a layer on another layer's pages, pages of 64."""
    raw = model(256, 301, [with_mlp(parallel(4, 2, 128, 128, 4, 64, 4, 2, 128, 128, 4, base=1e6), 128),
                           with_mlp(attention(8, 2, 128, 128, window=200, keep_first=7, rot=128), 64),
                           with_mlp(attention(4, 2, 128, 128, window=333, keep_first=3, rot=128, kv_from=1), None)], embed_scale=2.0)
    case = Case("big", tmp_path_factory.mktemp("big"), torch.bfloat16, raw=raw, requests=(700, 90))
    runner, cache = make_runner(case, dtype, DEV, page_tokens=64, n_pages=20, max_tokens=640, max_seq=1024)
    steps = [[("r0", 300), ("r1", 40)], [("r0", 399), ("r1", 1)], [("r0", 1), ("r1", 49)]]
    got = run_steps(runner, cache, case, steps)
    compare(case, got, *TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("marker,edge", [(20, "window"), (2, "kept")])
def test_window_and_kept_edges_in_prompts_and_in_decoding(marker, edge, dtype, tmp_path_factory):
    """A token that the rest of the sequence attends to strongly (its embedding is scaled up) sits just inside the
    window of one query and just outside the next one's, or is the last token that the mask keeps or the first that it
    does not.  The oracle with a mask one larger tells the positions apart by much more than the tolerance; the
    probes are the positions around the edge, once inside a prompt's portion and once decoded one by one."""
    def tweak(name, w):
        sharpen(name, w)
        w["embed"][7] = w["embed"][7] * 6.0

    window, keep = 9, (2 if edge == "window" else 3)
    raw = model(48, 50, [with_mlp(attention(4, 2, 16, 16, window=window, keep_first=keep, rot=16), None)])
    case = Case(f"edge_{edge}", tmp_path_factory.mktemp("edge"), torch.bfloat16, raw=raw, requests=(48, 48), tweak=tweak)
    for rid in case.tokens:
        t = [x if x != 7 else 8 for x in case.tokens[rid]]
        t[marker] = 7
        case.tokens[rid] = t
    ref = case.ref("r0")
    top = float(ref.abs().max())
    other = json.loads(json.dumps(case.cfg))
    if edge == "window":
        other["layers"][0]["mixer"]["mask"]["size"] = window + 1
        probe = marker + window          # the first position that no longer sees the marker
    else:
        other["layers"][0]["mixer"]["mask"]["keep_first"] = keep - 1
        probe = 30                       # far behind the window: only a kept token is seen
    moved = plain.forward(case.weights, other, case.tokens["r0"])
    assert float((moved[probe] - ref[probe]).abs().max()) > 20 * TOL[torch.float32][0] * top
    runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=16, max_tokens=128)
    first = marker + window - 3
    steps = [[("r0", 35), ("r1", first)]] + [[("r0", 13), ("r1", 1)]] + [[("r1", 1)]] * 6 + [[("r1", 48 - first - 7)]]
    got = run_steps(runner, cache, case, steps)
    compare(case, got, *TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_through_graphs_keeps_states_windows_and_kept_tokens(dtype, tmp_path_factory):
    """200 tokens decoded one by one for two requests side by side, replayed from CUDA graphs: the delta rule's state
    and both sides' convolution inputs are carried in their slot, the window's pages go back while the kept tokens'
    page stays, a later layer reads the earlier layer's pages."""
    raw = model(64, 83, [with_mlp(parallel(2, 1, 16, 16, 3, 8, 2, 1, 16, 16, 4), 32),
                         with_mlp(attention(4, 2, 16, 16, window=24, keep_first=3, rot=8), None),
                         with_mlp(parallel(4, 4, 16, 32, 2, 16, 4, 2, 8, 8, 2), None),
                         with_mlp(attention(2, 2, 16, 16, window=40, keep_first=1, rot=8, kv_from=1), 32)], embed_scale=2.0)
    case = Case("long", tmp_path_factory.mktemp("long"), torch.bfloat16, raw=raw)
    case.tokens["long0"] = draw(20 + 200, case.cfg["vocab"], 77)
    case.tokens["long1"] = draw(3 + 200, case.cfg["vocab"], 78)
    runner, cache = make_runner(case, dtype, DEV, page_tokens=16, n_pages=60, max_tokens=64, use_graphs=True)
    steps = [[("long0", 20), ("long1", 3)]] + [[("long0", 1), ("long1", 1)]] * 200
    got = run_steps(runner, cache, case, steps)
    assert runner.stats["graph_replays"] > 150
    compare(case, got, *TOL[dtype])


def _rand(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


def _dev(v):
    return torch.tensor(v, dtype=torch.int32).cuda()


def _close(a, b, rel):
    b = b.double()
    return float((a.detach().cpu().double() - b.cpu()).abs().max()) <= rel * max(float(b.abs().max()), 1e-30)


@pytest.mark.parametrize("aligned", [False, True], ids=["odd_offsets", "aligned"])
@pytest.mark.parametrize("heads,per_group,dim,v_dim", [(2, 1, 16, 8), (3, 1, 12, 10), (4, 2, 72, 40), (2, 2, 256, 33),
                                                       (6, 3, 5, 3), (2, 1, 128, 128), (2, 1, 64, 6), (1, 1, 200, 4)])
def test_delta_rule_against_its_twin(heads, per_group, dim, v_dim, aligned):
    """Segments of unequal length (one token, two, and more than a hundred) from states that are not zero, with steps
    of 0 and 1 and decays of 0 and 1 among them, against the twin in float64; then the same tokens cut in two
    launches, the state handed on through its slot; what lies in front of the heads in a slot is not touched."""
    import locus_b200.kernels as K

    G = heads // per_group
    segs, starts = [19, 1, 40, 2, 135], [0, 19, 20, 60, 62]
    T = sum(segs)
    # (q's and k's rows of a head on 16-byte boundaries: four rows are one load; otherwise one by one)
    off_q, off_k, off_v = (4, G * dim + 8, 2 * G * dim + 12) if aligned else (3, G * dim + 3, 2 * G * dim + 5)
    width = off_v + heads * v_dim + 2
    rows = _rand((T, -(-width // 4) * 4 if aligned else width + (1 - width % 2)), 5, 0.6)
    kcols = rows[:, off_k:off_k + G * dim].view(T, G, dim)
    kcols /= kcols.norm(dim=-1, keepdim=True)          # unit keys, as the mixer makes them
    beta = torch.rand(T, heads, generator=torch.Generator().manual_seed(2)).cuda()
    decay = torch.rand(T, heads, generator=torch.Generator().manual_seed(1)).cuda() * 0.5 + 0.5
    beta[3], beta[70], decay[5], decay[30] = 0.0, 1.0, 0.0, 1.0
    slots = _dev([2, 0, 3, 1, 4])
    state0 = _rand((5, 7 + heads * dim * v_dim), 6, 0.3)
    q0, qn = _dev(starts), _dev(segs)
    kw = dict(n_heads=heads, heads_per_group=per_group, dim=dim, v_dim=v_dim)

    def run(fn, rows_, beta_, decay_, state_, slots_, q0_, qn_, out_):
        fn(rows_, off_q, rows_, off_k, rows_, off_v, beta_, decay_, state_, 7, slots_, q0_, qn_, len(segs), out_, **kw)

    state, out = state0.clone(), torch.zeros(T, heads * v_dim, device="cuda")
    run(K.delta_rule, rows, beta, decay, state, slots, q0, qn, out)
    EK.PRECISE = True
    try:
        st_w, out_w = state0.cpu().double(), torch.zeros(T, heads * v_dim, dtype=torch.float64)
        run(EK.delta_rule, rows.cpu(), beta.cpu(), decay.cpu(), st_w, slots.cpu(), q0.cpu(), qn.cpu(), out_w)
    finally:
        EK.PRECISE = False
    assert _close(out, out_w, 3e-5) and _close(state, st_w, 3e-5)
    assert torch.equal(state[:, :7], state0[:, :7])
    state2, out2 = state0.clone(), torch.zeros(T, heads * v_dim, device="cuda")
    first = [n // 2 for n in segs]
    run(K.delta_rule, rows, beta, decay, state2, slots, q0, _dev(first), out2)
    run(K.delta_rule, rows, beta, decay, state2, slots, _dev([a + f for a, f in zip(starts, first)]),
        _dev([n - f for n, f in zip(segs, first)]), out2)
    assert _close(out2, out_w, 3e-5) and _close(state2, st_w, 3e-5)


@pytest.mark.parametrize("odt", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,v_dim,shared", [(2, 8, True), (3, 10, False), (1, 40, True), (4, 128, True)])
def test_delta_output_stage_and_gate_rows_against_their_twins(heads, v_dim, shared, odt):
    import locus_b200.kernels as K

    T, off_g = 37, 5
    o = _rand((T, heads * v_dim), 1, 2.0)
    proj = _rand((T, off_g + heads * v_dim + 3), 2, 1.5)
    w = _rand((v_dim if shared else heads * v_dim,), 3, 1.0, torch.bfloat16)
    out = torch.zeros(T, heads * v_dim, dtype=odt, device="cuda")
    K.delta_out(o, proj, off_g, w, 1e-5, out, n_heads=heads, v_dim=v_dim)
    want = torch.zeros(T, heads * v_dim, dtype=torch.float64)
    EK.PRECISE = True
    try:
        EK.delta_out(o.cpu(), proj.cpu(), off_g, w.cpu(), 1e-5, want, n_heads=heads, v_dim=v_dim)
        laid = -(-v_dim // 16) * 16
        rows = _rand((T, heads * laid), 4, 1.0, odt)
        gated = rows.clone()
        K.gate_rows(gated, proj, off_g, n_heads=heads, dim=v_dim, laid=laid)
        want_rows = rows.cpu().double()
        EK.gate_rows(want_rows, proj.cpu(), off_g, n_heads=heads, dim=v_dim, laid=laid)
    finally:
        EK.PRECISE = False
    tol = 1e-5 if odt == torch.float32 else 6e-3
    assert _close(out, want, tol) and _close(gated, want_rows, tol)


@pytest.mark.parametrize("odt", DTYPES, ids=IDS)
@pytest.mark.parametrize("heads,dims,taps,rot,norm,act,gated,paged", [
    ((4, 2, 2), (16, 16, 8), 3, 8, "rms", False, False, True),      # the attention side: rotation, head norms, pages
    ((2, 2, 4), (16, 16, 12), 4, 0, "unit", True, True, False),     # the delta rule's side: silu, unit norms, gates
    ((3, 1, 1), (10, 10, 6), 5, 6, "rms", False, False, True),      # nothing a multiple of 4, five taps
    ((1, 1, 3), (7, 7, 5), 1, 0, "unit", True, True, False),        # one tap: no inputs carried
    ((2, 1, 1), (128, 128, 128), 2, 64, None, False, False, True),  # wide heads, no norm
])
def test_head_prep_against_its_twin(heads, dims, taps, rot, norm, act, gated, paged, odt):
    """The convolution reads a portion's earlier inputs from the slot (not zero here), also when the portion is shorter
    than the convolution's reach, and moves them on; rotation by true positions; norms; gates; rows or pages."""
    import locus_b200.kernels as K

    segs, starts, pos0 = [9, 1, 2, 30], [0, 9, 10, 12], [0, 50, 3, 1000]
    T, page_tokens = sum(segs), 16
    widths = [h * d for h, d in zip(heads, dims)]
    offsets = (2, 2 + widths[0] + 1, 2 + widths[0] + 1 + widths[1] + 3)
    H = heads[2]
    off_b = offsets[2] + widths[2] + 1
    off_a = off_b + H
    proj = _rand((T, off_a + H + 2), 11, 1.2)
    C = sum(widths)
    conv = _rand((C, taps), 12, 0.7, torch.bfloat16)
    conv_off = 5
    state0 = _rand((6, conv_off + C * (taps - 1) + 2), 13, 0.8)
    slots_state = _dev([3, 0, 5, 2])
    positions = _dev([p + i for p, n in zip(pos0, segs) for i in range(n)])
    inv_freq = (1e4 ** (-torch.arange(0, rot, 2, dtype=torch.float32) / rot)).cuda() if rot else None
    laid = tuple(-(-d // 16) * 16 for d in dims) if paged else dims
    if paged:
        laid = (laid[0], max(laid[1], laid[2]), max(laid[1], laid[2]))
    a_log, dt_bias = _rand((H,), 14, 1.0), _rand((H,), 15, 1.0)
    cache_slots = torch.randperm(8 * page_tokens, generator=torch.Generator().manual_seed(16))[:T].to(torch.int32).cuda()

    def run(mod, dev):
        cv = (lambda t: t) if dev else (lambda t: None if t is None else t.cpu())
        dt = odt if dev else torch.float64
        mk = (lambda *s: torch.zeros(*s, dtype=dt, device="cuda" if dev else "cpu"))
        q = mk(T, heads[0] * laid[0])
        k = v = pool = None
        if paged:
            pool = mk(8, 2, heads[1], page_tokens, laid[1])
        else:
            k, v = mk(T, heads[1] * laid[1]), mk(T, heads[2] * laid[2])
        state = state0.clone() if dev else state0.cpu().double()
        beta = torch.zeros(T, H, dtype=torch.float32 if dev else torch.float64, device=q.device)
        decay = torch.zeros_like(beta)
        mod.head_prep(cv(proj), offsets=offsets, heads=heads, dims=dims, laid=laid, state_slots=cv(slots_state),
                      seg_q0=cv(_dev(starts)), seg_qn=cv(_dev(segs)), n_seg=len(segs), longest_new=max(segs),
                      positions=cv(positions), q_out=q, k_out=k, v_out=v, pool=pool, slots=cv(cache_slots) if paged else None,
                      page_tokens=page_tokens if paged else 0, conv=cv(conv), state=state, conv_offset=conv_off, act=act,
                      inv_freq=cv(inv_freq), rot=rot, norm=norm, eps=1e-6, q_scale=0.37,
                      gates=(beta, decay, off_b, off_a, cv(a_log), cv(dt_bias)) if gated else None)
        return q, k, v, pool, state, beta, decay

    got = run(K, True)
    EK.PRECISE = True
    try:
        want = run(EK, False)
    finally:
        EK.PRECISE = False
    tol = 2e-5 if odt == torch.float32 else 6e-3
    for g, w, t in zip(got, want, (tol, tol, tol, tol, 1e-6, 2e-5, 2e-5)):
        if g is not None:
            assert _close(g, w, t)
    assert torch.equal(got[4][:, :conv_off], state0[:, :conv_off])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_entry_point(dtype, cases):
    from locus_b200.engine.engine import Engine

    case = cases("mix")
    eng = Engine.from_model_dir(case.dir, dtype="float32" if dtype == torch.float32 else "bfloat16", ctx=512,
                                page_tokens=16, max_batch_tokens=64, chunk=32, max_running=3)
    prompts = [case.tokens[r] for r in ("r2", "r3", "r5", "r1")]
    outs = eng.generate(prompts, max_new_tokens=12)
    gap = 1e-3 if dtype == torch.float32 else 5e-2
    for p, o in zip(prompts, outs):
        seq = list(p)
        assert len(o) == 12
        for tok in o:
            lg = plain.forward(case.weights, case.cfg, seq)
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > gap * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()


def test_trace_replay_as_a_program(cases, tmp_path):
    """bin/trace_run on a model folder of this design: portions beside single tokens with four live requests and a
    pool that only holds them when pages are used again; logits against the plain implementation."""
    case = cases("mix")
    steps = schedules(case)["mixed"]
    fed, lines, want_rows = {}, [], []
    for n, step in enumerate(steps):
        entries, end = [], []
        for rid, k in step:
            a = fed.get(rid, 0)
            entries.append({"id": rid, "tokens": case.tokens[rid][a:a + k], "want": [0, k - 1] if k > 1 else [0]})
            want_rows += [(n, rid, a)] + ([(n, rid, a + k - 1)] if k > 1 else [])
            fed[rid] = a + k
            if fed[rid] == len(case.tokens[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", case.dir, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "320", "--page-tokens", "16"],
                           input="\n".join(lines) + "\n", text=True, capture_output=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {n}" for n in range(len(steps))]
        tol = TOL[torch.float32 if dtype == "float32" else torch.bfloat16][0]
        V, at = case.cfg["vocab"], {}
        for n, rid, pos in want_rows:
            rows = torch.from_file(str(out / f"{n}.f32"), size=os.path.getsize(out / f"{n}.f32") // 4,
                                   dtype=torch.float32).view(-1, V).double()
            i = at.get(n, 0)
            at[n] = i + 1
            ref = case.ref(rid)
            err, _ = errors_of(rows[i:i + 1], ref[pos:pos + 1], ref)
            assert err <= tol, f"{dtype} step {n} {rid} position {pos}: off by {err:.2e}"


def errors_of(out, ref_rows, ref_all):
    d = out - ref_rows
    d = d - d.mean(-1, keepdim=True)
    top = float((ref_all - ref_all.mean(-1, keepdim=True)).abs().max())
    return float(d.abs().max()) / top, top


def test_the_command_line_generates_from_a_folder_of_this_design(cases):
    """bin/locus-run: the architecture is found by config.json, the weights by name, and greedy generation gives the
    plain implementation's tokens (where its two best logits are not a near-tie)."""
    case = cases("mix")
    prompt = case.tokens["r3"][:12]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), case.dir, ",".join(map(str, prompt)), "8",
                        "--dtype", "float32", "--page-tokens", "16", "--ctx", "128"], capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.replace(",", " ").split() if x.lstrip("-").isdigit()]
    assert len(out) >= 8
    seq = list(prompt)
    for tok in out[-8:]:
        lg = plain.forward(case.weights, case.cfg, seq)
        top2 = torch.topk(lg[-1], 2).values
        if float(top2[0] - top2[1]) > 1e-3 * float(lg[-1].abs().max()):
            assert int(torch.argmax(lg[-1])) == tok
        seq.append(tok)
    archs = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "locus-run"), "--archs"], capture_output=True, text=True)
    assert "Mekizen" in archs.stdout


def _paged_attention_case(dtype, nh, nkv, hd, P, segs, window, keep_first, seed):
    """Requests (cached tokens, new tokens) on shuffled pages; a page that lies wholly between the kept first tokens
    and the window of the request's first new token has gone back (no entry in the table; the pool's unused pages are
    NaN), and so is NaN whatever lies in a request's pages behind its last token."""
    g = torch.Generator().manual_seed(seed)
    need = [-(-(c + n) // P) for c, n in segs]
    n_pages = sum(need) + 2
    pool = torch.randn(n_pages, 2, nkv, P, hd, generator=g).to(dtype)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(segs), max(need)), -1, dtype=torch.int32)
    used, q0s, T = 0, [], 0
    for s, (c, n) in enumerate(segs):
        lo = max(0, c - window + 1) if window else 0
        for pg in range(need[s]):
            page = perm[used]
            used += 1
            if window and pg * P >= keep_first and (pg + 1) * P <= lo:
                pool[page] = float("nan")
                continue
            table[s, pg] = page
        end = c + n
        if end % P:
            pool[int(table[s, end // P]), :, :, end % P:, :] = float("nan")
        q0s.append(T)
        T += n
    for page in perm[used:]:
        pool[page] = float("nan")
    q = torch.randn(T, nh * hd, generator=g).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    meta = dict(seg_q0=i32(q0s), seg_qn=i32([n for _, n in segs]), seg_ctx=i32([c for c, _ in segs]), block_table=table)
    return pool, q, meta, T


@pytest.mark.parametrize("nh,nkv,P,window,keep_first,sink", [(2, 2, 64, 100, 7, True), (4, 1, 128, 333, 130, True),
                                                             (2, 1, 64, 1, 3, False), (3, 3, 64, 200, 64, True),
                                                             (2, 2, 192, 0, 0, True), (2, 1, 64, 300, 500, False)])
def test_portion_kernels_with_kept_first_tokens_and_a_sink(nh, nkv, P, window, keep_first, sink):
    """Heads of 128 in bfloat16: the tcgen05 kernel whole and with its keys cut into ranges, the mma.sync kernel and
    the CUDA-core kernel against the twin, at contexts where the kept tokens fill no tile, one tile and more than one,
    touch the window, and where the window reaches the sequence's start."""
    import locus_b200.kernels as K

    dtype, hd = torch.bfloat16, 128
    segs = [(0, 5), (33, 17), (100, 2), (15, 140), (64, 64), (190, 200), (63, 1 + 128), (0, 450), (1000, 150), (700, 300)]
    pool, q, meta, T = _paged_attention_case(dtype, nh, nkv, hd, P, segs, window, keep_first, seed=window + 11)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=0.11, keep_first=keep_first, sink=sink)
    items64 = torch.tensor([(s, o) for s, (c, n) in enumerate(segs) for o in range(0, n, K.MMA_QUERY_TILE)], dtype=torch.int32)
    items16 = torch.tensor([(s, o) for s, (c, n) in enumerate(segs) for o in range(0, n, 16)], dtype=torch.int32)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.PRECISE = True
    try:
        EK.attn_chunk(q, pool, ref, items=items16, n_items=len(items16), **meta, **kw)
    finally:
        EK.PRECISE = False
    dev = {k: v.cuda() for k, v in meta.items()}

    def check(out, what):
        assert bool(torch.isfinite(out).all()), f"{what}: NaN (a page that went back was read)"
        assert _close(out, ref, 1.5e-2), what

    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
    K.attn_chunk_tc(q.cuda(), pool.cuda(), out, items=items64.cuda(), n_items=len(items64), **dev, **kw)
    assert K.attn_tc_error() == 0
    check(out, "attn_chunk_tc")
    for n_splits in (2, 5, 16):
        part_o = torch.full((T * nh * n_splits * hd,), float("nan"), device="cuda")
        part_ml = torch.full((T * nh * n_splits * 2,), float("nan"), device="cuda")
        out_s = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
        K.attn_chunk_tc(q.cuda(), pool.cuda(), out_s, items=items64.cuda(), n_items=len(items64), n_splits=n_splits,
                        part_o=part_o, part_ml=part_ml, **dev, **kw)
        assert K.attn_tc_error() == 0
        check(out_s, f"attn_chunk_tc in {n_splits} key ranges")
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
    K.attn_chunk_mma(q.cuda(), pool.cuda(), out, items=items64.cuda(), n_items=len(items64), **dev, **kw)
    check(out, "attn_chunk_mma")
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
    K.attn_chunk(q.cuda(), pool.cuda(), out, items=items16.cuda(), n_items=len(items16), **dev, **kw)
    check(out, "attn_chunk")


@pytest.mark.parametrize("dtype,hd", [(torch.bfloat16, 128), (torch.bfloat16, 96), (torch.float32, 64), (torch.bfloat16, 16)],
                         ids=["bf16_128", "bf16_96", "f32_64", "bf16_16"])
@pytest.mark.parametrize("nh,nkv,P,window,keep_first,sink", [(2, 2, 64, 100, 7, True), (4, 1, 128, 333, 130, True),
                                                             (2, 1, 64, 1, 3, False), (3, 3, 64, 200, 64, True),
                                                             (2, 1, 64, 40, 33, True), (2, 1, 64, 300, 500, False)])
def test_decode_kernels_with_kept_first_tokens_and_a_sink(nh, nkv, P, window, keep_first, sink, dtype, hd):
    """Single new tokens behind contexts in which the kept tokens lie inside the window, touch it, end in its first
    chunk of 32 and lie pages in front of it (those pages gone back): the streaming kernel in both of its variants
    (rows of 64 to 512 bytes) and the kernel of fixed ranges (other rows) against the twin, a batch and each alone."""
    import locus_b200.kernels as K

    ctxs = [0, 1, 2, 6, 7, 31, 32, 33, 63, 64, 99, 100, 101, 130, 131, 164, 200, 263, 333, 334, 461, 462, 463, 700, 1023, 1500]
    segs = [(c, 1) for c in ctxs]
    pool, q, meta, T = _paged_attention_case(dtype, nh, nkv, hd, P, segs, window, keep_first, seed=window + 5)
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, page_tokens=P, window=window, scale=0.13, keep_first=keep_first, sink=sink)
    items = torch.arange(len(segs), dtype=torch.int32)
    ref = torch.zeros(T, nh * hd, dtype=torch.float64)
    EK.PRECISE = True
    try:
        EK.attn_chunk(q, pool, ref, items=torch.stack([items, torch.zeros_like(items)], 1), n_items=len(items), **meta, **kw)
    finally:
        EK.PRECISE = False
    dev = {k: v.cuda() for k, v in meta.items()}
    max_splits = (max(ctxs) // K.DECODE_SPLIT) + 1
    units = K.decode_units(len(segs), nh, hd, dtype, max_splits, "cuda", page_tokens=P, fixed_ranges=keep_first > 0)
    part_o = torch.full((units * hd,), float("nan"), device="cuda")
    part_ml = torch.full((units * 2,), float("nan"), device="cuda")
    counters = torch.zeros(len(segs) * nh, dtype=torch.int32, device="cuda")
    tol = 1.5e-2 if dtype == torch.bfloat16 else 2e-5
    use_gqa = K.USE_GQA_DECODE
    try:
        for gqa, deep in [(g, d) for g in (True, False) for d in (None, True, False)]:
            if gqa and not K.attn_decode_gqa_takes(dtype, nh, nkv, hd, P, len(segs)):
                continue
            K.USE_GQA_DECODE = gqa
            K.attn_decode_variant(deep)
            K.attn_decode_gqa_variant(deep)
            what = f"{'grouped' if gqa else 'per head'}, variant {deep}"
            out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
            K.attn_decode(q.cuda(), pool.cuda(), out, items=items.cuda(), n_items=len(items), part_o=part_o, part_ml=part_ml,
                          counters=counters, max_splits=max_splits, **dev, **kw)
            assert K.attn_error() == 0 and K.attn_gqa_error() == 0
            assert bool(torch.isfinite(out).all()), f"{what}: NaN (a page that went back was read)"
            assert _close(out, ref, tol), what
            assert int(counters.abs().sum()) == 0
            # a few requests alone (the grouped kernel wants a batch: the last sixteen) give the same rows as in the batch
            for lo, hi in ((5, 6), (12, 13), (len(segs) - 1, len(segs)), (len(segs) - 16, len(segs))):
                one = torch.full((T, nh * hd), float("nan"), dtype=dtype, device="cuda")
                K.attn_decode(q.cuda(), pool.cuda(), one, items=items[lo:hi].cuda(), n_items=hi - lo, part_o=part_o,
                              part_ml=part_ml, counters=counters, max_splits=max_splits, **dev, **kw)
                assert _close(one[lo:hi], ref[lo:hi], tol), f"{what}, requests {lo} to {hi} alone"
    finally:
        K.USE_GQA_DECODE = use_gqa
        K.attn_decode_variant(None)
        K.attn_decode_gqa_variant(None)
