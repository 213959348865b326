"""The Mekizen design through the engine's host logic on the CPU (the kernels replaced by their plain torch twins):
configuration and plan, weights by name, a layer on an earlier layer's keys and values, window pages that go back
while the kept first tokens' stay, state slots that are freed and used again, whole prompts, decoding token by token,
portions down to two tokens, mixed batches, and greedy generation through the scheduler -- all against the plain
implementation, which shares no code with any of it.  The kernels themselves are covered by the gpu tests."""
import copy
import math

import pytest
import torch

import emulated_kernels as EK
import plain_mekizen as plain
from mekizen_cases import CONFIGS, Case, compare, make_runner, random_config, run_steps, schedules
import locus_b200.models  # noqa: F401  (registers the architectures)
from locus_b200.config import ConfigError, find_arch
from locus_b200.config.mekizen import MekizenConfig

TOL = (2e-5, 4e-6)   # max and mean |error| of the logits relative to the largest |logit|; float32 twins
F64 = torch.float64
SHOWS = 40 * TOL[0]   # what a fault must move the logits by to count as shown: far beyond the tolerance


@pytest.fixture(autouse=True)
def _emulate(monkeypatch):
    EK.install(monkeypatch)


def test_config_reads_every_size_and_refuses_what_is_wrong():
    cfg = MekizenConfig.from_dict(copy.deepcopy(CONFIGS["mix"]))
    assert find_arch("Mekizen").parse_config is not None
    p, a, b = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[3].mixer
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.conv, p.left.rot.dims) == (4, 2, 32, 16, 3, 16)
    assert (p.right.heads, p.right.kv_heads, p.right.dim, p.right.vdim, p.right.conv) == (4, 2, 16, 8, 4)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first, a.rot.base, a.kv_from) == (4, 2, 16, 32, 11, 3, 500.0, None)
    assert (b.window, b.keep_first, b.kv_from) == (20, 5, 1)
    assert cfg.layers[0].mlp.ff == 48 and cfg.layers[2].mlp is None and cfg.embedding_scale == 2.5 and cfg.eps == 1e-5
    odd = MekizenConfig.from_dict(copy.deepcopy(CONFIGS["odd"]))
    assert odd.embedding_scale == 1.0 and odd.layers[2].mixer.left.rot is None and odd.layers[3].mixer.window == 0
    assert odd.layers[3].mixer.rot is None and odd.layers[4].mixer.keep_first == 9
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "rot", "dims"), 18, "rot.dims"),
                              (("layers", 3, "mixer", "kv_from"), 0, "kv_from"), (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
                              (("layers", 3, "mixer", "dim"), 32, "dim"), (("layers", 0, "mlp", "kind"), "moe", "kind"),
                              (("norm",), None, "norm"), (("layers", 0, "mixer", "right", "conv"), 0, "conv"),
                              (("layers", 1, "mixer", "mask", "keep_first"), -1, "keep_first")):
        raw = copy.deepcopy(CONFIGS["mix"])
        node = raw
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            MekizenConfig.from_dict(raw)


def test_plan_shares_pages_between_layers_and_keeps_what_the_widest_mask_sees():
    from locus_b200.models.model import Model

    e = find_arch("Mekizen")
    m = Model(e.build_plan(e.parse_config(copy.deepcopy(CONFIGS["mix"]))), torch.float32, "cpu")
    needs = m.cache_needs()
    assert [c for _, _, c in needs] == [None, None, None, 1]
    # layer 1's pages serve layer 3's wider window and longer keep; heads are laid out at the kernels' size
    assert (needs[1][0].window, needs[1][0].keep_first, needs[1][0].head_dim) == (20, 5, 32) and needs[1][1] is None
    # a parallel layer: pages of the attention side, one state slot for the convolutions of both sides and the delta rule
    left, right = CONFIGS["mix"]["layers"][0]["mixer"]["left"], CONFIGS["mix"]["layers"][0]["mixer"]["right"]
    conv_l = (left["heads"] * left["dim"] + left["kv_heads"] * (left["dim"] + left["vdim"])) * (left["conv"] - 1)
    conv_r = (2 * right["kv_heads"] * right["dim"] + right["heads"] * right["vdim"]) * (right["conv"] - 1)
    assert needs[0][1].shape == (conv_l + right["heads"] * right["dim"] * right["vdim"] + conv_r,) and needs[0][0].window == 0
    shared = Model(e.build_plan(e.parse_config(copy.deepcopy(CONFIGS["shared_kv"]))), torch.float32, "cpu").cache_needs()
    assert shared[0][0].window == 0 and [c for _, _, c in shared] == [None, 0, 0]   # a reader without a mask: every page stays
    names = {s.name for _, s in m.tensor_sources()}
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.left.q.conv", "l0.mix.left.out", "l0.mix.right.A_log",
            "l0.mix.right.dt_bias", "l0.mix.right.b", "l1.mix.q.b", "l1.mix.g", "l1.mix.o.b", "l3.mix.q", "l0.mlp.up"} <= names
    assert not {"l3.mix.k", "l3.mix.v", "l3.mix.k.b", "l2.norm2", "l2.mlp.up", "l1.mix.g.b"} & names


def test_plain_mechanisms_against_their_closed_forms():
    g = torch.Generator().manual_seed(5)
    # the delta rule with unit decay, full steps and orthonormal keys stores each value and returns it to its own key
    T, d, dv = 6, 8, 3
    keys = torch.linalg.qr(torch.randn(d, d, generator=g, dtype=F64)).Q[:T]
    vals = torch.randn(T, dv, generator=g, dtype=F64)
    one = torch.ones(T, 1, dtype=F64)
    out = plain.delta_rule(keys[:, None], keys[:, None], vals[:, None], one, one)
    assert torch.allclose(out[:, 0], vals, atol=1e-12)
    out = plain.delta_rule(keys[[0] * T][:, None], keys[:, None], vals[:, None], one, one)    # the first key's value stays
    assert torch.allclose(out[:, 0], vals[[0] * T], atol=1e-12)
    # in general: the state unrolled as a product of (g_t (I - beta_t k_t k_t^T)) and additions beta_t k_t v_t^T
    q, k = torch.randn(T, 1, d, generator=g, dtype=F64), torch.randn(T, 1, d, generator=g, dtype=F64) * 0.4
    beta, dec = torch.rand(T, 1, generator=g, dtype=F64), torch.rand(T, 1, generator=g, dtype=F64)
    out = plain.delta_rule(q, k, vals[:, None], beta, dec)
    S = torch.zeros(d, dv, dtype=F64)
    for t in range(T):
        kt = k[t, 0]
        S = dec[t, 0] * (torch.eye(d, dtype=F64) - beta[t, 0] * torch.outer(kt, kt)) @ S + beta[t, 0] * torch.outer(kt, vals[t])
        assert torch.allclose(out[t, 0], S.T @ q[t, 0], atol=1e-12)
    # a window of 3 with 2 kept tokens, through a planted key that every query prefers while it sees it
    qq = torch.zeros(9, 1, 2, dtype=F64)
    kk = torch.zeros(9, 1, 2, dtype=F64)
    vv = torch.arange(9, dtype=F64).view(9, 1, 1) + 1.0
    qq[:, 0, 0] = 1.0
    for planted, seen_by in ((1, range(1, 9)), (2, range(2, 5)), (4, range(4, 7))):
        kk.zero_()
        kk[planted, 0, 0] = 60.0
        o = plain.softmax_attention(qq, kk, vv, 1.0, size=3, keep_first=2)
        for i in range(9):
            assert (abs(float(o[i, 0, 0]) - float(vv[planted])) < 1e-9) == (i in seen_by), (planted, i)
    assert [plain.visible(7, j, 3, 2) for j in range(9)] == [True, True, False, False, False, True, True, True, False]
    # the sink: p_j = exp(s_j) / (1 + sum exp(s)); scores far below zero give next to nothing, far above it the plain softmax
    s = torch.tensor([0.3, -1.2, 2.0], dtype=F64)
    o = plain.softmax_attention(torch.ones(3, 1, 1, dtype=F64), s.view(3, 1, 1), torch.eye(3, dtype=F64).view(3, 1, 3), 1.0, sink=True)
    assert torch.allclose(o[2, 0], torch.exp(s) / (1.0 + torch.exp(s).sum()), atol=1e-14)
    assert torch.allclose(o[0, 0, 0], torch.exp(s[0]) / (1.0 + torch.exp(s[0])), atol=1e-14)
    # the short convolution: the last column is the current token's, zeros before the start
    u = torch.randn(5, 2, generator=g, dtype=F64)
    w = torch.tensor([[0.5, -1.0, 2.0], [0.0, 0.0, 1.0]], dtype=F64)
    y = plain.short_conv(u, w)
    assert torch.allclose(y[:, 1], u[:, 1]) and math.isclose(float(y[0, 0]), 2.0 * float(u[0, 0]))
    assert math.isclose(float(y[3, 0]), 0.5 * float(u[1, 0]) - float(u[2, 0]) + 2.0 * float(u[3, 0]))
    # the rotation: pairs (i, i + dims/2) of the first dims, the rest untouched, position 0 unchanged
    x = torch.randn(4, 1, 6, generator=g, dtype=F64)
    r = plain.rotate(x, 100.0, 4)
    assert torch.equal(r[0], x[0]) and torch.equal(r[..., 4:], x[..., 4:])
    a = 3.0 * 100.0 ** (-2.0 / 4)
    assert math.isclose(float(r[3, 0, 1]), float(x[3, 0, 1]) * math.cos(a) - float(x[3, 0, 3]) * math.sin(a))
    assert math.isclose(float(r[3, 0, 3]), float(x[3, 0, 3]) * math.cos(a) + float(x[3, 0, 1]) * math.sin(a))


@pytest.mark.parametrize("name", ["mix", "odd", "shared_kv", "wide"])
def test_every_schedule_against_the_plain_implementation(tmp_path, name):
    lens = (41, 1, 23, 37, 2, 30) if name != "wide" else (90, 33, 5)
    case = Case(name, tmp_path, torch.float32, requests=lens)
    for sched, steps in schedules(case).items():
        runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=40, max_tokens=160, slots=4)
        got = run_steps(runner, cache, case, steps)
        compare(case, got, *TOL)
        assert cache.free_pages() == cache.total_pages(), sched


def test_a_drawn_configuration_in_mixed_batches(tmp_path):
    for seed in (3, 8):
        case = Case(f"drawn{seed}", tmp_path, torch.float32, raw=random_config(seed), requests=(70, 9, 44, 21), seed=seed)
        runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=16, n_pages=24, max_tokens=160, slots=4)
        got = run_steps(runner, cache, case, schedules(case)["mixed"])
        compare(case, got, 1e-4, 2e-5)


def test_the_sharpened_weights_show_each_fault(tmp_path):
    """What the comparisons rest on: with these weights a window or a count of kept tokens that is one off, a missing
    sink, a lost convolution input, a lost state, another rotated part, another scale, another epsilon's place and a far
    token each move the logits by far more than the tolerance."""
    case = Case("mix", tmp_path, torch.float32, requests=(60,))
    ref = case.ref("r0")
    scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())

    def moved(cfg=None, weights=None, toks=None, last=20, **kw):
        lg = plain.forward(weights or case.weights, cfg or case.cfg, toks or case.tokens["r0"], **kw)
        return float((lg[-last:] - ref[-last:]).abs().max()) / scale

    for layer in (1, 3):
        for key in ("size", "keep_first"):
            for delta in (-1, 1):
                cfg = copy.deepcopy(case.cfg)
                cfg["layers"][layer]["mixer"]["mask"][key] += delta
                assert moved(cfg) > SHOWS, (layer, key, delta)
    assert moved(sink=False) > SHOWS
    for key, value in ((("layers", 1, "mixer", "rot", "dims"), 4), (("layers", 0, "mixer", "left", "rot", "dims"), 8),
                       (("layers", 1, "mixer", "scale"), 0.3), (("layers", 0, "mixer", "left", "scale"), 0.3),
                       (("embedding", "scale"), 2.0), (("layers", 1, "mixer", "rot", "base"), 400.0)):
        cfg = copy.deepcopy(case.cfg)
        node = cfg
        for k in key[:-1]:
            node = node[k]
        node[key[-1]] = value
        assert moved(cfg) > SHOWS, key
    for side in ("left", "right"):       # the convolution sees one token less: its first column is taken away
        cfg = copy.deepcopy(case.cfg)
        cfg["layers"][0]["mixer"][side]["conv"] -= 1
        w = dict(case.weights)
        for n in ("q", "k", "v"):
            w[f"l0.mix.{side}.{n}.conv"] = w[f"l0.mix.{side}.{n}.conv"][:, 1:].contiguous()
        assert moved(cfg, w) > SHOWS, side
    for name in ("l0.mix.right.A_log", "l0.mix.right.dt_bias", "l1.mix.q.b", "l1.mix.o.b", "l0.mix.left.out", "l2.mix.right.norm"):
        w = dict(case.weights)
        w[name] = torch.zeros_like(w[name])
        assert moved(weights=w) > SHOWS, name
    # layer 3 with keys and values of its own kind (layer 1's projections once more, applied to its own input)
    assert moved(own_kv={3: 1}) > SHOWS
    # lost states and pages: a sequence that starts 25 tokens later has forgotten what came before
    lg = plain.forward(case.weights, case.cfg, case.tokens["r0"][25:])
    assert float((lg[-20:] - ref[-20:]).abs().max()) / scale > SHOWS
    toks = list(case.tokens["r0"])
    toks[1] = (toks[1] + 1) % case.cfg["vocab"]     # a token 40 and more back
    assert moved(toks=toks) > SHOWS


def test_far_tokens_reach_through_each_mechanism_alone(tmp_path):
    """One-layer models: a token 45 positions back moves the last logits through the delta rule's state alone (whose
    attention side is cut off by zeroing its output weight), through full attention alone, through a window's kept
    first tokens, and not through a window of 9 once the token is neither kept nor in the window."""
    for name, zero, at, reaches in (("delta_only", "l0.mix.left.out", 2, True), ("conv_attention_only", "l0.mix.right.out", 2, True),
                                    ("attention_only", None, 1, True), ("attention_only", None, 2, False)):
        case = Case(name, tmp_path, torch.float32, requests=(50,))
        w = dict(case.weights)
        if zero:
            w[zero] = torch.zeros_like(w[zero])
        ref = plain.forward(w, case.cfg, case.tokens["r0"])
        scale = float((ref - ref.mean(-1, keepdim=True)).abs().max())
        toks = list(case.tokens["r0"])
        toks[at] = (toks[at] + 1) % case.cfg["vocab"]
        lg = plain.forward(w, case.cfg, toks)
        move = float((lg[-3:] - ref[-3:]).abs().max()) / scale
        assert (move > SHOWS) == reaches, (name, at, move)


def test_window_pages_go_back_while_kept_pages_stay_and_slots_are_used_again(tmp_path):
    case = Case("attention_only", tmp_path, torch.float32, requests=(90, 90, 40, 40, 40))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=14, max_tokens=72, slots=2)
    steps = [[("r0", 30)], [("r0", 30)], [("r0", 30)], [("r1", 24), ("r2", 8)], [("r1", 33), ("r2", 32)],
             [("r1", 33), ("r3", 2)], [("r3", 38), ("r4", 1)], [("r4", 39)]]
    got = run_steps(runner, cache, case, steps)
    compare(case, got, *TOL)
    assert cache.free_pages() == cache.total_pages()
    # a request of 60 tokens holds, behind its last step, the page of its two kept tokens and what its window of 9 reaches
    from locus_b200.engine.step import StepEntry
    seq = cache.open("z")
    for a in (0, 20, 40):
        assert cache.ensure_capacity(seq, 20)
        runner.step([StepEntry(seq, case.tokens["r0"][a:a + 20], [19])])
    table = seq.page_tables()[0] if hasattr(seq, "page_tables") else None
    assert seq.pages_held(0) <= 4 < cache.pages_for(60)
    if table is not None:
        assert table[0] >= 0 and table[1] < 0 and table[2] < 0
    cache.release(seq)


def test_a_slot_used_again_starts_from_zero(tmp_path):
    """Two requests through the same state slot one after the other: the second one's delta-rule state and both
    sides' convolution inputs start at zero."""
    case = Case("mix", tmp_path, torch.float32, requests=(30, 30, 12))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=16, max_tokens=64, slots=1)
    got = run_steps(runner, cache, case, [[("r0", 30)], [("r1", 7)], [("r1", 23)], [("r2", 2)], [("r2", 10)]])
    compare(case, got, *TOL)


def test_long_decoding_token_by_token(tmp_path):
    case = Case("mix", tmp_path, torch.float32, requests=(120,))
    runner, cache = make_runner(case, torch.float32, "cpu", page_tokens=8, n_pages=20, max_tokens=32, slots=2)
    got = run_steps(runner, cache, case, [[("r0", 3)]] + [[("r0", 1)]] * 117)
    compare(case, got, *TOL)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from locus_b200.engine.engine import Engine
    from locus_b200.models import load_model

    case = Case("mix", tmp_path, torch.float32, requests=(9, 21, 3))
    m = load_model(case.dir, torch.float32, "cpu")
    eng = Engine.from_model(m, ctx=256, page_tokens=8, max_batch_tokens=16, chunk=8, max_running=2, use_graphs=False)
    prompts = [case.tokens[r] for r in ("r0", "r1", "r2")]
    outs = eng.generate(prompts, max_new_tokens=6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(case.weights, case.cfg, seq)
            top2 = torch.topk(lg[-1], 2).values
            if float(top2[0] - top2[1]) > 1e-4 * float(lg[-1].abs().max()):
                assert int(torch.argmax(lg[-1])) == tok
            seq.append(tok)
    assert eng.cache.free_pages() == eng.cache.total_pages()
