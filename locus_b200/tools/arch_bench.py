"""Prefill and decode throughput of the Lalepel, the Pozozen, the Mekizen or the Gugozen design at layer sizes that
resemble a real model's, beside the closest architecture at equal sizes (random weights, synthetic token ids, one GPU):
Qwen2-MoE for Lalepel and Pozozen; for Mekizen both Pozozen (the closest mixers: windowed attention beside a float32
recurrence) and Qwen2-MoE; for Gugozen both Lalepel (the closest mixers: latent attention and a float32 linear recurrence,
with routed experts) and Qwen2-MoE.

    python -m locus_b200.tools.arch_bench [--design lalepel|pozozen|mekizen|gugozen] [--size m|s] [--layers 4] [--prefill 2048]
                                          [--batch 8] [--context 4096] [--steps 16] [--warmup 3] [--dtype bf16|fp32]
                                          [--kernels]

Both models get the same width, head count and head sizes, experts, picks per token, expert and shared widths and
vocabulary; Lalepel's layers cycle through (latent attention, latent attention, retention, latent attention), all
with routed experts; Pozozen's through (attention beside a state-space mixer, matrix memory, matrix memory, attention
beside a state-space mixer) over two copies of the residual stream, with four identity experts beside the routed ones
in eight (or four) groups of which half stay open; Mekizen's through (convolved attention beside a gated delta rule,
windowed attention with kept first tokens and a sink, the same beside a delta rule again, attention on the second
layer's keys and values), all with a dense squared-ReLU feed-forward of four times the width; Gugozen's through
(grouped-query attention with a learned sink, gated linear attention, latent attention, latent attention on the third
layer's rows), all with clamped gated experts weighted on their input and a shared expert.  Timed on the device with CUDA events after warm-up; every step reads its weights (several
hundred MB: more than the L2 holds).  ``--kernels`` adds, for one eager prefill step and one eager decode step of
each model, the time by kernel entry point, and for the mixers' own kernels what their bytes or flops would take
at the measured peaks.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

SIZES = {
    # width, heads, head size (Qwen) = unrotated + rotated (Lalepel), value size, ranks, experts
    "m": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=512, window=4096, experts=60, top=4,
              ff=1408, shared=5632, vocab=151936, ret_dim=128, ssm_vdim=64, ssm_state=128),
    "s": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, q_rank=384, kv_rank=256, window=1024, experts=32, top=2,
              ff=704, shared=2816, vocab=32000, ret_dim=64, ssm_vdim=64, ssm_state=64),
}


def lalepel_config(z, n_layers):
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"]},
           "shared": {"ff": z["shared"]}}
    lat = {"type": "latent_attention", "mlp": moe, "mixer": {
        "heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "q_rank": z["q_rank"],
        "kv_rank": z["kv_rank"], "scale": (z["dim"] + z["rot"]) ** -0.5, "mask": {"size": z["window"]},
        "rot": {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 4.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}}
    ret = {"type": "retention", "mlp": moe, "mixer": {
        "heads": z["heads"], "dim": z["ret_dim"], "vdim": z["vdim"],
        "decay": [1.0 - 2.0 ** (-5 - 0.5 * i) for i in range(z["heads"])]}}
    return {"architecture": "Lalepel", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-6},
            "layers": [(ret if i % 4 == 2 else lat) for i in range(n_layers)]}


def pozozen_config(z, n_layers):
    ident = 4
    count = 8 if (z["experts"] + ident) % 8 == 0 else 4
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"], "identity": ident,
                                     "groups": {"count": count, "keep": count // 2}},
           "expert": {"ff": z["ff"]}, "shared": {"ff": z["shared"]}}
    par = {"type": "parallel", "mlp": moe, "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                 "mask": {"size": z["window"]}},
        "right": {"heads": 2 * z["width"] // z["ssm_vdim"], "vdim": z["ssm_vdim"], "state": z["ssm_state"], "groups": 1,
                  "conv": 4, "norm_groups": 1},
        "left_scale": 0.5, "right_scale": 0.5}}
    mem = {"type": "mlstm", "mlp": moe, "mixer": {"heads": z["heads"], "dim": z["ret_dim"], "vdim": z["vdim"], "gate_cap": 15.0}}
    return {"architecture": "Pozozen", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "streams": 2, "layers": [(mem if i % 4 in (1, 2) else par) for i in range(n_layers)]}


def mekizen_config(z, n_layers):
    rot = {"base": 10000.0, "dims": z["dim"]}
    mlp = {"kind": "dense", "ff": 4 * z["width"]}

    def attn(kv_from=None):
        m = {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
             "rot": rot, "mask": {"size": z["window"], "keep_first": 4}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "attention", "mlp": mlp, "mixer": m}

    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
                 "rot": rot, "conv": 4},
        "right": {"heads": z["heads"], "kv_heads": z["heads"], "dim": z["ret_dim"], "vdim": z["vdim"], "conv": 4}}}
    layers = []
    for i in range(n_layers):
        layers.append(par if i % 2 == 0 else attn(i - 2 if i % 4 == 3 else None))
    return {"architecture": "Mekizen", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "layers": layers}


def gugozen_config(z, n_layers):
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["ff"], "limit": 7.0},
           "shared": {"ff": z["shared"], "limit": 7.0}}
    att = {"type": "attention", "mlp": moe, "mixer": {
        "heads": z["heads"], "kv_heads": max(1, z["heads"] // 4), "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
        "rot": {"base": 1000000.0, "dims": z["dim"] // 2}}}
    rec = {"type": "gla", "mlp": moe, "mixer": {"heads": z["heads"], "dim": z["ret_dim"], "vdim": z["vdim"], "tau": 16.0}}

    def lat(kv_from=None):
        m = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["kv_rank"],
             "scale": (z["dim"] + z["rot"]) ** -0.5, "rot": {"base": 1000000.0, "dims": z["rot"]}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return {"type": "latent_attention", "mlp": moe, "mixer": m}

    layers = [(att, rec, lat(), lat(i - 1))[i % 4] if i % 4 != 3 else lat(i - 1) for i in range(n_layers)]
    return {"architecture": "Gugozen", "width": z["width"], "vocab": z["vocab"], "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}}, "layers": layers}


def qwen_config(z, n_layers, max_pos):
    hd = z["dim"] + z["rot"] if (z["dim"] + z["rot"]) in (64, 128) else z["dim"]
    return {"architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "num_hidden_layers": n_layers,
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": z["heads"],
            "head_dim": z["dim"], "vocab_size": z["vocab"], "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "max_position_embeddings": max_pos, "decoder_sparse_step": 1, "num_experts": z["experts"],
            "num_experts_per_tok": z["top"], "norm_topk_prob": False, "moe_intermediate_size": z["ff"],
            "shared_expert_intermediate_size": z["shared"], "intermediate_size": z["shared"], "qkv_bias": True,
            "tie_word_embeddings": False, "use_sliding_window": False, "mlp_only_layers": [], "hidden_act": "silu",
            "eos_token_id": -1, "_head": hd}


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def run(args) -> dict:
    import torch

    import locus_b200.kernels as K
    import locus_b200.models  # noqa: F401
    from locus_b200.cache import CacheManager
    from locus_b200.config import arch_name_of, find_arch
    from locus_b200.engine.step import ModelRunner, StepEntry
    from locus_b200.models.model import Model
    from locus_b200.weights.loader import RandomSource, load_weights

    dev = "cuda:0"
    torch.cuda.set_device(0)
    z = SIZES[args.size]
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    el = 2 if dtype == torch.bfloat16 else 4
    ctx, B, T = args.context, args.batch, args.prefill
    W, steps = max(3, args.warmup), args.steps
    pk = peaks()
    gen = torch.Generator().manual_seed(5)
    design = args.design
    own = {"lalepel": lalepel_config, "pozozen": pozozen_config, "mekizen": mekizen_config,
           "gugozen": gugozen_config}[design](z, args.layers)
    raws = {design: own}
    if design == "mekizen":
        raws["pozozen"] = pozozen_config(z, args.layers)
    if design == "gugozen":
        raws["lalepel"] = lalepel_config(z, args.layers)
    raws["qwen2_moe"] = qwen_config(z, args.layers, max(ctx, T) + 8)
    raws["qwen2_moe"].pop("_head")
    out = {}
    for name, raw in raws.items():
        entry = find_arch(arch_name_of(raw))
        cfg = entry.parse_config(raw)
        model = Model(entry.build_plan(cfg), dtype, dev)
        load_weights(model, RandomSource(model, 3, dtype, dev))
        P = 64
        n_pages = B * (-(-ctx // P) + 1) + -(-T // P) + 1
        cache = CacheManager(model.cache_needs(), page_tokens=P, n_pages=n_pages, n_state_slots=B + 1,
                             max_seq_tokens=max(ctx, T) + 8, dtype=dtype, device=dev)
        for g in cache.groups:
            g.pool.uniform_(-1.0, 1.0)
        runner = ModelRunner(model, cache, max_tokens=max(T, B), max_segments=B + 1, max_wanted=B + 1,
                             use_graphs=True)
        V = model.plan.vocab_size

        def ev():
            return torch.cuda.Event(enable_timing=True)

        prompt = torch.randint(0, V, (T,), generator=gen).tolist()

        def prefill_once():
            seq = cache.open("p")
            assert cache.ensure_capacity(seq, T)
            a, b = ev(), ev()
            a.record()
            runner.step([StepEntry(seq, prompt, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            cache.release(seq)
            return a.elapsed_time(b)

        pre = min([prefill_once() for _ in range(W + 3)][W:])
        seqs = [cache.open(f"d{i}") for i in range(B)]
        for s in seqs:
            assert cache.adopt(s, ctx - steps - W - 1)
        toks = torch.randint(0, V, (steps + W, B), generator=gen).tolist()

        def decode_once(i):
            for s in seqs:
                assert cache.ensure_capacity(s, 1)
            runner.step([StepEntry(s, [toks[i][j]], [0]) for j, s in enumerate(seqs)])

        for i in range(W):
            decode_once(i)
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for i in range(W, W + steps):
            decode_once(i)
        b.record()
        torch.cuda.synchronize()
        dec = a.elapsed_time(b) / steps
        res = {"weights_gb": model.param_bytes() / 1e9, "prefill_tokens": T, "prefill_ms": pre,
               "prefill_tokens_per_s": T / pre * 1e3, "decode_batch": B, "decode_context": ctx, "decode_ms": dec,
               "decode_tokens_per_s": B / dec * 1e3}
        if args.kernels:
            tables = {}
            with K.kernel_times() as kt:
                seq = cache.open("pk")
                assert cache.ensure_capacity(seq, T)
                runner.step([StepEntry(seq, prompt, [T - 1])])
                tables["prefill"] = {k: [n, round(ms, 4)] for k, (n, ms) in sorted(kt.table().items())}
                cache.release(seq)
            with K.kernel_times() as kt:
                for s in seqs:
                    assert cache.ensure_capacity(s, 1)
                runner.step([StepEntry(s, [toks[0][j]], [0]) for j, s in enumerate(seqs)])
                tables["decode"] = {k: [n, round(ms, 4)] for k, (n, ms) in sorted(kt.table().items())}
            res["kernel_ms"] = tables
        runner.check_device_errors()
        for s in seqs:
            cache.release(s)
        out[name] = res
        del runner, cache, model
        torch.cuda.empty_cache()
    # what the mixers' own kernels have to do per layer, at the measured peaks
    H, R = z["heads"], z["kv_rank"] + z["rot"]
    keys_avg = sum(min(p + 1, z["window"]) for p in range(T)) / T
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12       # float32 FMAs of the CUDA cores at the top clock
    if design == "gugozen":
        d, dv, G = z["ret_dim"], z["vdim"], max(1, H // 4)
        bounds = {
            "attn_prefill_us": 2.0 * T * (T + 1) / 2 * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
            "attn_decode_us": B * ctx * 2 * G * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            # the absorbed form multiplies the cached row (latent and rotated part) per score and the latent per value
            "latent_attn_prefill_us": 2.0 * T * (T + 1) / 2 * H * (R + z["kv_rank"]) / (pk["bf16_tflops"] * 1e12) * 1e6,
            "latent_attn_decode_us": B * ctx * R * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            # per token and head the decayed rank-one update and the read-out, float32 FMAs
            "gla_prefill_us": 2.0 * T * H * 2 * d * dv / (fma_tflops * 1e12) * 1e6,
            "gla_decode_us": B * H * d * dv * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            "retention_decode_us": B * H * d * dv * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            "qwen_attn_decode_us": B * ctx * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            "fp32_fma_tflops": fma_tflops,
        }
        return {"metric": f"prefill and decode tokens/s, Gugozen beside Lalepel and Qwen2-MoE at equal layer sizes "
                          f"({args.size}, {args.layers} layers, {args.dtype})",
                "size": z, "layers": args.layers, "dtype": args.dtype, "data": "synthetic", "designs": out,
                "bounds_per_layer": bounds, "peaks": pk,
                "l2": "no flush: every step reads its weights, more than the 126 MB L2"}
    if design == "mekizen":
        d, dv = z["ret_dim"], z["vdim"]
        chan = 2 * H * d + H * dv
        bounds = {
            # the left side sees every earlier token; a windowed layer the window and the kept tokens
            "attn_full_prefill_us": 2.0 * T * (T + 1) / 2 * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
            "attn_window_prefill_us": 2.0 * T * keys_avg * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
            "attn_full_decode_us": B * ctx * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            "attn_window_decode_us": B * min(ctx, z["window"] + 4) * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            # per token and head S^T k, S^T q and the decayed rank-one update, float32 FMAs
            "delta_prefill_us": 2.0 * T * H * 3 * d * dv / (fma_tflops * 1e12) * 1e6,
            "delta_decode_us": B * H * d * dv * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            # float32 rows in, float32 rows (the delta rule's side) or 16-bit rows and pages (the attention side) out
            "head_prep_delta_prefill_us": T * (chan + 2 * H) * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            "head_prep_attn_prefill_us": T * 3 * H * z["dim"] * (4 + el) / (pk["hbm_gbs"] * 1e9) * 1e6,
            "fp32_fma_tflops": fma_tflops,
        }
        return {"metric": f"prefill and decode tokens/s, Mekizen beside Pozozen and Qwen2-MoE at equal layer sizes "
                          f"({args.size}, {args.layers} layers, {args.dtype})",
                "size": z, "layers": args.layers, "dtype": args.dtype, "data": "synthetic", "designs": out,
                "bounds_per_layer": bounds, "peaks": pk,
                "l2": "no flush: every step reads its weights, more than the 126 MB L2"}
    if design == "pozozen":
        sh, sdv, sn = 2 * z["width"] // z["ssm_vdim"], z["ssm_vdim"], z["ssm_state"]

        def chunk_flops(heads, d, dvx):
            # per token and head: its row of Q K^T and of (Q K^T * D) V within a chunk of 32, Q S, and the state's update
            return 2.0 * T * heads * (32 * d + 32 * dvx + 2 * d * dvx)

        win_keys = sum(min(p + 1, z["window"]) for p in range(T)) / T
        bounds = {
            "attn_prefill_us": 2.0 * T * win_keys * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
            "attn_decode_us": B * min(ctx, z["window"]) * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            "ssm_recurrence_prefill_us": chunk_flops(sh, sn, sdv) / (fma_tflops * 1e12) * 1e6,
            "ssm_recurrence_decode_us": B * sh * sn * sdv * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            "mlstm_recurrence_prefill_us": chunk_flops(H, z["ret_dim"], z["vdim"] + 1) / (fma_tflops * 1e12) * 1e6,
            "mlstm_recurrence_decode_us": B * H * z["ret_dim"] * (z["vdim"] + 1) * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
            "qwen_attn_prefill_us": 2.0 * T * (T + 1) / 2 * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
            "qwen_attn_decode_us": B * ctx * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
            "fp32_fma_tflops": fma_tflops,
        }
        return {"metric": f"prefill and decode tokens/s, Pozozen beside Qwen2-MoE at equal layer sizes ({args.size}, "
                          f"{args.layers} layers, {args.dtype})",
                "size": z, "layers": args.layers, "dtype": args.dtype, "data": "synthetic", "designs": out,
                "bounds_per_layer": bounds, "peaks": pk,
                "l2": "no flush: every step reads its weights, more than the 126 MB L2"}
    bounds = {
        "latent_attn_prefill_us": 2.0 * T * keys_avg * H * (R + z["kv_rank"]) / (pk["bf16_tflops"] * 1e12) * 1e6,
        "qwen_attn_prefill_us": 2.0 * T * (T + 1) / 2 * H * 2 * z["dim"] / (pk["bf16_tflops"] * 1e12) * 1e6,
        "latent_attn_decode_us": B * min(ctx, z["window"]) * R * el / (pk["hbm_gbs"] * 1e9) * 1e6,
        "qwen_attn_decode_us": B * ctx * 2 * H * z["dim"] * el / (pk["hbm_gbs"] * 1e9) * 1e6,
        "retention_decode_us": B * H * z["ret_dim"] * z["vdim"] * 4 * 2 / (pk["hbm_gbs"] * 1e9) * 1e6,
        "retention_prefill_us": (T * (4 * H * z["ret_dim"] + 3 * H * z["vdim"]) * 4) / (pk["hbm_gbs"] * 1e9) * 1e6,
    }
    return {"metric": f"prefill and decode tokens/s, Lalepel beside Qwen2-MoE at equal layer sizes ({args.size}, "
                      f"{args.layers} layers, {args.dtype})",
            "size": z, "layers": args.layers, "dtype": args.dtype, "data": "synthetic", "designs": out,
            "bounds_per_layer": bounds, "peaks": pk,
            "l2": "no flush: every step reads its weights, more than the 126 MB L2"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="arch_bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("--design", default="lalepel", choices=["lalepel", "pozozen", "mekizen", "gugozen"])
    ap.add_argument("--size", default="m", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--kernels", action="store_true")
    args = ap.parse_args(argv)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
