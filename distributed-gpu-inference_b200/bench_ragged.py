"""``bench.py --compare petipel``: prompt-pass and decode throughput of the Petipel model class on the ragged step
engine beside a Llama-shaped model of equal width, depth and head layout on the paged decode engine, plus the time
of every mixer kernel of one prompt step and one decode step against its memory / math floor.

Random weights, synthetic token ids; bf16.  Timed with CUDA events on the launching stream after warm-up; the
inputs of a step (activations, weights, KV of all sequences) exceed L2 at the two larger sizes and the report says
so per size.  One JSON line on stdout; the default workload and output line of bench.py are untouched.

``bench.py --compare sanesun``: the same two steps for the Sanesun model class beside a Petipel model of equal width,
depth, head layout and feed-forward size (its closest relative here: attention layers alternating with a recurrence
on the same engine), with every kernel of both against its floor so that like kernels can be read side by side.

``bench.py --compare fibirax``: the same two steps for the Fibirax model class (a windowed attention AND a retention in
every layer, routed experts in every layer) beside a Petipel model of equal width, depth, head layout and expert sizes
whose layers alternate attention and recurrence, again with every kernel of both against its floor.

``bench.py --compare vatazen``: the same two steps for the Vatazen model class (latent layers with a decoupled rotated
key part and differential layers in turn, routed experts in every layer) beside a Fibirax model of equal width, depth,
head layout and expert sizes (its closest relative here: post-norm sublayers that read the residual itself, windowed sink
attention on the same tensor-core kernel, softmax routing over the same dispatch).
"""
from __future__ import annotations

import json
import math
import statistics
from typing import Any, Dict, List

import torch

SIZES = {
    # width, query heads, kv heads, head size; recurrent heads and their key / value sizes; feed-forward sizes
    "w1024": dict(width=1024, heads=8, kv=2, dk=128, dv=128, rheads=8, rdk=64, rdv=128, ff=4096, experts=8, eff=1024, top=2),
    "w2048": dict(width=2048, heads=16, kv=4, dk=128, dv=128, rheads=16, rdk=64, rdv=128, ff=8192, experts=8, eff=2048, top=2),
    "w4096": dict(width=4096, heads=32, kv=8, dk=128, dv=128, rheads=32, rdk=64, rdv=128, ff=14336, experts=8, eff=3584, top=2),
}
LAYERS = 4
VOCAB = 32000


def petipel_config(s: Dict[str, int]) -> Dict[str, Any]:
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["dk"], "vdim": s["dv"],
                                          "scale": 1.0 / math.sqrt(s["dk"]), "bias_max": 4096, "v_mix": True,
                                          "q_temp": {"coef": 0.1, "every": 512}}}
    rec = {"type": "hgrn2", "mixer": {"heads": s["rheads"], "dim": s["rdk"], "vdim": s["rdv"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]}}
    layers = []
    for i in range(LAYERS):
        layer = dict(rec if i % 2 == 0 else att)
        layer["mlp"] = dense if i % 4 < 2 else moe
        layers.append(layer)
    return {"architecture": "Petipel", "width": s["width"], "vocab": VOCAB, "residual_mult": 0.5,
            "norm": {"eps": 1e-6}, "layers": layers}


def _events_ms(pairs) -> float:
    return sum(a.elapsed_time(b) for a, b in pairs)


def _time_steps(fn, steps: int, warmup: int) -> float:
    """Median milliseconds of ``fn()`` over ``steps`` runs, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def run(args, measured_peaks, ClockSampler) -> None:
    from . import mixer_ops, ops
    from . import petipel_layer as P
    from .engine import PagedDecodeEngine
    from .ragged_engine import RaggedStepEngine
    from .testing import LlamaShapeConfig
    from .worker.distributed.model_shard import ModelShard

    dev = "cuda:0"
    peaks, how = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    B, Pn, ctx = 8, 2048, 2048          # prompt pass: 8 x 2048 tokens in one step; decode: 64 sequences at 2k context
    Bd = 64
    g = torch.Generator().manual_seed(0)
    sampler = ClockSampler(0)
    sampler.start()
    report: Dict[str, Any] = {}
    for name, s in SIZES.items():
        if args.compare_sizes and name not in args.compare_sizes.split(","):
            continue
        row: Dict[str, Any] = {}
        # ---- Petipel on the ragged step engine -----------------------------------------------------------------
        raw = petipel_config(s)
        cfg = P.PetipelConfig.from_dict(raw)
        shards = P.build_shards(cfg, P.random_checkpoint(cfg, seed=0), [(0, LAYERS)], dev, torch.bfloat16)
        eng = RaggedStepEngine(shards, max_tokens=Bd * (ctx + 64), max_seqs=Bd, fp32_logits=False)
        prompts = torch.randint(0, VOCAB, (Bd, ctx), generator=g).tolist()

        def prompt_step():
            eng.step([(i, prompts[i][:Pn], [Pn - 1]) for i in range(B)])
            for i in range(B):
                eng.finish(i)

        ms = _time_steps(prompt_step, steps, warmup)
        row["petipel_prefill_tok_s"] = round(B * Pn / ms * 1e3)
        mixer_ops.EVENTS = []
        prompt_step()
        torch.cuda.synchronize()
        ev_prompt, mixer_ops.EVENTS = mixer_ops.EVENTS, None
        for i in range(0, Bd, B):        # fill 64 sequences to the decode context
            eng.step([(j, prompts[j], []) for j in range(i, i + B)])
        nxt = [[1] for _ in range(Bd)]

        def decode_step():
            eng.step([(j, nxt[j], [0]) for j in range(Bd)])

        ms = _time_steps(decode_step, min(steps, 32), warmup)
        row["petipel_decode_tok_s"] = round(Bd / ms * 1e3)
        mixer_ops.EVENTS = []
        decode_step()
        torch.cuda.synchronize()
        ev_decode, mixer_ops.EVENTS = mixer_ops.EVENTS, None
        eng.release()
        row["kernels"] = _kernel_table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx + warmup + min(steps, 32), hbm, tf)
        del eng, shards
        torch.cuda.empty_cache()
        # ---- Llama shape of equal width / depth / heads on the paged engine ----------------------------------------
        lcfg = LlamaShapeConfig(hidden_size=s["width"], num_attention_heads=s["heads"], num_key_value_heads=s["kv"],
                                head_dim=s["dk"], intermediate_size=s["ff"], vocab_size=VOCAB, num_hidden_layers=LAYERS)
        shard = ModelShard.from_config(lcfg, 0, LAYERS, device=dev, dtype=torch.bfloat16, seed=0)
        leng = PagedDecodeEngine([shard], max_batch=Bd, max_seq_len=ctx + 64, fuse_projections=True)
        ids = torch.tensor(prompts, dtype=torch.int64)

        def llama_prompt():
            leng.allocate(B, Pn + 1)
            leng.prefill(ids[:B, :Pn])

        ms = _time_steps(llama_prompt, steps, warmup)
        row["llama_prefill_tok_s"] = round(B * Pn / ms * 1e3)
        ops.ATTN_EVENTS = []
        llama_prompt()
        torch.cuda.synchronize()
        ops.ATTN_EVENTS = None
        leng.allocate(Bd, ctx + 64)
        leng.prefill(ids)
        leng.ids_buf[:Bd, 0].fill_(1)
        ms = _time_steps(leng.decode_step_device, min(steps, 32), warmup)
        row["llama_decode_tok_s"] = round(Bd / ms * 1e3)
        leng.use_cuda_graph = False
        ops.ATTN_EVENTS = []
        leng.decode_step_device()
        torch.cuda.synchronize()
        pairs, ops.ATTN_EVENTS = ops.ATTN_EVENTS, None
        if pairs:
            t = _events_ms(pairs) / len(pairs) * 1e-3
            kv_bytes = Bd * (ctx + 40) * s["kv"] * 2 * s["dk"] * 2
            row["llama_decode_attention"] = {"us": round(t * 1e6, 1), "of_copy_peak": round(kv_bytes / t / hbm, 3)}
        leng.release()
        del leng, shard
        torch.cuda.empty_cache()
        row["inputs_exceed_l2"] = bool(Bd * ctx * s["kv"] * (s["dk"] + s["dv"]) * 2 > 126e6)
        report[name] = row
    clocks = sampler.stop()
    print(json.dumps({"bench": "petipel_vs_llama", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic",
                      "layers": LAYERS, "prompt_step": f"{B} x {Pn} tokens", "decode_step": f"{Bd} sequences at {ctx}",
                      "peaks": how, "sizes": report, "clocks": clocks}), flush=True)


def _kernel_table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx, hbm, tf) -> Dict[str, Any]:
    """Per kernel: mean microseconds in the prompt step and in the decode step, and the fraction of the floor
    max(bytes / copy peak, flops / bf16 peak) for the ones whose traffic is easy to state."""
    out: Dict[str, Any] = {}
    W, H, G, dk, dv = s["width"], s["heads"], s["kv"], s["dk"], s["dv"]
    RH, rdk, rdv = s["rheads"], s["rdk"], s["rdv"]
    for phase, events, n_tok, past in (("prompt", ev_prompt, B * Pn, 0), ("decode", ev_decode, Bd, ctx)):
        by: Dict[str, List[float]] = {}
        for name, a, b in events:
            by.setdefault(name, []).append(a.elapsed_time(b) * 1e-3)
        per_seq = n_tok // (B if phase == "prompt" else Bd)
        n_seq = n_tok // per_seq
        floors = {
            "offset_rmsnorm": (n_tok * W * 6, 0),
            "postnorm_residual": (n_tok * W * (4 + 4 + 2 + 2), 0),
            "value_prep_append": (n_tok * G * (dk + dv) * 2 * 2 + n_tok * G * dv * 2, 0),
            "biased_paged_attention": (n_seq * (past + per_seq) * G * (dk + dv) * 2 + n_tok * H * (dk + dv) * 2,
                                       n_seq * H * 2 * (dk + dv) * (per_seq * past + per_seq * (per_seq + 1) // 2)),
            "biased_prompt_attention": (n_seq * (past + per_seq) * G * (dk + dv) * 2 + n_tok * H * (dk + dv) * 2,
                                        n_seq * H * 2 * (dk + dv) * (per_seq * past + per_seq * (per_seq + 1) // 2)),
            "gated_scan": (n_tok * RH * (2 * rdk + rdv) * 2 + n_tok * RH * rdv * 4 + 2 * n_seq * RH * rdk * rdv * 4, 0),
            "head_rmsnorm": (n_tok * RH * rdv * 6, 0),
            "polynorm": (n_tok * s["ff"] * 4, 0),
            "clamped_glu": (n_tok * s["top"] * s["eff"] * 6, 0),
            "scaled_gather": (n_tok * s["top"] * W * 4, 0),
            "expert_combine": (n_tok * s["top"] * W * 2 + n_tok * W * 4, 0),
        }
        for name, ts in by.items():
            t = statistics.mean(ts)
            entry = {"us": round(t * 1e6, 1), "calls": len(ts)}
            if name in floors:
                nbytes, flops = floors[name]
                floor = max(nbytes / hbm, flops / tf)
                entry["of_floor"] = round(floor / t, 3)
                entry["bound"] = "math" if flops / tf > nbytes / hbm else "memory"
            out.setdefault(phase, {})[name] = entry
    return out


# ---- Sanesun beside Petipel ------------------------------------------------------------------------------------------
SANESUN_WINDOW, SANESUN_KEEP, LATENT_RANK = 512, 4, 256


def sanesun_config(s: Dict[str, int]) -> Dict[str, Any]:
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["dk"], "vdim": s["dv"],
                                          "scale": 1.0 / math.sqrt(s["dk"]),
                                          "mask": {"size": SANESUN_WINDOW, "keep_first": SANESUN_KEEP},
                                          "rot": {"base": 10000.0, "dims": s["dk"] // 2}}}
    lat = {"type": "latent_attention", "mixer": {"heads": s["heads"], "dim": s["dk"], "vdim": s["dv"],
                                                 "kv_rank": LATENT_RANK, "q_rank": s["width"] // 2,
                                                 "scale": 1.0 / math.sqrt(s["dk"])}}
    rec = {"type": "channel_delta", "mixer": {"heads": s["rheads"], "kv_heads": s["rheads"], "dim": s["rdk"],
                                              "vdim": s["rdv"], "conv": 4}}
    layers = [dict(m, mlp={"kind": "dense", "ff": s["ff"]}) for m in (rec, att, rec, lat)]
    return {"architecture": "Sanesun", "width": s["width"], "vocab": VOCAB, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": layers}


def petipel_dense_config(s: Dict[str, int]) -> Dict[str, Any]:
    raw = petipel_config(s)
    for layer in raw["layers"]:
        layer["mlp"] = {"kind": "dense", "ff": s["ff"]}
    return raw


def run_sanesun(args, measured_peaks, ClockSampler) -> None:
    from . import mixer_ops
    from . import petipel_layer as P
    from . import sanesun_layer as S
    from .ragged_engine import RaggedStepEngine

    dev = "cuda:0"
    peaks, how = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    B, Pn, ctx, Bd = 8, 2048, 2048, 64
    g = torch.Generator().manual_seed(0)
    sampler = ClockSampler(0)
    sampler.start()
    report: Dict[str, Any] = {}
    for name, s in SIZES.items():
        if args.compare_sizes and name not in args.compare_sizes.split(","):
            continue
        row: Dict[str, Any] = {}
        prompts = torch.randint(0, VOCAB, (Bd, ctx), generator=g).tolist()
        for label, mod, raw in (("sanesun", S, sanesun_config(s)), ("petipel", P, petipel_dense_config(s))):
            cfg = (S.SanesunConfig if mod is S else P.PetipelConfig).from_dict(raw)
            shards = mod.build_shards(cfg, mod.random_checkpoint(cfg, seed=0), [(0, LAYERS)], dev, torch.bfloat16)
            eng = RaggedStepEngine(shards, max_tokens=Bd * (ctx + 64), max_seqs=Bd, fp32_logits=False)

            def prompt_step():
                eng.step([(i, prompts[i][:Pn], [Pn - 1]) for i in range(B)])
                for i in range(B):
                    eng.finish(i)

            ms = _time_steps(prompt_step, steps, warmup)
            row[label + "_prefill_tok_s"] = round(B * Pn / ms * 1e3)
            mixer_ops.EVENTS = []
            prompt_step()
            torch.cuda.synchronize()
            ev_prompt, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            for i in range(0, Bd, B):
                eng.step([(j, prompts[j], []) for j in range(i, i + B)])
            nxt = [[1] for _ in range(Bd)]

            def decode_step():
                eng.step([(j, nxt[j], [0]) for j in range(Bd)])

            n_dec = min(steps, 32)
            ms = _time_steps(decode_step, n_dec, warmup)
            row[label + "_decode_tok_s"] = round(Bd / ms * 1e3)
            mixer_ops.EVENTS = []
            decode_step()
            torch.cuda.synchronize()
            ev_decode, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            eng.release()
            table = _kernel_table if mod is P else _sanesun_kernel_table
            row[label + "_kernels"] = table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx + warmup + n_dec, hbm, tf)
            del eng, shards
            torch.cuda.empty_cache()
        row["inputs_exceed_l2"] = bool(Bd * ctx * s["kv"] * (s["dk"] + s["dv"]) * 2 > 126e6)
        report[name] = row
    clocks = sampler.stop()
    print(json.dumps({"bench": "sanesun_vs_petipel", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic",
                      "layers": LAYERS, "prompt_step": f"{B} x {Pn} tokens", "decode_step": f"{Bd} sequences at {ctx}",
                      "peaks": how, "sizes": report, "clocks": clocks}), flush=True)


def _sanesun_kernel_table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx, hbm, tf) -> Dict[str, Any]:
    """Like ``_kernel_table`` for the Sanesun kernels.  The two attention layers share one kernel; their calls are
    told apart by their order in a step (layer 1: windowed, layer 3: latent) and reported under two names."""
    out: Dict[str, Any] = {}
    W, H, G, dk, dv = s["width"], s["heads"], s["kv"], s["dk"], s["dv"]
    RH, rdk, rdv, r = s["rheads"], s["rdk"], s["rdv"], LATENT_RANK
    C = 2 * RH * rdk + RH * rdv
    for phase, events, n_tok, past in (("prompt", ev_prompt, B * Pn, 0), ("decode", ev_decode, Bd, ctx)):
        by: Dict[str, List[float]] = {}
        seen_attn = 0
        for name, a, b in events:
            if name in ("mixed_paged_attention", "mixed_prompt_attention"):
                name = ("windowed_attention", "latent_attention")[seen_attn % 2]
                seen_attn += 1
            by.setdefault(name, []).append(a.elapsed_time(b) * 1e-3)
        per_seq = n_tok // (B if phase == "prompt" else Bd)
        n_seq = n_tok // per_seq
        # keys a query sees: all earlier ones (latent), or the window and the kept prefix (windowed)
        pairs_full = per_seq * past + per_seq * (per_seq + 1) // 2
        seen_w = [min(past + t + 1, SANESUN_WINDOW + SANESUN_KEEP) for t in range(per_seq)]
        pairs_win = sum(seen_w)
        keys_win = min(past + per_seq, (SANESUN_WINDOW + SANESUN_KEEP + per_seq))
        floors = {
            "rms_norm": (n_tok * W * 6, 0),
            "residual_add2_norm": (n_tok * W * (4 + 4 + 2 + 2 + 2), 0),
            "xielu": (n_tok * s["ff"] * 4, 0),
            "rotary_kv_append": (n_tok * (H * dk * 2 + G * (dk + dv) * 2) * 2, 0),
            "norm_append": (n_tok * r * 4, 0),
            "windowed_attention": (n_seq * keys_win * G * (dk + dv) * 2 + n_tok * H * (dk + dv) * 2,
                                   n_seq * H * 2 * (dk + dv) * pairs_win),
            "latent_attention": (n_seq * (past + per_seq) * r * 2 + n_tok * H * 2 * r * 2, n_seq * H * 2 * 2 * r * pairs_full),
            "causal_conv_silu": (n_tok * C * 4, 0),
            "delta_scan": (n_tok * RH * (3 * rdk + rdv) * 2 + n_tok * RH * rdv * 4 + 2 * n_seq * RH * rdk * rdv * 4, 0),
            "head_rmsnorm_gated": (n_tok * RH * rdv * 8, 0),
        }
        for name, ts in by.items():
            t = statistics.mean(ts)
            entry = {"us": round(t * 1e6, 1), "calls": len(ts)}
            if name in floors:
                nbytes, flops = floors[name]
                floor = max(nbytes / hbm, flops / tf)
                entry["of_floor"] = round(floor / t, 3)
                entry["bound"] = "math" if flops / tf > nbytes / hbm else "memory"
            out.setdefault(phase, {})[name] = entry
    return out


# ---- Fibirax beside Petipel ------------------------------------------------------------------------------------------
FIBIRAX_WINDOW = 512


def fibirax_config(s: Dict[str, int]) -> Dict[str, Any]:
    left = {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["dk"], "vdim": s["dv"], "scale": 1.0 / math.sqrt(s["dk"]),
            "softcap": 30.0, "mask": {"size": FIBIRAX_WINDOW},
            "rot": {"base": 10000.0, "dims": s["dk"] // 2,
                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    right = {"heads": s["rheads"], "dim": s["rdk"], "vdim": s["rdv"],
             "decay": [1.0 - 2.0 ** (-5 - (i % 8)) for i in range(s["rheads"])]}
    mlp = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0}, "shared": {"ff": s["eff"], "limit": 7.0},
           "router": {"experts": s["experts"], "identity": 2, "top": s["top"], "groups": {"count": 2, "keep": 1}}}
    layer = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.8, "right_scale": 0.5}, "mlp": mlp}
    return {"architecture": "Fibirax", "width": s["width"], "vocab": VOCAB, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": [layer] * LAYERS}


def petipel_moe_config(s: Dict[str, int]) -> Dict[str, Any]:
    raw = petipel_config(s)
    for layer in raw["layers"]:
        layer["mlp"] = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0},
                        "router": {"experts": s["experts"], "top": s["top"]}}
    return raw


def run_fibirax(args, measured_peaks, ClockSampler) -> None:
    from . import fibirax_layer as Fx
    from . import mixer_ops
    from . import petipel_layer as P
    from .ragged_engine import RaggedStepEngine

    dev = "cuda:0"
    peaks, how = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    B, Pn, ctx, Bd = 8, 2048, 2048, 64
    g = torch.Generator().manual_seed(0)
    sampler = ClockSampler(0)
    sampler.start()
    report: Dict[str, Any] = {}
    for name, s in SIZES.items():
        if args.compare_sizes and name not in args.compare_sizes.split(","):
            continue
        row: Dict[str, Any] = {}
        prompts = torch.randint(0, VOCAB, (Bd, ctx), generator=g).tolist()
        for label, mod, raw in (("fibirax", Fx, fibirax_config(s)), ("petipel", P, petipel_moe_config(s))):
            cfg = (Fx.FibiraxConfig if mod is Fx else P.PetipelConfig).from_dict(raw)
            shards = mod.build_shards(cfg, mod.random_checkpoint(cfg, seed=0), [(0, LAYERS)], dev, torch.bfloat16)
            eng = RaggedStepEngine(shards, max_tokens=Bd * (ctx + 64), max_seqs=Bd, fp32_logits=False)

            def prompt_step():
                eng.step([(i, prompts[i][:Pn], [Pn - 1]) for i in range(B)])
                for i in range(B):
                    eng.finish(i)

            ms = _time_steps(prompt_step, steps, warmup)
            row[label + "_prefill_tok_s"] = round(B * Pn / ms * 1e3)
            mixer_ops.EVENTS = []
            prompt_step()
            torch.cuda.synchronize()
            ev_prompt, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            for i in range(0, Bd, B):
                eng.step([(j, prompts[j], []) for j in range(i, i + B)])
            nxt = [[1] for _ in range(Bd)]

            def decode_step():
                eng.step([(j, nxt[j], [0]) for j in range(Bd)])

            n_dec = min(steps, 32)
            ms = _time_steps(decode_step, n_dec, warmup)
            row[label + "_decode_tok_s"] = round(Bd / ms * 1e3)
            mixer_ops.EVENTS = []
            decode_step()
            torch.cuda.synchronize()
            ev_decode, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            eng.release()
            table = _kernel_table if mod is P else _fibirax_kernel_table
            row[label + "_kernels"] = table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx + warmup + n_dec, hbm, tf)
            del eng, shards
            torch.cuda.empty_cache()
        row["inputs_exceed_l2"] = bool(Bd * ctx * s["kv"] * (s["dk"] + s["dv"]) * 2 > 126e6)
        report[name] = row
    clocks = sampler.stop()
    print(json.dumps({"bench": "fibirax_vs_petipel", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic",
                      "layers": LAYERS, "prompt_step": f"{B} x {Pn} tokens", "decode_step": f"{Bd} sequences at {ctx}",
                      "peaks": how, "sizes": report, "clocks": clocks}), flush=True)


def _fibirax_kernel_table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx, hbm, tf) -> Dict[str, Any]:
    """Like ``_kernel_table`` for the Fibirax kernels (the clamped GLU runs for the routed and for the shared expert:
    its floor is stated for the mean of the two)."""
    out: Dict[str, Any] = {}
    W, H, G, dk, dv = s["width"], s["heads"], s["kv"], s["dk"], s["dv"]
    RH, rdk, rdv, top = s["rheads"], s["rdk"], s["rdv"], s["top"]
    for phase, events, n_tok, past in (("prompt", ev_prompt, B * Pn, 0), ("decode", ev_decode, Bd, ctx)):
        by: Dict[str, List[float]] = {}
        for name, a, b in events:
            by.setdefault(name, []).append(a.elapsed_time(b) * 1e-3)
        per_seq = n_tok // (B if phase == "prompt" else Bd)
        n_seq = n_tok // per_seq
        pairs_win = sum(min(past + t + 1, FIBIRAX_WINDOW) for t in range(per_seq))
        keys_win = min(past + per_seq, FIBIRAX_WINDOW + per_seq)
        attn = (n_seq * keys_win * G * (dk + dv) * 2 + n_tok * H * (dk + dv) * 2, n_seq * H * 2 * (dk + dv) * pairs_win)
        floors = {
            "cast_rows": (n_tok * W * 6, 0),
            "rms_norm": (n_tok * W * 6, 0),
            "branch_postnorm_residual": (n_tok * W * (4 + 4 + 2 + 2), 0),
            "qknorm_rotary_append": (n_tok * (H * dk * 2 + G * (dk + dv) * 2) * 2, 0),
            "mixed_prompt_attention": attn,
            "mixed_paged_attention": attn,
            "retention_scan": (n_tok * RH * (2 * rdk + rdv) * 2 + n_tok * RH * rdv * 4 + 2 * n_seq * RH * rdk * rdv * 4, 0),
            "head_norm_act_gate": (n_tok * RH * rdv * 8, 0),
            "clamped_glu": (n_tok * (top + 1) // 2 * s["eff"] * 6, 0),
            "gather_rows": (n_tok * top * W * 4, 0),
            "weighted_expert_combine": (n_tok * top * W * 2 + n_tok * W * (4 + 4 + 2), 0),
        }
        for name, ts in by.items():
            t = statistics.mean(ts)
            entry = {"us": round(t * 1e6, 1), "calls": len(ts)}
            if name in floors:
                nbytes, flops = floors[name]
                floor = max(nbytes / hbm, flops / tf)
                entry["of_floor"] = round(floor / t, 3)
                entry["bound"] = "math" if flops / tf > nbytes / hbm else "memory"
            out.setdefault(phase, {})[name] = entry
    return out


# ---- Vatazen beside Fibirax ------------------------------------------------------------------------------------------
VATAZEN_WINDOW = 512      # the latent layers' window; the differential layers see blocks of this many positions too
VATAZEN_RANK, VATAZEN_ROT, VATAZEN_SIDE = 256, 64, 64


def vatazen_config(s: Dict[str, int]) -> Dict[str, Any]:
    """Latent and differential layers in turn.  A differential layer runs two maps per head, so it gets half the heads of
    the size's head layout: both layer types then put ``heads`` score maps on the attention kernel."""
    lat = {"heads": s["heads"], "dim": s["dk"], "rot_dim": VATAZEN_ROT, "vdim": s["dv"], "kv_rank": VATAZEN_RANK,
           "scale": 1.0 / math.sqrt(s["dk"] + VATAZEN_ROT), "mask": {"size": VATAZEN_WINDOW},
           "rot": {"base": 10000.0, "dims": VATAZEN_ROT,
                   "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}}
    dif = {"heads": s["heads"] // 2, "kv_heads": max(s["kv"] // 2, 1), "dim": s["dk"], "vdim": s["dv"], "diff": 0.3,
           "scale": 1.0 / math.sqrt(s["dk"]), "mask": {"size": VATAZEN_WINDOW}}
    mlp = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    layers = [{"type": "latent_attention" if i % 2 == 0 else "attention", "mixer": lat if i % 2 == 0 else dif, "mlp": mlp}
              for i in range(LAYERS)]
    return {"architecture": "Vatazen", "width": s["width"], "vocab": VOCAB, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "token_side": {"dim": VATAZEN_SIDE}, "layers": layers}


def run_vatazen(args, measured_peaks, ClockSampler) -> None:
    from . import fibirax_layer as Fx
    from . import mixer_ops
    from . import vatazen_layer as Vz
    from .ragged_engine import RaggedStepEngine

    dev = "cuda:0"
    peaks, how = measured_peaks()
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = max(3, args.steps), max(3, args.warmup)
    B, Pn, ctx, Bd = 8, 2048, 2048, 64
    g = torch.Generator().manual_seed(0)
    sampler = ClockSampler(0)
    sampler.start()
    report: Dict[str, Any] = {}
    for name, s in SIZES.items():
        if args.compare_sizes and name not in args.compare_sizes.split(","):
            continue
        row: Dict[str, Any] = {}
        prompts = torch.randint(0, VOCAB, (Bd, ctx), generator=g).tolist()
        for label, mod, raw in (("vatazen", Vz, vatazen_config(s)), ("fibirax", Fx, fibirax_config(s))):
            cfg = (Vz.VatazenConfig if mod is Vz else Fx.FibiraxConfig).from_dict(raw)
            shards = mod.build_shards(cfg, mod.random_checkpoint(cfg, seed=0), [(0, LAYERS)], dev, torch.bfloat16)
            eng = RaggedStepEngine(shards, max_tokens=Bd * (ctx + 64), max_seqs=Bd, fp32_logits=False)

            def prompt_step():
                eng.step([(i, prompts[i][:Pn], [Pn - 1]) for i in range(B)])
                for i in range(B):
                    eng.finish(i)

            ms = _time_steps(prompt_step, steps, warmup)
            row[label + "_prefill_tok_s"] = round(B * Pn / ms * 1e3)
            mixer_ops.EVENTS = []
            prompt_step()
            torch.cuda.synchronize()
            ev_prompt, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            for i in range(0, Bd, B):
                eng.step([(j, prompts[j], []) for j in range(i, i + B)])
            nxt = [[1] for _ in range(Bd)]

            def decode_step():
                eng.step([(j, nxt[j], [0]) for j in range(Bd)])

            n_dec = min(steps, 32)
            ms = _time_steps(decode_step, n_dec, warmup)
            row[label + "_decode_tok_s"] = round(Bd / ms * 1e3)
            mixer_ops.EVENTS = []
            decode_step()
            torch.cuda.synchronize()
            ev_decode, mixer_ops.EVENTS = mixer_ops.EVENTS, None
            eng.release()
            table = _vatazen_kernel_table if mod is Vz else _fibirax_kernel_table
            row[label + "_kernels"] = table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx + warmup + n_dec, hbm, tf)
            del eng, shards
            torch.cuda.empty_cache()
        row["inputs_exceed_l2"] = bool(Bd * ctx * (VATAZEN_RANK + VATAZEN_ROT) * 2 * LAYERS > 126e6)
        report[name] = row
    clocks = sampler.stop()
    print(json.dumps({"bench": "vatazen_vs_fibirax", "unit": "tokens/s", "dtype": "bf16", "data": "synthetic",
                      "layers": LAYERS, "prompt_step": f"{B} x {Pn} tokens", "decode_step": f"{Bd} sequences at {ctx}",
                      "peaks": how, "sizes": report, "clocks": clocks}), flush=True)


def _vatazen_kernel_table(s, ev_prompt, ev_decode, B, Pn, Bd, ctx, hbm, tf) -> Dict[str, Any]:
    """Like ``_kernel_table`` for the Vatazen kernels.  The attention kernel serves latent and differential layers in
    turn; its calls are listed per layer type (even calls of a step are latent layers)."""
    out: Dict[str, Any] = {}
    W, H, G, dk, dv, top = s["width"], s["heads"], s["kv"], s["dk"], s["dv"], s["top"]
    r, dr = VATAZEN_RANK, VATAZEN_ROT
    Hd, Gd = H // 2, max(G // 2, 1)
    for phase, events, n_tok, past in (("prompt", ev_prompt, B * Pn, 0), ("decode", ev_decode, Bd, ctx)):
        by: Dict[str, List[float]] = {}
        n_attn = 0
        for name, a, b in events:
            if name in ("mixed_prompt_attention", "mixed_paged_attention"):
                name += "[latent]" if n_attn % 2 == 0 else "[differential]"
                n_attn += 1
            by.setdefault(name, []).append(a.elapsed_time(b) * 1e-3)
        per_seq = n_tok // (B if phase == "prompt" else Bd)
        n_seq = n_tok // per_seq
        pairs_win = sum(min(past + t + 1, VATAZEN_WINDOW) for t in range(per_seq))
        pairs_blk = sum((past + t) % VATAZEN_WINDOW + 1 for t in range(per_seq))
        keys_win = min(past + per_seq, VATAZEN_WINDOW + per_seq)
        keys_blk = min(past + per_seq, (past % VATAZEN_WINDOW) + per_seq)
        lat = (n_seq * keys_win * (r + dr) * 2 + n_tok * H * (2 * r + dr) * 2, n_seq * H * 2 * (2 * r + dr) * pairs_win)
        dif = (n_seq * keys_blk * Gd * (2 * dk + dv) * 2 + n_tok * 2 * Hd * (dk + dv) * 2, n_seq * 2 * Hd * 2 * (dk + dv) * pairs_blk)
        floors = {
            "token_shift": (n_tok * W * 7, 0),
            "latent_rotary_append": (n_tok * (H * dr + r + dr) * 4, 0),
            "qknorm_rotary_append": (n_tok * (2 * Hd * dk * 2 + Gd * (2 * dk + dv) * 2) * 2, 0),
            "mixed_prompt_attention[latent]": lat,
            "mixed_paged_attention[latent]": lat,
            "mixed_prompt_attention[differential]": dif,
            "mixed_paged_attention[differential]": dif,
            "head_diff_norm": (n_tok * Hd * dv * 10, 0),      # two fp32 maps in, one 16-bit row out
            "gated_postnorm_residual": (n_tok * W * 14, 0),
            "relu_squared": (n_tok * top * s["eff"] * 4, 0),
            "gated_table_rows": (n_tok * VATAZEN_SIDE * 6, 0),
            "router_logits": (n_tok * W * 4, 0),
            "gather_rows": (n_tok * top * W * 4, 0),
            "weighted_expert_combine": (n_tok * top * W * 2 + n_tok * W * (4 + 4), 0),
        }
        for name, ts in by.items():
            t = statistics.mean(ts)
            entry = {"us": round(t * 1e6, 1), "calls": len(ts)}
            if name in floors:
                nbytes, flops = floors[name]
                floor = max(nbytes / hbm, flops / tf)
                entry["of_floor"] = round(floor / t, 3)
                entry["bound"] = "math" if flops / tf > nbytes / hbm else "memory"
            out.setdefault(phase, {})[name] = entry
    return out
