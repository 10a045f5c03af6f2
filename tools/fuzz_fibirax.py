"""Random Fibirax configurations (head layouts and sizes on and off the tensor-core grid, windows, rotary widths with and
without frequency rescaling, soft caps, decays, branch weights, expert counts, groups, identity and shared experts,
layers without a feed-forward): the ragged step engine in fp32 and bf16, two requests cut into random portions and mixed
in steps, against oracle/fibirax_ref.py.  ``python tools/fuzz_fibirax.py [n_seeds]`` on a B200; prints one line per seed
and ``bad <count>``."""
import json
import os
import random
import sys
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

import dgi_b200  # noqa: E402,F401
from dgi_b200 import fibirax_layer as Fx  # noqa: E402
from dgi_b200.ragged_engine import RaggedStepEngine  # noqa: E402
from oracle import fibirax_ref as R  # noqa: E402


def rand_layer(rng):
    G = rng.choice([1, 2, 3, 4])
    H = G * rng.choice([1, 2, 3, 4, 8])
    dk = rng.choice([4, 8, 16, 24, 32, 48, 64, 96, 128])
    dv = rng.choice([4, 8, 16, 24, 32, 48, 64, 96, 128, 2 * rng.randint(2, 40)])
    left = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": rng.choice([dk ** -0.5, 0.1, 0.3])}
    if rng.random() < 0.85:
        left["mask"] = {"size": rng.choice([1, 2, 7, 16, 31, 32, 33, 64, 100, 1000])}
    if rng.random() < 0.8:
        left["softcap"] = rng.choice([1.0, 5.0, 20.0, 50.0])
    dims = rng.choice([0, 2, 4, dk // 2 - (dk // 2) % 2, dk])
    if dims:
        left["rot"] = {"base": rng.choice([50.0, 10000.0, 500000.0, 1e6]), "dims": dims}
        if rng.random() < 0.7:
            left["rot"]["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                                      "original": rng.choice([16, 64, 1024])}
    Hr = rng.choice([1, 2, 3, 4])
    right = {"heads": Hr, "dim": rng.choice([2, 4, 8, 16, 32, 33, 64, 96, 128, 160, 256]),
             "vdim": rng.choice([2, 4, 16, 31, 32, 64, 100]),
             "decay": [rng.choice([1.0, 0.999, 1 - 2.0 ** -10, 0.97, 0.9, 0.5, 0.1]) for _ in range(Hr)]}
    mlp = None
    if rng.random() < 0.8:
        groups = rng.choice([1, 1, 2, 3, 4])
        per = rng.randint(1, 4)
        total = groups * per
        ident = rng.randint(0, min(total - 1, 3))
        keep = rng.randint(1, groups)
        top = rng.randint(1, min(4, keep * per))
        mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 24, 40, 64, 136]), "limit": rng.choice([0.5, 1.0, 7.0])},
               "router": {"experts": total - ident, "identity": ident, "top": top}}
        if groups > 1 or rng.random() < 0.5:
            mlp["router"]["groups"] = {"count": groups, "keep": keep}
        if rng.random() < 0.6:
            mlp["shared"] = {"ff": rng.choice([8, 40, 96]), "limit": rng.choice([0.5, 1.5])}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": rng.choice([0.8, 1.0, 0.3, -0.5, 0.0]),
                                          "right_scale": rng.choice([0.5, 1.0, 2.0, -1.0, 0.0])}, "mlp": mlp}


def rand_cfg(rng):
    return {"architecture": "Fibirax", "width": rng.choice([16, 32, 48, 64, 96, 128, 200]), "vocab": rng.choice([17, 64, 301]),
            "embedding": {"scale": rng.choice([0.5, 1.0, 4.0])}, "norm": {"eps": rng.choice([1e-6, 1e-5])},
            "layers": [rand_layer(rng) for _ in range(rng.randint(1, 5))]}


bad = 0
for seed in range(int(sys.argv[1]) if len(sys.argv) > 1 else 24):
    rng = random.Random(seed)
    raw = rand_cfg(rng)
    try:
        cfg = Fx.FibiraxConfig.from_dict(raw)
        tensors = Fx.random_checkpoint(cfg, seed=seed)
        g = torch.Generator().manual_seed(seed)
        n1, n2 = rng.randint(40, 150), rng.randint(1, 60)
        t1 = torch.randint(0, raw["vocab"], (n1,), generator=g).tolist()
        t2 = torch.randint(0, raw["vocab"], (n2,), generator=g).tolist()
        ref1, ref2 = R.forward(raw, tensors, t1), R.forward(raw, tensors, t2)
        for dt, tol in ((torch.float32, 5e-5), (torch.bfloat16, 4e-2)):
            eng = RaggedStepEngine(Fx.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], "cuda:0", dt), max_tokens=256,
                                   max_seqs=2)
            got1, got2, a1, a2 = [], [], 0, 0
            while a1 < n1 or a2 < n2:
                entries = []
                c1 = min(n1 - a1, rng.choice([1, 1, 2, 3, 17, 40]))
                c2 = min(n2 - a2, rng.choice([0, 1, 2, 9]))
                if c1:
                    entries.append(("a", t1[a1:a1 + c1], list(range(c1))))
                if c2:
                    entries.append(("b", t2[a2:a2 + c2], list(range(c2))))
                if rng.random() < 0.5:
                    entries.reverse()
                out, o = eng.step(entries), 0
                for rid, toks, _ in entries:
                    (got1 if rid == "a" else got2).append(out[o:o + len(toks)])
                    o += len(toks)
                a1 += c1
                a2 += c2
            eng.release()
            for got, ref in ((got1, ref1), (got2, ref2)):
                gg = torch.cat(got).cpu().double()
                if dt == torch.float32:
                    err = float((gg - ref).abs().max() / max(1.0, ref.abs().max()))
                else:
                    # a routing near-tie that 16-bit rounding flips changes a token's whole feed-forward output: judge
                    # the median token, and bound the mean loosely
                    per_tok = (gg - ref).pow(2).mean(dim=1).sqrt() / ref.pow(2).mean().sqrt()
                    err = float(per_tok.median())
                    if float(per_tok.pow(2).mean().sqrt()) > 0.25:
                        err = float("inf")
                if not (err <= tol):
                    bad += 1
                    print("MISMATCH seed", seed, dt, err, json.dumps(raw), flush=True)
        print("seed", seed, "ok", [(l["mixer"]["left"]["dim"], l["mixer"]["left"]["vdim"], l["mixer"]["right"]["dim"])
                                   for l in raw["layers"]], flush=True)
    except Exception as e:  # noqa: BLE001
        bad += 1
        print("ERROR seed", seed, type(e).__name__, str(e)[:300], json.dumps(raw), flush=True)
        traceback.print_exc()
print("bad", bad)
