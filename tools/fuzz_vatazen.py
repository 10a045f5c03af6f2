"""Random Vatazen configurations (layer orders, head layouts and sizes on and off the tensor-core grid, latent ranks and
rotated widths, rotary widths with and without YaRN rescaling, windows, blocks, expert counts, layers without a
feed-forward, models without the token table): the ragged step engine in fp32 and bf16, two requests cut into random
portions and mixed in steps with slots used again, against oracle/vatazen_ref.py.
``python tools/fuzz_vatazen.py [n_seeds]`` on a B200; prints one line per seed and ``bad <count>``."""
import json
import os
import random
import sys
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

import dgi_b200  # noqa: E402,F401
from dgi_b200 import vatazen_layer as Vz  # noqa: E402
from dgi_b200.ragged_engine import RaggedStepEngine  # noqa: E402
from oracle import vatazen_ref as R  # noqa: E402


def rand_layer(rng):
    mlp = None
    if rng.random() < 0.85:
        E = rng.choice([1, 2, 3, 4, 6, 8, 12, 16, 40])
        mlp = {"kind": "moe", "expert": {"ff": rng.choice([8, 24, 40, 64, 96, 136])},
               "router": {"experts": E, "top": rng.randint(1, min(E, 4))}}
    if rng.random() < 0.5:
        H = rng.choice([1, 2, 3, 4, 6, 8, 12, 16, 20, 33])
        dn = rng.choice([2, 4, 8, 16, 24, 32, 64, 96])
        dr = rng.choice([2, 4, 8, 16, 32, 64])
        rank = rng.choice([4, 8, 24, 32, 48, 56, 64, 96, 128, 192, 256, 2 * rng.randint(2, 60)])
        dims = rng.choice([dr, dr, dr, max(2, dr // 2 - (dr // 2) % 2)])
        m = {"heads": H, "dim": dn, "rot_dim": dr, "vdim": rng.choice([2, 8, 16, 24, 32, 64, 100]), "kv_rank": rank,
             "scale": rng.choice([(dn + dr) ** -0.5, 0.1, 0.3]),
             "mask": {"size": rng.choice([1, 2, 7, 16, 31, 32, 33, 40, 64, 100, 1000])},
             "rot": {"base": rng.choice([50.0, 10000.0, 500000.0, 1e6]), "dims": dims}}
        if rng.random() < 0.75:
            m["rot"]["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0, 40.0]), "original": rng.choice([16, 64, 2048, 4096]),
                                   "fast": rng.choice([32.0, 8.0, 2.0]), "slow": rng.choice([1.0, 0.5, 2.0])}
        return {"type": "latent_attention", "mixer": m, "mlp": mlp}
    G = rng.choice([1, 2, 3, 4])
    H = G * rng.choice([1, 2, 3, 4, 8])
    dk = rng.choice([4, 8, 16, 24, 32, 48, 64, 128])
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": rng.choice([4, 8, 16, 24, 32, 64, 128, 2 * rng.randint(2, 40)]),
         "diff": rng.choice([0.0, 0.1, 0.3, 0.5, 0.8]), "scale": rng.choice([dk ** -0.5, 0.1, 0.3]),
         "mask": {"size": rng.choice([1, 2, 7, 16, 31, 32, 33, 64, 100, 1000])}}
    if rng.random() < 0.3:
        del m["kv_heads"]
        m["heads"] = rng.choice([1, 2, 5, 8])
    return {"type": "attention", "mixer": m, "mlp": mlp}


def rand_cfg(rng):
    raw = {"architecture": "Vatazen", "width": rng.choice([16, 32, 48, 64, 96, 128, 200]), "vocab": rng.choice([17, 64, 301]),
           "embedding": {"scale": rng.choice([0.5, 1.0, 4.0])}, "norm": {"eps": rng.choice([1e-6, 1e-5])},
           "layers": [rand_layer(rng) for _ in range(rng.randint(1, 6))]}
    # the sublayers read the residual itself, which grows by three unit-RMS updates per layer, and a latent layer's
    # queries and rotated keys are not normed: keep its scores O(1) so that the softmax stays well conditioned and the
    # tolerances below can be fixed numbers
    for i, layer in enumerate(raw["layers"]):
        if layer["type"] == "latent_attention":
            m = layer["mixer"]
            m["scale"] = rng.choice([0.5, 1.0, 2.0]) / (4.0 * (1 + 3 * i) * (m["dim"] + m["rot_dim"]) ** 0.5)
    if rng.random() < 0.8:
        raw["token_side"] = {"dim": rng.choice([1, 4, 8, 24, 30])}
    if rng.random() < 0.2:
        del raw["embedding"]
    return raw


def main():
    bad = 0
    for seed in range(int(sys.argv[1]) if len(sys.argv) > 1 else 24):
        rng = random.Random(seed)
        raw = rand_cfg(rng)
        try:
            cfg = Vz.VatazenConfig.from_dict(raw)
            tensors = Vz.random_checkpoint(cfg, seed=seed)
            g = torch.Generator().manual_seed(seed)
            n1, n2 = rng.randint(40, 150), rng.randint(1, 60)
            t1 = torch.randint(0, raw["vocab"], (n1,), generator=g).tolist()
            t2 = torch.randint(0, raw["vocab"], (n2,), generator=g).tolist()
            ref1, ref2 = R.forward(raw, tensors, t1), R.forward(raw, tensors, t2)
            # what fp32 arithmetic alone does to this model (the same statement in fp32): the yardstick for the fp32 engine
            cond = max(float((R.forward(raw, tensors, t, dtype=torch.float32).double() - ref).abs().max() / max(1.0, ref.abs().max()))
                       for t, ref in ((t1, ref1), (t2, ref2)))
            # 16-bit storage rounds 2^16 times coarser but far less often; a model that amplifies fp32 rounding amplifies it too
            for dt, tol in ((torch.float32, max(5e-5, 4.0 * cond)), (torch.bfloat16, max(6e-2, 3000.0 * cond))):
                eng = RaggedStepEngine(Vz.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], "cuda:0", dt), max_tokens=256,
                                       max_seqs=2)
                eng.step([("z", t2[:7], [])])        # a request that leaves: its slot and page are used again
                eng.finish("z")
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
                        # the median token
                        per_tok = (gg - ref).pow(2).mean(dim=1).sqrt() / ref.pow(2).mean().sqrt()
                        err = float(per_tok.median())
                    if not (err <= tol):
                        bad += 1
                        print("MISMATCH seed", seed, dt, err, "allowed", tol, json.dumps(raw), flush=True)
            print("seed", seed, "ok", [(l["type"][:3], l["mixer"]["heads"], l["mixer"]["dim"], l["mixer"]["vdim"]) for l in raw["layers"]],
                  flush=True)
        except Exception as e:  # noqa: BLE001
            bad += 1
            print("ERROR seed", seed, type(e).__name__, str(e)[:300], json.dumps(raw), flush=True)
            traceback.print_exc()
    print("bad", bad)
    return bad


if __name__ == "__main__":
    sys.exit(1 if main() else 0)
