"""CPU: configuration, registry, pools and checkpoint layout of the Vatazen model class, and sanity of its oracle."""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from dgi_b200 import model_registry
from dgi_b200 import vatazen_layer as Vz
from oracle import vatazen_ref as R

F64 = torch.float64
CFG = {
    "architecture": "Vatazen", "width": 24, "vocab": 19, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "token_side": {"dim": 3},
    "layers": [
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 10, "kv_rank": 14, "scale": 0.3, "mask": {"size": 7},
                   "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 2.0, "slow": 1.0}}},
         "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 4, "top": 2}}},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "diff": 0.25, "scale": 0.35, "mask": {"size": 5}},
         "mlp": None},
    ],
}


def test_config_names_pools_and_states():
    cfg = Vz.VatazenConfig.from_dict(CFG)
    assert cfg.num_hidden_layers == 2 and cfg.hidden_size == 24 and cfg.vocab_size == 19 and cfg.embed_scale == 2.0
    assert cfg.side_dim == 3
    assert cfg.kv_shape(0) == (1, 18, 0) and cfg.state_shape(0) == (24,)      # one row [latent | rotated key part] per token
    assert cfg.kv_shape(1) == (2, 16, 6) and cfg.state_shape(1) == (24,)      # both maps' keys of a kv head side by side
    with pytest.raises(NotImplementedError):
        Vz.VatazenConfig.from_dict(dict(CFG, layers=[dict(CFG["layers"][0], type="retention")]))
    bad = dict(CFG["layers"][0], mlp=dict(CFG["layers"][0]["mlp"], kind="dense"))
    with pytest.raises(NotImplementedError):
        Vz.VatazenConfig.from_dict(dict(CFG, layers=[bad]))
    odd = dict(CFG["layers"][1], mixer=dict(CFG["layers"][1]["mixer"], kv_heads=3))
    with pytest.raises(ValueError):
        Vz.VatazenConfig.from_dict(dict(CFG, layers=[odd]))
    plain = Vz.VatazenConfig.from_dict({k: v for k, v in CFG.items() if k not in ("token_side", "embedding")})
    assert plain.side_dim == 0 and plain.embed_scale == 1.0
    assert model_registry.architecture_of(CFG).name == "Vatazen"
    assert "Vatazen" in model_registry.known_architectures()


def test_random_checkpoint_has_the_checkpoint_names():
    cfg = Vz.VatazenConfig.from_dict(CFG)
    t = Vz.random_checkpoint(cfg, seed=1)
    assert tuple(t["side.embed"].shape) == (19, 6) and "head" not in t
    assert tuple(t["l0.mix.q"].shape) == (20, 24) and tuple(t["l0.mix.dkv"].shape) == (18, 24)
    assert tuple(t["l0.mix.dkv.norm"].shape) == (14,) and tuple(t["l0.mix.uk"].shape) == (12, 14)
    assert tuple(t["l0.mix.uv"].shape) == (20, 14) and tuple(t["l0.mix.sink"].shape) == (2,)
    assert tuple(t["l1.mix.q"].shape) == (64, 24) and tuple(t["l1.mix.k"].shape) == (32, 24) and tuple(t["l1.mix.v.b"].shape) == (12,)
    assert tuple(t["l1.mix.q.norm"].shape) == (8,) and tuple(t["l1.mix.lk2"].shape) == (8,) and tuple(t["l1.mix.o.b"].shape) == (24,)
    assert tuple(t["l0.mlp.router"].shape) == (4, 24) and tuple(t["l0.mlp.router.b"].shape) == (4,)
    assert "l0.mlp.e3.down" in t and "l0.mlp.e4.up" not in t and "l1.mlp.router" not in t and "l1.norm2" not in t
    assert tuple(t["l1.shift"].shape) == (24,) and tuple(t["l1.rg1"].shape) == (24, 24) and "l1.rg2" not in t
    assert tuple(t["l1.side.gate"].shape) == (3, 24) and tuple(t["l1.side.proj"].shape) == (24, 3)
    logits = R.forward(CFG, t, [1, 5, 7, 2, 2, 18, 0, 3, 9, 11])
    assert logits.shape == (10, 19) and torch.isfinite(logits).all()


def test_frequency_table_against_the_oracle():
    sc = {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 1.0}
    for dims, base in ((12, 50.0), (32, 10000.0), (2, 7.0)):
        for scaling in (sc, None):
            f, gain = Vz.yarn_frequencies(dims, base, scaling)
            fr, gr = R.yarn_frequencies(dims, base, scaling)
            assert torch.allclose(f, fr, rtol=1e-14) and abs(gain - gr) < 1e-15


def test_oracle_properties():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=F64)
    pos = torch.arange(5)
    f, _ = R.yarn_frequencies(4, 50.0, None)
    part = R.rotate_pairs(x, pos, f, 1.0)
    assert (part[..., 4:] == x[..., 4:]).all() and (part[0] == x[0]).all()          # position 0 turns nothing
    assert torch.allclose(part.norm(dim=-1), x.norm(dim=-1))
    assert torch.allclose(R.rotate_pairs(x, pos, f, 1.3)[..., :4], 1.3 * part[..., :4])   # the gain scales the turned part only
    # a rotation enters a score by the distance only
    a, b = R.rotate_pairs(x[:1].expand(5, 2, 8), pos, f, 1.0), R.rotate_pairs(x[1:2].expand(5, 2, 8), pos + 3, f, 1.0)
    s = (a * b).sum(-1)
    assert torch.allclose(s, s[:1].expand_as(s))
    # the shift reads the UNSHIFTED previous row; mu = 0 changes nothing, mu = 1 hands every token its predecessor
    h = torch.randn(6, 3, generator=g, dtype=F64)
    assert torch.equal(R.token_shift(h, torch.zeros(3, dtype=F64)), h)
    assert torch.allclose(R.token_shift(h, torch.ones(3, dtype=F64))[1:], h[:-1], atol=1e-14)
    assert torch.allclose(R.token_shift(h[2:], torch.ones(3, dtype=F64), before=h[1])[0], h[1], atol=1e-14)
    # masks: a window as long as the sequence and a block as long as the sequence are plain causal
    assert torch.equal(R.visible(7, window=7), R.visible(7)) and torch.equal(R.visible(7, chunk=7), R.visible(7))
    assert R.visible(9, chunk=4)[5].tolist() == [False] * 4 + [True, True] + [False] * 3
    assert R.visible(9, window=3)[5].tolist() == [False] * 3 + [True] * 3 + [False] * 3
    # the sink only shrinks: alone with one key the weight is e^s / (e^s + e^sink)
    q, k, v = (torch.randn(4, 2, 6, generator=g, dtype=F64) for _ in range(3))
    sink = torch.tensor([0.3, -1.0], dtype=F64)
    o = R.softmax_attention(q, k, v, 0.5, R.visible(4), sink)
    e0 = math.exp(float((q[0, 0] @ k[0, 0]) * 0.5))
    assert torch.allclose(o[0, 0], v[0, 0] * e0 / (e0 + math.exp(0.3)))
    # routing: the softmax over the chosen equals the softmax over all, renormalised over the chosen
    z = torch.randn(50, 12, generator=g, dtype=F64)
    ids, w = R.route(z, 3)
    full = torch.softmax(z, dim=-1).gather(1, ids)
    assert torch.allclose(w, full / full.sum(-1, keepdim=True)) and torch.allclose(w.sum(-1), torch.ones(50, dtype=F64))
    assert torch.equal(ids.sort(dim=1).values, z.topk(3, dim=-1).indices.sort(dim=1).values)
