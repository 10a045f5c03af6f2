"""CPU: configuration, registry, pools and checkpoint layout of the Fibirax model class, and sanity of its oracle."""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from dgi_b200 import fibirax_layer as Fx
from dgi_b200 import model_registry
from oracle import fibirax_ref as R

F64 = torch.float64
CFG = {
    "architecture": "Fibirax", "width": 24, "vocab": 19, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.35, "softcap": 3.0, "mask": {"size": 7},
                            "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}}},
                   "right": {"heads": 3, "dim": 6, "vdim": 10, "decay": [0.9, 0.5, 0.99]}, "left_scale": 0.7, "right_scale": 1.2},
         "mlp": {"kind": "moe", "expert": {"ff": 12, "limit": 1.5}, "shared": {"ff": 8, "limit": 0.7},
                 "router": {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 2}}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 2, "dim": 4, "vdim": 4, "scale": 0.5},
                   "right": {"heads": 1, "dim": 4, "vdim": 2, "decay": [1.0]}, "left_scale": 1.0, "right_scale": 1.0},
         "mlp": None},
    ],
}


def test_config_names_pools_and_states():
    cfg = Fx.FibiraxConfig.from_dict(CFG)
    assert cfg.num_hidden_layers == 2 and cfg.hidden_size == 24 and cfg.vocab_size == 19 and cfg.embed_scale == 2.0
    assert cfg.kv_shape(0) == (2, 8, 6) and cfg.state_shape(0) == (3, 6, 10)     # every layer keeps pages AND a state
    assert cfg.kv_shape(1) == (2, 4, 4) and cfg.state_shape(1) == (1, 4, 2)      # kv_heads defaults to heads
    with pytest.raises(NotImplementedError):
        Fx.FibiraxConfig.from_dict(dict(CFG, layers=[dict(CFG["layers"][0], type="serial")]))
    bad = dict(CFG["layers"][0], mlp=dict(CFG["layers"][0]["mlp"], kind="dense"))
    with pytest.raises(NotImplementedError):
        Fx.FibiraxConfig.from_dict(dict(CFG, layers=[bad]))
    short = dict(CFG["layers"][0]["mixer"], right=dict(CFG["layers"][0]["mixer"]["right"], decay=[0.5]))
    with pytest.raises(ValueError):
        Fx.FibiraxConfig.from_dict(dict(CFG, layers=[dict(CFG["layers"][0], mixer=short)]))
    assert model_registry.architecture_of(CFG).name == "Fibirax"
    assert "Fibirax" in model_registry.known_architectures()


def test_random_checkpoint_has_the_checkpoint_names():
    cfg = Fx.FibiraxConfig.from_dict(CFG)
    t = Fx.random_checkpoint(cfg, seed=1)
    assert tuple(t["l0.mix.left.q"].shape) == (32, 24) and tuple(t["l0.mix.left.v"].shape) == (12, 24)
    assert tuple(t["l0.mix.left.q.norm"].shape) == (8,) and tuple(t["l0.mix.left.o"].shape) == (24, 24)
    assert tuple(t["l0.mix.right.g"].shape) == (30, 24) and tuple(t["l0.mix.right.o"].shape) == (24, 30)
    assert tuple(t["l0.mlp.router"].shape) == (6, 24) and tuple(t["l0.mlp.correction"].shape) == (6,)
    assert "l0.mlp.e3.down" in t and "l0.mlp.e4.gate" not in t and tuple(t["l0.mlp.shared.up"].shape) == (8, 24)
    assert "l1.mlp.router" not in t and "l1.norm2" not in t and tuple(t["l1.ls1"].shape) == (24,)
    logits = R.forward(CFG, t, [1, 5, 7, 2, 2, 18, 0, 3, 9, 11])
    assert logits.shape == (10, 19) and torch.isfinite(logits).all()


def test_frequency_table_against_the_oracle():
    sc = {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 40}
    for dims, base in ((12, 50.0), (32, 10000.0), (2, 7.0)):
        assert torch.allclose(Fx.wavelength_scaled_frequencies(dims, base, sc), R.rotary_frequencies(dims, base, sc), rtol=1e-14)
        assert torch.allclose(Fx.wavelength_scaled_frequencies(dims, base, None), R.rotary_frequencies(dims, base, None), rtol=1e-14)


def test_oracle_properties():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=F64)
    pos = torch.arange(5)
    f = R.rotary_frequencies(4, 50.0, None)
    part = R.rotate_pairs(x, pos, f)
    assert (part[..., 4:] == x[..., 4:]).all() and (part[0] == x[0]).all()          # position 0 turns nothing
    assert torch.allclose(part.norm(dim=-1), x.norm(dim=-1))
    # a rotation enters a score by the distance only
    a, b = R.rotate_pairs(x[:1].expand(5, 2, 8), pos, f), R.rotate_pairs(x[1:2].expand(5, 2, 8), pos + 3, f)
    s = (a * b).sum(-1)
    assert torch.allclose(s, s[:1].expand_as(s))
    # decay 1 and orthonormal keys: the state returns what was stored under a key
    n, dk, dv = 3, 4, 2
    k = torch.eye(dk, dtype=F64)[:n].view(n, 1, dk)
    v = torch.randn(n, 1, dv, generator=g, dtype=F64)
    o, S = R.retention_scan(k, k, v, [1.0])
    assert (o - v).abs().max() < 1e-12 and S.shape == (1, dk, dv)
    o2, _ = R.retention_scan(k[:1], k[:1], v[:1], [0.5], state=S)                   # one more step from a carried state
    assert torch.allclose(o2[0, 0], 0.5 * v[0, 0] + v[0, 0])
    # a window as long as the sequence is plain causal attention; a huge cap is no cap; the sink only shrinks
    q, kk, vv = (torch.randn(7, 2, 4, generator=g, dtype=F64) for _ in range(3))
    full = R.capped_window_attention(q, kk, vv, 0.5)
    assert (R.capped_window_attention(q, kk, vv, 0.5, 7) - full).abs().max() < 1e-12
    assert (R.capped_window_attention(q, kk, vv, 0.5, 0, 1e6) - full).abs().max() < 1e-9
    plain = R.capped_window_attention(q, kk, vv, 0.5, sink=False)
    e0 = math.exp(float((q[0, 0] @ kk[0, 0]) * 0.5))
    assert torch.allclose(full[0, 0], plain[0, 0] * e0 / (1 + e0))
    # routing: weights sum to one, a dropped group is never chosen even when every choice score is negative
    z = torch.randn(50, 12, generator=g, dtype=F64)
    corr = -2.0 - torch.rand(12, generator=g, dtype=F64)
    ids, w = R.route(z, corr, 3, 4, 1)
    assert torch.allclose(w.sum(-1), torch.ones(50, dtype=F64)) and all(len({int(e) // 3 for e in row}) == 1 for row in ids)
    ids_all, _ = R.route(z, torch.zeros(12, dtype=F64), 3, 1, 1)
    assert torch.equal(ids_all.sort(dim=1).values, z.topk(3, dim=-1).indices.sort(dim=1).values)
