"""GPU: the Vatazen model class on the ragged step engine against the plain float64 statement in oracle/vatazen_ref.py.

Small configurations with random weights; sizes are chosen so that nothing is a multiple of a warp, a page or a key
tile by accident (kv heads fewer than heads, one head, key sizes 2 / 12 / 40, latent ranks 4 / 22 / 40 / 48 / 72, rotated
widths that are turned in part, in full and over one pair, windows and blocks of 1, 5, 7, 9, 19, 24 and longer than the
sequence, expert counts of 1, 3, 5 and 8 with 1 to all of them chosen, a layer without a feed-forward, a model without
the token table or an embedding scale).  Where random weights would hide a fault the inputs are made so that it shows: one
key gets a score that dominates just inside and just outside a window or a block, all scores are pushed far below the
sink's, one far key among hundreds is the only one a query matches.
"""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from oracle import vatazen_ref as R

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def latent(heads, dim, rot_dim, vdim, rank, size, rot_dims=None, base=10000.0, scale=None, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "scale": scale or 1.0 / math.sqrt(dim + rot_dim), "mask": {"size": size},
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if scaling:
        m["rot"]["scaling"] = scaling
    return m


def differential(heads, kv, dim, vdim, size, diff, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "diff": diff, "mask": {"size": size},
            "scale": scale or 1.0 / math.sqrt(dim)}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


SCALING = {"factor": 3.0, "original": 24, "fast": 2.0, "slow": 0.5}

CFG_A = {   # sizes off every grid: the row kernels serve both storage types
    "architecture": "Vatazen", "width": 56, "vocab": 53, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "token_side": {"dim": 5},
    "layers": [
        layer("latent_attention", latent(3, 12, 6, 20, 22, 9, base=50.0, scale=0.3, scaling=SCALING), moe(5, 3, 40)),
        layer("attention", differential(4, 2, 12, 10, 7, 0.2, scale=0.35), None),
        layer("latent_attention", latent(1, 8, 4, 8, 40, 200, rot_dims=2, base=7.0), moe(3, 1, 16)),
        layer("attention", differential(3, 1, 40, 33, 33, 0.5), moe(5, 5, 24)),
    ],
}
CFG_B = {   # sizes the tensor-core attention and the grouped expert GEMM take in 16-bit storage
    "architecture": "Vatazen", "width": 64, "vocab": 41, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "token_side": {"dim": 8},
    "layers": [
        layer("latent_attention", latent(10, 16, 16, 24, 48, 19, base=200.0, scaling=SCALING), moe(8, 2, 32)),
        layer("attention", differential(8, 2, 16, 40, 24, 0.3), moe(4, 4, 48)),
        layer("latent_attention", latent(2, 32, 8, 16, 72, 40), None),
        layer("attention", differential(4, 4, 32, 8, 5, 0.1), moe(8, 1, 16)),
    ],
}
CFG_D = {   # many heads over one latent row: steps of single tokens put the heads on the rows of the attention's tiles
    "architecture": "Vatazen", "width": 64, "vocab": 37, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
    "layers": [layer("latent_attention", latent(20, 8, 8, 8, 24, 11, base=100.0), moe(4, 2, 16)),
               layer("latent_attention", latent(16, 16, 16, 16, 48, 300), None)],
}
CFG_C = {   # the smallest of everything, without the token table and the embedding scale
    "architecture": "Vatazen", "width": 16, "vocab": 11, "norm": {"eps": 1e-6},
    "layers": [layer("latent_attention", latent(1, 2, 2, 2, 4, 1), moe(1, 1, 8)),
               layer("attention", differential(1, 1, 4, 2, 1, 0.0), moe(2, 2, 8))],
}


def build(cfg_raw, dtype=torch.float32, seed=0, max_tokens=512, max_seqs=4):
    from dgi_b200 import vatazen_layer as Vz
    from dgi_b200.ragged_engine import RaggedStepEngine

    cfg = Vz.VatazenConfig.from_dict(cfg_raw)
    tensors = Vz.random_checkpoint(cfg, seed=seed)
    shards = Vz.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], DEV, dtype)
    return RaggedStepEngine(shards, max_tokens=max_tokens, max_seqs=max_seqs), tensors


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def whole(engine, rid, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    out = engine.step([(rid, toks, want)]).cpu()
    engine.finish(rid)
    return out


def close(got, ref, tol):
    err = (got.to(F64) - ref.to(F64)).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), f"max abs error {err}"


def rounding_close(got, ref, median=0.05, tail=0.15, tail_share=0.2):
    """16-bit storage against a wider statement, row by row (error rms over the statement's rms): the typical row is within
    rounding; a few rows may differ more, where rounding flips an expert's choice, but not many."""
    row = (got.to(F64) - ref.to(F64)).pow(2).mean(dim=1).sqrt() / ref.to(F64).pow(2).mean().sqrt()
    assert row.median() <= median, f"median row error {row.median().item()}"
    assert (row > tail).to(F64).mean() <= tail_share, f"rows over {tail}: {(row > tail).sum().item()} of {row.numel()}"


def paged(rows_by_pool, bs=16, seed=0):
    """Pools holding ``rows [n, G, d]`` (one per entry) in the same shuffled blocks, and the block table that finds them."""
    n = rows_by_pool[0].shape[0]
    nb = (n + bs - 1) // bs
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed))[:nb]
    pools = []
    for rows in rows_by_pool:
        pool = torch.full((nb + 3, rows.shape[1], bs, rows.shape[2]), float("nan"), dtype=rows.dtype)
        for t in range(n):
            pool[perm[t // bs], :, t % bs] = rows[t]
        pools.append(pool.to(DEV))
    return pools, perm.to(torch.int32).view(1, -1).to(DEV)


def seqs_of(spans):
    return torch.tensor(spans, dtype=torch.int32, device=DEV)


def tiles_of(cuts):
    tiles, at = [], 0
    for c in cuts:
        tiles.append((at, c, 0))
        at += c
    return torch.tensor(tiles, dtype=torch.int32, device=DEV), at


# ---- mechanisms, one at a time -------------------------------------------------------------------------------------
def test_frequency_table_ramp_and_gain():
    from dgi_b200 import vatazen_layer as Vz

    for dims, base, sc in ((6, 50.0, SCALING), (32, 10000.0, {"factor": 8.0, "original": 512, "fast": 16.0, "slow": 2.0}),
                           (2, 7.0, SCALING), (16, 200.0, None), (4, 3.0, {"factor": 1.0, "original": 8, "fast": 1.0, "slow": 1.0})):
        f, gain = Vz.yarn_frequencies(dims, base, sc)
        fr, gr = R.yarn_frequencies(dims, base, sc)
        assert torch.allclose(f, fr, rtol=1e-14) and abs(gain - gr) < 1e-15
    # the fast end keeps its frequency, the slow end is divided by the factor, the gain grows with the factor
    f, gain = Vz.yarn_frequencies(32, 10000.0, {"factor": 8.0, "original": 512, "fast": 16.0, "slow": 2.0})
    plain, one = Vz.yarn_frequencies(32, 10000.0, None)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 8.0) < 1e-18 and one == 1.0
    assert abs(gain - (0.1 * math.log(8.0) + 1.0)) < 1e-15


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)], ids=["fp32", "bf16"])
def test_token_shift_carries_the_last_row_per_slot(dt, tol):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(1)
    W = 150
    mu = torch.rand(W, generator=g).to(dt)
    state = torch.full((3, W), float("nan"), device=DEV)
    a, b = torch.randn(101, W, generator=g), torch.randn(40, W, generator=g)
    ref_a, ref_b = R.token_shift(a.to(F64), mu.to(F64)), R.token_shift(b.to(F64), mu.to(F64))
    # step 1: a's first 70 rows (three runs of a CTA) beside b's first row; both fresh, in slots 2 and 0
    x = torch.cat([a[:70], b[:1]]).to(DEV)
    out, cast = M.token_shift(x, mu.to(DEV), state, seqs_of([(0, 70, 2, 1), (70, 1, 0, 1)]), 70, want_cast=True)
    close(out[:70].cpu(), ref_a[:70], tol)
    close(out[70:].cpu(), ref_b[:1], tol)
    close(cast.cpu(), x.cpu(), tol)
    assert torch.equal(state[2].cpu(), a[69]) and torch.equal(state[0].cpu(), b[0]) and torch.isnan(state[1]).all()
    # step 2: single rows of both, then the rest; the row before comes from the slot
    x = torch.cat([b[1:2], a[70:71]]).to(DEV)
    out, cast = M.token_shift(x, mu.to(DEV), state, seqs_of([(0, 1, 0, 0), (1, 1, 2, 0)]), 1)
    assert cast is None
    close(out[:1].cpu(), ref_b[1:2], tol)
    close(out[1:].cpu(), ref_a[70:71], tol)
    x = torch.cat([a[71:], b[2:]]).to(DEV)
    out, _ = M.token_shift(x, mu.to(DEV), state, seqs_of([(0, 30, 2, 0), (30, 38, 0, 0)]), 38)
    close(out[:30].cpu(), ref_a[71:], tol)
    close(out[30:].cpu(), ref_b[2:], tol)
    # a new sequence in a used slot starts from zero, not from what the last owner left
    out, _ = M.token_shift(b[:5].to(DEV), mu.to(DEV), state, seqs_of([(0, 5, 2, 1)]), 5)
    close(out.cpu(), ref_b[:5], tol)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)], ids=["fp32", "bf16"])
@pytest.mark.parametrize("H,dn,dr,rank,dims,sc", [(3, 12, 6, 22, 6, SCALING), (1, 8, 4, 40, 2, None), (10, 16, 16, 48, 16, SCALING),
                                                  (2, 4, 2, 5, 0, None)])
def test_latent_norm_rotation_and_append(dt, tol, H, dn, dr, rank, dims, sc):
    from dgi_b200 import mixer_ops as M, vatazen_layer as Vz

    g = torch.Generator().manual_seed(H + rank)
    n, bs, nb = 37, 16, 5
    proj = torch.randn(n, H * (dn + dr) + rank + dr + 3, generator=g).to(dt)      # q | dkv inside one wider buffer
    w = (1.0 + 0.2 * torch.randn(rank, generator=g)).to(dt)
    pos = torch.randint(0, 3000, (n,), generator=g).to(torch.int32)
    slots = torch.randperm(nb * bs, generator=g)[:n].to(torch.int64)
    slots[5] = -1                                                                 # a skipped token stores nothing
    freqs, gain = Vz.yarn_frequencies(dims, 50.0, sc)
    pool = torch.full((nb, 1, bs, rank + dr), float("nan"), dtype=dt, device=DEV)
    dev = proj.to(DEV)
    q = dev[:, :H * (dn + dr)].unflatten(1, (H, dn + dr))
    q_out = torch.full((n, H, rank + dr), float("nan"), dtype=dt, device=DEV)
    M.latent_rotary_append(q[:, :, dn:], q_out[:, :, rank:], dev[:, H * (dn + dr):H * (dn + dr) + rank + dr], w.to(DEV), 1e-5,
                           freqs.to(DEV) if dims else None, gain, pool, slots.to(DEV), pos.to(DEV))
    p64 = proj.to(F64)
    dkv = p64[:, H * (dn + dr):H * (dn + dr) + rank + dr]
    c = R.rms(dkv[:, :rank], 1e-5) * w.to(F64)
    k_rot = R.rotate_pairs(dkv[:, rank:].reshape(n, 1, dr), pos, freqs, gain)[:, 0]
    q_rot = R.rotate_pairs(p64[:, :H * (dn + dr)].reshape(n, H, dn + dr)[..., dn:], pos, freqs, gain)
    close(q_out[:, :, rank:].cpu(), q_rot, tol)
    assert torch.isnan(q_out[:, :, :rank]).all()
    flat = pool.view(nb * bs, rank + dr).cpu()
    for t in range(n):
        if slots[t] >= 0:
            close(flat[slots[t], :rank], c[t], tol)
            close(flat[slots[t], rank:], k_rot[t], tol)
    used = set(int(s) for s in slots if s >= 0)
    assert all(torch.isnan(flat[s]).all() for s in range(nb * bs) if s not in used)


def _latent_reference(q, rows, rank, scale, window, sink):
    """Absorbed form: one shared row per token serves as key over its whole width and as value over ``rank`` columns."""
    n, H, _ = q.shape
    k = rows.expand(n, H, rows.shape[2])
    return R.softmax_attention(q.to(F64), k.to(F64), k[..., :rank].to(F64), scale, R.visible(n, window=window), sink.to(F64))


def test_window_edges_sink_and_values_inside_wider_rows_fp32():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(5)
    n, H, D, rank, win = 75, 3, 28, 22, 9
    q, rows = torch.randn(n, H, D, generator=g), torch.randn(n, 1, D, generator=g)
    sink = torch.randn(H, generator=g)
    # the last query of head 0 matches key n - win (just inside), the one before it key n - 1 - win (just outside for it)
    rows[n - win, 0] = 3.0 * q[n - 1, 0]
    rows[n - 2 - win, 0] = 3.0 * q[n - 2, 1]
    ref = _latent_reference(q, rows, rank, 0.3, win, sink)
    (pool,), table = paged([rows])
    out = torch.empty((n, H, rank), device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    M.mixed_paged_attention(out, q.to(DEV), pool, pool, table, torch.zeros(n, dtype=torch.int32, device=DEV), pos, 0.3,
                            sink=sink.to(DEV), window=win, value_width=rank)
    close(out.cpu(), ref, 2e-5)
    assert (out[n - 1, 0].cpu() - rows[n - win, 0, :rank]).abs().max() < 1e-3          # the inside key takes all the weight
    wrong = _latent_reference(q, rows, rank, 0.3, win + 1, sink)
    assert (wrong[n - 2, 1] - ref[n - 2, 1]).abs().max() > 0.1                          # one token more would have shown
    # the sink: with every score far below it the outputs vanish; alone with one key it takes its share
    far = _latent_reference(q.abs(), -rows.abs(), rank, 5.0, win, sink)
    (pool2,), table2 = paged([-rows.abs()])
    M.mixed_paged_attention(out, q.abs().to(DEV), pool2, pool2, table2, torch.zeros(n, dtype=torch.int32, device=DEV), pos,
                            5.0, sink=sink.to(DEV), window=win, value_width=rank)
    close(out.cpu(), far, 2e-5)
    assert out.abs().max() < 1e-3
    s0 = float((q[0, 0] @ rows[0, 0]) * 0.3)
    share = math.exp(s0) / (math.exp(s0) + math.exp(float(sink[0])))
    assert torch.allclose(ref[0, 0], rows[0, 0, :rank].to(F64) * share, atol=1e-9)


def _differential_reference(q, k, v, scale, chunk):
    """q ``[n, 2H, dk]`` laid out (kv head, map, head in group), k ``[n, 2G, dk]`` (kv head, map), v ``[n, G, dv]``."""
    n, H2, _ = q.shape
    G = v.shape[1]
    rep = H2 // (2 * G)
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(2 * rep, dim=1)
    return R.softmax_attention(q.to(F64), kk.to(F64), vv.to(F64), scale, R.visible(n, chunk=chunk))


def test_block_edges_and_two_maps_over_one_value_head_fp32():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(6)
    n, H, G, dk, dv, chunk = 80, 4, 2, 12, 10, 7
    q, k, v = (torch.randn(n, h, d, generator=g) for h, d in ((2 * H, dk), (2 * G, dk), (G, dv)))
    i = 10 * chunk + 3                                   # a position in the middle of a block
    k[10 * chunk, 0] = 6.0 * q[i, 0]                     # the block's first key: just inside
    k[10 * chunk - 1, 1] = 6.0 * q[i, 2]                 # the key before it: just outside (query head 2 reads key head 1)
    ref = _differential_reference(q, k, v, 0.35, chunk)
    (kp, vp), table = paged([k, v])
    out = torch.empty((n, 2 * H, dv), device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    M.mixed_paged_attention(out, q.to(DEV), kp, vp, table, torch.zeros(n, dtype=torch.int32, device=DEV), pos, 0.35,
                            chunk=chunk, value_div=2)
    close(out.cpu(), ref, 2e-5)
    assert (out[i, 0].cpu() - v[10 * chunk, 0]).abs().max() < 1e-3
    whole_causal = _differential_reference(q, k, v, 0.35, 0)
    assert (whole_causal[i, 2] - ref[i, 2]).abs().max() > 0.1
    # the first position of a block sees itself only
    assert torch.allclose(ref[3 * chunk], v.repeat_interleave(4, dim=1)[3 * chunk].to(F64), atol=1e-12)
    close(out[3 * chunk].cpu(), ref[3 * chunk], 2e-5)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("H,D,rank,win", [(10, 64, 48, 19), (2, 80, 72, 40), (16, 192, 128, 33), (3, 48, 8, 1), (37, 96, 64, 70),
                                          (32, 320, 256, 100)])
def test_tensor_core_latent_attention_matches_the_statement(dt, H, D, rank, win):
    from dgi_b200 import mixer_ops as M

    assert M.mixed_prompt_attention_supported(H, 1, D, rank, False, True, False, dt)
    g = torch.Generator().manual_seed(H + D)
    n = 150
    q, rows = torch.randn(n, H, D, generator=g).to(dt), torch.randn(n, 1, D, generator=g).to(dt)
    sink = torch.randn(H, generator=g)
    rows[n - win, 0] = (2.0 * q[n - 1, 0].float()).to(dt)
    if win < n - 2:
        rows[n - 2 - win, 0] = (2.0 * q[n - 2, H - 1].float()).to(dt)
    ref = _latent_reference(q, rows, rank, 0.2, win, sink)
    (pool,), table = paged([rows])
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    for cuts in ([16] * 9 + [6], [5, 16, 3, 16, 16, 1, 13, 16, 16, 16, 16, 16]):     # tiles that straddle pages and key tiles
        tiles, at = tiles_of(cuts)
        out = torch.full((H, n, rank), float("nan"), dtype=dt, device=DEV).transpose(0, 1)     # head-major, as the layer has it
        M.mixed_prompt_attention(out, q.to(DEV), pool, pool, table, tiles, pos, 0.2, sink=sink.to(DEV), window=win,
                                 value_width=rank)
        close(out[:at].cpu(), ref[:at], tol)
    # decoded tokens: three rows of the same sequence as three one-token tiles, their keys split over CTAs and merged
    last = torch.tensor([n - 1, n - 2, 40])
    out = torch.empty((3, H, rank), dtype=dt, device=DEV)
    M.mixed_prompt_attention(out, q[last].to(DEV), pool, pool, table.expand(3, -1).contiguous(),
                             torch.tensor([(0, 1, 0), (1, 1, 1), (2, 1, 2)], dtype=torch.int32, device=DEV),
                             last.to(torch.int32).to(DEV), 0.2, sink=sink.to(DEV), window=win, max_context=n, value_width=rank)
    close(out.cpu(), ref[last], tol)
    # the same three tokens with 16 heads on the rows of a tile, head-major outputs, with and without key splits
    for ctx in (n, 0):
        out = torch.full((H, 3, rank), float("nan"), dtype=dt, device=DEV).transpose(0, 1)
        M.mixed_prompt_attention(out, q[last].to(DEV), pool, pool, table.expand(3, -1).contiguous(),
                                 torch.tensor([(0, 1, 0), (1, 1, 1), (2, 1, 2)], dtype=torch.int32, device=DEV),
                                 last.to(torch.int32).to(DEV), 0.2, sink=sink.to(DEV), window=win, max_context=ctx,
                                 value_width=rank, heads_as_rows=True)
        close(out.cpu(), ref[last], tol)
    # and the row kernel says the same
    out2 = torch.empty((n, H, rank), dtype=dt, device=DEV)
    M.mixed_paged_attention(out2, q.to(DEV), pool, pool, table, torch.zeros(n, dtype=torch.int32, device=DEV), pos, 0.2,
                            sink=sink.to(DEV), window=win, value_width=rank)
    close(out2.cpu(), ref, tol)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("H,G,dk,dv,chunk", [(8, 2, 16, 40, 24), (4, 4, 32, 8, 5), (12, 1, 16, 64, 64), (2, 2, 64, 128, 33)])
def test_tensor_core_differential_maps_match_the_statement(dt, H, G, dk, dv, chunk):
    from dgi_b200 import mixer_ops as M

    assert M.mixed_prompt_attention_supported(2 * H, 2 * G, dk, dv, False, False, False, dt)
    g = torch.Generator().manual_seed(H + dv)
    n = 150
    q, k, v = (torch.randn(n, h, d, generator=g).to(dt) for h, d in ((2 * H, dk), (2 * G, dk), (G, dv)))
    first = ((n - 1) // chunk) * chunk                       # the first key of the last position's block
    k[first, 0] = (2.0 * q[n - 1, 0].float()).to(dt)         # just inside
    if first > 0:
        k[first - 1, 2 * G - 1] = (2.0 * q[n - 1, 2 * H - 1].float()).to(dt)     # just outside
    ref = _differential_reference(q, k, v, 0.25, chunk)
    (kp, vp), table = paged([k, v])
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    tol = 2e-2 if dt == torch.bfloat16 else 4e-3
    for cuts in ([16] * 9 + [6], [5, 16, 3, 16, 16, 1, 13, 16, 16, 16, 16, 16]):
        tiles, at = tiles_of(cuts)
        for odt in (dt, torch.float32):                      # outputs in the storage type, and unrounded
            out = torch.full((n, 2 * H, dv), float("nan"), dtype=odt, device=DEV)
            M.mixed_prompt_attention(out, q.to(DEV), kp, vp, table, tiles, pos, 0.25, chunk=chunk, value_div=2)
            close(out[:at].cpu(), ref[:at], tol)
    last = torch.tensor([n - 1, first, max(first - 1, 0)])
    out = torch.empty((3, 2 * H, dv), dtype=torch.float32, device=DEV)
    M.mixed_prompt_attention(out, q[last].to(DEV), kp, vp, table.expand(3, -1).contiguous(),
                             torch.tensor([(0, 1, 0), (1, 1, 1), (2, 1, 2)], dtype=torch.int32, device=DEV),
                             last.to(torch.int32).to(DEV), 0.25, chunk=chunk, max_context=n, value_div=2)
    close(out.cpu(), ref[last], tol)
    for odt in (dt, torch.float32):
        out2 = torch.empty((n, 2 * H, dv), dtype=odt, device=DEV)
        M.mixed_paged_attention(out2, q.to(DEV), kp, vp, table, torch.zeros(n, dtype=torch.int32, device=DEV), pos, 0.25,
                                chunk=chunk, value_div=2)
        close(out2.cpu(), ref, tol)


def test_one_far_key_among_hundreds_inside_a_long_window():
    """A latent layer whose window is longer than the sequence: the last query matches one key 600 tokens back."""
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(8)
    n, H, D, rank = 700, 2, 80, 72
    q, rows = 0.2 * torch.randn(n, H, D, generator=g), 0.2 * torch.randn(n, 1, D, generator=g)
    rows[100, 0] = 40.0 * q[n - 1, 1]
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2e-2)):
        qq, rr = q.to(dt), rows.to(dt)
        ref = _latent_reference(qq, rr, rank, 1.0, 1000, torch.zeros(H))
        (pool,), table = paged([rr])
        out = torch.empty((1, H, rank), dtype=dt, device=DEV)
        args = (qq[n - 1:].to(DEV), pool, pool, table)
        pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        M.mixed_paged_attention(out, *args, torch.zeros(1, dtype=torch.int32, device=DEV), pos, 1.0,
                                sink=torch.zeros(H, device=DEV), window=1000, value_width=rank)
        close(out.cpu(), ref[n - 1:], tol)
        assert (out[0, 1].float().cpu() - rr[100, 0, :rank].float()).abs().max() < 0.05
        if dt != torch.float32:
            M.mixed_prompt_attention(out, *args, torch.tensor([(0, 1, 0)], dtype=torch.int32, device=DEV), pos, 1.0,
                                     sink=torch.zeros(H, device=DEV), window=1000, max_context=n, value_width=rank)
            close(out.cpu(), ref[n - 1:], tol)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)], ids=["fp32", "bf16"])
@pytest.mark.parametrize("H,rep,dv", [(4, 2, 10), (3, 3, 33), (8, 1, 64), (1, 1, 2)])
def test_head_difference_norm(dt, tol, H, rep, dv):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(H + dv)
    n, lam, diff = 19, 0.37, 0.2
    buf = torch.randn(n, 2 * H * dv + 4, generator=g).to(dt)
    a = buf[:, :2 * H * dv].unflatten(1, (2 * H, dv))
    a64 = a.to(F64).reshape(n, H // rep, 2, rep, dv)               # (kv head, map, head in group)
    o = (a64[:, :, 0] - lam * a64[:, :, 1]).reshape(n, H, dv)
    want = (R.rms(o, 1e-5) * (1.0 - diff)).reshape(n, H * dv)
    close(M.head_diff_norm(a.to(DEV), lam, 1.0 - diff, 1e-5, rep).cpu(), want, tol)
    out = M.head_diff_norm(a.float().to(DEV), lam, 1.0 - diff, 1e-5, rep, dtype=dt)      # fp32 maps, rounded at the end
    assert out.dtype == dt
    close(out.cpu(), want, tol)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)], ids=["fp32", "bf16"])
def test_gated_post_norm_residual_update(dt, tol):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(3)
    n, W = 21, 150
    x, y32 = torch.randn(n, W, generator=g), torch.randn(n, W, generator=g)
    y, gate, w = y32.to(dt), torch.randn(n, W, generator=g).to(dt), (0.1 * torch.randn(W, generator=g)).to(dt)
    for a, gt, off in ((y, gate, 1.0), (y32, gate, 1.0), (y, None, 0.0)):
        xd = x.clone().to(DEV)
        copy = M.gated_postnorm_residual(xd, a.to(DEV), gt.to(DEV) if gt is not None else None, w.to(DEV), off, 1e-5)
        z = a.to(F64) * (torch.sigmoid(gt.to(F64)) if gt is not None else 1.0)
        ref = x.to(F64) + R.rms(z, 1e-5) * (off + w.to(F64))
        close(xd.cpu(), ref, 2e-6)                                   # the residual itself stays fp32
        close(copy.cpu(), ref, tol)
        assert copy.dtype == dt


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)], ids=["fp32", "bf16"])
def test_squared_relu_and_gated_table_rows(dt, tol):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(4)
    for rows, ff in ((13, 40), (7, 33), (1, 8)):
        z = torch.randn(rows, ff + 8, generator=g).to(dt)
        out = M.relu_squared(z.to(DEV)[:, :ff])
        close(out.cpu(), torch.relu(z[:, :ff].to(F64)) ** 2, tol)
    n, d, vocab, L = 17, 5, 23, 3
    table = torch.randn(vocab, d * L, generator=g).to(dt)
    z = (2.0 * torch.randn(n, d, generator=g)).to(dt)
    tok = torch.randint(0, vocab, (n,), generator=g)
    for layer_idx in range(L):
        out = M.gated_table_rows(z.to(DEV), table.to(DEV), layer_idx * d, tok.to(DEV))
        close(out.cpu(), R.gelu_tanh(z.to(F64)) * table.to(F64)[tok][:, layer_idx * d:(layer_idx + 1) * d], tol)


@pytest.mark.parametrize("spec,W", [(moe(5, 3, 40), 56), (moe(8, 2, 32), 64), (moe(1, 1, 8), 16), (moe(4, 4, 48), 64)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_routed_feed_forward_softmax_over_the_chosen(dt, spec, W):
    from dgi_b200 import vatazen_layer as Vz

    g = torch.Generator().manual_seed(W + spec["router"]["experts"])
    E, ff = spec["router"]["experts"], spec["expert"]["ff"]
    t = {"router": (3.0 * torch.randn(E, W, generator=g) / math.sqrt(W)).to(dt), "router.b": torch.randn(E, generator=g).to(dt)}
    for e in range(E):
        t[f"e{e}.up"] = (torch.randn(ff, W, generator=g) / math.sqrt(W)).to(dt)
        t[f"e{e}.down"] = (torch.randn(W, ff, generator=g) / math.sqrt(ff)).to(dt)
    mod = Vz.SquaredReluMoE(spec, t, DEV, dt)
    x = torch.randn(45, W, generator=g)
    h = x.to(dt)
    got = mod(h.to(DEV), h.to(torch.float32).to(DEV))
    ref = R.routed_ff(h.to(F64), spec, {k: v.to(F64) for k, v in t.items()})
    close(got.cpu(), ref, 3e-5 if dt == torch.float32 else 3e-2)
    ids, w = R.route(torch.randn(9, 6, generator=g, dtype=F64), 2)
    assert torch.allclose(w.sum(-1), torch.ones(9, dtype=F64)) and ids.shape == (9, 2)


@pytest.mark.parametrize("n,E,W", [(45, 5, 56), (1, 1, 16), (300, 12, 200), (33, 40, 130), (9, 8, 2048)])
def test_router_logits_do_not_depend_on_the_batch(n, E, W):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(n + E)
    x, w, b = torch.randn(n, W, generator=g), torch.randn(E, W, generator=g), torch.randn(E, generator=g)
    got = M.router_logits(x.to(DEV), w.to(DEV), b.to(DEV))
    close(got.cpu(), x.to(F64) @ w.to(F64).T + b.to(F64), 2e-6 * W ** 0.5)
    close(M.router_logits(x.to(DEV), w.to(DEV)).cpu(), x.to(F64) @ w.to(F64).T, 2e-6 * W ** 0.5)
    one = M.router_logits(x[n // 2:n // 2 + 1].contiguous().to(DEV), w.to(DEV), b.to(DEV))      # a row alone: the same bits
    assert torch.equal(one[0], got[n // 2])


# ---- the model through the engine ----------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C], ids=["A", "B", "C"])
def test_whole_prompt_fp32(cfg):
    engine, tensors = build(cfg)
    toks = tokens(90, cfg["vocab"], 11)
    layers = []
    ref = R.forward(cfg, tensors, toks, layers_out=layers)
    engine.layer_trace = []
    got = whole(engine, "a", toks)
    for mine, theirs in zip(engine.layer_trace, layers):                    # the residual after every layer
        close(mine.cpu(), theirs, 3e-5)
    engine.layer_trace = None
    close(got, ref, 3e-5)
    one = tokens(1, cfg["vocab"], 12)                                       # the first token alone
    close(whole(engine, "b", one), R.forward(cfg, tensors, one), 3e-5)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C], ids=["A", "B", "C"])
def test_whole_prompt_bf16(cfg):
    engine, tensors = build(cfg, dtype=torch.bfloat16)
    toks = tokens(70, cfg["vocab"], 13)
    ref = R.forward(cfg, tensors, toks)
    rounding_close(whole(engine, "a", toks), ref)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["A", "B"])
def test_prefill_then_long_decode_matches_the_whole_prompt(cfg):
    engine, tensors = build(cfg)
    toks = tokens(120, cfg["vocab"], 14)
    ref = R.forward(cfg, tensors, toks)
    got = [engine.step([("a", toks[:30], list(range(30)))])]
    for t in range(30, len(toks)):                               # 90 decoded tokens: every window and block passes over them
        got.append(engine.step([("a", [toks[t]], [0])]))
    engine.finish("a")
    close(torch.cat(got).cpu(), ref, 3e-5)
    got = [engine.step([("b", [t], [0])]) for t in toks[:40]]    # decoding from the very first token
    engine.finish("b")
    close(torch.cat(got).cpu(), ref[:40], 3e-5)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["A", "B"])
def test_portions_of_any_size_down_to_two_tokens(cfg):
    engine, tensors = build(cfg)
    toks = tokens(131, cfg["vocab"], 15)
    ref = R.forward(cfg, tensors, toks)
    for cuts in ([2, 2, 13, 3, 16, 17, 2, 31, 33, 2, 1, 9], [64, 2, 65], [15, 1, 16, 1, 31, 1, 2, 64], [8, 1, 9, 1, 10, 102]):
        got, at = [], 0
        for c in cuts:
            c = min(c, len(toks) - at)
            got.append(engine.step([("a", toks[at:at + c], list(range(c)))]))
            at += c
        engine.finish("a")
        close(torch.cat(got).cpu(), ref[:at], 3e-5)


def test_mixed_batches_match_each_request_alone_and_reuse_pages_and_slots():
    cfg = CFG_A
    engine, tensors = build(cfg, max_tokens=256, max_seqs=3)
    prompts = {r: tokens(n, cfg["vocab"], 20 + i) for i, (r, n) in enumerate((("a", 70), ("b", 33), ("c", 5), ("d", 90), ("e", 48)))}
    ref = {r: R.forward(cfg, tensors, t) for r, t in prompts.items()}
    at = {r: 0 for r in prompts}
    got = {r: [] for r in prompts}

    def feed(plan):
        entries = []
        for r, c in plan:
            entries.append((r, prompts[r][at[r]:at[r] + c], list(range(c))))
        out = engine.step(entries)
        o = 0
        for r, c in plan:
            got[r].append(out[o:o + c])
            o, at[r] = o + c, at[r] + c
            if at[r] == len(prompts[r]):
                engine.finish(r)

    feed([("a", 40), ("b", 2), ("c", 5)])                        # c ends: its slot and page are free again
    feed([("a", 1), ("b", 30), ("d", 17)])                       # d takes c's slot (and must not read c's last row)
    feed([("b", 1), ("d", 2), ("a", 1)])                         # b ends
    feed([("e", 31), ("a", 1), ("d", 1)])                        # e takes b's slot and pages
    feed([("d", 70), ("a", 27), ("e", 2)])                       # a and d end
    feed([("e", 15)])
    for r in prompts:
        assert at[r] == len(prompts[r])
        close(torch.cat(got[r]).cpu(), ref[r], 3e-5)
    assert engine.free_slots == 3 and engine.free_blocks == 256 // 16


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["A", "B"])
def test_logits_do_not_depend_on_the_batch_or_the_cut_beyond_rounding_bf16(cfg):
    engine, _ = build(cfg, dtype=torch.bfloat16)
    a, b = tokens(80, cfg["vocab"], 31), tokens(37, cfg["vocab"], 32)
    alone = whole(engine, "a", a)
    out = engine.step([("b", b[:20], []), ("a", a[:50], list(range(50)))])
    out2 = engine.step([("a", a[50:], list(range(30))), ("b", b[20:], [])])
    engine.release()
    rounding_close(torch.cat([out, out2]).cpu(), alone)


def test_long_prompt_whole_in_portions_and_decoded_bf16_against_fp32():
    """600 tokens through the tensor-core kernels: the whole prompt, portions beside another request, and single
    tokens agree with the fp32 engine within 16-bit rounding."""
    cfg = CFG_B
    e32, _ = build(cfg, max_tokens=1024, max_seqs=2)
    e16, _ = build(cfg, dtype=torch.bfloat16, max_tokens=1024, max_seqs=2)
    toks = tokens(600, cfg["vocab"], 16)
    want = [0, 100, 255, 256, 300, 400, 511, 512, 550, 590, 599]
    ref = whole(e32, "a", toks, want)
    rounding_close(whole(e16, "a", toks, want), ref)
    got = [e16.step([("b", toks[:100], [0])]), e16.step([("b", toks[100:590], [0, 155, 156, 200, 300, 411, 412, 450]), ("c", toks[:3], [])])]
    got += [e16.step([("b", [t], [0] if i in (0, 9) else [])]) for i, t in enumerate(toks[590:])]
    e16.release()
    rounding_close(torch.cat([g for g in got if g is not None]).cpu(), ref)


def test_single_token_steps_with_heads_on_the_rows_bf16_against_fp32():
    cfg = CFG_D
    e32, _ = build(cfg, max_tokens=512, max_seqs=3)
    e16, _ = build(cfg, dtype=torch.bfloat16, max_tokens=512, max_seqs=3)
    prompts = {r: tokens(n, cfg["vocab"], 60 + i) for i, (r, n) in enumerate((("a", 150), ("b", 40), ("c", 75)))}
    ref = {r: whole(e32, r, t) for r, t in prompts.items()}
    got = {r: [] for r in prompts}
    out = e16.step([(r, t[:len(t) - 30], list(range(len(t) - 30))) for r, t in prompts.items()])
    o = 0
    for r, t in prompts.items():
        got[r].append(out[o:o + len(t) - 30])
        o += len(t) - 30
    for i in range(30):                                       # 30 steps of three single tokens
        out = e16.step([(r, [t[len(t) - 30 + i]], [0]) for r, t in prompts.items()])
        for j, r in enumerate(prompts):
            got[r].append(out[j:j + 1])
    e16.release()
    for r in prompts:
        rounding_close(torch.cat(got[r]).cpu(), ref[r])


def test_greedy_generation_through_the_scheduler():
    cfg = CFG_B
    engine, tensors = build(cfg, max_tokens=256, max_seqs=2)
    prompts = [tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate((9, 30, 3))]     # three requests, two slots
    out = engine.generate(prompts, max_new_tokens=6, prefill_chunk=7, token_budget=12)
    for p, o in zip(prompts, out):
        want = R.greedy(cfg, tensors, p, 6)
        # a near-tie may flip a token in fp32; up to the first difference the texts must agree and it must be a near-tie
        for k, (x, y) in enumerate(zip(o, want)):
            if x != y:
                lg = R.forward(cfg, tensors, p + want[:k])[-1]
                assert abs(lg[x] - lg[y]) < 1e-4
                break
    assert engine.free_slots == 2


def test_registry_serves_a_checkpoint_folder(tmp_path):
    import json

    from dgi_b200 import model_registry, vatazen_layer as Vz
    from dgi_b200.ragged_engine import RaggedStepEngine
    from dgi_b200.safetensors_io import write_safetensors

    cfg = Vz.VatazenConfig.from_dict(CFG_A)
    tensors = Vz.random_checkpoint(cfg, seed=5)
    (tmp_path / "config.json").write_text(json.dumps(CFG_A))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    arch, _, shards = model_registry.load_model_dir(str(tmp_path), device=DEV, dtype=torch.float32)
    assert arch.name == "Vatazen" and arch.engine == "ragged"
    engine = RaggedStepEngine(shards, max_tokens=128, max_seqs=1)
    toks = tokens(20, CFG_A["vocab"], 50)
    close(whole(engine, "a", toks), R.forward(CFG_A, tensors, toks), 3e-5)


def test_two_shards_carry_the_token_table_and_the_tied_head():
    from dgi_b200 import vatazen_layer as Vz
    from dgi_b200.ragged_engine import RaggedStepEngine

    cfg = Vz.VatazenConfig.from_dict(CFG_A)
    tensors = Vz.random_checkpoint(cfg, seed=6)
    shards = Vz.build_shards(cfg, tensors, [(0, 1), (1, 4)], DEV, torch.float32)
    engine = RaggedStepEngine(shards, max_tokens=128, max_seqs=2)
    toks = tokens(45, CFG_A["vocab"], 51)
    ref = R.forward(CFG_A, tensors, toks)
    got = [engine.step([("a", toks[:20], list(range(20)))]), engine.step([("a", toks[20:], list(range(25)))])]
    close(torch.cat(got).cpu(), ref, 3e-5)
