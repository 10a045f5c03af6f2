"""Vatazen: a decoder whose sublayers read the fp32 residual stream ITSELF, are gated by a sigmoid of a linear map of
that stream, and are normed on the way out:

    x <- x + N1(sigmoid(R1 x + r1) * mixer(shift(x)));   x <- x + N2(sigmoid(R2 x + r2) * ff(x));   x <- x + side(x, token)

N is an RMS norm whose weight is stored around zero.  ``shift`` blends every row with the row of the token before it,
per channel (``h_t + (h_(t-1) - h_t) * mu``, with the unshifted previous row); only the mixer reads shifted rows, and
the last row of every live sequence is carried in a state slot per layer.  ``side`` reads a per-layer slice ``e`` of a
second embedding table: ``y = P (gelu_tanh(G x) * e)``, added as ``y / rms(y) * w``.  One of two mixers per layer:

  ``latent_attention``  softmax attention whose keys and values are up-projections of one normed latent row per token,
                        plus one rotated key part that all heads share; queries carry an unrotated and a rotated part per
                        head.  Rotary pairs are (2i, 2i + 1) with YaRN-rescaled frequencies and a common gain on cos and
                        sin.  A position sees its last ``mask.size`` positions; a learned sink logit per head joins the
                        softmax denominator.  Served in the absorbed form: the key up-projection moves to the query side,
                        the value up-projection behind the attention, so the kernel is a multi-query attention over a
                        one-head pool whose rows ``[latent | rotated key part]`` serve as keys over their whole width and
                        as values over the latent columns.
  ``attention``         differential attention: two softmax maps per head (RMS-normed q and k per head and map, no
                        positions) over the same values, ``o = a1 - lambda a2`` made unit-RMS per head and scaled by
                        ``1 - diff``; a position sees the keys of its own block of ``mask.size`` positions, counted from
                        the sequence's start.  The maps run as twice the heads of one attention launch: query heads are
                        laid out (kv head, map, head in group), key heads (kv head, map), and two key heads read one
                        value head.

Feed-forward: a mixture of experts ``W_down relu(W_up h)^2`` chosen by the largest router logits (fp32, with bias) and
weighted by the softmax over the chosen logits.  The head is the embedding table itself (unscaled).

The modules follow the calling convention of ``ModelShard.forward`` (reference:
worker/distributed/model_shard.py:205-215): ``layer(h, attention_mask=, position_ids=, past_key_value=, use_cache=)
-> (h, present)`` with ``h`` the packed fp32 residual ``[n_tok, width]`` of one step and ``past_key_value`` a
``RaggedLayerCache`` (pages AND a state slot for every layer).  Matrix products are torch GEMMs; everything between them
is a kernel of ``mixer_ops``.  There is no dense / CPU mode.

Checkpoint names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2|shift|rg1|rg1.b|rg2|rg2.b``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.side.gate|proj|norm``, ``final.norm``; linear weights are ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import mixer_ops
from .fibirax_layer import GroupedSoftmaxMoE
from .paged_layer import RaggedLayerCache
from .petipel_layer import OffsetRMSNorm, _param
from .sanesun_layer import ScaledFloatEmbedding, _pad8
from .worker.distributed.model_shard import ModelShard

MIXERS = ("latent_attention", "attention")
YARN_GAIN_SLOPE = 0.1      # cos and sin are multiplied by 0.1 ln(factor) + 1; fixed by the design
YARN_MIN_SPAN = 0.001      # floor under hi - lo of the frequency ramp; fixed by the design


class VatazenConfig:
    """``config.json`` of the design, plus the attribute names the rest of the framework reads from a config."""

    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.architecture = raw.get("architecture", "Vatazen")
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.width = int(raw["width"])
        self.vocab = int(raw["vocab"])
        self.eps = float(raw["norm"]["eps"])
        self.embed_scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        self.side_dim = int((raw.get("token_side") or {}).get("dim", 0))
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise NotImplementedError(f"layer {i}: unknown mixer type {layer['type']!r}")
            m = layer["mixer"]
            if layer["type"] == "attention" and int(m["heads"]) % int(m.get("kv_heads", m["heads"])):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if layer["type"] == "latent_attention":
                rot = m.get("rot") or {}
                if int(rot.get("dims", 0)) > int(m["rot_dim"]) or int(rot.get("dims", 0)) % 2:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "moe") != "moe":
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        # names shared with the other model classes
        self.hidden_size = self.width
        self.vocab_size = self.vocab
        self.num_hidden_layers = len(self.layers)
        self.num_attention_heads = max(int(l["mixer"]["heads"]) for l in self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VatazenConfig":
        return cls(raw)

    def kv_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        """``(kv heads, key row, value row)`` of a layer's pages.  A latent layer keeps one row ``[latent | rotated key
        part]`` per token and no value pool; a differential layer keeps both maps' keys of a kv head side by side."""
        kind, m = self.layers[i]["type"], self.layers[i]["mixer"]
        if kind == "latent_attention":
            return 1, int(m["kv_rank"]) + int(m["rot_dim"]), 0
        return int(m.get("kv_heads", m["heads"])), 2 * int(m["dim"]), int(m["vdim"])

    def state_shape(self, i: int):
        """Per live sequence and layer: the last row the mixer read, before its shift."""
        return (self.width,)


def yarn_frequencies(dims: int, base: float, scaling: Optional[Dict[str, Any]]) -> Tuple[torch.Tensor, float]:
    """``(float64 [dims / 2], gain)``: ``f_i = base^(-2i / dims)``; with ``scaling`` (factor, original, fast, slow) let
    ``d(t) = dims ln(original / (2 pi t)) / (2 ln base)``, ``lo = max(floor(d(fast)), 0)``, ``hi = min(ceil(d(slow)),
    dims - 1)`` and ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``: the frequency becomes ``r_i f_i / factor +
    (1 - r_i) f_i`` and cos and sin are multiplied by ``gain = 0.1 ln(factor) + 1``."""
    out, gain = [], 1.0
    lo = hi = 0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def d(t: float) -> float:
            return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(d(float(scaling["fast"]))), 0)
        hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
        gain = YARN_GAIN_SLOPE * math.log(factor) + 1.0
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            r = min(max((i - lo) / max(hi - lo, YARN_MIN_SPAN), 0.0), 1.0)
            f = f / factor * r + f * (1.0 - r)
        out.append(f)
    return torch.tensor(out, dtype=torch.float64), gain


class LatentRotaryAttention(nn.Module):
    """The ``latent_attention`` mixer in absorbed form.  Launches per step: the input GEMM (q | down-projection), norm +
    rotary + append, the batched key up-projection on the query side, attention, the batched value up-projection, the
    output GEMM."""

    HEADS_AS_ROWS_FROM = 16    # heads from which a step of single tokens puts heads on the rows of the attention's tiles

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.H, self.dn, self.dr = int(spec["heads"]), int(spec["dim"]), int(spec["rot_dim"])
        self.dv, self.rank = int(spec["vdim"]), int(spec["kv_rank"])
        self.scale, self.eps = float(spec["scale"]), eps
        self.window = int((spec.get("mask") or {}).get("size", 0))
        rot = spec.get("rot") or {}
        freqs, self.gain = yarn_frequencies(int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), rot.get("scaling"))
        self.register_buffer("freqs", freqs.to(device) if freqs.numel() else None, persistent=False)
        sections = [t["q"], t["dkv"]]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        self.c_norm = _param(t["dkv.norm"], device, dtype)
        self.w_uk = _param(t["uk"].reshape(self.H, self.dn, self.rank), device, dtype)                  # [H, dn, r]
        self.w_uv = _param(t["uv"].reshape(self.H, self.dv, self.rank).transpose(1, 2), device, dtype)  # [H, r, dv]
        self.sink = _param(t["sink"], device, torch.float32) if "sink" in t else None
        self.w_o = _param(t["o"], device, dtype)
        D = self.rank + self.dr
        self.tensor_cores = D % 8 == 0 and mixer_ops.mixed_prompt_attention_supported(
            self.H, 1, D, self.rank, False, True, False, self.w_in.dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st, n = cache.state, h.shape[0]
        H, dn, dr, r, c = self.H, self.dn, self.dr, self.rank, self.cuts
        proj = F.linear(h, self.w_in)
        q = proj[:, :H * (dn + dr)].unflatten(1, (H, dn + dr))
        q_lat = torch.empty((n, H, r + dr), dtype=h.dtype, device=h.device)       # [W_uk^T q_plain | turned q part]
        mixer_ops.latent_rotary_append(q[:, :, dn:], q_lat[:, :, r:], proj[:, c[1]:c[1] + r + dr], self.c_norm, self.eps,
                                       self.freqs, self.gain, cache.k_pool, st.slot_mapping, st.tok_pos)
        torch.bmm(q[:, :, :dn].transpose(0, 1), self.w_uk, out=q_lat[:, :, :r].transpose(0, 1))
        o_lat = torch.empty((H, n, r), dtype=h.dtype, device=h.device)
        if self.tensor_cores:
            tiles, _ = st.prompt_tiles(1, mixer_ops.PROMPT_TILE_TOKENS)
            # steps of single tokens: all heads read the same rows, so 16 heads share a tensor-core tile
            mixer_ops.mixed_prompt_attention(o_lat.transpose(0, 1), q_lat, cache.k_pool, cache.k_pool, st.block_tables,
                                             tiles, st.tok_pos, self.scale, sink=self.sink, window=self.window,
                                             max_context=st.max_context(), value_width=r,
                                             heads_as_rows=H >= self.HEADS_AS_ROWS_FROM and st.max_count() == 1)
        else:
            mixer_ops.mixed_paged_attention(o_lat.transpose(0, 1), q_lat, cache.k_pool, cache.k_pool, st.block_tables,
                                            st.tok_row, st.tok_pos, self.scale, sink=self.sink, window=self.window,
                                            value_width=r)
        o = torch.bmm(o_lat, self.w_uv)                                           # [H, n, dv]
        return F.linear(o.transpose(0, 1).reshape(n, H * self.dv), self.w_o)


class DifferentialAttention(nn.Module):
    """The ``attention`` mixer.  Launches per step: the input GEMM with biases (q | k | v), q/k norm + append, one
    attention launch over both maps, the head difference norm, the output GEMM with bias."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.H, self.G = int(spec["heads"]), int(spec.get("kv_heads", spec["heads"]))
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.scale, self.eps, self.diff = float(spec["scale"]), eps, float(spec["diff"])
        self.chunk = int((spec.get("mask") or {}).get("size", 0))
        H, G, dk = self.H, self.G, self.dk
        self.rep = H // G

        def by_group(w: torch.Tensor) -> torch.Tensor:
            """Query rows (head, map, d) -> (kv head, map, head in group, d)."""
            tail = w.shape[1:]
            return w.reshape(G, self.rep, 2, dk, *tail).transpose(1, 2).reshape(2 * H * dk, *tail)

        def bias(name: str, rows: int) -> torch.Tensor:
            return t[name + ".b"] if name + ".b" in t else torch.zeros(rows, dtype=t[name].dtype)

        sections = [by_group(t["q"]), t["k"], t["v"]]
        biases = [by_group(bias("q", 2 * H * dk)), bias("k", 2 * G * dk), bias("v", G * self.dv)]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        self.b_in = _param(torch.cat([_pad8(b) for b in biases], dim=0), device, dtype)
        self.q_norm = _param(t["q.norm"], device, dtype) if "q.norm" in t else None
        self.k_norm = _param(t["k.norm"], device, dtype) if "k.norm" in t else None
        f32 = lambda name: t[name].to(torch.float32)  # noqa: E731
        self.lam = float(torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum())) + self.diff
        self.w_o = _param(t["o"], device, dtype)
        self.b_o = _param(t["o.b"], device, dtype) if "o.b" in t else None
        self.tensor_cores = self.dv % 8 == 0 and mixer_ops.mixed_prompt_attention_supported(
            2 * H, 2 * G, dk, self.dv, False, False, False, self.w_in.dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st, n, c = cache.state, h.shape[0], self.cuts
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        proj = F.linear(h, self.w_in, self.b_in)
        q, k, v = proj[:, :2 * H * dk], proj[:, c[1]:c[1] + 2 * G * dk], proj[:, c[2]:c[2] + G * dv]
        nb, _g, bs, _w = cache.k_pool.shape
        k_pool = cache.k_pool.view(nb, 2 * G, bs, dk)        # the pool's rows as (kv head, map) key heads
        mixer_ops.qknorm_rotary_append(q, k, v, self.q_norm, self.k_norm, self.eps, None, k_pool, cache.v_pool,
                                       st.slot_mapping, st.tok_pos, 2 * H)
        maps = torch.empty((n, 2 * H, dv), dtype=torch.float32, device=h.device)    # rounded only after their difference
        if self.tensor_cores:
            tiles, _ = st.prompt_tiles(1, mixer_ops.PROMPT_TILE_TOKENS)
            mixer_ops.mixed_prompt_attention(maps, q.unflatten(1, (2 * H, dk)), k_pool, cache.v_pool, st.block_tables, tiles,
                                             st.tok_pos, self.scale, chunk=self.chunk, max_context=st.max_context(),
                                             value_div=2)
        else:
            mixer_ops.mixed_paged_attention(maps, q.unflatten(1, (2 * H, dk)), k_pool, cache.v_pool, st.block_tables,
                                            st.tok_row, st.tok_pos, self.scale, chunk=self.chunk, value_div=2)
        o = mixer_ops.head_diff_norm(maps, self.lam, 1.0 - self.diff, self.eps, self.rep, dtype=h.dtype)
        return F.linear(o, self.w_o, self.b_o)


class SquaredReluMoE(GroupedSoftmaxMoE):
    """Experts ``W_down relu(W_up h)^2`` under the dispatch of ``GroupedSoftmaxMoE``: the router's fp32 logits carry a
    bias, the ``top`` largest are chosen and weighted by the softmax over the chosen ones (the softmax over all,
    renormalised over the chosen, is the same numbers)."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], device, dtype):
        nn.Module.__init__(self)
        r = spec["router"]
        self.E, self.ident, self.top = int(r["experts"]), 0, int(r["top"])
        self.groups = self.keep = 1
        self.correction = None
        self.w_router = _param(t["router"], device, torch.float32)
        self.b_router = _param(t["router.b"], device, torch.float32) if "router.b" in t else None
        if self.w_router.shape[0] != self.E:
            raise ValueError("the router has one output per expert")
        self.w_gu = _param(torch.stack([t[f"e{e}.up"] for e in range(self.E)]), device, dtype)        # [E, ff, W]
        self.w_down = _param(torch.stack([t[f"e{e}.down"] for e in range(self.E)]), device, dtype)    # [E, W, ff]
        self.grouped = (mixer_ops.grouped_linear_supported(self.w_gu.shape[2], self.w_gu.dtype)
                        and mixer_ops.grouped_linear_supported(self.w_down.shape[2], self.w_down.dtype))
        self._ar = None
        self.ws_gu = self.ws_down = None

    def _route(self, x: torch.Tensor):
        return mixer_ops.softmax_group_topk(mixer_ops.router_logits(x, self.w_router, self.b_router), None, self.top)

    def _activate(self, z: torch.Tensor) -> torch.Tensor:
        return mixer_ops.relu_squared(z)


class TokenSideInput(nn.Module):
    """``x += w * y / rms(y)`` with ``y = P (gelu_tanh(G x) * e)``, ``e`` the token's row of this layer's columns of a
    second embedding table (shared by the layers; plain norm weight)."""

    def __init__(self, table: torch.Tensor, col0: int, t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.table, self.col0, self.eps = table, col0, eps
        self.w_gate, self.w_proj = _param(t["side.gate"], device, dtype), _param(t["side.proj"], device, dtype)
        self.norm = _param(t["side.norm"], device, dtype)

    def forward(self, x: torch.Tensor, h: torch.Tensor, tokens: torch.Tensor, want_copy: bool) -> Optional[torch.Tensor]:
        g = mixer_ops.gated_table_rows(F.linear(h, self.w_gate), self.table, self.col0, tokens)
        return mixer_ops.gated_postnorm_residual(x, F.linear(g, self.w_proj), None, self.norm, 0.0, self.eps,
                                                 want_copy=want_copy)


class VatazenDecoderLayer(nn.Module):
    """One layer; see the module docstring.  Every residual update also hands the next reader its input: the new residual
    in the weights' dtype (nothing when the weights are fp32, which read the residual itself)."""

    def __init__(self, config: VatazenConfig, layer_idx: int, t: Dict[str, torch.Tensor], side_table: Optional[torch.Tensor],
                 device=None, dtype=None):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx, self.kind, self.eps = layer_idx, spec["type"], config.eps
        mix = {k[4:]: v for k, v in t.items() if k.startswith("mix.")}
        if self.kind == "latent_attention":
            self.mixer = LatentRotaryAttention(spec["mixer"], mix, self.eps, device, dtype)
        else:
            self.mixer = DifferentialAttention(spec["mixer"], mix, self.eps, device, dtype)
        self.shift = _param(t["shift"], device, dtype)
        self.norm1 = _param(t["norm1"], device, dtype)
        self.w_rg1, self.b_rg1 = _param(t["rg1"], device, dtype), _param(t["rg1.b"], device, dtype)
        self.mlp = None
        if spec.get("mlp") is not None:
            self.mlp = SquaredReluMoE(spec["mlp"], {k[4:]: v for k, v in t.items() if k.startswith("mlp.")}, device, dtype)
            self.norm2 = _param(t["norm2"], device, dtype)
            self.w_rg2, self.b_rg2 = _param(t["rg2"], device, dtype), _param(t["rg2.b"], device, dtype)
        self.side = None
        if side_table is not None:
            self.side = TokenSideInput(side_table, layer_idx * config.side_dim, t, self.eps, device, dtype)
        self.low_precision = self.norm1.dtype != torch.float32

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None,
                past_key_value: Optional[RaggedLayerCache] = None, use_cache: bool = True):
        if not isinstance(past_key_value, RaggedLayerCache):
            raise TypeError("VatazenDecoderLayer needs a RaggedLayerCache handle in past_key_value")
        x, st = hidden_states, past_key_value.state
        if x.dtype != torch.float32 or x.dim() != 2:
            raise TypeError("the residual stream is a packed fp32 [n_tok, width] tensor")
        lp = self.low_precision
        # the mixer reads shifted rows, its gate the rows themselves
        shifted, h = mixer_ops.token_shift(x, self.shift, past_key_value.rstate, st.scan_seqs, st.max_count(),
                                           want_cast=lp and st.pending_norm is None)
        if lp and st.pending_norm is not None:
            h = st.pending_norm
        st.pending_norm = None
        if not lp:
            h = x
        gate = F.linear(h, self.w_rg1, self.b_rg1)
        y = self.mixer(shifted, past_key_value)
        h = mixer_ops.gated_postnorm_residual(x, y, gate, self.norm1, 1.0, self.eps, want_copy=lp)
        if self.mlp is not None:
            if not lp:
                h = x
            gate = F.linear(h, self.w_rg2, self.b_rg2)
            y = self.mlp(h, x)
            h = mixer_ops.gated_postnorm_residual(x, y, gate, self.norm2, 1.0, self.eps, want_copy=lp)
        if self.side is not None:
            h = self.side(x, h if lp else x, st.token_ids, lp)
        st.pending_norm = h if lp else None
        return x, (past_key_value if use_cache else None)


def build_shards(config: VatazenConfig, tensors: Dict[str, torch.Tensor], ranges: Sequence[Tuple[int, int]],
                 device: str, dtype: torch.dtype) -> List[ModelShard]:
    """``ModelShard``s for layer ranges holding the weights of a checkpoint's name -> tensor dict."""
    shards = []
    total = config.num_hidden_layers
    for start, end in ranges:
        side_table = None
        if config.side_dim > 0 and end > start:
            side_table = tensors["side.embed"].to(device=device, dtype=dtype).contiguous()
        layers = []
        for i in range(start, end):
            pre = f"l{i}."
            layers.append(VatazenDecoderLayer(config, i, {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)},
                                              side_table, device, dtype))
        embed = norm = head = None
        if start == 0:
            embed = ScaledFloatEmbedding(config.vocab, config.width, device=device, dtype=dtype, scale=config.embed_scale)
            embed.weight.requires_grad_(False)
            with torch.no_grad():
                embed.weight.copy_(tensors["embed"])
        if end == total:
            norm = OffsetRMSNorm(config.width, config.eps, device, dtype)
            head = nn.Linear(config.width, config.vocab, bias=False, device=device, dtype=dtype)
            head.weight.requires_grad_(False)
            with torch.no_grad():
                norm.weight.copy_(tensors["final.norm"])
            if embed is not None:
                head.weight = embed.weight            # the head IS the embedding table
            else:
                with torch.no_grad():
                    head.weight.copy_(tensors["embed"])
        shards.append(ModelShard.from_layers(config, layers, start, end, device, dtype, embed, norm, head,
                                             model_id="vatazen").eval())
    return shards


def random_checkpoint(config: VatazenConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights with the checkpoint's names and shapes (for tests and benchmarks; not a trained model).
    Projections ~ N(0, gain / fan_in); norm weights, shifts, gates, sinks and biases are chosen so that every term of the
    design contributes."""
    g = torch.Generator().manual_seed(seed)
    W = config.width

    def lin(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def vec(n, s=1.0, mean=0.0):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)

    t: Dict[str, torch.Tensor] = {"embed": (torch.randn(config.vocab, W, generator=g) / config.embed_scale).to(dtype)}
    if config.side_dim > 0:
        t["side.embed"] = torch.randn(config.vocab, config.side_dim * len(config.layers), generator=g).to(dtype)
    for i, layer in enumerate(config.layers):
        pre, m = f"l{i}.mix.", layer["mixer"]
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        if layer["type"] == "latent_attention":
            r, dr = int(m["kv_rank"]), int(m["rot_dim"])
            t[pre + "q"] = lin(H * (dk + dr), W, 2.0)
            t[pre + "dkv"], t[pre + "dkv.norm"] = lin(r + dr, W, 2.0), vec(r, 0.1, 1.0)
            t[pre + "uk"], t[pre + "uv"] = lin(H * dk, r, 1.5), lin(H * dv, r)
            t[pre + "sink"] = vec(H)
            t[pre + "o"] = lin(W, H * dv)
        else:
            G = int(m.get("kv_heads", H))
            for name, rows in (("q", 2 * H * dk), ("k", 2 * G * dk), ("v", G * dv)):
                t[pre + name] = lin(rows, W, 1.5)
                t[pre + name + ".b"] = vec(rows, 0.1)
            t[pre + "q.norm"], t[pre + "k.norm"] = vec(dk, 0.3, 1.5), vec(dk, 0.3, 1.5)
            for name in ("lq1", "lk1", "lq2", "lk2"):
                t[pre + name] = vec(dk, 0.1)
            t[pre + "o"], t[pre + "o.b"] = lin(W, H * dv), vec(W, 0.1)
        pre = f"l{i}."
        t[pre + "shift"] = torch.rand(W, generator=g).to(dtype)
        t[pre + "norm1"] = vec(W, 0.1)
        t[pre + "rg1"], t[pre + "rg1.b"] = lin(W, W), vec(W, 0.5)
        mlp = layer.get("mlp")
        if mlp:
            E, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            for e in range(E):
                t[pre + f"mlp.e{e}.up"], t[pre + f"mlp.e{e}.down"] = lin(ff, W, 1.5), lin(W, ff)
            t[pre + "mlp.router"], t[pre + "mlp.router.b"] = lin(E, W, 3.0), vec(E, 0.5)
            t[pre + "norm2"] = vec(W, 0.1)
            t[pre + "rg2"], t[pre + "rg2.b"] = lin(W, W), vec(W, 0.5)
        if config.side_dim > 0:
            t[pre + "side.gate"], t[pre + "side.proj"] = lin(config.side_dim, W, 2.0), lin(W, config.side_dim)
            t[pre + "side.norm"] = vec(W, 0.1, 0.5)
    t["final.norm"] = vec(W, 0.1)
    return t
