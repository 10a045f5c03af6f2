"""Fibirax: a decoder whose sublayers read the fp32 residual stream ITSELF and are normed on the way out,

    x <- x + s1 * N1(mixer(x));        x <- x + s2 * N2(ff(x)),

with N an RMS norm and s1 / s2 per-channel layer scales.  The one mixer type, ``parallel``, runs two mixers side by side
on the same input and adds them with fixed weights, ``a_l * left + a_r * right``:

  left    grouped-query softmax attention: q and k are RMS-normed per head and rotated over their first dimensions (pair
          (2i, 2i + 1), frequencies rescaled by wavelength), the scaled scores pass ``c * tanh(s / c)``, a position sees
          its last ``mask.size`` positions only, and the softmax denominator carries an extra 1 (a sink of score 0
          without a value).  Keys and values live in the paged pools.
  right   retention: linear attention with one fixed decay per head, ``S <- d_h S + (k / sqrt(dk)) v^T``, ``o = S^T q``;
          each head's read-out is made unit-RMS, gated by ``silu(W_g x)`` and projected.  The fp32 state lives in a slot
          pool per live sequence.

So a layer keeps pages AND a state slot.  One GEMM produces every projection of both mixers; both write their head
outputs side by side into one buffer, and one GEMM over the two output projections placed side by side forms the mixer's
result.  The branch weights ride along: ``N(a_l L + a_r R) = sign(a_l) N'(L + (a_r / a_l) R)`` with N' using ``eps /
a_l^2``, so ``a_r / a_l`` scales the right branch's fp32 read-outs before they are rounded and nothing else changes.

Feed-forward: a mixture of experts with softmax scores over the routed AND identity experts, a selection bias, expert
groups of which only the best may be chosen, weights renormalised over the chosen, identity experts that return the
token's own row, and a shared expert for every token.  Experts are clamped GLUs.

The modules follow the calling convention of ``ModelShard.forward`` (reference:
worker/distributed/model_shard.py:205-215): ``layer(h, attention_mask=, position_ids=, past_key_value=, use_cache=)
-> (h, present)`` with ``h`` the packed fp32 residual ``[n_tok, width]`` of one step and ``past_key_value`` a
``RaggedLayerCache``.  Matrix products are torch GEMMs; everything between them is a kernel of ``mixer_ops``.  There
is no dense / CPU mode.

Checkpoint names: ``embed``, ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``; linear weights are ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import mixer_ops
from .paged_layer import RaggedLayerCache
from .petipel_layer import _param
from .sanesun_layer import PlainRMSNorm, ScaledFloatEmbedding, _pad8
from .worker.distributed.model_shard import ModelShard

GLU_ALPHA = 1.702          # the experts' gate is g * sigmoid(1.702 g); fixed by the design
WEIGHT_SUM_FLOOR = 1e-20   # added to the sum of the chosen scores before the weights are divided by it


class FibiraxConfig:
    """``config.json`` of the design, plus the attribute names the rest of the framework reads from a config."""

    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.architecture = raw.get("architecture", "Fibirax")
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.width = int(raw["width"])
        self.vocab = int(raw["vocab"])
        self.eps = float(raw["norm"]["eps"])
        self.embed_scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        for i, layer in enumerate(self.layers):
            if layer["type"] != "parallel":
                raise NotImplementedError(f"layer {i}: unknown mixer type {layer['type']!r}")
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            if int(left["heads"]) % int(left.get("kv_heads", left["heads"])):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if len(right["decay"]) != int(right["heads"]):
                raise ValueError(f"layer {i}: one decay per retention head")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise NotImplementedError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
                r = mlp["router"]
                total = int(r["experts"]) + int(r.get("identity", 0))
                groups = r.get("groups") or {}
                if total % int(groups.get("count", 1)):
                    raise ValueError(f"layer {i}: experts do not divide into {groups['count']} groups")
        # names shared with the other model classes
        self.hidden_size = self.width
        self.vocab_size = self.vocab
        self.num_hidden_layers = len(self.layers)
        self.num_attention_heads = max(int(l["mixer"]["left"]["heads"]) for l in self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FibiraxConfig":
        return cls(raw)

    def kv_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        m = self.layers[i]["mixer"]["left"]
        return int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])

    def state_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        m = self.layers[i]["mixer"]["right"]
        return int(m["heads"]), int(m["dim"]), int(m["vdim"])


def wavelength_scaled_frequencies(dims: int, base: float, scaling: Optional[Dict[str, Any]]) -> torch.Tensor:
    """float64 ``[dims / 2]``: ``f_i = base^(-2i / dims)``; with ``scaling`` (factor, low, high, original) a frequency
    whose wavelength ``l = 2 pi / f`` is below ``original / high`` is kept, above ``original / low`` divided by
    ``factor``, and in between blended with ``s = (original / l - low) / (high - low)``: ``(1 - s) f / factor + s f``."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > orig / low:
                f = f / factor
            elif wave >= orig / high:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


class ParallelMixer(nn.Module):
    """Soft-capped windowed sink attention beside retention; see the module docstring.  Launches per step: the input
    GEMM, q/k norm + rotary + append, attention, retention scan, gated head norm, the output GEMM."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        left, right = spec["left"], spec["right"]
        lt = {k[5:]: v for k, v in t.items() if k.startswith("left.")}
        rt = {k[6:]: v for k, v in t.items() if k.startswith("right.")}
        self.eps = eps
        # left
        self.H, self.G = int(left["heads"]), int(left.get("kv_heads", left["heads"]))
        self.dk, self.dv = int(left["dim"]), int(left["vdim"])
        self.scale = float(left["scale"])
        self.softcap = float(left.get("softcap") or 0.0)
        self.window = int((left.get("mask") or {}).get("size", 0))
        rot = left.get("rot") or {}
        freqs = wavelength_scaled_frequencies(int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), rot.get("scaling"))
        self.register_buffer("freqs", freqs.to(device) if freqs.numel() else None, persistent=False)
        self.q_norm = _param(lt["q.norm"], device, dtype) if "q.norm" in lt else None
        self.k_norm = _param(lt["k.norm"], device, dtype) if "k.norm" in lt else None
        self.register_buffer("sink", torch.zeros(self.H, dtype=torch.float32, device=device), persistent=False)
        # right
        self.Hr, self.dkr, self.dvr = int(right["heads"]), int(right["dim"]), int(right["vdim"])
        self.register_buffer("decay", torch.tensor([float(d) for d in right["decay"]], dtype=torch.float32, device=device),
                             persistent=False)
        sections = [lt["q"], lt["k"], lt["v"], rt["q"], rt["k"], rt["v"], rt["g"]]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        # the two output projections side by side; the branch weights are folded as the module docstring says
        a_l, a_r = float(spec["left_scale"]), float(spec["right_scale"])
        c = a_l if a_l != 0.0 else 1.0
        self.right_gain = a_r / c
        self.norm_sign = 1.0 if c > 0 else -1.0
        self.norm_eps = eps / (c * c)
        self.Kl, self.Kr = self.H * self.dv, self.Hr * self.dvr
        w_ol = lt["o"] if a_l != 0.0 else torch.zeros_like(lt["o"])
        w_out = torch.cat([w_ol, rt["o"]], dim=1)
        pad = -w_out.shape[1] % 8
        if pad:
            w_out = torch.cat([w_out, w_out.new_zeros(w_out.shape[0], pad)], dim=1)
        self.K_pad = pad
        self.w_out = _param(w_out, device, dtype)
        self.tensor_cores = mixer_ops.mixed_prompt_attention_supported(self.H, self.G, self.dk, self.dv, False, False, False,
                                                                       self.w_in.dtype) and self.Kl % 2 == 0

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st, n, c = cache.state, h.shape[0], self.cuts
        H, G, dk, dv, Hr, dkr, dvr = self.H, self.G, self.dk, self.dv, self.Hr, self.dkr, self.dvr
        proj = F.linear(h, self.w_in)
        buf = torch.empty((n, self.w_out.shape[1]), dtype=h.dtype, device=h.device)
        if self.K_pad:
            buf[:, self.Kl + self.Kr:].zero_()
        # left: attention over the pages
        q, k, v = proj[:, c[0]:c[0] + H * dk], proj[:, c[1]:c[1] + G * dk], proj[:, c[2]:c[2] + G * dv]
        mixer_ops.qknorm_rotary_append(q, k, v, self.q_norm, self.k_norm, self.eps, self.freqs, cache.k_pool, cache.v_pool,
                                       st.slot_mapping, st.tok_pos, H, interleaved=True)
        attn = buf[:, :self.Kl].unflatten(1, (H, dv))
        if self.tensor_cores:
            tiles, _ = st.prompt_tiles(1, mixer_ops.PROMPT_TILE_TOKENS)
            mixer_ops.mixed_prompt_attention(attn, q.unflatten(1, (H, dk)), cache.k_pool, cache.v_pool, st.block_tables,
                                             tiles, st.tok_pos, self.scale, sink=self.sink, window=self.window,
                                             max_context=st.max_context(), softcap=self.softcap)
        else:
            mixer_ops.mixed_paged_attention(attn, q.unflatten(1, (H, dk)), cache.k_pool, cache.v_pool, st.block_tables,
                                            st.tok_row, st.tok_pos, self.scale, sink=self.sink, window=self.window,
                                            softcap=self.softcap)
        # right: retention over the state slots
        o = mixer_ops.retention_scan(proj[:, c[3]:c[3] + Hr * dkr], proj[:, c[4]:c[4] + Hr * dkr],
                                     proj[:, c[5]:c[5] + Hr * dvr], self.decay, dkr ** -0.5, cache.rstate, st.scan_seqs,
                                     plan=st.scan_plan(ctas_per_seq=Hr * ((dvr + 31) // 32)))
        mixer_ops.head_norm_act_gate(o, None, proj[:, c[6]:c[6] + Hr * dvr], self.eps, h.dtype, gate_act="silu",
                                     out_scale=self.right_gain, out=buf[:, self.Kl:self.Kl + self.Kr])
        return F.linear(buf, self.w_out)


class GroupedSoftmaxMoE(nn.Module):
    """Routed experts weighted on the way OUT, identity experts, a shared expert; see the module docstring.  The router
    reads the fp32 residual; tokens are sorted by expert and pushed through the experts' clamped GLUs: one grouped launch
    each way (this library's kernel for steps of few rows, the vendor's grouped GEMM for long prompt steps, both with
    the experts' row offsets read on the device), or one vendor GEMM per expert in fp32."""

    GROUPED_MAX_ROWS = 2048

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], device, dtype):
        super().__init__()
        r = spec["router"]
        self.E, self.ident, self.top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
        groups = r.get("groups") or {}
        self.groups, self.keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
        self.limit = float(spec["expert"]["limit"])
        self.w_router = _param(t["router"], device, torch.float32)
        self.correction = _param(t["correction"], device, torch.float32) if "correction" in t else None
        if self.w_router.shape[0] != self.E + self.ident:
            raise ValueError("the router has one output per routed and identity expert")
        self.w_gu = self.w_down = None
        if self.E:
            self.w_gu = _param(torch.stack([torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]], dim=0) for e in range(self.E)]),
                               device, dtype)                                                        # [E, 2 ff, W]
            self.w_down = _param(torch.stack([t[f"e{e}.down"] for e in range(self.E)]), device, dtype)  # [E, W, ff]
        self.grouped = bool(self.E) and (mixer_ops.grouped_linear_supported(self.w_gu.shape[2], self.w_gu.dtype)
                                         and mixer_ops.grouped_linear_supported(self.w_down.shape[2], self.w_down.dtype))
        self._ar: Optional[torch.Tensor] = None
        self.shared_limit = 0.0
        self.ws_gu = self.ws_down = None
        if spec.get("shared"):
            self.shared_limit = float(spec["shared"]["limit"])
            self.ws_gu = _param(torch.cat([t["shared.gate"], t["shared.up"]], dim=0), device, dtype)
            self.ws_down = _param(t["shared.down"], device, dtype)

    def _arange(self, n: int, device) -> torch.Tensor:
        """``arange(n)`` on the device, cut from a cached longer one."""
        if self._ar is None or self._ar.numel() < n or self._ar.device != device:
            self._ar = torch.arange(max(n, 4096), device=device)
        return self._ar[:n]

    def _route(self, x: torch.Tensor):
        """``(expert ids int32 [n, top], weights fp32 [n, top])`` from the fp32 residual rows."""
        return mixer_ops.softmax_group_topk(F.linear(x, self.w_router), self.correction, self.top, self.groups, self.keep,
                                            sum_floor=WEIGHT_SUM_FLOOR)

    def _activate(self, z: torch.Tensor) -> torch.Tensor:
        """What stands between an expert's two matrices; subclasses with other experts override this and ``_route``."""
        if z.shape[0] == 0:
            return z[:, :z.shape[1] // 2]
        return mixer_ops.clamped_glu(z, self.limit, GLU_ALPHA)

    def forward(self, h: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """``h``: the sublayer's input in the experts' dtype, ``x``: the same rows in fp32 (the residual)."""
        n, top, E = h.shape[0], self.top, self.E
        ids, w = self._route(x)
        # rows in expert order; where each expert's rows start comes from the sorted ids themselves (a search, not a
        # count: no value ever travels to the host)
        # 16-bit keys: the radix sort takes two passes where 64-bit keys take eight (expert counts stay far below 2^15)
        sorted_ids, order = torch.sort(ids.reshape(-1).to(torch.int16), stable=True)
        where = torch.empty_like(order)
        where[order] = self._arange(n * top, h.device)
        ys = h.new_empty((0, h.shape[1]))
        if E:
            offsets = torch.searchsorted(sorted_ids, self._arange(E + 1, h.device).to(torch.int16)).to(torch.int32)
            xs = mixer_ops.gather_rows(h, order, top)      # identity rows ride at the end and are never multiplied
            if self.grouped and n * top <= self.GROUPED_MAX_ROWS:
                y = self._activate(mixer_ops.grouped_linear(xs, self.w_gu, offsets))
                ys = mixer_ops.grouped_linear(y, self.w_down, offsets)
            elif self.grouped and hasattr(torch, "_grouped_mm"):
                # long prompt steps: the vendor's grouped GEMM, which also reads the offsets on the device
                ends = offsets[1:]
                y = self._activate(torch._grouped_mm(xs, self.w_gu.transpose(1, 2), offs=ends))
                ys = torch._grouped_mm(y, self.w_down.transpose(1, 2), offs=ends)
            else:
                # fp32, or sizes off the 16-byte grid: one vendor GEMM per expert; the counts come to the host once
                bounds = offsets.tolist()
                gu = torch.empty((n * top, self.w_gu.shape[1]), dtype=h.dtype, device=h.device)
                for e in range(E):
                    lo, hi = bounds[e], bounds[e + 1]
                    if hi > lo:
                        torch.mm(xs[lo:hi], self.w_gu[e].t(), out=gu[lo:hi])
                routed = bounds[E]
                y = self._activate(gu[:routed])
                ys = torch.empty((n * top, h.shape[1]), dtype=h.dtype, device=h.device)
                for e in range(E):
                    lo, hi = bounds[e], bounds[e + 1]
                    if hi > lo:
                        torch.mm(y[lo:hi], self.w_down[e].t(), out=ys[lo:hi])
        shared = None
        if self.ws_gu is not None:
            shared = F.linear(mixer_ops.clamped_glu(F.linear(h, self.ws_gu), self.shared_limit, GLU_ALPHA), self.ws_down)
        return mixer_ops.weighted_expert_combine(ys, where, ids, w, x, shared, E)


class FibiraxDecoderLayer(nn.Module):
    """One layer; see the module docstring.  The residual update also hands the next sublayer its input: the new
    residual in the weights' dtype (``pending_norm`` of the step's shared state; nothing when the weights are fp32)."""

    def __init__(self, config: FibiraxConfig, layer_idx: int, t: Dict[str, torch.Tensor], device=None, dtype=None):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx, self.kind, self.eps = layer_idx, spec["type"], config.eps
        self.mixer = ParallelMixer(spec["mixer"], {k[4:]: v for k, v in t.items() if k.startswith("mix.")}, self.eps,
                                   device, dtype)
        self.norm1 = _param(t["norm1"], device, dtype)
        self.ls1 = _param(t["ls1"], device, dtype) if "ls1" in t else None
        self.mlp = None
        if spec.get("mlp") is not None:
            self.mlp = GroupedSoftmaxMoE(spec["mlp"], {k[4:]: v for k, v in t.items() if k.startswith("mlp.")}, device, dtype)
            self.norm2 = _param(t["norm2"], device, dtype)
            self.ls2 = _param(t["ls2"], device, dtype) if "ls2" in t else None
        self.low_precision = self.norm1.dtype != torch.float32

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None,
                past_key_value: Optional[RaggedLayerCache] = None, use_cache: bool = True):
        if not isinstance(past_key_value, RaggedLayerCache):
            raise TypeError("FibiraxDecoderLayer needs a RaggedLayerCache handle in past_key_value")
        x, st = hidden_states, past_key_value.state
        if x.dtype != torch.float32 or x.dim() != 2:
            raise TypeError("the residual stream is a packed fp32 [n_tok, width] tensor")
        lp = self.low_precision
        h = x
        if lp:
            h = st.pending_norm if st.pending_norm is not None else mixer_ops.cast_rows(x, self.norm1.dtype)
        st.pending_norm = None
        y = self.mixer(h, past_key_value)
        h = mixer_ops.branch_postnorm_residual(x, y, self.mixer.norm_sign, None, 0.0, self.norm1, self.ls1,
                                               self.mixer.norm_eps, want_copy=lp)
        if self.mlp is not None:
            y = self.mlp(h if lp else x, x)
            h = mixer_ops.branch_postnorm_residual(x, y, 1.0, None, 0.0, self.norm2, self.ls2, self.eps, want_copy=lp)
        st.pending_norm = h if lp else None
        return x, (past_key_value if use_cache else None)


def build_shards(config: FibiraxConfig, tensors: Dict[str, torch.Tensor], ranges: Sequence[Tuple[int, int]],
                 device: str, dtype: torch.dtype) -> List[ModelShard]:
    """``ModelShard``s for layer ranges holding the weights of a checkpoint's name -> tensor dict."""
    shards = []
    total = config.num_hidden_layers
    for start, end in ranges:
        layers = []
        for i in range(start, end):
            pre = f"l{i}."
            layers.append(FibiraxDecoderLayer(config, i, {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)},
                                              device, dtype))
        embed = norm = head = None
        if start == 0:
            embed = ScaledFloatEmbedding(config.vocab, config.width, device=device, dtype=dtype, scale=config.embed_scale)
            embed.weight.requires_grad_(False)
            with torch.no_grad():
                embed.weight.copy_(tensors["embed"])
        if end == total:
            norm = PlainRMSNorm(config.width, config.eps, device, dtype)
            head = nn.Linear(config.width, config.vocab, bias=False, device=device, dtype=dtype)
            head.weight.requires_grad_(False)
            with torch.no_grad():
                norm.weight.copy_(tensors["final.norm"])
                head.weight.copy_(tensors["head"])
        shards.append(ModelShard.from_layers(config, layers, start, end, device, dtype, embed, norm, head,
                                             model_id="fibirax").eval())
    return shards


def random_checkpoint(config: FibiraxConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights with the checkpoint's names and shapes (for tests and benchmarks; not a trained model).
    Projections ~ N(0, gain / fan_in); norm weights, layer scales and the selection bias are chosen so that every term
    of the design contributes."""
    g = torch.Generator().manual_seed(seed)
    W = config.width

    def lin(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def near_one(*shape, s=0.1):
        return (1.0 + s * torch.randn(*shape, generator=g)).to(dtype)

    t: Dict[str, torch.Tensor] = {"embed": (torch.randn(config.vocab, W, generator=g) / config.embed_scale).to(dtype)}
    for i, layer in enumerate(config.layers):
        pre = f"l{i}."
        left, right = layer["mixer"]["left"], layer["mixer"]["right"]
        H, G, dk, dv = int(left["heads"]), int(left.get("kv_heads", left["heads"])), int(left["dim"]), int(left["vdim"])
        t[pre + "mix.left.q"], t[pre + "mix.left.k"] = lin(H * dk, W, 2.0), lin(G * dk, W, 2.0)
        t[pre + "mix.left.v"], t[pre + "mix.left.o"] = lin(G * dv, W), lin(W, H * dv)
        t[pre + "mix.left.q.norm"], t[pre + "mix.left.k.norm"] = near_one(dk, s=0.3), near_one(dk, s=0.3)
        Hr, dkr, dvr = int(right["heads"]), int(right["dim"]), int(right["vdim"])
        t[pre + "mix.right.q"], t[pre + "mix.right.k"] = lin(Hr * dkr, W), lin(Hr * dkr, W)
        t[pre + "mix.right.v"], t[pre + "mix.right.g"] = lin(Hr * dvr, W), lin(Hr * dvr, W, 2.0)
        t[pre + "mix.right.o"] = lin(W, Hr * dvr)
        t[pre + "norm1"], t[pre + "ls1"] = near_one(W), (0.5 + 0.1 * torch.randn(W, generator=g)).to(dtype)
        mlp = layer.get("mlp")
        if mlp:
            r = mlp["router"]
            E, ident, ff = int(r["experts"]), int(r.get("identity", 0)), int(mlp["expert"]["ff"])
            for e in range(E):
                t[pre + f"mlp.e{e}.gate"], t[pre + f"mlp.e{e}.up"] = lin(ff, W, 2.0), lin(ff, W, 2.0)
                t[pre + f"mlp.e{e}.down"] = lin(W, ff)
            t[pre + "mlp.router"] = lin(E + ident, W, 3.0)
            t[pre + "mlp.correction"] = (0.1 * torch.randn(E + ident, generator=g)).to(dtype)
            if mlp.get("shared"):
                fs = int(mlp["shared"]["ff"])
                t[pre + "mlp.shared.gate"], t[pre + "mlp.shared.up"] = lin(fs, W, 2.0), lin(fs, W, 2.0)
                t[pre + "mlp.shared.down"] = lin(W, fs)
            t[pre + "norm2"], t[pre + "ls2"] = near_one(W), (0.5 + 0.1 * torch.randn(W, generator=g)).to(dtype)
    t["final.norm"] = near_one(W)
    t["head"] = lin(config.vocab, W)
    return t
