"""Plain, slow Vatazen forward pass in torch (float64 by default), one function per mechanism, written from the
design's equations.  Shares no code with the served path: whole sequences, dense masks, a loop over experts.

Notation: ``x`` residual ``[T, W]``.  Per layer

    x <- x + N1(sigmoid(R1 x + r1) * mixer(shift(x)));   x <- x + N2(sigmoid(R2 x + r2) * ff(x));   x <- x + side(x, tok)

with N an RMS norm whose weight is stored around zero, ``shift`` a per-channel blend of a token's row with the row of
the token before it, and ``side`` a small gated read of a per-layer slice of a second embedding table.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h: torch.Tensor, mu: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row t becomes h_t + (h_(t-1) - h_t) * mu with the UNSHIFTED previous row; ``before`` (zeros when None) stands
    in front of row 0."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1).to(h.dtype)
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mu


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """``(frequencies [dims/2] float64, gain)``.  f_i = base^(-2i/dims).  With scaling: d(t) = dims ln(original /
    (2 pi t)) / (2 ln base); lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1); r_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1); the frequency is r_i f_i / factor + (1 - r_i) f_i and cos and sin are both multiplied by
    gain = 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def d(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor, gain: float) -> torch.Tensor:
    """x ``[T, ..., d]``: entries (2i, 2i + 1), i < len(freqs), are turned by pos * f_i; cos and sin carry ``gain``."""
    r = 2 * freqs.numel()
    ang = pos.to(torch.float64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [freqs.numel()]
    c = (torch.cos(ang) * gain).to(x.dtype).reshape(shape)
    s = (torch.sin(ang) * gain).to(x.dtype).reshape(shape)
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out = x.clone()
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


def visible(T: int, window: int = 0, chunk: int = 0) -> torch.Tensor:
    """bool ``[T, T]``: j <= i, within the last ``window`` positions (window > 0), in the same block of ``chunk``
    positions counted from 0 (chunk > 0)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & (i - j < window)
    if chunk > 0:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[T, H, dk]``, k ``[T, H, dk]``, v ``[T, H, dv]`` -> ``[T, H, dv]``; ``sink [H]`` adds exp(sink_h) to the
    denominator only."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(s.dtype)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype)[:, None, None] - m)
    return torch.einsum("hij,jhd->ihd", e / den, v)


def latent_attention(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """Keys and values are up-projections of one normed latent row; one rotated key part is shared by the heads."""
    T = h.shape[0]
    H, dn, dr, dv, rank = (int(spec[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    pos = torch.arange(T)
    rot = spec["rot"]
    freqs, gain = yarn_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    q = (h @ t["q"].T).reshape(T, H, dn + dr)
    down = h @ t["dkv"].T
    c = rms(down[:, :rank], eps) * t["dkv.norm"]
    k_rot = rotate_pairs(down[:, rank:].reshape(T, 1, dr), pos, freqs, gain)
    q_rot = rotate_pairs(q[..., dn:], pos, freqs, gain)
    k_plain = (c @ t["uk"].T).reshape(T, H, dn)
    v = (c @ t["uv"].T).reshape(T, H, dv)
    qq = torch.cat([q[..., :dn], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, dr)], dim=-1)
    window = int((spec.get("mask") or {}).get("size", 0))
    o = softmax_attention(qq, kk, v, float(spec["scale"]), visible(T, window=window), t.get("sink"))
    return o.reshape(T, H * dv) @ t["o"].T


def differential_attention(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, combined as a1 - lambda a2, made unit-RMS per head and scaled
    by 1 - diff; keys of one block of ``mask.size`` positions only."""
    T = h.shape[0]
    H, G, dk, dv = int(spec["heads"]), int(spec.get("kv_heads", spec["heads"])), int(spec["dim"]), int(spec["vdim"])
    diff = float(spec["diff"])
    q = (h @ t["q"].T + t["q.b"]).reshape(T, H, 2, dk)
    k = (h @ t["k"].T + t["k.b"]).reshape(T, G, 2, dk)
    v = (h @ t["v"].T + t["v.b"]).reshape(T, G, dv)
    q = rms(q, eps) * t["q.norm"]
    k = rms(k, eps) * t["k.norm"]
    rep = H // G
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    chunk = int((spec.get("mask") or {}).get("size", 0))
    mask = visible(T, chunk=chunk)
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, float(spec["scale"]), mask)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, float(spec["scale"]), mask)
    lam = torch.exp((t["lq1"] * t["lk1"]).sum()) - torch.exp((t["lq2"] * t["lk2"]).sum()) + diff
    o = rms(a1 - lam * a2, eps) * (1.0 - diff)
    return o.reshape(T, H * dv) @ t["o"].T + t["o.b"]


def route(z: torch.Tensor, top: int):
    """The ``top`` largest logits per row (ties: lowest index) and the softmax over just those."""
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1)


def routed_ff(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor]) -> torch.Tensor:
    """Experts W_down relu(W_up h)^2, weighted by the softmax over the chosen router logits."""
    E, top = int(spec["router"]["experts"]), int(spec["router"]["top"])
    ids, w = route(h @ t["router"].T + t["router.b"], top)
    out = torch.zeros_like(h)
    for e in range(E):
        y = torch.relu(h @ t[f"e{e}.up"].T) ** 2 @ t[f"e{e}.down"].T
        out = out + y * (w * (ids == e)).sum(dim=-1, keepdim=True)
    return out


def side_input(x: torch.Tensor, e: torch.Tensor, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """What the per-layer token input adds: ``e [T, d]`` are the tokens' rows of this layer's slice of the table."""
    y = (gelu_tanh(x @ t["side.gate"].T) * e) @ t["side.proj"].T
    return rms(y, eps) * t["side.norm"]


def layer_forward(x: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor], eps: float,
                  side_rows: Optional[torch.Tensor]) -> torch.Tensor:
    mix = {k[4:]: v for k, v in t.items() if k.startswith("mix.")}
    h = token_shift(x, t["shift"])
    if spec["type"] == "latent_attention":
        y = latent_attention(h, spec["mixer"], mix, eps)
    elif spec["type"] == "attention":
        y = differential_attention(h, spec["mixer"], mix, eps)
    else:
        raise NotImplementedError(spec["type"])
    y = y * torch.sigmoid(x @ t["rg1"].T + t["rg1.b"])
    x = x + rms(y, eps) * (1.0 + t["norm1"])
    if spec.get("mlp") is not None:
        y = routed_ff(x, spec["mlp"], {k[4:]: v for k, v in t.items() if k.startswith("mlp.")})
        y = y * torch.sigmoid(x @ t["rg2"].T + t["rg2.b"])
        x = x + rms(y, eps) * (1.0 + t["norm2"])
    if side_rows is not None:
        x = x + side_input(x, side_rows, t, eps)
    return x


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence; ``layers_out`` (a list) receives the residual after every layer."""
    t = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    tok = torch.tensor(list(tokens), dtype=torch.int64)
    x = t["embed"][tok] * float((config.get("embedding") or {}).get("scale", 1.0))
    sd = int((config.get("token_side") or {}).get("dim", 0))
    for i, spec in enumerate(config["layers"]):
        pre = f"l{i}."
        lt = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
        rows = t["side.embed"][tok][:, i * sd:(i + 1) * sd] if sd > 0 else None
        x = layer_forward(x, spec, lt, eps, rows)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * (1.0 + t["final.norm"])
    return x @ t["embed"].T


def greedy(config: dict, tensors: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(config, tensors, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
