"""Plain, slow Fibirax forward pass in torch (float64 by default), one function per mechanism, written from the
design's equations.  Shares no code with the served path: whole sequences, dense masks, token-by-token recurrences.

Notation: ``x`` residual ``[T, W]``; per layer  x <- x + s1 * N1(mixer(x));  x <- x + s2 * N2(ff(x))  with N an RMS norm
and s1 / s2 per-channel layer scales.  The mixer runs a windowed softmax attention ("left") and a fixed-decay linear
attention ("right") side by side on the same input and returns  a_l * left + a_r * right.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y * w if w is not None else y


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict], dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2i/dims), then the wavelength-dependent rescaling: long waves are slowed by ``factor``, short
    ones kept, the band between is blended linearly in original/wavelength."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(f.numel()):
        wave = 2.0 * math.pi / float(f[n])
        if wave < orig / high:
            continue
        if wave > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / wave - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """x ``[T, heads, d]``: the first 2 * len(freqs) entries are turned pairwise, (2i, 2i + 1) by pos * f_i."""
    r = 2 * freqs.numel()
    ang = pos.to(freqs.dtype)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out = x.clone()
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


def capped_window_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0,
                            cap: float = 0.0, sink: bool = True) -> torch.Tensor:
    """q ``[T, H, dk]``, k ``[T, G, dk]``, v ``[T, G, dv]`` of one sequence -> ``[T, H, dv]``.  Scores are scaled, bounded
    by cap * tanh(s / cap), limited to the last ``window`` positions, and normalised with 1 + sum exp (``sink``)."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    seen = (dist >= 0) & ((dist < window) if window > 0 else torch.ones_like(dist, dtype=torch.bool))
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // rep].T) * scale
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        out[:, hd] = (e / ((1.0 if sink else 0.0) + e.sum(dim=1, keepdim=True))) @ v[:, hd // rep]
    return out


def window_sink_attention(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """The left mixer: projections, per-head q / k norm, partial rotation, the attention above, output projection."""
    T = h.shape[0]
    H, G, dk, dv = int(spec["heads"]), int(spec.get("kv_heads", spec["heads"])), int(spec["dim"]), int(spec["vdim"])
    q = (h @ t["q"].T).view(T, H, dk)
    k = (h @ t["k"].T).view(T, G, dk)
    v = (h @ t["v"].T).view(T, G, dv)
    if "q.norm" in t:
        q = rms(q, eps, t["q.norm"])
    if "k.norm" in t:
        k = rms(k, eps, t["k.norm"])
    rot = spec.get("rot")
    if rot and int(rot.get("dims", 0)) > 0:
        f = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"), dtype=h.dtype)
        q, k = rotate_pairs(q, torch.arange(T), f), rotate_pairs(k, torch.arange(T), f)
    out = capped_window_attention(q, k, v, float(spec["scale"]), int((spec.get("mask") or {}).get("size", 0)),
                                  float(spec.get("softcap") or 0.0))
    return out.reshape(T, H * dv) @ t["o"].T


def retention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay, state: Optional[torch.Tensor] = None):
    """q, k ``[T, H, dk]`` (k already scaled), v ``[T, H, dv]``: S_t = d_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by
    token.  Returns (o ``[T, H, dv]``, the final state ``[H, dk, dv]``)."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for n in range(T):
        for hd in range(H):
            S[hd] = float(decay[hd]) * S[hd] + torch.outer(k[n, hd], v[n, hd])
            o[n, hd] = S[hd].T @ q[n, hd]
    return o, S


def retention(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """The right mixer: k scaled by dk^-1/2, the scan above, every head's read-out made unit-RMS, gated by silu(W_g h)
    and projected."""
    T = h.shape[0]
    H, dk, dv = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
    q = (h @ t["q"].T).view(T, H, dk)
    k = (h @ t["k"].T).view(T, H, dk) * dk ** -0.5
    v = (h @ t["v"].T).view(T, H, dv)
    o, _ = retention_scan(q, k, v, spec["decay"])
    g = h @ t["g"].T
    return (rms(o, eps).reshape(T, H * dv) * (g * torch.sigmoid(g))) @ t["o"].T


def clamped_expert(h: torch.Tensor, t: Dict[str, torch.Tensor], pre: str, limit: float) -> torch.Tensor:
    g = (h @ t[pre + "gate"].T).clamp(max=limit)
    u = (h @ t[pre + "up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[pre + "down"].T


def route(z: torch.Tensor, corr: torch.Tensor, top: int, groups: int, keep: int):
    """Softmax scores; the choice uses score + correction restricted to the ``keep`` groups whose best choice score is
    largest; the weights are the chosen plain scores over their sum.  Returns (ids ``[T, top]``, weights)."""
    s = torch.softmax(z, dim=-1)
    c = s + corr
    T, E = c.shape
    if groups > 1 and keep < groups:
        per = E // groups
        best = c.view(T, groups, per).max(dim=-1).values
        kept = torch.zeros(T, groups, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        c = torch.where(kept[:, :, None].expand(T, groups, per).reshape(T, E), c, torch.full_like(c, float("-inf")))
    ids = c.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def routed_ff(h: torch.Tensor, spec: dict, t: Dict[str, torch.Tensor]) -> torch.Tensor:
    r = spec["router"]
    E, ident, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    grp = r.get("groups") or {}
    corr = t["correction"].to(h.dtype) if "correction" in t else torch.zeros(E + ident, dtype=h.dtype)
    ids, w = route(h @ t["router"].to(h.dtype).T, corr, top, int(grp.get("count", 1)),
                   int(grp.get("keep", grp.get("count", 1))))
    out = torch.zeros_like(h)
    limit = float(spec["expert"]["limit"])
    for n in range(h.shape[0]):
        for j in range(top):
            e = int(ids[n, j])
            y = clamped_expert(h[n:n + 1], t, f"e{e}.", limit)[0] if e < E else h[n]
            out[n] += w[n, j] * y
    if spec.get("shared"):
        out = out + clamped_expert(h, t, "shared.", float(spec["shared"]["limit"]))
    return out


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` (a list) receives the residual after every layer."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        lt = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
        if layer["type"] != "parallel":
            raise NotImplementedError(layer["type"])
        m = layer["mixer"]
        left = window_sink_attention(x, m["left"], {k[9:]: v for k, v in lt.items() if k.startswith("mix.left.")}, eps)
        right = retention(x, m["right"], {k[10:]: v for k, v in lt.items() if k.startswith("mix.right.")}, eps)
        y = float(m["left_scale"]) * left + float(m["right_scale"]) * right
        y = rms(y, eps, lt["norm1"])
        x = x + (y * lt["ls1"] if "ls1" in lt else y)
        if layer.get("mlp") is not None:
            y = routed_ff(x, layer["mlp"], {k[4:]: v for k, v in lt.items() if k.startswith("mlp.")})
            y = rms(y, eps, lt["norm2"])
            x = x + (y * lt["ls2"] if "ls2" in lt else y)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms(x, eps, t["final.norm"]) @ t["head"].T


def greedy(config: dict, tensors: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(config, tensors, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out
